"""The reference arm of bench.py runs on host cores only: check on CPU that it prints one JSON line with the
keys the bench contract names, for the same workload string as the main arm."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-seconds", "1"], capture_output=True, text=True, timeout=600,
                         cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["metric"] == "w8a8_grouped_gemm_tops" and line["unit"] == "TOPS"
    assert line["config"]["workload"].startswith("moe_grouped_slice_m_w8a8: 64 experts, K=7168, N=4096")
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["value"] > 0


def test_reference_arm_config_equals_the_main_arm_config():
    """Both arms describe the workload with the same `config` object (the reference arm adds one key)."""
    import sys as _sys
    _sys.path.insert(0, ROOT)
    import bench
    cfg = bench.moe_config(bench.MOE, "split", 1)
    assert set(cfg) == {"workload", "placement", "rows_per_rank", "l2", "weights"}
    assert cfg["rows_per_rank"] == [131072]
    assert sum(bench.moe_config(bench.MOE, "split", 8)["rows_per_rank"]) == 131072


def test_recorded_dram_traffic_matches_the_kernel_sources():
    """The profiler figures the bench quotes name the tile constants they were captured with."""
    from catlass_b200 import kernel_facts
    assert kernel_facts.check() == []
    assert kernel_facts.traffic("w8a8_pair_kernel/moe_small", 8.0) == 8 * kernel_facts.DRAM_TRAFFIC["w8a8_pair_kernel/moe_small"]["bytes"]
