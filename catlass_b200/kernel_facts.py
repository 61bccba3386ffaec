"""Measured facts about the kernels that the benchmark quotes next to its own timings.

DRAM traffic per launch cannot be measured by the benchmark itself (it needs the profiler's counters), so the
figures below are carried from single-launch `ncu` captures (`dram__bytes_read.sum + dram__bytes_write.sum`) of the
named workloads; each entry names the kernel build facts it was captured with.  `check()` compares those facts
with the kernel sources, so a figure cannot silently outlive a change of the tiling it was measured on: when it
fails, re-capture and update the entry.
"""
import os
import re

_CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")

DRAM_TRAFFIC = {
    # grouped W8A8 on CTA pairs, `moe_small` workload (8 experts, 16384 rows, K=7168, N=4096, Zipf loads):
    # traffic grows in proportion to rows and experts, so a launch over R rows of the full workload moves
    # bytes * R / 16384
    "w8a8_pair_kernel/moe_small": {
        "bytes": 540.7e6, "rows": 16384,
        "facts": {"w8a8_gemm_pair.cuh": {"kPairTileM": 256, "kPairBN": 256, "kStages": 6}},
    },
    # few-token W8A8, decode_a (16 x 14336 x 4096)
    "w8a8_smallm_kernel/decode_a": {
        "bytes": 59.2e6,
        "facts": {"w8a8_smallm.cuh": {"kSmallMTileN": 128, "kSmallMMaxSplits": 8}},
    },
    # W4A8, M=128 N=8192 K=8192 group 128
    "w4a8_gemm_kernel/w4a8": {
        "bytes": 36.8e6,
        "facts": {"w4a8_gemm.cuh": {"kW4Channels": 128, "kW4Tokens": 128}},
    },
    # MX 8192^3 (E4M3, E2M1) on the single-CTA kernel (CB200_MX_PAIR=0 in developer builds)
    "mx_gemm_kernel/mxfp8": {
        "bytes": 342.4e6,
        "facts": {"mx_gemm.cuh": {"kMxBlockN": 256, "kMxStages": 4}},
    },
    # MX 8192^3 on CTA pairs (the default for large dense problems)
    "mx_pair_kernel/mxfp8": {
        "bytes": 444.3e6,
        "facts": {"mx_gemm_pair.cuh": {"kMxPairStages": 6}, "mx_gemm.cuh": {"kMxBlockN": 256}},
    },
    "mx_pair_kernel/mxfp4": {
        "bytes": 211.4e6,
        "facts": {"mx_gemm_pair.cuh": {"kMxPairStages": 6}, "mx_gemm.cuh": {"kMxBlockN": 256}},
    },
    "mx_gemm_kernel/mxfp4": {
        "bytes": 184.4e6,
        "facts": {"mx_gemm.cuh": {"kMxBlockN": 256, "kMxStages": 4}},
    },
    # quantisers, bf16 32768 x 7168 (rows staged through shared memory)
    "quant_int8_staged_kernel/quant_int8": {
        "bytes": 669.0e6,
        "facts": {"quant_int8.cuh": {"kQuantInt8Threads": 256}},
    },
    "mx_quantize_staged_kernel/quant_mx": {
        "bytes": 676.7e6,
        "facts": {"mx_quantize.cuh": {"kMxQuantThreads": 256}},
    },
}


def _constant(source_text, name):
    m = re.search(r"constexpr\s+int\s+" + re.escape(name) + r"\s*=\s*(\d+)\s*;", source_text)
    return int(m.group(1)) if m else None


def check():
    """Returns the list of entries whose recorded build facts no longer match the kernel sources."""
    stale = []
    for key, entry in DRAM_TRAFFIC.items():
        for fname, facts in entry["facts"].items():
            text = open(os.path.join(_CSRC, fname)).read()
            for name, value in facts.items():
                if _constant(text, name) != value:
                    stale.append(f"{key}: {fname} {name} is {_constant(text, name)}, captured with {value}")
    return stale


def traffic(key, scale=1.0):
    """DRAM bytes per launch for `key`, or None when the entry is stale."""
    entry = DRAM_TRAFFIC.get(key)
    if entry is None or any(s.startswith(key + ":") for s in check()):
        return None
    return entry["bytes"] * scale
