"""The reference's own pytest assertions for the quantized-matmul operators
(tests/optest/tests/test_{07,10,12,32,42,47,48,53,54}_*.py), run against this library through the binding that
mirrors the reference's torch_catlass package: same call, same expected value, same tolerance, device "cuda"."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_catlass(cuda):
    from catlass_b200 import torch_catlass as tc
    return tc


def test_quant_matmul(torch_catlass):
    """tests/optest/tests/test_12_quant_matmul.py:11-20"""
    m, n, k = 128, 64, 256
    a = torch.randint(-8, 8, (m, k), dtype=torch.int8, device="cuda")
    b = torch.randint(-8, 8, (k, n), dtype=torch.int8, device="cuda")
    s = torch.randn(n, dtype=torch.float16, device="cuda").abs() * 0.1
    ps = torch.randn(m, dtype=torch.float16, device="cuda").abs() * 0.1
    r = torch_catlass.quant_matmul(a, b, s, ps)
    e = torch.matmul(a.float(), b.float()) * s * ps.unsqueeze(1)
    assert r.shape == (m, n) and r.dtype == torch.float16
    assert torch.allclose(r.float(), e, rtol=1e-1, atol=1e-1)


def test_quant_optimized_matmul_tla(torch_catlass):
    """tests/optest/tests/test_42_*: bf16 output, B given transposed (the op's default), scales (1, N) / (1, M)."""
    m, n, k = 256, 512, 1024
    a = torch.randint(-8, 8, (m, k), dtype=torch.int8, device="cuda")
    b = torch.randint(-8, 8, (n, k), dtype=torch.int8, device="cuda")
    s = torch.randn(1, n, dtype=torch.float32, device="cuda").abs() * 0.1
    ps = torch.randn(1, m, dtype=torch.float32, device="cuda").abs() * 0.1
    r = torch_catlass.quant_optimized_matmul_tla(a, b, s, ps)
    e = torch.matmul(a.float(), b.float().t()) * s * ps.reshape(m, 1)
    assert r.shape == (m, n) and r.dtype == torch.bfloat16
    assert torch.allclose(r.float(), e, rtol=1e-1, atol=1e-1)


def _grouped_expected(a, b, scale, per_token_scale, group_sizes):
    out, offset = [], 0
    for i, size in enumerate(group_sizes):
        part = torch.matmul(a[offset:offset + size].float(), b[i].float())
        out.append(part * scale[i].float() * per_token_scale[offset:offset + size].float().unsqueeze(1))
        offset += size
    return torch.cat(out, dim=0)


def test_grouped_matmul_slice_m_per_token_dequant_moe(torch_catlass):
    """tests/optest/tests/test_07_*.py:11-39: int32 prefix-sum list, float scales, half output."""
    g, m_total, n, k = 4, 512, 128, 64
    group_list = torch.tensor([128, 256, 384, 512], dtype=torch.int32, device="cuda")
    a = torch.randint(-8, 8, (m_total, k), dtype=torch.int8, device="cuda")
    b = torch.randint(-8, 8, (g, k, n), dtype=torch.int8, device="cuda")
    scale = torch.randn(g, n, dtype=torch.float32, device="cuda").abs() * 0.1
    pts = torch.randn(m_total, dtype=torch.float32, device="cuda").abs() * 0.1
    result = torch_catlass.grouped_matmul_slice_m_per_token_dequant(a, b, group_list, scale, pts)
    expected = _grouped_expected(a, b, scale, pts, [128] * 4)
    assert result.shape == (m_total, n) and result.dtype == torch.float16 and result.device.type == "cuda"
    assert torch.allclose(result.float(), expected, rtol=1e-1, atol=1e-1)


def test_grouped_matmul_slice_m_per_token_dequant_multistage_and_950(torch_catlass):
    """Examples 10 and 47: int64 list, bf16 scales, bf16 output; ragged groups."""
    sizes = [100, 0, 300, 112]
    g, n, k = len(sizes), 256, 128
    m_total = sum(sizes)
    group_list = torch.tensor(sizes, dtype=torch.int64).cumsum(0).cuda()
    a = torch.randint(-8, 8, (m_total, k), dtype=torch.int8, device="cuda")
    b = torch.randint(-8, 8, (g, k, n), dtype=torch.int8, device="cuda")
    scale = (torch.randn(g, n, device="cuda").abs() * 0.1).to(torch.bfloat16)
    pts = (torch.randn(m_total, device="cuda").abs() * 0.1).to(torch.bfloat16)
    expected = _grouped_expected(a, b, scale, pts, sizes)
    for op in (torch_catlass.grouped_matmul_slice_m_per_token_dequant_multistage,
               torch_catlass.ascend950_grouped_matmul_slice_m_per_token_dequant):
        result = op(a, b, group_list, scale, pts)
        assert result.shape == (m_total, n) and result.dtype == torch.bfloat16
        assert torch.allclose(result.float(), expected, rtol=1e-1, atol=1e-1)


@pytest.mark.parametrize("quant_mode", [0, 1], ids=["per_tensor", "per_channel"])
def test_grouped_per_tensor_per_channel_dequant(torch_catlass, quant_mode):
    """tests/optest/tests/test_48_*.py: fp32 scale bits zero-extended to 64-bit words, half output."""
    import struct
    group_sizes, n, k, scale_per_tensor = (128, 128), 128, 256, 0.5
    m_total = sum(group_sizes)
    a = torch.randint(-4, 4, (m_total, k), dtype=torch.int8)
    b = torch.randint(-4, 4, (len(group_sizes), k, n), dtype=torch.int8)
    pcs = torch.randn(n, dtype=torch.float32).abs() * 0.1
    words = [struct.unpack("<I", struct.pack("<f", float(v)))[0] for v in pcs]
    pcs_u64 = torch.tensor(words, dtype=torch.int64).cuda()
    group_list = torch.tensor(group_sizes, dtype=torch.int64).cumsum(0).cuda()
    result = torch_catlass.ascend950_grouped_matmul_slice_m_per_tensor_per_channel_dequant(
        a.cuda(), b.cuda(), group_list, pcs_u64, scalePerTensor=scale_per_tensor, quantMode=quant_mode)
    expected, offset = [], 0
    for gid, size in enumerate(group_sizes):
        part = a[offset:offset + size].float() @ b[gid].float()
        expected.append(part * scale_per_tensor if quant_mode == 0 else part * pcs.unsqueeze(0))
        offset += size
    expected = torch.cat(expected, dim=0)
    assert result.shape == (m_total, n) and result.dtype == torch.float16
    assert torch.allclose(result.float().cpu(), expected, rtol=1e-2, atol=1e-2)


def _pack_int4(data):
    """The packer of tests/optest/tests/test_32_w4a8_matmul.py:11-28 (pairs along the last axis, low nibble first)."""
    k, n = data.shape
    if n % 2 != 0:
        data = torch.cat([data, torch.zeros(k, 1, dtype=torch.int8)], dim=1)
    pairs = data.reshape(-1, 2)
    packed = ((pairs[:, 1].int() & 0x0F) << 4) | (pairs[:, 0].int() & 0x0F)
    return packed.to(torch.int8).reshape(k, -1)


def test_w4a8_matmul(torch_catlass):
    """tests/optest/tests/test_32_w4a8_matmul.py:31-70: C = 1.5 * (A @ B), half output, B packed along N."""
    m, n, k = 256, 256, 256
    a = torch.randint(-8, 8, (m, k), dtype=torch.int8, device="cuda")
    b_orig = torch.randint(-8, 8, (k, n), dtype=torch.int8)
    result = torch_catlass.w4a8_matmul(a, _pack_int4(b_orig).cuda(), "float16", transA=False, transB=False)
    expected = (torch.matmul(a.float().cpu(), b_orig.float()) * 1.5).to(torch.float16)
    assert result.shape == (m, n) and result.dtype == torch.float16 and result.device.type == "cuda"
    assert torch.allclose(result.float().cpu(), expected.float(), rtol=1e-1, atol=1e-1)


def _quantize_axis_last(matrix, emax=8, fp8_max=448.0):
    """E4M3 MX quantisation of the rows of `matrix` in blocks of 32 (the rule of mx_golden.py:177-221)."""
    m, n = matrix.shape
    blocks = (n + 31) // 32
    padded = torch.zeros(m, blocks * 32)
    padded[:, :n] = matrix
    view = padded.view(m, blocks, 32)
    exp = (torch.floor(torch.log2(view.abs().amax(dim=-1).clamp(min=1e-12))) - emax).clamp(-128, 127)
    scale = torch.exp2(exp)
    q = (view / scale.unsqueeze(-1)).clamp(-fp8_max, fp8_max).to(torch.float8_e4m3fn)
    deq = (q.float() * scale.unsqueeze(-1)).reshape(m, blocks * 32)[:, :n].contiguous()
    q = q.reshape(m, blocks * 32)[:, :n].contiguous()
    ks = (blocks + 1) // 2 * 2
    sp = torch.ones(m, ks)
    sp[:, :blocks] = scale
    return q, sp.to(torch.float8_e8m0fnu), deq


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)],
                         ids=["nn", "nt", "tn", "tt"])
def test_ascend950_fp8_mx_matmul_aswt(torch_catlass, trans_a, trans_b):
    """tests/optest/tests/test_53_ascend950_fp8_mx_matmul_aswt.py:21-55 with the input layouts of
    mx_golden.py:prepare_fp8_mx_inputs."""
    m, n, k = 256, 512, 1024
    a32 = torch.randn(m, k) * 10.0 - 5.0
    b32 = torch.randn(k, n) * 10.0 - 5.0
    a8, a_scale, a_deq = _quantize_axis_last(a32)
    bt8, bt_scale, bt_deq = _quantize_axis_last(b32.t().contiguous())
    b8, b_deq = bt8.t().contiguous(), bt_deq.t().contiguous()
    a_scale = a_scale.reshape(m, a_scale.shape[1] // 2, 2).contiguous()
    b_scale = bt_scale.reshape(n, bt_scale.shape[1] // 2, 2).contiguous()          # [n, KS/2, 2]
    if trans_a:
        a8 = a8.t().contiguous()
        a_scale = a_scale.permute(1, 0, 2).contiguous()
    if trans_b:
        b8 = b8.t().contiguous()
    else:
        b_scale = b_scale.permute(1, 0, 2).contiguous()                            # [KS/2, n, 2]
    expected = a_deq @ b_deq
    result = torch_catlass.ascend950_fp8_mx_matmul_aswt(a8.cuda(), b8.cuda(), a_scale.cuda(), b_scale.cuda(),
                                                        transA=trans_a, transB=trans_b)
    assert result.shape == (m, n) and result.dtype == torch.float32 and result.device.type == "cuda"
    assert torch.allclose(result.cpu(), expected, rtol=1e-2, atol=1e-2), \
        f"max diff = {(result.cpu() - expected).abs().max().item()}"


@pytest.mark.parametrize("trans_b", [False, True], ids=["b_kn", "b_nk"])
def test_ascend950_mx_grouped_matmul_slice_m(torch_catlass, trans_b):
    """tests/optest/tests/test_55_*.py with the inputs of mx_golden.py:prepare_fp8_mx_grouped_slice_m_inputs: group
    sizes (not prefix sums), per-group B and B scales, fp32 output, allclose(1e-2)."""
    group_sizes, n, k = (128, 128), 128, 256
    m = sum(group_sizes)
    a32 = torch.randn(m, k) * 10.0 - 5.0
    a8, a_scale, a_deq = _quantize_axis_last(a32)
    a_scale = a_scale.reshape(m, a_scale.shape[1] // 2, 2).contiguous()
    b_list, s_list, expected, offset = [], [], [], 0
    for size in group_sizes:
        b32 = torch.randn(k, n) * 10.0 - 5.0
        bt8, bt_scale, bt_deq = _quantize_axis_last(b32.t().contiguous())        # [n][k], scales [n][KS]
        scale = bt_scale.reshape(n, bt_scale.shape[1] // 2, 2)                   # [n, KS/2, 2]
        if trans_b:
            b_list.append(bt8.contiguous())
            s_list.append(scale.contiguous())
        else:
            b_list.append(bt8.t().contiguous())                                  # [k][n]
            s_list.append(scale.permute(1, 0, 2).contiguous())                   # [KS/2, n, 2]
        expected.append(a_deq[offset:offset + size] @ bt_deq.t())
        offset += size
    result = torch_catlass.ascend950_mx_grouped_matmul_slice_m(
        a8.cuda(), torch.stack(b_list).cuda(), torch.tensor(group_sizes, dtype=torch.int64).cuda(), a_scale.cuda(),
        torch.stack(s_list).cuda(), transA=False, transB=trans_b)
    expected = torch.cat(expected, dim=0)
    assert result.shape == (m, n) and result.dtype == torch.float32
    assert torch.allclose(result.cpu(), expected, rtol=1e-2, atol=1e-2)


def test_ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant(torch_catlass):
    """The reference op's signature (tests/optest/torch_catlass/ops/ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant.py)
    on the example's own run (4 groups, m = 256, n = 512, k = 1024): the dequantised output within the example's
    tolerance (2^-4 relative, doubled) of SwiGLU applied to the dequantised matmul."""
    group_sizes, n, k = (64, 64, 64, 64), 512, 1024
    m = sum(group_sizes)
    a32 = torch.randn(m, k)
    a8, a_scale, a_deq = _quantize_axis_last(a32)
    a_scale = a_scale.reshape(m, a_scale.shape[1] // 2, 2).contiguous()
    b_list, s_list, expected, offset = [], [], [], 0
    for size in group_sizes:
        b32 = torch.randn(k, n)
        bt8, bt_scale, bt_deq = _quantize_axis_last(b32.t().contiguous())
        b_list.append(bt8.contiguous())
        s_list.append(bt_scale.reshape(n, bt_scale.shape[1] // 2, 2).contiguous())
        c = a_deq[offset:offset + size] @ bt_deq.t()
        act, gate = c.chunk(2, dim=-1)
        expected.append(act / (torch.exp(-act) + 1) * gate)
        offset += size
    expected = torch.cat(expected, dim=0)
    q, q_scale = torch_catlass.ascend950_fp8_mx_grouped_matmul_slice_m_swiglu_mx_quant(
        a8.cuda(), torch.stack(b_list).cuda(), a_scale.cuda(), torch.stack(s_list).cuda(),
        torch.tensor(group_sizes, dtype=torch.int64).cuda(), transB=True)
    assert q.shape == (m, n // 2) and q.dtype == torch.float8_e4m3fn and q_scale.shape == (m, n // 64)
    scales = torch.pow(2.0, q_scale.view(torch.uint8).cpu().float() - 127.0).repeat_interleave(32, dim=1)
    deq = q.cpu().float() * scales
    err = (deq - expected).abs() / expected.abs().clamp(min=1.0)
    assert err.max().item() <= 2 * 2.0 ** -4, err.max().item()


@pytest.mark.parametrize("deterministic", [False, True], ids=["no_deter", "deter"])
def test_ascend950_fp8_mx_grouped_matmul_finalize_routing_no_deter(torch_catlass, deterministic):
    """The reference op's signature (tests/optest/torch_catlass/ops/
    ascend950_fp8_mx_grouped_matmul_finalize_routing_no_deter.py) on the example's own run
    (4 groups, m = n = k = 128, prefix-sum list, batch 16, dp 2) with bias and shared input switched on."""
    g, m, n, k, batch, dp = 4, 128, 128, 128, 16, 2
    sizes = [12, 25, 38, 53]
    a8, a_scale, a_deq = _quantize_axis_last(torch.randn(m, k))
    a_scale = a_scale.reshape(m, a_scale.shape[1] // 2, 2).contiguous()
    b_list, s_list, c_parts, offset = [], [], [], 0
    bias = torch.randn(g, n).to(torch.bfloat16)
    for i, size in enumerate(sizes):
        bt8, bt_scale, bt_deq = _quantize_axis_last(torch.randn(k, n).t().contiguous())
        b_list.append(bt8.t().contiguous())                                                  # [k][n]
        s_list.append(bt_scale.reshape(n, bt_scale.shape[1] // 2, 2).permute(1, 0, 2).contiguous())
        c_parts.append(a_deq[offset:offset + size] @ bt_deq.t() + bias[i].float().unsqueeze(0))
        offset += size
    c = torch.cat(c_parts, dim=0)
    logit = torch.randn(m)
    row_index = torch.arange(m, dtype=torch.int64) % batch
    shared = torch.randn(batch // dp, n).to(torch.bfloat16)
    expected = torch.zeros(batch, n)
    expected[3:3 + batch // dp] += 0.5 * shared.float()
    expected.index_add_(0, row_index, logit.unsqueeze(1) * c)
    group_list = torch.tensor(sizes, dtype=torch.int64).cumsum(0)
    op = (torch_catlass.ascend950_fp8_mx_grouped_matmul_finalize_routing if deterministic
          else torch_catlass.ascend950_fp8_mx_grouped_matmul_finalize_routing_no_deter)
    result = op(
        a8.cuda(), torch.stack(b_list).cuda(), a_scale.cuda(), torch.stack(s_list).cuda(), group_list.cuda(),
        logit.cuda(), row_index.cuda(), bias.cuda(), shared.cuda(), batch, data_parallel_size=dp,
        shared_input_weight=0.5, shared_input_offset=3, group_list_type=0, trans_a=False, trans_b=False)
    assert result.shape == (batch, n) and result.dtype == torch.float32
    assert torch.allclose(result.cpu(), expected, rtol=1e-2, atol=1e-2), (result.cpu() - expected).abs().max().item()


def test_grouped_matmul_slice_k_per_token_dequant(torch_catlass):
    """tests/optest/tests/test_11_grouped_matmul_slice_k_per_token_dequant.py:11-40"""
    g, m, n, k_total = 4, 128, 128, 256
    group_list = torch.tensor([64, 128, 192, 256], dtype=torch.int64, device="cuda")
    a = torch.randint(-8, 8, (k_total, m), dtype=torch.int8, device="cuda")
    b = torch.randint(-8, 8, (k_total, n), dtype=torch.int8, device="cuda")
    scale = (torch.randn(g, n, device="cuda").abs() * 0.1).to(torch.bfloat16)
    pts = (torch.randn(g, m, device="cuda").abs() * 0.1).to(torch.bfloat16)
    result = torch_catlass.grouped_matmul_slice_k_per_token_dequant(a, b, group_list, scale, pts, transA=True)
    expected, offset = [], 0
    for i in range(g):
        part = torch.matmul(a[offset:offset + 64].T.float(), b[offset:offset + 64].float())
        expected.append(part * scale[i].float() * pts[i].float().unsqueeze(1))
        offset += 64
    expected = torch.stack(expected, dim=0)
    assert result.shape == (g, m, n) and result.dtype == torch.bfloat16
    assert torch.allclose(result.float(), expected, rtol=1e-1, atol=1e-1)
