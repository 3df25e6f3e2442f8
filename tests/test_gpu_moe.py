"""GPU parity of the mixture-of-experts steps around the grouped GEMM: block alignment (bit-exact against
the reference's stored outputs and the oracle), row gather (bit-exact), silu_and_mul (the reference's
tolerance), the fused silu_and_mul + MXFP4 quantisation, the weighted combine, and the whole expert MLP.
Mirrors tests/kernel/moe/moe_align_block_size_test.py and tests/kernel/moe_test.py of the reference."""

import numpy as np
import pytest
import torch

import wave_b200 as wb
from conftest import GOLDEN
from oracle import moe_oracle
from oracle import mxfp4_oracle as orc
from wave_b200 import moe, ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_align(topk_ids, experts, block, with_inverse=True):
    n = topk_ids.numel()
    cap = n + experts * (block - 1)
    sorted_ids = torch.empty(cap, dtype=torch.int32, device=DEV)
    expert_ids = torch.full((-(cap // -block),), -1, dtype=torch.int32, device=DEV)
    post = torch.empty(1, dtype=torch.int32, device=DEV)
    inverse = torch.empty(n, dtype=torch.int32, device=DEV) if with_inverse else None
    wb.moe_align_block_size(topk_ids.to(DEV), experts, block, sorted_ids, expert_ids, post, inverse)
    return sorted_ids.cpu().numpy(), expert_ids.cpu().numpy(), int(post.item()), None if inverse is None else inverse.cpu().numpy()


def test_moe_align_block_size_golden():
    g = np.load(GOLDEN / "moe_align.npz")
    ci = 0
    while f"case{ci}_params" in g.files:
        tokens, topk, block, experts = (int(v) for v in g[f"case{ci}_params"])
        ids = torch.from_numpy(g[f"case{ci}_topk_ids"])
        sorted_ids, expert_ids, post, inverse = run_align(ids, experts, block)
        assert post == int(g[f"case{ci}_post_pad"][0])
        assert np.array_equal(sorted_ids, g[f"case{ci}_sorted_ids"])
        assert np.array_equal(expert_ids, g[f"case{ci}_expert_ids"])
        assert np.array_equal(sorted_ids[inverse], np.arange(tokens * topk))
        ci += 1
    assert ci >= 6


@pytest.mark.parametrize("num_tokens", [1, 33, 256, 4096])
@pytest.mark.parametrize("block_size", [16, 32, 64, 128])
@pytest.mark.parametrize("num_experts", [4, 8, 64, 256])
def test_moe_align_block_size_matches_oracle(num_tokens, block_size, num_experts):
    """The reference test's sweep (moe_align_block_size_test.py:14-17), widened; int32 and int64 ids."""
    g = torch.Generator().manual_seed(num_tokens * 7 + block_size + num_experts)
    _, topk_ids = torch.topk(torch.rand(num_tokens, num_experts, generator=g), k=2, dim=1)
    exp = moe_oracle.moe_align_block_size(topk_ids.numpy(), num_experts, block_size,
                                          topk_ids.numel() + num_experts * (block_size - 1),
                                          -((topk_ids.numel() + num_experts * (block_size - 1)) // -block_size))
    for ids in (topk_ids, topk_ids.to(torch.int32)):
        sorted_ids, expert_ids, post, inverse = run_align(ids, num_experts, block_size)
        assert post == exp[2] and post % block_size == 0
        assert np.array_equal(sorted_ids, exp[0]) and np.array_equal(expert_ids, exp[1]) and np.array_equal(inverse, exp[3])


def test_moe_align_block_size_skewed_and_empty():
    ids = torch.full((1000, 2), 3, dtype=torch.int64)  # every pair on one expert, all others empty
    exp = moe_oracle.moe_align_block_size(ids.numpy(), 8, 128, 2000 + 8 * 127, -((2000 + 8 * 127) // -128))
    sorted_ids, expert_ids, post, inverse = run_align(ids, 8, 128)
    assert post == 2048 and np.array_equal(sorted_ids, exp[0]) and np.array_equal(expert_ids, exp[1])
    with pytest.raises(ValueError):  # outputs too small for the worst case
        wb.moe_align_block_size(ids.to(DEV), 8, 128, torch.empty(2000, dtype=torch.int32, device=DEV),
                                torch.empty(30, dtype=torch.int32, device=DEV), torch.empty(1, dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("row_bytes", [256, 8, 100])
def test_gather_rows_bit_exact(row_bytes):
    g = torch.Generator().manual_seed(row_bytes)
    src = torch.randint(0, 256, (50, row_bytes), dtype=torch.uint8, generator=g)
    _, ids = torch.topk(torch.rand(50, 8, generator=g), k=2, dim=1)
    sorted_ids, _, post, _ = run_align(ids, 8, 16, with_inverse=False)
    out = torch.full((post, row_bytes), 0xAB, dtype=torch.uint8, device=DEV)
    moe.gather_rows(src.to(DEV), torch.from_numpy(sorted_ids).to(DEV), 100, 2, out)
    exp = torch.zeros(post, row_bytes, dtype=torch.uint8)
    real = torch.from_numpy(sorted_ids[:post]) < 100
    exp[real] = src[torch.from_numpy(sorted_ids[:post])[real].long() // 2]
    assert torch.equal(out.cpu(), exp)


@pytest.mark.parametrize("m,n", [(1, 128), (33, 1024), (64, 200), (5, 30)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_silu_and_mul_as_the_reference_tests_it(m, n, dtype):
    """get_wave_silu_and_mul_kernel / silu_and_mul of tests/kernel/moe_test.py:43-79 (rtol 1e-1, atol 1e-2 there)."""
    kernel, symbols = wb.get_silu_and_mul_kernel(m, n, dtype)
    silu = wb.wave_compile(wb.WaveCompileOptions(subs=symbols, canonicalize=True, schedule=wb.SchedulingType.NONE), kernel)
    g = torch.Generator().manual_seed(m + n)
    gate = torch.randn(m, n, generator=g).to(dtype)
    up = torch.randn(m, n, generator=g).to(dtype)
    out = torch.zeros(m, n, dtype=dtype, device=DEV)
    silu(gate.to(DEV), up.to(DEV), out)
    ref = moe_oracle.silu_and_mul(gate, up)
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-1, atol=1e-2)
    # and much tighter: the kernel's fast exponential and division are good to ~1e-6 relative, then one
    # rounding to the output type
    if dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-6)
    else:
        assert int(orc.bf16_ulp_distance(out, ref).max()) <= 1


def test_silu_and_mul_on_column_halves_with_fused_quantisation():
    rows, inter = 300, 512
    g = torch.Generator().manual_seed(3)
    h = (torch.randn(rows, 2 * inter, generator=g) * 2).to(torch.bfloat16)
    hd = h.to(DEV)
    out, q, s = wb.silu_and_mul(hd[:, :inter], hd[:, inter:], out=torch.empty(rows, inter, dtype=torch.bfloat16, device=DEV),
                                quantize=True)
    ref = moe_oracle.silu_and_mul(h[:, :inter], h[:, inter:])
    assert int(orc.bf16_ulp_distance(out, ref).max()) <= 1
    # The codes come from the kernel's own f32 values, which differ from the oracle's by a few ulps, so a value
    # next to a rounding boundary may land on the neighbouring code: nearly all codes and scales are those of the
    # oracle's quantiser, and every dequantised value is within the quantiser's worst-case error of the reference
    # (2 units of the block's scale: values between 6 and 8 units are clamped to 6).
    q_ref, s_ref = orc.quantize_mxfp4(ref)
    assert float((s.cpu() != s_ref).float().mean()) < 1e-3
    qc, qr = q.cpu(), q_ref
    nib_diff = ((qc & 0xF) != (qr & 0xF)).float().mean() + ((qc >> 4) != (qr >> 4)).float().mean()
    assert float(nib_diff) < 2e-3
    deq = orc.dequant_mxfp4(qc, s.cpu())
    unit = orc.e8m0_to_f32(s.cpu().float()).repeat_interleave(32, dim=1)
    assert bool(((deq - ref).abs() <= unit * 2.0 + 1e-6).all())
    # quantise-only form gives the same codes
    _, q2, s2 = wb.silu_and_mul(hd[:, :inter], hd[:, inter:], quantize=True)
    assert torch.equal(q, q2) and torch.equal(s, s2)


def test_combine_matches_weighted_sum():
    T, k, cols = 77, 2, 200
    g = torch.Generator().manual_seed(9)
    y = torch.randn(300, cols, generator=g).to(torch.bfloat16)
    row_of = torch.randint(0, 300, (T * k,), generator=g, dtype=torch.int32)
    row_of[5] = -1
    w = torch.rand(T * k, generator=g)
    out = torch.empty(T, cols, dtype=torch.bfloat16, device=DEV)
    moe.combine(y.to(DEV), row_of.to(DEV), w.to(DEV), k, out)
    contrib = torch.where((row_of >= 0).view(-1, 1), w.view(-1, 1) * y.float()[row_of.clamp(min=0).long()], torch.zeros(1))
    ref = contrib.view(T, k, cols).sum(1)
    assert int(orc.bf16_ulp_distance(out, ref).max()) <= 1


@pytest.mark.parametrize("T,E,K,inter", [(33, 8, 512, 256), (256, 4, 1024, 512), (1, 8, 256, 128)])
def test_expert_mlp_against_oracle(T, E, K, inter):
    """Whole MXFP4 expert MLP against the oracle's expert loop (torch_ref_moe's structure). Tolerance: the
    reference's own MoE tolerance (rtol 1e-1, atol 1e-2, tests/kernel/moe_test.py:258), which absorbs the
    re-quantisation of hidden activations whose f32 values differ from the oracle's in the last bits."""
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    w1, w1s, w2, w2s = [], [], [], []
    for e in range(E):
        q, s = orc.quantize_mxfp4(torch.randn(2 * inter, K, generator=g) * 0.05)
        w1.append(q); w1s.append(s)
        q, s = orc.quantize_mxfp4(torch.randn(K, inter, generator=g) * 0.05)
        w2.append(q); w2s.append(s)
    mlp = wb.MXFP4ExpertMLP([t.to(DEV) for t in w1], [t.to(DEV) for t in w1s], [t.to(DEV) for t in w2],
                            [t.to(DEV) for t in w2s], top_k=2)
    out = mlp(x.to(DEV), logits.to(DEV))
    ref = moe_oracle.expert_mlp(x, w1, w1s, w2, w2s, logits, 2)
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-1, atol=1e-2)
    # and relative to the output's own scale: mean error well under one percent of the rms
    rel = (out.cpu().float() - ref).abs().mean() / ref.pow(2).mean().sqrt()
    assert float(rel) < 2e-2
    ops.check_device_status()


def test_device_driven_grouped_gemm_matches_host_offsets_form():
    """wb200_mxfp4_moe_gemm (routing read from the alignment kernel's device outputs) against
    wb200_mxfp4_grouped_gemm (row offsets given by the host) on the same routed rows: identical bits."""
    from wave_b200.grouped import ExpertWeights, grouped_scaled_gemm, moe_scaled_gemm
    T, E, K, N, k = 700, 5, 512, 384, 2
    g = torch.Generator().manual_seed(21)
    _, ids = torch.topk(torch.rand(T, E, generator=g), k=k, dim=1)
    ids[:, :] = torch.where(ids == 3, torch.zeros_like(ids), ids)  # expert 3 gets no rows
    n = T * k
    cap = (n + E * 255 + 255) // 256 * 256
    sorted_ids, expert_ids, post, _ = run_align(ids, E, 256)
    sorted_ids = np.concatenate([sorted_ids, np.full(cap - sorted_ids.size, n, dtype=np.int32)])
    xq = torch.randint(0, 256, (T, K // 2), dtype=torch.uint8, generator=g)
    xs = torch.randint(122, 129, (T, K // 32), dtype=torch.uint8, generator=g)
    w = [torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g) for _ in range(E)]
    ws = [torch.randint(122, 129, (N, K // 32), dtype=torch.uint8, generator=g) for _ in range(E)]
    experts = ExpertWeights([t.to(DEV) for t in w], [t.to(DEV) for t in ws])
    a = torch.empty(cap, K // 2, dtype=torch.uint8, device=DEV)
    a_s = torch.empty(cap, K // 32, dtype=torch.uint8, device=DEV)
    sid = torch.from_numpy(sorted_ids).to(DEV)
    moe.gather_rows(xq.to(DEV), sid, n, k, a)
    moe.gather_rows(xs.to(DEV), sid, n, k, a_s)
    c_dev = torch.full((cap, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    eid = torch.full((cap // 256,), -1, dtype=torch.int32, device=DEV)
    eid[: expert_ids.size] = torch.from_numpy(expert_ids).to(DEV)[: cap // 256]
    moe_scaled_gemm(a, a_s, experts, eid, torch.tensor([post], dtype=torch.int32, device=DEV), c_dev)
    counts = torch.bincount(ids.reshape(-1), minlength=E).tolist()
    offsets = [0]
    for cnt in counts:
        offsets.append(offsets[-1] + (cnt + 255) // 256 * 256)
    assert offsets[-1] == post
    c_host = torch.empty(post, N, dtype=torch.bfloat16, device=DEV)
    grouped_scaled_gemm(a[:post], a_s[:post], experts, offsets, c_host)
    assert torch.equal(c_dev[:post].view(torch.int16), c_host.view(torch.int16))
    assert bool(c_dev[post:].isnan().all())  # row blocks past the padded total are not touched
    # and against the oracle for one expert's rows
    e = 1
    rows = slice(offsets[e], offsets[e] + counts[e])
    ref = orc.scaled_gemm(a[rows].cpu(), a_s[rows].cpu(), w[e], ws[e])
    assert int(orc.bf16_ulp_distance(c_dev[rows], ref).max()) <= 1
    ops.check_device_status()


def test_expert_mlp_forward_can_be_captured_in_a_cuda_graph():
    """No step of the forward pass reads the routing back to the host."""
    T, E, K, inter = 64, 4, 512, 256
    g = torch.Generator().manual_seed(2)
    w1, w1s, w2, w2s = [], [], [], []
    for e in range(E):
        q, s = orc.quantize_mxfp4(torch.randn(2 * inter, K, generator=g) * 0.05)
        w1.append(q.to(DEV)); w1s.append(s.to(DEV))
        q, s = orc.quantize_mxfp4(torch.randn(K, inter, generator=g) * 0.05)
        w2.append(q.to(DEV)); w2s.append(s.to(DEV))
    mlp = wb.MXFP4ExpertMLP(w1, w1s, w2, w2s, top_k=2)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    logits = torch.randn(T, E, generator=g).to(DEV)
    eager = mlp(x, logits)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = mlp(x, logits)
    x.copy_(torch.randn(T, K, generator=g).to(torch.bfloat16))  # new tokens, same buffers
    graph.replay()
    torch.cuda.synchronize()
    again = mlp(x, logits)
    torch.cuda.synchronize()
    assert torch.equal(captured, again) and not torch.equal(captured, eager)
    ops.check_device_status()


def test_quantize_scatter_equals_quantise_then_gather_on_routed_rows():
    T, E, K, k = 300, 6, 1024, 2
    g = torch.Generator().manual_seed(31)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    _, ids = torch.topk(torch.rand(T, E, generator=g), k=k, dim=1)
    sorted_ids, _, post, inverse = run_align(ids, E, 256)
    cap = (T * k + E * 255 + 255) // 256 * 256
    q = torch.full((cap, K // 2), 0xEE, dtype=torch.uint8, device=DEV)
    s = torch.full((cap, K // 32), 0xEE, dtype=torch.uint8, device=DEV)
    moe.quantize_scatter(x.to(DEV), torch.from_numpy(inverse).to(DEV), k, q, s)
    q_ref, s_ref = orc.quantize_mxfp4(x.float())
    routed = torch.from_numpy(sorted_ids[:post]).long()
    real = routed < T * k
    pos = torch.arange(post)[real]
    assert torch.equal(q.cpu()[pos], q_ref[routed[real] // k]) and torch.equal(s.cpu()[pos], s_ref[routed[real] // k])
    untouched = torch.ones(cap, dtype=torch.bool)
    untouched[pos] = False
    assert bool((q.cpu()[untouched] == 0xEE).all()) and bool((s.cpu()[untouched] == 0xEE).all())


def test_silu_and_mul_row_limit_from_device():
    rows, n = 512, 256
    g = torch.Generator().manual_seed(8)
    h = torch.randn(rows, 2 * n, generator=g).to(torch.bfloat16).to(DEV)
    out = torch.full((rows, n), -3.0, dtype=torch.bfloat16, device=DEV)
    limit = torch.tensor([384], dtype=torch.int32, device=DEV)
    wb.silu_and_mul(h[:, :n], h[:, n:], out=out, num_rows=limit)
    ref = moe_oracle.silu_and_mul(h[:384, :n].cpu(), h[:384, n:].cpu())
    assert int(orc.bf16_ulp_distance(out[:384], ref).max()) <= 1
    assert bool((out[384:] == -3.0).all())
