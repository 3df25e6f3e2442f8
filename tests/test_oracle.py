"""The CPU oracle against the golden vectors generated from the reference itself
(tests/golden/make_golden.py). Runs without a GPU."""

import hashlib

import numpy as np
import torch

from conftest import GOLDEN
from oracle import mxfp4_oracle as orc


def _bits_equal(a: torch.Tensor, b: np.ndarray) -> bool:
    a = a.numpy()
    return bool(((a.view(np.int32) == b.view(np.int32)) | (np.isnan(a) & np.isnan(b))).all())


def test_e2m1_table_all_bytes():
    g = np.load(GOLDEN / "kat_codecs.npz")
    out = orc.mxfp4_to_f32(torch.from_numpy(g["bytes"]))
    assert _bits_equal(out, g["e2m1_f32"])  # includes the sign of -0.0 (code 8)


def test_e8m0_table_all_codes():
    g = np.load(GOLDEN / "kat_codecs.npz")
    out = orc.e8m0_to_f32(torch.arange(256, dtype=torch.uint8))
    assert _bits_equal(out, g["e8m0_f32"])
    assert torch.isnan(out[255]) and out[127] == 1.0 and out[0] == 2.0 ** -127


def test_input_generator_matches_reference_seed5():
    g = np.load(GOLDEN / "gemm_seed5_64x96x128.npz")
    x, w, xs, ws = orc.generate_gemm_afp4wfp4_inputs((64, 96, 128))
    assert w.shape == (64, 96) and not w.is_contiguous()  # transposed view, as the reference returns it
    assert np.array_equal(x.numpy(), g["x"]) and np.array_equal(w.numpy(), g["w"])
    assert np.array_equal(xs.numpy(), g["x_scales"]) and np.array_equal(ws.numpy(), g["w_scales"])


def test_input_generator_1024_digests():
    g = np.load(GOLDEN / "gemm_seed5_1024_sample.npz")
    x, w, xs, ws = orc.generate_gemm_afp4wfp4_inputs((1024, 1024, 1024))
    for name, t in dict(x=x, w=w, x_scales=xs, w_scales=ws).items():
        digest = hashlib.sha256(np.ascontiguousarray(t.numpy()).tobytes()).hexdigest()
        assert digest == str(g[f"sha256_{name}"]), name


def test_gemm_matches_reference_small():
    g = np.load(GOLDEN / "gemm_seed5_64x96x128.npz")
    x, w, xs, ws = (torch.from_numpy(g[k]) for k in ("x", "w", "x_scales", "w_scales"))
    torch.set_num_threads(1)
    out = orc.torch_scaled_gemm_mxfp4(x, w, xs, ws)
    torch.testing.assert_close(out, torch.from_numpy(g["out"]), rtol=1e-6, atol=1e-5)
    # the [N, K/2] entry point agrees with the transposed-view one
    out2 = orc.scaled_gemm(x, xs, w.T.contiguous(), ws)
    torch.testing.assert_close(out2, torch.from_numpy(g["out"]), rtol=1e-6, atol=1e-5)


def test_gemm_matches_reference_wide_scales_and_dequant_bits():
    g = np.load(GOLDEN / "gemm_wide_scales_48x80x256.npz")
    a, b, a_s, b_s = (torch.from_numpy(g[k]) for k in ("a", "b", "a_scale", "b_scale"))
    assert _bits_equal(orc.dequant_mxfp4(a, a_s), g["a_deq"])
    out = orc.scaled_gemm(a, a_s, b, b_s)
    torch.testing.assert_close(out, torch.from_numpy(g["out"]), rtol=1e-6, atol=1e-4)
    # NaN code 255 and the extreme scale codes 0, 1, 254
    assert _bits_equal(orc.dequant_mxfp4(a, torch.from_numpy(g["edge_scale"])), g["edge_deq"])


def test_gemm_1024_sample():
    g = np.load(GOLDEN / "gemm_seed5_1024_sample.npz")
    x, w, xs, ws = orc.generate_gemm_afp4wfp4_inputs((1024, 1024, 1024))
    out = orc.torch_scaled_gemm_mxfp4(x, w, xs, ws)
    torch.testing.assert_close(out[::64, ::64], torch.from_numpy(g["out_sample"]), rtol=1e-5, atol=1e-3)


def test_pack_scales_layout():
    """Every (row, K-block) lands at the documented byte; padding is 127."""
    rows, kb = 200, 10
    s = torch.arange(rows * kb, dtype=torch.int64).reshape(rows, kb).remainder(251).to(torch.uint8)
    packed = orc.pack_scales(s).numpy()
    ka = 2 * ((kb * 32 + 255) // 256)
    assert packed.size == 2 * ka * 512
    for r in (0, 1, 31, 32, 95, 127, 128, 199):
        for j in (0, 3, 4, 9):
            off = ((r // 128) * ka + j // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + j % 4
            assert packed[off] == s[r, j]
    # a padded row and a padded K block
    assert packed[(1 * ka + 0) * 512 + (255 % 32) * 16 + ((255 % 128) // 32) * 4] == orc.SF_PAD
    assert packed[(0 * ka + 2) * 512 + 0 * 16 + 0 * 4 + 2] == orc.SF_PAD  # K block 10


def test_quantizer_round_trip_properties():
    torch.manual_seed(3)
    x = torch.randn(16, 256)
    q, s = orc.quantize_mxfp4(x)
    assert q.shape == (16, 128) and s.shape == (16, 8)
    deq = orc.dequant_mxfp4(q, s)
    # requantising dequantised values is the identity (idempotence)
    q2, s2 = orc.quantize_mxfp4(deq)
    assert torch.equal(orc.dequant_mxfp4(q2, s2), deq)
    # block maxima map into the top octave of E2M1: scaled amax in [4, 8) before clamping
    amax = x.reshape(16, 8, 32).abs().amax(dim=2)
    scaled = amax / torch.pow(torch.tensor(2.0), s.float() - 127)
    assert bool(((scaled >= 4) & (scaled < 8)).all())
    # error bounded by half the largest grid step (2 between 4 and 6, so 1) times the scale,
    # and by the clamp at 6 for values scaled into (6, 8)
    err = (deq - x).abs().reshape(16, 8, 32)
    bound = 2.0 * torch.pow(torch.tensor(2.0), s.float() - 127).unsqueeze(2)
    assert bool((err <= bound).all())
    # all-zero block: scale byte 127, codes 0
    q0, s0 = orc.quantize_mxfp4(torch.zeros(1, 32))
    assert int(s0[0, 0]) == 127 and int(q0.sum()) == 0
    # ties go to the even code: 0.25 -> 0 (code 0), 0.75 -> 1.0 (code 2), 2.5 -> 2 (code 4), 5 -> 4 (code 6)
    t = torch.zeros(1, 32)
    t[0, :5] = torch.tensor([6.0, 0.25, 0.75, 2.5, 5.0])
    qt, st = orc.quantize_mxfp4(t)
    codes = [(int(qt[0, i // 2]) >> (4 * (i % 2))) & 0xF for i in range(5)]
    assert int(st[0, 0]) == 127 and codes == [7, 0, 2, 4, 6]


def test_tolerance_helpers():
    ref = torch.tensor([[1.0, -2.0, 0.0]])
    c = ref.to(torch.bfloat16)
    assert int(orc.bf16_ulp_distance(c, ref).max()) == 0
    up = torch.tensor([[1.0078125, -2.0, -0.0]]).to(torch.bfloat16)  # 1 ulp above 1.0; -0.0 equals +0.0
    assert orc.bf16_ulp_distance(up, ref).flatten().tolist() == [1, 0, 0]


def test_moe_align_block_size_oracle_matches_reference_outputs():
    """oracle/moe_oracle.py against the stored outputs of the reference's moe_align_block_size_pytorch."""
    from oracle import moe_oracle
    g = np.load(GOLDEN / "moe_align.npz")
    ncases = sum(1 for k in g.files if k.endswith("_params"))
    assert ncases >= 6
    for ci in range(ncases):
        tokens, topk, block, experts = (int(v) for v in g[f"case{ci}_params"])
        ref_sorted, ref_experts = g[f"case{ci}_sorted_ids"], g[f"case{ci}_expert_ids"]
        sorted_ids, expert_ids, total, inverse = moe_oracle.moe_align_block_size(
            g[f"case{ci}_topk_ids"], experts, block, ref_sorted.size, ref_experts.size)
        assert total == int(g[f"case{ci}_post_pad"][0])
        assert np.array_equal(sorted_ids, ref_sorted)
        assert np.array_equal(expert_ids, ref_experts)
        assert np.array_equal(sorted_ids[inverse], np.arange(tokens * topk))


def test_mxfp8_oracle_matches_reference_outputs():
    """oracle/mxfp8_oracle.py against the stored outputs of the reference's own MXFP8 generator and oracle."""
    from oracle import mxfp8_oracle
    g = np.load(GOLDEN / "gemm_mxfp8_seed5_64x96x128.npz")
    x, w, xs, ws = mxfp8_oracle.generate_gemm_afp8wfp8_inputs((64, 96, 128))
    assert np.array_equal(x.view(torch.uint8).numpy(), g["x"])
    assert np.array_equal(w.T.contiguous().view(torch.uint8).numpy(), g["w"])
    assert np.array_equal(xs.numpy(), g["x_scales"]) and np.array_equal(ws.numpy(), g["w_scales"])
    torch.set_num_threads(1)
    out = mxfp8_oracle.torch_scaled_gemm_mxfp8(x, w, xs, ws)
    assert np.array_equal(out.numpy(), g["out"])


def test_amd_preshuffle_index_maps_match_reference_outputs():
    """The reference's AMD scale and B pre-shuffles (mxfp_utils.py:98-128), restated as index maps, against the
    outputs the reference itself produced (tests/golden/preshuffle.npz, written by make_golden.py)."""
    g = np.load(GOLDEN / "preshuffle.npz")
    scale, b = torch.from_numpy(g["scale"]), torch.from_numpy(g["b"])
    assert torch.equal(orc.amd_e8m0_shuffle(scale), torch.from_numpy(g["scale_shuffled"]))
    assert torch.equal(orc.amd_b_preshuffle(b), torch.from_numpy(g["b_shuffled"]))
    # a caller who holds weights in the reference's pre-shuffled order gets the row-major bytes back
    assert torch.equal(orc.amd_b_unshuffle(torch.from_numpy(g["b_shuffled"])), b)
    # on aligned shapes the scale shuffle is a permutation
    s2 = torch.randint(0, 255, (512, 64), dtype=torch.uint8, generator=torch.Generator().manual_seed(3))
    assert sorted(orc.amd_e8m0_shuffle(s2).reshape(-1).tolist()) == sorted(s2.reshape(-1).tolist())


def test_mixed_pair_oracle_matches_reference_output():
    """8-bit activations x packed E2M1 weights: the oracle against the output stored from the reference's own
    generators and dequantisation functions (tests/golden/make_golden.py, step 8)."""
    import numpy as np
    from conftest import GOLDEN
    from oracle import mxfp8_oracle as orc8
    g = np.load(GOLDEN / "gemm_mxfp8_mxfp4_seed5_64x96x128.npz")
    x = torch.from_numpy(g["x"]).view(torch.float8_e5m2)
    w = torch.from_numpy(g["w"])  # [N, K/2] packed E2M1
    out = orc8.torch_scaled_gemm_mxfp8_mxfp4(x, w, torch.from_numpy(g["x_scales"]), torch.from_numpy(g["w_scales"]))
    torch.testing.assert_close(out, torch.from_numpy(g["out"]), rtol=1e-6, atol=1e-6 * float(np.abs(g["out"]).max()))
