"""Generate the golden fixtures in this folder from the reference itself.

Run where a checkout of the reference (iree-org/wave) is at hand, giving its path:

    python tests/golden/make_golden.py <path to the reference checkout>

It imports the reference's own module `wave_lang/kernel/wave/utils/mxfp_utils.py` and the torch
helper `tests/kernel/moe/torch_kernels.py` (both pure torch; they run on the CPU without the
reference's compiler stack) and stores their outputs on seeded inputs as small .npz files. The tests compare the oracle in `oracle/` and, on a GPU, the CUDA kernels
against these files, so the pin travels to machines that do not have the reference.
"""

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main(ref_root: str, only_mixed: bool = False) -> None:
    sys.path.insert(0, ref_root)
    from wave_lang.kernel.wave.utils import mxfp_utils as ref  # noqa: E402

    if only_mixed:  # adds the newest fixture without rewriting the others (their archives carry timestamps)
        mixed_pair(ref, reference_mxfp8_functions(ref_root, ref))
        return

    torch.set_num_threads(1)  # fixed summation order inside torch.mm for the stored GEMM outputs

    # 1. Known-answer tables: every packed byte, every scale code.
    all_bytes = torch.arange(256, dtype=torch.uint8).reshape(1, 256)
    e2m1 = ref.mxfp4_to_f32(all_bytes.clone())
    e8m0 = ref.e8m0_to_f32(torch.arange(256, dtype=torch.float32))
    np.savez_compressed(HERE / "kat_codecs.npz", bytes=all_bytes.numpy(), e2m1_f32=e2m1.numpy(),
                        e8m0_f32=e8m0.numpy())

    # 2. The reference's own input generator (seed 5) and GEMM on a small shape.
    shape = (64, 96, 128)
    x, w, xs, ws = ref.generate_gemm_afp4wfp4_inputs(shape, device=torch.device("cpu"))
    out = ref.torchScaledGemmMXFP4(x, w, xs, ws)
    np.savez_compressed(HERE / "gemm_seed5_64x96x128.npz", x=x.numpy(), w=np.ascontiguousarray(w.numpy()),
                        x_scales=xs.numpy(), w_scales=ws.numpy(), out=out.numpy())

    # 3. Wider scale range [124, 130] (the 1024^3 config's distribution) on a ragged small shape,
    #    with the NaN code and the extreme scale codes planted in known places.
    g = torch.Generator().manual_seed(77)
    M, N, K = 48, 80, 256
    a = torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, generator=g)
    b = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=g)
    a_s = torch.randint(124, 131, (M, K // 32), dtype=torch.uint8, generator=g)
    b_s = torch.randint(124, 131, (N, K // 32), dtype=torch.uint8, generator=g)
    out = ref.torchScaledGemmMXFP4(a, b.T, a_s, b_s)
    a_deq = ref.mxfp4_to_f32(a.clone()) * ref.e8m0_to_f32(a_s.repeat_interleave(32, dim=1).to(torch.float32))
    edge_s = a_s.clone()
    edge_s[0, 0], edge_s[1, 1], edge_s[2, 2], edge_s[3, 3] = 255, 0, 254, 1
    edge_deq = ref.mxfp4_to_f32(a.clone()) * ref.e8m0_to_f32(edge_s.repeat_interleave(32, dim=1).to(torch.float32))
    np.savez_compressed(HERE / "gemm_wide_scales_48x80x256.npz", a=a.numpy(), b=b.numpy(), a_scale=a_s.numpy(),
                        b_scale=b_s.numpy(), out=out.numpy(), a_deq=a_deq.numpy(), edge_scale=edge_s.numpy(),
                        edge_deq=edge_deq.numpy())

    # 4. The reference's AMD preshuffles (kept in the API for parity).
    sc = torch.randint(0, 256, (300, 40), dtype=torch.uint8, generator=g)
    bb = torch.randint(0, 256, (64, 128), dtype=torch.uint8, generator=g)
    np.savez_compressed(HERE / "preshuffle.npz", scale=sc.numpy(), scale_shuffled=ref.e8m0_shuffle(sc).numpy(),
                        b=bb.numpy(), b_shuffled=ref.b_preshuffle(bb).numpy())

    # 5. The 1024^3 seed-5 case of the reference's tests: digests of the inputs and a strided
    #    sample of the output (the full arrays are too large to commit).
    x, w, xs, ws = ref.generate_gemm_afp4wfp4_inputs((1024, 1024, 1024), device=torch.device("cpu"))
    torch.set_num_threads(8)
    out = ref.torchScaledGemmMXFP4(x, w, xs, ws)
    digest = {k: hashlib.sha256(np.ascontiguousarray(v.numpy()).tobytes()).hexdigest()
              for k, v in dict(x=x, w=w, x_scales=xs, w_scales=ws).items()}
    np.savez_compressed(HERE / "gemm_seed5_1024_sample.npz", out_sample=out[::64, ::64].numpy(),
                        **{f"sha256_{k}": np.array(v) for k, v in digest.items()})
    # 6. Block alignment of routed tokens: the reference's own torch function
    #    (tests/kernel/moe/torch_kernels.py, pure torch), on the shapes its test sweeps
    #    (tests/kernel/moe/moe_align_block_size_test.py:14-17) plus a case with empty experts.
    import importlib.util
    spec = importlib.util.spec_from_file_location("ref_moe_torch_kernels", Path(ref_root) / "tests/kernel/moe/torch_kernels.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    store = {}
    gen = torch.Generator().manual_seed(0)
    cases = [(1, 2, 16, 4), (33, 2, 32, 8), (256, 2, 64, 64), (33, 2, 16, 64), (256, 2, 128, 8), (7, 3, 16, 5)]
    for ci, (tokens, topk, block, experts) in enumerate(cases):
        scores = torch.rand(tokens, experts, generator=gen)
        _, topk_ids = torch.topk(scores, k=topk, dim=1)
        cap = topk_ids.numel() + experts * (block - 1)
        sorted_ids = torch.empty(cap, dtype=torch.int32)
        expert_ids = torch.full((-(cap // -block),), -1, dtype=torch.int32)
        post = torch.empty(1, dtype=torch.int32)
        mod.moe_align_block_size_pytorch(topk_ids, experts, block, sorted_ids, expert_ids, post)
        store[f"case{ci}_params"] = np.array([tokens, topk, block, experts])
        store[f"case{ci}_topk_ids"] = topk_ids.numpy()
        store[f"case{ci}_sorted_ids"] = sorted_ids.numpy()
        store[f"case{ci}_expert_ids"] = expert_ids.numpy()
        store[f"case{ci}_post_pad"] = post.numpy()
    np.savez_compressed(HERE / "moe_align.npz", **store)

    # 7. MXFP8: the reference keeps its generator and its oracle for this variant inside a test file
    #    (tests/kernel/wave_gemm_mxfp_test.py:64-91) whose other imports need the compiler stack, so the
    #    two function definitions are taken out of that file's syntax tree and executed as they are, with
    #    the CPU forms of the helpers they call.
    ns = reference_mxfp8_functions(ref_root, ref)
    torch.set_num_threads(1)
    x, w, xs, ws = ns["generate_gemm_afp8wfp8_inputs"]((64, 96, 128))
    out = ns["torchScaledGemmMXFP8"](x, w, xs, ws)
    np.savez_compressed(HERE / "gemm_mxfp8_seed5_64x96x128.npz", x=x.view(torch.uint8).numpy(),
                        w=np.ascontiguousarray(w.T.contiguous().view(torch.uint8).numpy()),  # stored as [N, K] bytes
                        x_scales=np.ascontiguousarray(xs.numpy()), w_scales=np.ascontiguousarray(ws.numpy()),
                        out=out.numpy())
    mixed_pair(ref, ns)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


def reference_mxfp8_functions(ref_root: str, ref) -> dict:
    import ast
    test_src = (Path(ref_root) / "tests/kernel/wave_gemm_mxfp_test.py").read_text()
    wanted = [n for n in ast.parse(test_src).body
              if isinstance(n, ast.FunctionDef) and n.name in ("generate_gemm_afp8wfp8_inputs", "torchScaledGemmMXFP8")]
    assert len(wanted) == 2
    ns = {"torch": torch, "SCALE_GROUP_SIZE": ref.SCALE_GROUP_SIZE, "e8m0_to_f32": ref.e8m0_to_f32,
          "device_randn": torch.randn, "device_randint": torch.randint}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), "wave_gemm_mxfp_test.py", "exec"), ns)
    return ns


def mixed_pair(ref, ns) -> None:
    """8. The mixed pair of the same scaled MMA: the reference's 8-bit activations (its MXFP8 generator) against its packed
    E2M1 weights (its MXFP4 generator), each dequantised by the reference's own functions, then its f32 torch.mm."""
    torch.set_num_threads(1)
    shape = (64, 96, 128)
    x, _, xs, _ = ns["generate_gemm_afp8wfp8_inputs"](shape)
    _, w, _, ws = ref.generate_gemm_afp4wfp4_inputs(shape)  # w: [K/2, N] view, ws: [N, K/32]
    x_f32 = x.to(torch.float32) * ref.e8m0_to_f32(xs.repeat_interleave(ref.SCALE_GROUP_SIZE, dim=1).to(torch.float32))
    w_f32 = ref.mxfp4_to_f32(w.T).T * ref.e8m0_to_f32(ws.repeat_interleave(ref.SCALE_GROUP_SIZE, dim=1).to(torch.float32)).T
    out = torch.mm(x_f32, w_f32)
    np.savez_compressed(HERE / "gemm_mxfp8_mxfp4_seed5_64x96x128.npz", x=x.view(torch.uint8).numpy(),
                        w=np.ascontiguousarray(w.T.contiguous().numpy()),  # stored as [N, K/2] packed bytes
                        x_scales=np.ascontiguousarray(xs.numpy()), w_scales=np.ascontiguousarray(ws.numpy()), out=out.numpy())


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: make_golden.py <path to the reference checkout> [--only-mixed]")
    main(sys.argv[1], only_mixed="--only-mixed" in sys.argv[2:])
