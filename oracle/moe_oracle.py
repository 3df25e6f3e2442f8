"""CPU oracle for the mixture-of-experts steps around the grouped GEMM — TEST INFRASTRUCTURE, not a product path.

Restates, with numpy / torch on the CPU, the reference's own CPU code for these steps:
`moe_align_block_size_pytorch` (tests/kernel/moe/torch_kernels.py:10-97), `silu_and_mul_ref`
(tests/kernel/moe_test.py:39-40) and the expert loop with its weighted sum, `torch_ref_moe`
(tests/kernel/moe_test.py:102-127). Only `tests/` may import this module.

Parity is pinned for the integer step: `tests/golden/make_golden.py` runs the reference's
`moe_align_block_size_pytorch` itself on seeded routings and stores its outputs in
`tests/golden/moe_align.npz`; `tests/test_oracle.py` checks `moe_align_block_size` here against
them. The floating-point steps are one-line formulas restated from the cited lines.
"""

from __future__ import annotations

import numpy as np
import torch

from . import mxfp4_oracle as orc


def moe_align_block_size(topk_ids: np.ndarray, num_experts: int, block_size: int, sorted_capacity: int,
                         expert_capacity: int):
    """tests/kernel/moe/torch_kernels.py:30-97, as plain loops. Returns (sorted_ids [sorted_capacity] int32 filled
    with the padding value topk_ids.size, expert_ids [expert_capacity] int32 with -1 where the reference leaves
    the entry unwritten, num_tokens_post_pad, inverse [n])."""
    flat = np.asarray(topk_ids).reshape(-1).astype(np.int64)
    n = flat.size
    sorted_ids = np.full(sorted_capacity, n, dtype=np.int32)          # :34
    expert_ids = np.full(expert_capacity, -1, dtype=np.int32)
    counts = np.bincount(flat, minlength=num_experts)                  # :39
    padded = (counts + block_size - 1) // block_size * block_size      # :42-43
    starts = np.cumsum(padded) - padded                                # :48
    total = int(padded.sum())                                          # :44
    blk = 0
    for e in range(num_experts):                                       # :52-55
        for _ in range(int(padded[e]) // block_size):
            expert_ids[blk] = e
            blk += 1
    inverse = np.full(n, -1, dtype=np.int32)
    fill = starts.copy()
    for i in range(n):                                                 # :66-97: stable by original position
        e = int(flat[i])
        sorted_ids[fill[e]] = i
        inverse[i] = fill[e]
        fill[e] += 1
    return sorted_ids, expert_ids, total, inverse


def silu_and_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """tests/kernel/moe_test.py:39-40, evaluated in f32."""
    g, u = gate.float(), up.float()
    return g * u / (1 + torch.exp(-g))


def expert_mlp(x: torch.Tensor, w1_q, w1_s, w2_q, w2_s, router_logits: torch.Tensor, top_k: int) -> torch.Tensor:
    """The expert loop of torch_ref_moe (tests/kernel/moe_test.py:102-127) on MXFP4 operands: tokens are
    quantised to MXFP4 (the harness quantiser of `mxfp4_oracle.quantize_mxfp4`), every product uses the
    dequantised operands in f32, the hidden activations are rounded to bf16 after the first projection
    (the type the kernel writes them in), quantised again after silu_and_mul, and the output rows are
    rounded to bf16 before the weighted sum. Returns f32 [T, K_out]."""
    T = x.shape[0]
    score = torch.softmax(router_logits.float(), dim=-1, dtype=torch.float32)   # :111
    weight, ids = torch.topk(score, top_k)                                      # :112
    xq, xs = orc.quantize_mxfp4(x.float())
    xd = orc.dequant_mxfp4(xq, xs)
    out = torch.zeros(T, w2_q[0].shape[0], dtype=torch.float32)
    for e in range(len(w1_q)):                                                  # :115-121
        w1 = orc.dequant_mxfp4(w1_q[e], w1_s[e])
        w2 = orc.dequant_mxfp4(w2_q[e], w2_s[e])
        for j in range(top_k):
            sel = (ids[:, j] == e).nonzero().squeeze(-1)
            if sel.numel() == 0:
                continue
            h = (xd[sel] @ w1.T).to(torch.bfloat16).float()
            d = h.shape[1] // 2
            a = silu_and_mul(h[:, :d], h[:, d:])
            aq, a_s = orc.quantize_mxfp4(a)
            y = (orc.dequant_mxfp4(aq, a_s) @ w2.T).to(torch.bfloat16).float()
            out[sel] += weight[sel, j:j + 1] * y                                # :123-127
    return out
