"""Generates the golden vectors under tests/golden/ by running the REFERENCE project's own code.

Run once, in a container where the reference checkout is available (pass its path as the first
argument, or set REFERENCE_ROOT); the produced .npz files are committed, this script is only
re-run to regenerate them.  Nothing here is imported by the tests.

What runs:
  * build_groups_from_block_mask (fa2_custom_mask/fa2_custom_mask.py:15-38), natively on CPU;
  * the forward kernel _attn_fwd (fa2_custom_mask/fa2_fwd.py:108-206) under the Triton CPU
    interpreter, launched the way _attention.forward launches it
    (fa2_custom_mask/fa2_custom_mask.py:77-87) but without the autotuner, BLOCK_M = BLOCK_N = 64;
  * reorder_kernel / inv_reorder_kernel through apply_head_wise_reorder / apply_inv_reorder
    (fa2_custom_mask/functional.py:5-20, 46-62) under the interpreter.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT", "")
if not REF or not os.path.isdir(REF):
    raise SystemExit("usage: make_golden.py <path to the reference checkout>")
sys.path.insert(0, REF)
HERE = os.path.dirname(os.path.abspath(__file__))

from fa2_custom_mask.fa2_custom_mask import build_groups_from_block_mask  # noqa: E402
from fa2_custom_mask.fa2_fwd import _attn_fwd  # noqa: E402
from fa2_custom_mask.functional import apply_head_wise_reorder, apply_inv_reorder  # noqa: E402


def mask_cases():
    g = torch.Generator().manual_seed(1234)
    cases = {}
    cases["b1h1_nb4_p50"] = torch.rand(1, 1, 4, 4, generator=g) < 0.5
    cases["b2h3_nb7_p30"] = torch.rand(2, 3, 7, 7, generator=g) < 0.3      # odd nb, empty rows
    cases["b1h2_nb5_full"] = torch.ones(1, 2, 5, 5, dtype=torch.bool)
    cases["b2h1_nb3_empty"] = torch.zeros(2, 1, 3, 3, dtype=torch.bool)    # -> (None, None)
    single = torch.zeros(1, 1, 6, 6, dtype=torch.bool)
    single[0, 0, 4, 1] = True
    cases["b1h1_nb6_single"] = single
    cases["b1h2_nb33_p10"] = (torch.rand(1, 2, 33, 33, generator=g) < 0.1) | torch.eye(33, dtype=torch.bool)
    cases["b1h1_nb16_causal"] = torch.tril(torch.rand(1, 1, 16, 16, generator=g) < 0.25, -1) | torch.eye(16, dtype=torch.bool)
    return cases


def gen_groups():
    out = {}
    for name, m in mask_cases().items():
        groups, n_list = build_groups_from_block_mask(m)
        out[name + "/mask"] = m.numpy()
        if groups is None:
            out[name + "/none"] = np.asarray([1], dtype=np.int32)
        else:
            out[name + "/groups"] = groups.numpy()
            out[name + "/n_list"] = n_list.numpy()
    np.savez_compressed(os.path.join(HERE, "groups.npz"), **out)
    print("groups.npz:", len(mask_cases()), "cases")


def run_ref_fwd(q, k, v, mask, sm_scale):
    B, H, N, D = q.shape
    groups, nlist = build_groups_from_block_mask(mask)
    o = torch.full_like(q, float("nan"))
    M = torch.full((B, H, N), float("nan"), dtype=torch.float32)
    _attn_fwd.fn[(groups.shape[0],)](
        q, k, v, groups, nlist, sm_scale, M, o,
        *q.stride(), *k.stride(), *v.stride(), *o.stride(),
        B, H, N, HEAD_DIM=D, BLOCK_M=64, BLOCK_N=64)
    return o, M


def gen_fwd():
    out = {}
    specs = [
        # name, B, H, N, dtype, density, diagonal, seed
        ("f32_b1h2_n256", 1, 2, 256, torch.float32, 0.5, True, 11),
        ("f16_b2h1_n256_emptyrows", 2, 1, 256, torch.float16, 0.3, False, 12),
        # bf16 is left out: the Triton CPU interpreter does not emulate bf16 arithmetic (it returns
        # values of order 1e9 for this kernel), so only fp32 and fp16 vectors are trustworthy.
        ("f16_b1h1_n192_oddnb", 1, 1, 192, torch.float16, 0.6, True, 13),
        ("f16_b1h1_n512_p10", 1, 1, 512, torch.float16, 0.1, True, 14),
    ]
    for name, B, H, N, dt, dens, diag, seed in specs:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, H, N, 64, generator=g).to(dt)
        k = torch.randn(B, H, N, 64, generator=g).to(dt)
        v = torch.randn(B, H, N, 64, generator=g).to(dt)
        nb = N // 64
        mask = torch.rand(B, H, nb, nb, generator=g) < dens
        if diag:
            mask |= torch.eye(nb, dtype=torch.bool)
        sm_scale = 0.125
        o, M = run_ref_fwd(q, k, v, mask, sm_scale)
        out[name + "/q"] = q.float().numpy()
        out[name + "/k"] = k.float().numpy()
        out[name + "/v"] = v.float().numpy()
        out[name + "/mask"] = mask.numpy()
        out[name + "/o"] = o.float().numpy()
        out[name + "/M"] = M.numpy()
        out[name + "/meta"] = np.asarray([{torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dt]], dtype=np.int32)
        out[name + "/sm_scale"] = np.asarray([sm_scale], dtype=np.float64)
        print(name, "done")
    np.savez_compressed(os.path.join(HERE, "fwd.npz"), **out)


def gen_reorder():
    out = {}
    perms = torch.tensor([[0, 1, 2], [0, 2, 1], [1, 2, 0], [1, 0, 2], [2, 1, 0], [2, 0, 1]], dtype=torch.int32)
    perms_inv = torch.tensor([[0, 1, 2], [0, 2, 1], [2, 0, 1], [1, 0, 2], [2, 1, 0], [1, 2, 0]], dtype=torch.int32)
    for name, B, F, H, W, D in [("g2x3x4_d8", 2, 2, 3, 4, 8), ("g3x5x2_d16", 1, 3, 5, 2, 16)]:
        g = torch.Generator().manual_seed(77)
        heads = 6
        T = F * H * W
        x = torch.randn(B, heads, T, D, generator=g)
        idx = torch.arange(6)
        fwd = apply_head_wise_reorder(x.contiguous(), perms[idx], F, H, W)
        back = apply_inv_reorder(fwd.contiguous(), perms[idx], perms_inv[idx], F, H, W)
        out[name + "/x"] = x.numpy()
        out[name + "/fwd"] = fwd.numpy()
        out[name + "/back"] = back.numpy()
        out[name + "/dims"] = np.asarray([B, heads, F, H, W, D], dtype=np.int32)
        print(name, "roundtrip exact:", bool(torch.equal(back, x)))
    np.savez_compressed(os.path.join(HERE, "reorder.npz"), **out)


if __name__ == "__main__":
    gen_groups()
    gen_fwd()
    gen_reorder()
