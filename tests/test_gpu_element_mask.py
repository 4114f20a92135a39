"""Element-level (dense) masks: the op applies them inside the 64x64 blocks that are only partly
kept, so that its result is the naive masked softmax of kernel-test.py:37-40 for any boolean mask
(the in-tile mask the reference kernel sketches in fa2_custom_mask/fa2_fwd.py:57-75), in forward
and backward.  Tolerances (stated by the task): 2e-2 on O, 5e-2 on the gradients."""
import math

import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
O_TOL, G_TOL, LSE_TOL = 2e-2, 5e-2, 2e-3


def _masks(B, H, N, seed):
    g = torch.Generator().manual_seed(seed)
    nb = N // 64
    causal = torch.ones(N, N, dtype=torch.bool).tril()                       # diagonal blocks partial
    band = causal & ~torch.ones(N, N, dtype=torch.bool).tril(-(N // 3) - 7)  # sliding window, ragged edges
    rand = torch.rand(B, H, N, N, generator=g) < 0.3                         # every block partial
    rand[..., torch.arange(N), torch.arange(N)] = True
    sparse = oracle.expand_block_mask(oracle.make_block_mask(B, H, nb, 0.4, seed=seed)) & \
        (torch.rand(B, H, N, N, generator=g) < 0.9)                          # partial and empty blocks
    hole = oracle.expand_block_mask(oracle.make_block_mask(B, H, nb, 0.5, seed=seed + 1))
    hole[:, :, 5] = False                                                    # a row with nothing kept
    hole[:, :, 70, :64] = False
    return {"causal": causal, "band": band, "random": rand, "sparse": sparse, "hole": hole}


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kind", ["causal", "band", "random", "sparse", "hole"])
def test_forward_and_gradients_with_element_masks(lib, kind, dtype):
    from fa2_custom_mask import flash_attention_custom_mask
    B, H, N = 1, 2, 320
    q, k, v, do = oracle.make_qkv(B, H, N, 64, seed=7, dtype=dtype, n=4)
    dense = _masks(B, H, N, seed=3)[kind]
    full = dense.expand(B, H, N, N)
    qc, kc, vc = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = flash_attention_custom_mask(qc, kc, vc, dense.cuda(), 0.125)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    o_ref, _, dq, dk, dv = oracle.attn_forward_backward_dense(q, k, v, full, 0.125, do)
    assert torch.isfinite(o).all() and torch.isfinite(qc.grad).all()
    assert (o.detach().float().cpu() - o_ref).abs().max().item() <= O_TOL
    for name, got, ref in (("dq", qc.grad, dq), ("dk", kc.grad, dk), ("dv", vc.grad, dv)):
        err = (got.float().cpu() - ref).abs().max().item()
        assert err <= G_TOL, f"{kind} {name} max-abs err {err}"


def test_lse_rowmax_and_both_entry_points(lib):
    """LSE and row maxima under an element mask, list mode against mask mode, and the marks of
    the reduced block mask."""
    from fa2_custom_mask import (attention_forward, attention_forward_masked, build_tile_lists,
                                 reduce_dense_mask)
    B, H, N = 2, 1, 256
    q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=11, dtype=torch.float16))
    dense = _masks(B, H, N, seed=5)["sparse"]
    dense[:, :, 100] = False
    block = reduce_dense_mask(dense.cuda(), mark_partial=True)
    assert block.dtype == torch.uint8
    blocks = dense.reshape(B, H, N // 64, 64, N // 64, 64)
    any_, all_ = blocks.any(-1).any(-2), blocks.all(-1).all(-2)
    assert torch.equal(block.cpu() == 0, ~any_) and torch.equal(block.cpu() == 2, any_ & ~all_)
    o1, lse1, rm1 = attention_forward_masked(q, k, v, block, 0.125, want_rowmax=True, dense=dense.cuda())
    lists = build_tile_lists(block, want_csc=False)
    flagged = (lists.col_idx[: int(lists.meta[0])] >> 30) & 1
    assert int(flagged.sum()) == int((block == 2).sum())
    o2, lse2, rm2 = attention_forward(q, k, v, lists, 0.125, want_rowmax=True, dense=dense.cuda())
    torch.cuda.synchronize()
    assert torch.equal(o1, o2) and torch.equal(lse1, lse2) and torch.equal(rm1, rm2)
    o_ref, lse_ref = oracle.attn_forward_dense(q.cpu(), k.cpu(), v.cpu(), dense, 0.125)
    assert (o1.float().cpu() - o_ref).abs().max().item() <= O_TOL
    live = torch.isfinite(lse_ref)
    assert not live.all()                                   # row 100 keeps nothing
    assert torch.equal(torch.isfinite(lse1.cpu()), live)
    assert (lse1.cpu()[live] * math.log(2.0) - lse_ref[live]).abs().max().item() <= LSE_TOL
    assert (o1[:, :, 100] == 0).all()
    # without the dense mask the same block mask attends the marked blocks in full
    o3, _, _ = attention_forward_masked(q, k, v, block, 0.125)
    o3_ref, _ = oracle.attn_forward(q.cpu(), k.cpu(), v.cpu(), block.cpu() != 0, 0.125)
    assert (o3.float().cpu() - o3_ref).abs().max().item() <= O_TOL


def test_causal_mask_at_a_baseline_size(lib):
    """A token-level causal mask at N = 6400 (BASELINE config 2's length): 100 partly kept
    diagonal blocks, 4,950 full ones; against the fp32 arithmetic evaluated on the GPU in chunks."""
    from fa2_custom_mask import flash_attention_custom_mask
    N = 6400
    q, k, v = (t.cuda() for t in oracle.make_qkv(1, 1, N, 64, seed=N, dtype=torch.bfloat16))
    dense = torch.ones(N, N, dtype=torch.bool, device="cuda").tril()
    with torch.no_grad():
        o = flash_attention_custom_mask(q, k, v, dense, 0.125)
    worst = 0.0
    for r0 in range(0, N, 1600):
        s = (q[0, 0, r0:r0 + 1600].float() @ k[0, 0].float().T) * 0.125
        s = s.masked_fill(~dense[r0:r0 + 1600], float("-inf"))
        ref = torch.softmax(s, -1) @ v[0, 0].float()
        worst = max(worst, (o[0, 0, r0:r0 + 1600].float() - ref).abs().max().item())
    assert worst <= O_TOL, worst
