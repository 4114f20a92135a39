"""Head-wise token reorder kernels: bit-exact against the oracle and the reference's vectors."""
import numpy as np
import pytest
import torch

from conftest import golden_cases
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_golden_vectors(lib, golden):
    from fa2_custom_mask import apply_head_wise_reorder, apply_inv_reorder
    g = golden["reorder"]
    perms = torch.from_numpy(oracle.PERMUTATIONS).cuda()
    inv = torch.from_numpy(oracle.PERMUTATIONS_INV).cuda()
    for case in golden_cases(g):
        B, heads, F, H, W, D = (int(x) for x in g[case + "/dims"])
        x = torch.from_numpy(g[case + "/x"]).cuda()
        fwd = apply_head_wise_reorder(x, perms, F, H, W)
        assert torch.equal(fwd.cpu(), torch.from_numpy(g[case + "/fwd"]))
        back = apply_inv_reorder(fwd, perms, inv, F, H, W)
        assert torch.equal(back.cpu(), torch.from_numpy(g[case + "/back"]))


@pytest.mark.parametrize("dtype,D", [(torch.float16, 64), (torch.bfloat16, 64), (torch.float32, 5),
                                     (torch.uint8, 3), (torch.float64, 2)])
def test_matches_oracle_all_vector_widths(lib, dtype, D):
    from fa2_custom_mask import apply_head_wise_reorder, apply_inv_reorder
    B, heads, F, H, W = 2, 7, 3, 4, 5
    g = torch.Generator().manual_seed(D)
    x = (torch.randn(B, heads, F * H * W, D, generator=g) * 50).to(dtype)
    idx = torch.tensor([0, 1, 2, 3, 4, 5, 2])
    orders = torch.from_numpy(oracle.PERMUTATIONS)[idx]
    inv = torch.from_numpy(oracle.PERMUTATIONS_INV)[idx]
    fwd = apply_head_wise_reorder(x.cuda(), orders.cuda(), F, H, W)
    assert torch.equal(fwd.cpu(), oracle.reorder(x, orders.numpy(), F, H, W))
    back = apply_inv_reorder(fwd, orders.cuda(), inv.cuda(), F, H, W)
    assert torch.equal(back.cpu(), x)


def test_permute_qkv_roundtrip_default_grid(lib):
    """The reference's default video grid: 13 x 30 x 45 image tokens after 226 text tokens."""
    from fa2_custom_mask import permute_qkv_triton, inv_permute_attn_triton
    heads, T, n_text = 6, 13 * 30 * 45, 226
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, heads, n_text + T, 64, generator=g).half().cuda()
    k, v = q.clone() + 1, q.clone() + 2
    orig = q.clone()
    plan = {"permute": torch.tensor([[0, 1, 2, 3, 4, 5]]).cuda()}
    q2, k2, v2 = permute_qkv_triton(q, k, v, plan, 0)
    assert q2.data_ptr() == q.data_ptr()                      # mutates and returns its inputs
    assert torch.equal(q[:, :, :n_text], orig[:, :, :n_text])  # text tokens untouched
    ref = oracle.reorder_by_view(orig[:, :, n_text:].cpu(), oracle.PERMUTATIONS, 13, 30, 45)
    assert torch.equal(q[:, :, n_text:].cpu(), ref)
    assert torch.equal(k[:, :, n_text:].cpu(), ref + 1)
    out = inv_permute_attn_triton(q, plan, 0)
    assert out.data_ptr() == q.data_ptr() and torch.equal(q, orig)
