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


def test_strided_views_and_shared_stride_entry(lib):
    """Slices are read where they lie (separate in/out strides); the reference-shaped entry point
    with one stride set for both tensors gives the same bytes."""
    from fa2_custom_mask import apply_head_wise_reorder, apply_inv_reorder, _lib
    B, heads, F, H, W, D, n_text = 2, 6, 3, 5, 4, 64, 7
    T = F * H * W
    g = torch.Generator().manual_seed(3)
    full = torch.randn(B, heads, n_text + T + 2, D, generator=g).half().cuda()
    image = full[:, :, n_text:n_text + T]                      # non-contiguous view, offset base
    orders = torch.from_numpy(oracle.PERMUTATIONS).cuda()
    inv = torch.from_numpy(oracle.PERMUTATIONS_INV).cuda()
    before = full.clone()
    fwd = apply_head_wise_reorder(image, orders, F, H, W)
    want = oracle.reorder(image.cpu().contiguous(), oracle.PERMUTATIONS, F, H, W)
    assert fwd.is_contiguous() and torch.equal(fwd.cpu(), want)
    assert torch.equal(full, before)                           # the source is only read
    # head-transposed source ([B, T, heads, D] storage): another stride set, same result
    x_t = image.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
    assert torch.equal(apply_head_wise_reorder(x_t, orders, F, H, W).cpu(), want)
    # inverse straight out of a slice
    full2 = torch.zeros_like(full)
    full2[:, :, n_text:n_text + T] = fwd
    back = apply_inv_reorder(full2[:, :, n_text:n_text + T], orders, inv, F, H, W)
    assert torch.equal(back, image)
    # strided destination through the C ABI: write into the slice of a third tensor
    dst = torch.zeros_like(full)
    dview = dst[:, :, n_text:n_text + T]
    o32 = orders.to(torch.int32).contiguous()
    rc = lib.bsa_reorder_strided(_lib.ptr(image), _lib.strides4(image), _lib.ptr(dview),
                                 _lib.strides4(dview), _lib.ptr(o32), B, heads, T, D, F, H, W, 2,
                                 _lib.stream_ptr(full.device))
    assert rc == 0
    assert torch.equal(dview.cpu(), want)
    assert int(dst[:, :, :n_text].abs().sum()) == 0 and int(dst[:, :, n_text + T:].abs().sum()) == 0
    # the reference-shaped entry (one stride set): slice to slice
    dst2 = torch.zeros_like(full)
    d2 = dst2[:, :, n_text:n_text + T]
    rc = lib.bsa_reorder(_lib.ptr(image), _lib.ptr(d2), _lib.strides4(image), _lib.ptr(o32), B, heads,
                         T, D, F, H, W, 2, _lib.stream_ptr(full.device))
    assert rc == 0 and torch.equal(d2.cpu(), want)
    i32 = inv.to(torch.int32).contiguous()
    d3 = torch.zeros_like(full)[:, :, n_text:n_text + T]
    rc = lib.bsa_inv_reorder(_lib.ptr(d2), _lib.ptr(d3), _lib.strides4(d2), _lib.ptr(o32),
                             _lib.ptr(i32), B, heads, T, D, F, H, W, 2, _lib.stream_ptr(full.device))
    assert rc == 0 and torch.equal(d3, image)
