"""Mask preprocessing kernels against the oracle and the reference's golden vectors: bit-exact."""
import numpy as np
import pytest
import torch

from conftest import golden_cases
from oracle import oracle

pytestmark = pytest.mark.gpu


def _lists_to_numpy(tl):
    meta = tl.meta.cpu().numpy()
    nnz, G = (int(x) for x in meta[:2])
    assert not meta[2:].any()
    out = dict(meta=meta[:2])
    out["row_ptr"] = tl.row_ptr.cpu().numpy()
    out["col_ptr"] = tl.col_ptr.cpu().numpy()
    out["col_idx"] = tl.col_idx.cpu().numpy()[:nnz]
    out["row_idx"] = tl.row_idx.cpu().numpy()[:nnz]
    out["groups"] = tl.groups.cpu().numpy()[:5 * G].reshape(G, 5)
    return out


def _check_lists(mask_cpu, lib):
    from fa2_custom_mask import build_tile_lists
    tl = build_tile_lists(mask_cpu.cuda(), want_groups=True)
    got = _lists_to_numpy(tl)
    ref = oracle.tile_lists(mask_cpu.numpy())
    for key in ("meta", "row_ptr", "col_idx", "col_ptr", "row_idx"):
        np.testing.assert_array_equal(got[key], ref[key], err_msg=key)
    if ref["groups"] is None:
        assert got["groups"].shape[0] == 0
    else:
        np.testing.assert_array_equal(got["groups"], ref["groups"])


def test_lists_match_reference_golden(lib, golden):
    from fa2_custom_mask import build_groups_from_block_mask
    g = golden["groups"]
    for case in golden_cases(g):
        mask = torch.from_numpy(g[case + "/mask"])
        groups, n_list = build_groups_from_block_mask(mask.cuda())
        if case + "/none" in g.files:
            assert groups is None and n_list is None
        else:
            assert groups.dtype == torch.int32 and n_list.dtype == torch.int32
            assert groups.is_cuda and groups.is_contiguous()
            np.testing.assert_array_equal(groups.cpu().numpy(), g[case + "/groups"])
            np.testing.assert_array_equal(n_list.cpu().numpy(), g[case + "/n_list"])
        _check_lists(mask, lib)


@pytest.mark.parametrize("B,H,nb,p,diag,causal", [
    (1, 1, 1, 1.0, True, False), (1, 1, 2, 0.5, False, False), (2, 3, 9, 0.3, False, False),
    (1, 2, 100, 0.1, True, False), (1, 1, 274, 0.1, True, False), (1, 1, 274, 1.0, True, False),
    (2, 2, 64, 0.25, True, True), (1, 4, 257, 0.02, False, False),
    # more than 8192 rows: the offset scan carries over from one tile of counts to the next
    (1, 32, 500, 0.1, True, False), (2, 16, 300, 0.05, False, True),
])
def test_lists_match_oracle(lib, B, H, nb, p, diag, causal):
    _check_lists(oracle.make_block_mask(B, H, nb, p, seed=nb, diagonal=diag, causal=causal), lib)


def test_lists_on_broadcast_and_strided_masks(lib):
    from fa2_custom_mask import build_tile_lists
    base = oracle.make_block_mask(1, 1, 12, 0.4, seed=1)
    expanded = base.cuda().expand(2, 3, 12, 12)          # stride 0 over batch and heads
    tl = build_tile_lists(expanded, want_csr=True, want_csc=False)
    ref = oracle.tile_lists(base.expand(2, 3, 12, 12).numpy())
    np.testing.assert_array_equal(tl.row_ptr.cpu().numpy(), ref["row_ptr"])
    np.testing.assert_array_equal(tl.col_idx.cpu().numpy()[:ref["col_idx"].size], ref["col_idx"])
    sliced = oracle.make_block_mask(1, 2, 20, 0.4, seed=2).cuda()[:, :, 3:15, 5:17]  # non-contiguous
    tl = build_tile_lists(sliced, want_csr=True, want_csc=True)
    ref = oracle.tile_lists(sliced.cpu().numpy())
    np.testing.assert_array_equal(tl.col_ptr.cpu().numpy(), ref["col_ptr"])
    np.testing.assert_array_equal(tl.row_idx.cpu().numpy()[:ref["row_idx"].size], ref["row_idx"])
    np.testing.assert_array_equal(tl.row_ptr.cpu().numpy(), ref["row_ptr"])
    np.testing.assert_array_equal(tl.col_idx.cpu().numpy()[:ref["col_idx"].size], ref["col_idx"])


@pytest.mark.parametrize("B,H,N,p", [(1, 1, 64, 1.0), (2, 2, 320, 0.4), (1, 1, 1024, 0.1),
                                     (1, 1, 6400, 0.1), (1, 1, 17536, 0.1)])
def test_mask_reduce_roundtrip(lib, B, H, N, p):
    from fa2_custom_mask import reduce_dense_mask
    block = oracle.make_block_mask(B, H, N // 64, p, seed=N, diagonal=False)
    dense = oracle.expand_block_mask(block.cuda())
    got, partial = reduce_dense_mask(dense, return_partial=True)
    assert got.dtype == torch.bool and got.shape == block.shape
    assert torch.equal(got.cpu(), block)                 # reduce(expand(block)) == block, bit-exact
    assert int(partial) == 0


def test_mask_reduce_partial_tiles_and_layouts(lib):
    from fa2_custom_mask import reduce_dense_mask
    g = torch.Generator().manual_seed(5)
    dense = (torch.rand(2, 1, 256, 256, generator=g) < 0.0005)
    got, partial = reduce_dense_mask(dense.cuda(), return_partial=True)
    assert torch.equal(got.cpu(), oracle.reduce_dense_mask(dense))
    assert int(partial) == oracle.count_partial_tiles(dense)
    # 2-D mask, broadcast view and a misaligned slice (falls back to a contiguous copy)
    d2 = dense[0, 0].cuda()
    assert torch.equal(reduce_dense_mask(d2).cpu(), oracle.reduce_dense_mask(dense[0, 0]))
    big = (torch.rand(1, 1, 200, 200, generator=g) < 0.01).cuda()
    sl = big[:, :, 3:131, 5:133]
    assert torch.equal(reduce_dense_mask(sl).cpu(), oracle.reduce_dense_mask(sl.cpu()))
    # a single kept element in the last row/column of a tile is seen
    one = torch.zeros(1, 1, 1088, 1088, dtype=torch.bool)
    one[0, 0, 1087, 1087] = True
    one[0, 0, 63, 960] = True
    assert torch.equal(reduce_dense_mask(one.cuda()).cpu(), oracle.reduce_dense_mask(one))
