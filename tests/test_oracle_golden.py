"""The CPU oracle against the vectors the reference's own code produced (tests/golden/*.npz)."""
import numpy as np
import torch

from conftest import golden_cases
from oracle import oracle

DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def test_build_groups_matches_reference(golden):
    g = golden["groups"]
    for case in golden_cases(g):
        mask = g[case + "/mask"]
        groups, n_list = oracle.build_groups(mask)
        if case + "/none" in g.files:
            assert groups is None and n_list is None
        else:
            assert groups.dtype == np.int32 and n_list.dtype == np.int32
            np.testing.assert_array_equal(groups, g[case + "/groups"])
            np.testing.assert_array_equal(n_list, g[case + "/n_list"])


def test_tile_lists_consistent_with_groups(golden):
    g = golden["groups"]
    for case in golden_cases(g):
        mask = g[case + "/mask"]
        tl = oracle.tile_lists(mask)
        B, H, nb, _ = mask.shape
        if case + "/none" in g.files:
            assert tl["meta"][0] == 0 and tl["meta"][1] == 0
            continue
        np.testing.assert_array_equal(tl["col_idx"], g[case + "/n_list"])
        ref_groups = g[case + "/groups"]
        # groups rows are the non-empty CSR rows
        lens = np.diff(tl["row_ptr"])
        rows = np.flatnonzero(lens)
        np.testing.assert_array_equal(ref_groups[:, 3], tl["row_ptr"][rows])
        np.testing.assert_array_equal(ref_groups[:, 4], lens[rows])
        np.testing.assert_array_equal(ref_groups[:, 2], rows % nb)
        # both CSR forms decode back to the mask
        rebuilt = np.zeros((B * H * nb, nb), dtype=bool)
        rebuilt_t = np.zeros((B * H, nb, nb), dtype=bool)
        for r in range(B * H * nb):
            rebuilt[r, tl["col_idx"][tl["row_ptr"][r]:tl["row_ptr"][r + 1]]] = True
            bh, n = divmod(r, nb)
            rebuilt_t[bh, tl["row_idx"][tl["col_ptr"][r]:tl["col_ptr"][r + 1]], n] = True
        np.testing.assert_array_equal(rebuilt.reshape(mask.shape), mask)
        np.testing.assert_array_equal(rebuilt_t.reshape(mask.shape), mask)


def test_forward_tiled_and_naive_match_reference_kernel(golden):
    g = golden["fwd"]
    for case in golden_cases(g):
        dt = DT[int(g[case + "/meta"][0])]
        q, k, v = (torch.from_numpy(g[case + "/" + n]).to(dt) for n in "qkv")
        mask = torch.from_numpy(g[case + "/mask"])
        sm_scale = float(g[case + "/sm_scale"][0])
        o_ref = torch.from_numpy(g[case + "/o"])
        m_ref = torch.from_numpy(g[case + "/M"])
        written = ~torch.isnan(m_ref)

        groups, n_list = oracle.build_groups(mask.numpy())
        o_t, m_t = oracle.attn_forward_tiled(q, k, v, groups, n_list, sm_scale)
        # same rows written as the reference kernel; its row maximum reproduced
        assert torch.equal(~torch.isnan(m_t), written)
        tol = 1e-5 if dt == torch.float32 else 2e-3
        assert torch.allclose(m_t[written], m_ref[written], atol=1e-4, rtol=1e-5)
        o_t_cast = o_t.to(dt).float()
        assert (o_t_cast[written] - o_ref[written]).abs().max() <= (1e-5 if dt == torch.float32 else 1e-2)

        # the naive form (the oracle used at every size) agrees on the rows the kernel writes
        o_n, lse = oracle.attn_forward(q, k, v, mask, sm_scale)
        err = (o_n[written] - o_ref[written]).abs().max().item()
        assert err <= (2e-5 if dt == torch.float32 else 2e-2), (case, err)
        # M is the row maximum of the scaled logits in the exp2 domain, never above the LSE
        lse2 = lse / np.log(2.0)
        assert (m_ref[written] <= lse2[written] + 1e-3).all()
        # rows the reference leaves unwritten are exactly the rows with no kept block
        assert torch.equal(torch.isinf(lse) & (lse < 0), ~written)


def test_reorder_matches_reference_kernels(golden):
    g = golden["reorder"]
    for case in golden_cases(g):
        B, heads, F, H, W, D = (int(x) for x in g[case + "/dims"])
        x = torch.from_numpy(g[case + "/x"])
        orders = oracle.PERMUTATIONS[np.arange(6)]
        inv = oracle.PERMUTATIONS_INV[np.arange(6)]
        fwd = oracle.reorder(x, orders, F, H, W)
        assert torch.equal(fwd, torch.from_numpy(g[case + "/fwd"]))
        assert torch.equal(oracle.reorder_by_view(x, orders, F, H, W), fwd)
        back = oracle.inv_reorder(fwd, orders, inv, F, H, W)
        assert torch.equal(back, torch.from_numpy(g[case + "/back"]))
        assert torch.equal(back, x)


def test_dense_block_roundtrip():
    m = oracle.make_block_mask(2, 3, 5, 0.4, seed=3, diagonal=False)
    dense = oracle.expand_block_mask(m)
    assert dense.shape == (2, 3, 320, 320)
    assert torch.equal(oracle.reduce_dense_mask(dense), m)
    assert oracle.count_partial_tiles(dense) == 0
    dense[0, 0, 0, 0] = ~dense[0, 0, 0, 0]
    assert oracle.count_partial_tiles(dense) == 1


def test_autograd_oracle_matches_formulas():
    # dS = P (dP - delta), dQ = s dS K, dK = s dS^T Q, dV = P^T dO  (fa2_bwd.py:56-74,116-130)
    q, k, v, do = oracle.make_qkv(1, 2, 128, 64, seed=5, n=4)
    mask = oracle.make_block_mask(1, 2, 2, 0.5, seed=5)
    s = 0.125
    o, lse, dq, dk, dv = oracle.attn_forward_backward(q, k, v, mask, s, do)
    dense = oracle.expand_block_mask(mask)
    p = torch.exp((q @ k.mT) * s - lse[..., None]).masked_fill(~dense, 0.0)
    delta = (o * do).sum(-1, keepdim=True)
    ds = p * (do @ v.mT - delta)
    assert torch.allclose(dq, s * ds @ k, atol=1e-4)
    assert torch.allclose(dk, s * ds.mT @ q, atol=1e-4)
    assert torch.allclose(dv, p.mT @ do, atol=1e-4)
