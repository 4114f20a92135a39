"""Host-side logic that needs no GPU: argument validation of the Python surface and the work
partitioning across ranks (checked with a 2-process gloo group)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle


def test_public_names_match_the_reference_package(lib):
    import fa2_custom_mask as pkg
    for name in ("flash_attention_custom_mask", "permute_qkv_triton", "apply_head_wise_reorder",
                 "inv_permute_attn_triton", "apply_inv_reorder"):
        assert hasattr(pkg, name)
    from fa2_custom_mask.fa2_custom_mask import _attention, build_groups_from_block_mask  # noqa: F401
    import inspect
    sig = inspect.signature(_attention.forward)
    assert list(sig.parameters) == ["ctx", "q", "k", "v", "mask", "sm_scale"]
    assert sig.parameters["sm_scale"].default == 1.3 and sig.parameters["mask"].default is None
    from fa2_custom_mask import functional
    sig = inspect.signature(functional.permute_qkv_triton)
    assert [(p.name, p.default) for p in sig.parameters.values()][4:] == [
        ("i_block", inspect._empty), ("F", 13), ("H", 30), ("W", 45), ("n_text_tokens", 226)][0:5]


def test_cpu_tensors_are_rejected_not_computed(lib):
    from fa2_custom_mask import flash_attention_custom_mask, apply_head_wise_reorder
    q = torch.randn(1, 1, 64, 64, dtype=torch.float16)
    mask = torch.ones(1, 1, 1, 1, dtype=torch.bool)
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_attention_custom_mask(q, q, q, mask, 0.125)
    with pytest.raises(RuntimeError, match="no CPU path"):
        apply_head_wise_reorder(torch.randn(1, 1, 8, 4), torch.zeros(1, 3, dtype=torch.int32), 2, 2, 2)


def test_shape_checks(lib):
    from fa2_custom_mask import flash_attention_custom_mask
    mask = torch.ones(1, 1, 1, 1, dtype=torch.bool)
    q = torch.randn(1, 1, 64, 48, dtype=torch.float16)
    with pytest.raises(AssertionError):
        flash_attention_custom_mask(q, q, q, mask, 0.125)          # D not in the reference's set
    q = torch.randn(1, 1, 64, 128, dtype=torch.float16)
    with pytest.raises(NotImplementedError):
        flash_attention_custom_mask(q, q, q, mask, 0.125)
    q = torch.randn(1, 1, 100, 64, dtype=torch.float16)
    with pytest.raises(AssertionError):
        flash_attention_custom_mask(q, q, q, mask, 0.125)          # N % 64


def test_shard_heads_partitions_exactly():
    from fa2_custom_mask.sharding import shard_heads, shard_rows_by_tiles, plan
    for units in (1, 7, 32, 33):
        for ws in (1, 2, 4, 8):
            spans = [shard_heads(units, ws, r) for r in range(ws)]
            assert spans[0][0] == 0 and spans[-1][1] == units
            assert all(spans[i][1] == spans[i + 1][0] for i in range(ws - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    mask = oracle.make_block_mask(1, 1, 274, 0.1, seed=2)
    tiles = mask[0, 0].sum(-1).tolist()
    for ws in (2, 4, 8):
        spans = shard_rows_by_tiles(tiles, ws)
        assert spans[0][0] == 0 and spans[-1][1] == 274
        assert all(spans[i][1] == spans[i + 1][0] for i in range(ws - 1))
        loads = [sum(tiles[a:b]) for a, b in spans]
        assert max(loads) <= 1.05 * sum(tiles) / ws
    # uneven rows: every row is counted once, for the rank that gets it
    assert [sum([1, 9, 1, 1, 1, 1, 1, 1][a:b]) for a, b in
            shard_rows_by_tiles([1, 9, 1, 1, 1, 1, 1, 1], 2)] == [10, 6]
    loads = [sum(range(1, 17)[a:b]) for a, b in shard_rows_by_tiles(list(range(1, 17)), 4)]
    assert loads == [36, 30, 39, 31] and sum(loads) == 136
    # all tiles in one row, or more ranks than rows: empty ranges, still a partition
    for tiles_, ws in (([10, 0, 0, 0], 4), ([3, 3], 5), ([0, 0, 0], 2), ([], 3)):
        spans = shard_rows_by_tiles(tiles_, ws)
        assert len(spans) == ws and spans[0][0] == 0 and spans[-1][1] == len(tiles_)
        assert all(a <= b for a, b in spans)
        assert all(spans[i][1] == spans[i + 1][0] for i in range(ws - 1))
    assert plan(1, 32, 8, 3)[0] == "heads"
    assert plan(1, 1, 8, 3, tiles)[0] == "rows"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, B, H, nb):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fa2_custom_mask.sharding import shard_heads
        a, b = shard_heads(B * H, world, rank)
        # every rank builds the same seeded problem, computes only its heads with the CPU oracle,
        # and the pieces are gathered; no data-path exchange is needed to get the full result
        q, k, v = oracle.make_qkv(B, H, nb * 64, 64, seed=9)
        mask = oracle.make_block_mask(B, H, nb, 0.5, seed=9)
        flat = lambda t: t.reshape(B * H, *t.shape[2:])
        o_mine, _ = oracle.attn_forward(flat(q)[a:b, None], flat(k)[a:b, None], flat(v)[a:b, None],
                                        flat(mask)[a:b, None], 0.125)
        tiles = torch.tensor([int(flat(mask)[a:b].sum())])
        dist.all_reduce(tiles)
        assert int(tiles) == int(mask.sum())
        pieces = [None] * world
        dist.all_gather_object(pieces, (a, b, o_mine.squeeze(1)))
        if rank == 0:
            full, _ = oracle.attn_forward(q, k, v, mask, 0.125)
            got = torch.cat([p[2] for p in sorted(pieces, key=lambda p: p[0])]).reshape(full.shape)
            assert torch.allclose(got, full, atol=1e-6)
    finally:
        dist.destroy_process_group()


def test_head_sharding_two_ranks_gloo():
    mp.spawn(_rank_main, args=(2, _free_port(), 1, 3, 2), nprocs=2, join=True)


def _rank_rows(rank, world, port, nb):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from fa2_custom_mask.sharding import plan
        # one head, fewer (b, h) units than ranks: every rank holds all of K and V and computes
        # its share of the query-block rows, balanced by listed tiles
        q, k, v = oracle.make_qkv(1, 1, nb * 64, 64, seed=4)
        mask = oracle.make_block_mask(1, 1, nb, 0.4, seed=4, causal=True)
        kind, (r0, r1) = plan(1, 1, world, rank, mask[0, 0].sum(-1).tolist())
        assert kind == "rows"
        o_mine, _ = oracle.attn_forward(q[:, :, 64 * r0:64 * r1], k, v, mask[:, :, r0:r1], 0.125)
        pieces = [None] * world
        dist.all_gather_object(pieces, (r0, r1, o_mine))
        if rank == 0:
            full, _ = oracle.attn_forward(q, k, v, mask, 0.125)
            spans = sorted((a, b) for a, b, _ in pieces)
            assert spans[0][0] == 0 and spans[-1][1] == nb
            got = torch.cat([p[2] for p in sorted(pieces, key=lambda p: p[0])], dim=2)
            assert torch.allclose(got, full, atol=1e-6)
    finally:
        dist.destroy_process_group()


def test_row_sharding_two_ranks_gloo():
    mp.spawn(_rank_rows, args=(2, _free_port(), 6), nprocs=2, join=True)
