"""Forward kernel (through the C ABI) against the fp32 oracle and the reference's golden vectors.
Tolerance (stated by the task): max-abs 2e-2 on O for fp16/bf16 inputs."""
import math

import numpy as np
import pytest
import torch

from conftest import golden_cases
from oracle import oracle

pytestmark = pytest.mark.gpu
O_TOL = 2e-2
LSE_TOL = 2e-3
DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def _run(q, k, v, mask, sm_scale, want_rowmax=True, mode="lists"):
    """mode "lists": bsa_tile_lists_build + bsa_attn_fwd; mode "mask": bsa_attn_fwd_block_mask."""
    from fa2_custom_mask import attention_forward, attention_forward_masked, build_tile_lists
    if mode == "mask":
        o, lse2, rowmax = attention_forward_masked(q.cuda(), k.cuda(), v.cuda(), mask.cuda(),
                                                   sm_scale, want_rowmax)
        torch.cuda.synchronize()
        return o.float().cpu(), lse2.cpu(), (rowmax.cpu() if rowmax is not None else None)
    lists = build_tile_lists(mask.cuda(), want_csc=False)
    o, lse2, rowmax = attention_forward(q.cuda(), k.cuda(), v.cuda(), lists, sm_scale, want_rowmax)
    torch.cuda.synchronize()
    return o.float().cpu(), lse2.cpu(), (rowmax.cpu() if rowmax is not None else None)


def _compare(q, k, v, mask, sm_scale, o, lse2):
    o_ref, lse_ref = oracle.attn_forward(q, k, v, mask, sm_scale)
    err = (o - o_ref).abs().max().item()
    assert err <= O_TOL, f"O max-abs err {err}"
    live = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse2), live)
    assert (lse2[~live] == -math.inf).all()
    lerr = (lse2[live] * math.log(2.0) - lse_ref[live]).abs().max().item()
    assert lerr <= LSE_TOL, f"LSE max-abs err {lerr}"
    return err


def test_golden_vectors_of_the_reference_kernel(lib, golden):
    g = golden["fwd"]
    for case in golden_cases(g):
        dt = DT[int(g[case + "/meta"][0])]
        run_dt = torch.float16 if dt == torch.float32 else dt   # the kernel is 16-bit only
        q, k, v = (torch.from_numpy(g[case + "/" + n]).to(run_dt) for n in "qkv")
        mask = torch.from_numpy(g[case + "/mask"])
        sm_scale = float(g[case + "/sm_scale"][0])
        o, lse2, rowmax = _run(q, k, v, mask, sm_scale, mode="mask")
        o_l, lse2_l, rowmax_l = _run(q, k, v, mask, sm_scale, mode="lists")
        assert torch.equal(o, o_l) and torch.equal(lse2, lse2_l) and torch.equal(rowmax, rowmax_l)
        o_ref = torch.from_numpy(g[case + "/o"])
        m_ref = torch.from_numpy(g[case + "/M"])
        written = ~torch.isnan(m_ref)
        assert (o[written] - o_ref[written]).abs().max().item() <= O_TOL, case
        # the reference's M buffer is the running row maximum in the exp2 domain
        assert (rowmax[written] - m_ref[written]).abs().max().item() <= 2e-2, case
        # rows the reference never writes: zeros and -inf here
        assert (o[~written] == 0).all() and (lse2[~written] == -math.inf).all()


@pytest.mark.parametrize("mode", ["lists", "mask"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,N,p,diag,causal", [
    (1, 1, 64, 1.0, True, False),       # one tile, odd block count
    (1, 1, 128, 1.0, True, False),      # one full pair
    (1, 2, 192, 0.5, True, False),      # odd nb: last pair has one block
    (2, 3, 256, 0.5, False, False),     # rows with no tile
    (1, 1, 1024, 0.1, True, False),     # BASELINE config 1 shape
    (1, 2, 1024, 1.0, True, False),     # dense
    (2, 2, 512, 0.25, True, True),      # block-causal sparse
])
def test_forward_matches_oracle(lib, mode, dtype, B, H, N, p, diag, causal):
    q, k, v = oracle.make_qkv(B, H, N, 64, seed=N + B, dtype=dtype)
    mask = oracle.make_block_mask(B, H, N // 64, p, seed=N, diagonal=diag, causal=causal)
    o, lse2, _ = _run(q, k, v, mask, 0.125, mode=mode)
    _compare(q, k, v, mask, 0.125, o, lse2)


def test_single_tile_and_diagonal_only(lib):
    q, k, v = oracle.make_qkv(1, 1, 384, 64, seed=3, dtype=torch.float16)
    single = torch.zeros(1, 1, 6, 6, dtype=torch.bool)
    single[0, 0, 4, 1] = True
    o, lse2, _ = _run(q, k, v, single, 0.125)
    _compare(q, k, v, single, 0.125, o, lse2)
    diag = torch.eye(6, dtype=torch.bool)[None, None]
    o, lse2, _ = _run(q, k, v, diag, 0.125)
    _compare(q, k, v, diag, 0.125, o, lse2)


def test_large_logits_trigger_the_lazy_rescale(lib):
    # keys grow along the sequence so the running maximum rises by far more than 2^8 between tiles
    q, k, v = oracle.make_qkv(1, 1, 512, 64, seed=4, dtype=torch.float16)
    ramp = torch.linspace(0.2, 6.0, 512)[None, None, :, None]
    k = (k.float() * ramp).half()
    mask = torch.ones(1, 1, 8, 8, dtype=torch.bool)
    for s in (0.125, 1.3):          # 1.3 is the reference's default sm_scale
        o, lse2, _ = _run(q, k, v, mask, s)
        _compare(q, k, v, mask, s, o, lse2)


def test_public_op_block_and_dense_masks(lib):
    from fa2_custom_mask import flash_attention_custom_mask
    q, k, v = (t.cuda() for t in oracle.make_qkv(2, 2, 256, 64, seed=6, dtype=torch.bfloat16))
    mask = oracle.make_block_mask(2, 2, 4, 0.5, seed=6)
    o_ref, _ = oracle.attn_forward(q.cpu(), k.cpu(), v.cpu(), mask, 0.125)
    o1 = flash_attention_custom_mask(q, k, v, mask.cuda(), 0.125)
    assert o1.dtype == q.dtype and o1.shape == q.shape
    assert (o1.float().cpu() - o_ref).abs().max() <= O_TOL
    o2 = flash_attention_custom_mask(q, k, v, oracle.expand_block_mask(mask).cuda(), 0.125)
    assert torch.equal(o1, o2)                       # dense mask reduces to the same block mask
    shared = mask[:1, :1]
    o3 = flash_attention_custom_mask(q, k, v, shared.cuda(), 0.125)     # broadcast over B, H
    o3_ref, _ = oracle.attn_forward(q.cpu(), k.cpu(), v.cpu(), shared.expand(2, 2, 4, 4), 0.125)
    assert (o3.float().cpu() - o3_ref).abs().max() <= O_TOL
    empty = torch.zeros(2, 2, 4, 4, dtype=torch.bool).cuda()
    assert (flash_attention_custom_mask(q, k, v, empty, 0.125) == 0).all()   # fa2_custom_mask.py:49-51
    # non-contiguous inputs ([B,N,H,D] storage viewed as [B,H,N,D])
    qt = q.transpose(1, 2).contiguous().transpose(1, 2)
    o4 = flash_attention_custom_mask(qt, k, v, mask.cuda(), 0.125)
    assert torch.equal(o4, o1)


def test_mask_mode_strided_and_wide_masks(lib):
    # a mask row wider than one pass of the in-kernel lister (nb > 352) and a non-contiguous mask
    q, k, v = oracle.make_qkv(1, 1, 64 * 400, 64, seed=31, dtype=torch.float16)
    wide = oracle.make_block_mask(1, 1, 400, 0.02, seed=31)
    a = _run(q, k, v, wide, 0.125, mode="mask")
    b = _run(q, k, v, wide, 0.125, mode="lists")
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    from fa2_custom_mask import attention_forward_masked
    q, k, v = (t.cuda() for t in oracle.make_qkv(1, 2, 512, 64, seed=32, dtype=torch.bfloat16))
    big = oracle.make_block_mask(1, 2, 20, 0.4, seed=32).cuda()
    sl = big[:, :, 3:11, 5:13]                      # strided view, 8 x 8 blocks
    o, lse2, _ = attention_forward_masked(q, k, v, sl, 0.125)
    o_ref, _ = oracle.attn_forward(q.cpu(), k.cpu(), v.cpu(), sl.cpu(), 0.125)
    assert (o.float().cpu() - o_ref).abs().max() <= O_TOL


def test_run_to_run_determinism(lib):
    q, k, v = oracle.make_qkv(1, 2, 1024, 64, seed=8, dtype=torch.float16)
    mask = oracle.make_block_mask(1, 2, 16, 0.3, seed=8)
    a = _run(q, k, v, mask, 0.125)
    b = _run(q, k, v, mask, 0.125)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def _chunked_fp32_check(q, k, v, mask, o, lse2, chunk=2048):
    """The oracle's fp32 naive arithmetic evaluated on the GPU in query-row chunks, per (b, h)."""
    B, H, N, _ = q.shape
    worst = 0.0
    for b in range(B):
        for h in range(H):
            kf, vf = k[b, h].float(), v[b, h].float()
            for r0 in range(0, N, chunk):
                r1 = min(N, r0 + chunk)
                s = (q[b, h, r0:r1].float() @ kf.T) * 0.125
                dense = mask[b, h, r0 // 64:(r1 + 63) // 64].repeat_interleave(64, 0) \
                    .repeat_interleave(64, 1)
                s = s.masked_fill(~dense[: r1 - r0], float("-inf"))
                ref = torch.softmax(s, -1) @ vf
                worst = max(worst, (o[b, h, r0:r1].float() - ref).abs().max().item())
                lerr = (lse2[b, h, r0:r1] * math.log(2.0) - torch.logsumexp(s, -1)).abs().max().item()
                assert lerr <= LSE_TOL
    return worst


@pytest.mark.parametrize("H,N,p,dtype", [
    (1, 6400, 0.1, torch.float16), (1, 6400, 1.0, torch.float16),          # BASELINE config 2
    (1, 17536, 0.1, torch.float16), (1, 17536, 1.0, torch.float16),        # config 3, sparse and dense
    (2, 32000, 0.1, torch.bfloat16),                                       # config 4, two of its heads
])
def test_baseline_sizes_against_gpu_fp32_reference(lib, H, N, p, dtype):
    """Full BASELINE sizes (per-head masks), both entry points: the same fp32 naive arithmetic as
    the oracle, evaluated on the GPU in query-row chunks (the CPU oracle would need minutes),
    plus a linearity property in V."""
    from fa2_custom_mask import attention_forward, attention_forward_masked, build_tile_lists
    q, k, v = (t.cuda() for t in oracle.make_qkv(1, H, N, 64, seed=N, dtype=dtype))
    mask = oracle.make_block_mask(1, H, N // 64, p, seed=N).cuda()
    lists = build_tile_lists(mask, want_csc=False)
    o, lse2, _ = attention_forward(q, k, v, lists, 0.125)
    om, lse2m, _ = attention_forward_masked(q, k, v, mask, 0.125)
    assert torch.equal(o, om) and torch.equal(lse2, lse2m)
    worst = _chunked_fp32_check(q, k, v, mask, o, lse2)
    assert worst <= O_TOL, worst
    # attention is linear in V: O(2V) == 2 O(V) up to output rounding
    o2, _, _ = attention_forward(q, k, (v.float() * 2).to(dtype), lists, 0.125)
    assert (o2.float() - 2 * o.float()).abs().max().item() <= (2e-2 if dtype == torch.float16 else 4e-2)


@pytest.mark.parametrize("B,H,N", [
    (2, 8, 2048),     # 512 query blocks: several per CTA, handed out in index order
    (1, 4, 4096),     # 256 query blocks: at most two per CTA, the second round longest first
])
def test_work_counter_hand_out_equals_fixed_stride(lib, B, H, N):
    """With a work counter the CTAs draw query blocks dynamically; the result must not depend on
    who computes which block, and the counter must be back at zero for the next call."""
    from fa2_custom_mask import _lib, fa2_custom_mask as host
    q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=5, dtype=torch.float16))
    mask = oracle.make_block_mask(B, H, N // 64, 0.3, seed=6, diagonal=False).cuda()
    m4 = host._as_4d(host._as_bytes(mask))
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    for word in (None, counter, counter, counter):
        o = torch.empty_like(q)
        lse2 = torch.empty(B, H, N, dtype=torch.float32, device="cuda")
        rc = lib.bsa_attn_fwd_block_mask(
            _lib.ptr(q), _lib.strides4(q), _lib.ptr(k), _lib.strides4(k), _lib.ptr(v),
            _lib.strides4(v), _lib.ptr(o), _lib.strides4(o), _lib.ptr(lse2), None, _lib.ptr(m4),
            _lib.strides4(m4), B, H, 0.125, _lib.dtype_code(q.dtype), B, H, N, 64,
            _lib.ptr(word), None, _lib.stream_ptr(q.device))
        assert rc == 0
        torch.cuda.synchronize()
        assert int(counter.item()) == 0
        outs.append((o, lse2))
    for o, lse2 in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(lse2, outs[0][1])
    _compare(q.cpu(), k.cpu(), v.cpu(), mask.cpu(), 0.125, outs[1][0].float().cpu(), outs[1][1].cpu())


def test_two_streams_and_graph_replay(lib):
    """Calls on different streams get a work counter each and may overlap on the GPU; a call captured
    into a CUDA graph replays with the same result."""
    from fa2_custom_mask import attention_forward_masked
    cases = []
    for seed in (11, 12):
        q, k, v = (t.cuda() for t in oracle.make_qkv(1, 4, 2048, 64, seed=seed, dtype=torch.float16))
        mask = oracle.make_block_mask(1, 4, 32, 0.3, seed=seed).cuda()
        ref = attention_forward_masked(q, k, v, mask, 0.125)[0]
        cases.append((q, k, v, mask, ref))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [[], []]
    for _ in range(8):                      # interleaved launches on the two streams
        for s, (q, k, v, mask, _) , o in zip(streams, cases, outs):
            with torch.cuda.stream(s):
                o.append(attention_forward_masked(q, k, v, mask, 0.125)[0])
    torch.cuda.synchronize()
    for (_, _, _, _, ref), o in zip(cases, outs):
        assert all(torch.equal(x, ref) for x in o)

    q, k, v, mask, ref = cases[0]
    s = streams[0]
    with torch.cuda.stream(s):
        attention_forward_masked(q, k, v, mask, 0.125)      # the stream's counter exists before capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            out = attention_forward_masked(q, k, v, mask, 0.125)[0]
        for _ in range(3):
            out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, ref)


def test_public_op_with_dense_mask_in_a_graph(lib):
    """Dense mask -> block mask -> forward, the whole public call, holds no host synchronisation:
    it can be captured into a CUDA graph and replays on new inputs (mask included) written into
    the same buffers."""
    from fa2_custom_mask import flash_attention_custom_mask
    B, H, N = 1, 2, 1024
    q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=21, dtype=torch.bfloat16))
    block = oracle.make_block_mask(B, H, N // 64, 0.4, seed=21)
    dense = oracle.expand_block_mask(block).cuda()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s), torch.no_grad():
        flash_attention_custom_mask(q, k, v, dense, 0.125)   # loads the library outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            out = flash_attention_custom_mask(q, k, v, dense, 0.125)
        for seed in (22, 23):
            q2, k2, v2 = oracle.make_qkv(B, H, N, 64, seed=seed, dtype=torch.bfloat16)
            block2 = oracle.make_block_mask(B, H, N // 64, 0.3, seed=seed)
            q.copy_(q2); k.copy_(k2); v.copy_(v2)
            dense.copy_(oracle.expand_block_mask(block2))
            graph.replay()
            torch.cuda.synchronize()
            ref, _ = oracle.attn_forward(q2, k2, v2, block2, 0.125)
            assert (out.float().cpu() - ref).abs().max() <= O_TOL


def test_maximum_sequence_length(lib):
    """N = 131072 (2048 key blocks per row, the most a CTA can list) runs and is right on sampled
    query blocks; one block more is refused with BSA_ERR_TOO_LARGE before any launch."""
    from fa2_custom_mask import _lib, attention_forward_masked
    N, nb = 131072, 2048
    g = torch.Generator(device="cuda").manual_seed(3)
    q, k, v = (torch.randn(1, 1, N, 64, device="cuda", generator=g).half() for _ in range(3))
    mask = torch.rand(1, 1, nb, nb, device="cuda", generator=g) < 0.003
    mask |= torch.eye(nb, dtype=torch.bool, device="cuda")
    mask[0, 0, 7, :] = True                       # one row that lists every key block
    mask[0, 0, 9, :] = False                      # and one that lists none
    o, lse2, _ = attention_forward_masked(q, k, v, mask, 0.125)
    torch.cuda.synchronize()
    for mb in (0, 7, 9, 1000, nb - 1):
        rows = slice(64 * mb, 64 * mb + 64)
        s = (q[0, 0, rows].float() @ k[0, 0].float().T) * 0.125
        dense = mask[0, 0, mb].repeat_interleave(64)[None, :].expand(64, N)
        s = s.masked_fill(~dense, float("-inf"))
        if mb == 9:
            assert (o[0, 0, rows] == 0).all() and (lse2[0, 0, rows] == -math.inf).all()
            continue
        ref = torch.softmax(s, -1) @ v[0, 0].float()
        assert (o[0, 0, rows].float() - ref).abs().max().item() <= O_TOL
        lse_ref = torch.logsumexp(s, -1)
        assert (lse2[0, 0, rows] * math.log(2.0) - lse_ref).abs().max().item() <= LSE_TOL
    # one block more than a CTA can list
    N2 = N + 64
    big = torch.empty(1, 1, N2, 64, device="cuda", dtype=torch.float16)
    m2 = torch.zeros(1, 1, nb + 1, nb + 1, dtype=torch.uint8, device="cuda")
    lse = torch.empty(1, 1, N2, dtype=torch.float32, device="cuda")
    rc = lib.bsa_attn_fwd_block_mask(
        _lib.ptr(big), _lib.strides4(big), _lib.ptr(big), _lib.strides4(big), _lib.ptr(big),
        _lib.strides4(big), _lib.ptr(big), _lib.strides4(big), _lib.ptr(lse), None, _lib.ptr(m2),
        _lib.strides4(m2), 1, 1, 0.125, _lib.dtype_code(big.dtype), 1, 1, N2, 64, None, None,
        _lib.stream_ptr(big.device))
    assert rc == -8   # BSA_ERR_TOO_LARGE


def test_bounded_wait_runs_out_and_reports(lib):
    """A wait that nothing satisfies gives up after the wait limit, reports through the status
    word and leaves the context usable (no trap, no endless loop).  With a device word the
    host-side check raises; with the public op's own word, which lives in pinned host memory, the
    next call of the op raises without any synchronisation, and the call after that is right."""
    import time
    from fa2_custom_mask import (_lib, attention_forward_masked, check_status,
                                 flash_attention_custom_mask, new_status_word)
    from fa2_custom_mask import fa2_custom_mask as host
    q, k, v = (t.cuda() for t in oracle.make_qkv(1, 2, 512, 64, seed=31, dtype=torch.float16))
    mask = oracle.make_block_mask(1, 2, 8, 0.5, seed=31).cuda()
    ref = attention_forward_masked(q, k, v, mask, 0.125)[0]
    status = new_status_word(q.device)
    report = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    t0 = time.time()
    rc = lib.bsa_selftest_bounded_wait(_lib.ptr(status), _lib.ptr(report), _lib.stream_ptr(q.device))
    assert rc == 0
    with pytest.raises(_lib.BsaError) as err:
        check_status(status)
    assert err.value.status == -9                                 # BSA_ERR_DEVICE_TIMEOUT
    assert time.time() - t0 < 30
    r = report.cpu().tolist()
    assert r[:3] == [0, 0, 1] and 1000 <= r[3] <= 10000           # gave up after about 2 s
    assert int(status.item()) == 99
    out = attention_forward_masked(q, k, v, mask, 0.125)[0]       # the context is still usable
    torch.cuda.synchronize()
    assert torch.equal(out, ref)

    with torch.no_grad():
        o1 = flash_attention_custom_mask(q, k, v, mask, 0.125)
        state = host._stream_state(q.device, _lib.stream_ptr(q.device).value or 0)
        assert state is not None and not state.status.is_cuda and int(state.status[0]) == 0
        rc = lib.bsa_selftest_bounded_wait(_lib.ptr(state.status), _lib.ptr(report),
                                           _lib.stream_ptr(q.device))
        assert rc == 0
        torch.cuda.synchronize()
        with pytest.raises(_lib.BsaError) as err:
            flash_attention_custom_mask(q, k, v, mask, 0.125)
        assert err.value.status == -9
        o2 = flash_attention_custom_mask(q, k, v, mask, 0.125)    # the report was consumed
        torch.cuda.synchronize()
    assert torch.equal(o1, o2) and torch.equal(o1, ref)


@pytest.mark.parametrize("mode", ["lists", "mask"])
def test_row_ranges_concatenate_to_the_whole_launch(lib, mode):
    """The forward restricted to query-block rows [r0, r1) touches nothing else, and the ranges of
    a split (balanced by listed tiles, as the multi-GPU fallback split does) put together are
    bit-equal to the unsplit launch."""
    from fa2_custom_mask import (attention_forward, attention_forward_masked, build_tile_lists,
                                 sharding)
    B, H, N = 1, 2, 4096
    nb = N // 64
    q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=41, dtype=torch.float16))
    mask = oracle.make_block_mask(B, H, nb, 0.2, seed=41, causal=True).cuda()
    lists = build_tile_lists(mask, want_csc=False)

    def run(rows=None, out=None):
        if mode == "lists":
            return attention_forward(q, k, v, lists, 0.125, rows=rows, out=out)
        return attention_forward_masked(q, k, v, mask, 0.125, rows=rows, out=out)

    whole_o, whole_lse, _ = run()
    row_tiles = mask.sum(dim=(0, 1, 3)).cpu().tolist()
    for parts in (2, 4, 8):
        o = torch.full_like(whole_o, float("nan"))
        lse = torch.full_like(whole_lse, float("nan"))
        ranges = sharding.shard_rows_by_tiles(row_tiles, parts)
        assert ranges[0][0] == 0 and ranges[-1][1] == nb
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        for r0, r1 in ranges:
            run(rows=(r0, r1), out=(o, lse))
        torch.cuda.synchronize()
        assert torch.equal(o, whole_o) and torch.equal(lse, whole_lse)
    # a single range leaves the other rows alone, an empty one launches nothing
    o = torch.full_like(whole_o, 7.0)
    lse = torch.full_like(whole_lse, 7.0)
    run(rows=(5, 9), out=(o, lse))
    run(rows=(9, 9), out=(o, lse))
    torch.cuda.synchronize()
    assert torch.equal(o[:, :, 320:576], whole_o[:, :, 320:576])
    assert (o[:, :, :320] == 7).all() and (o[:, :, 576:] == 7).all()
    assert (lse[:, :, :320] == 7).all() and (lse[:, :, 576:] == 7).all()
    with pytest.raises(ValueError):
        run(rows=(3, nb + 1))


def test_negative_scale_is_refused(lib):
    from fa2_custom_mask import _lib, attention_forward_masked
    q, k, v = (t.cuda() for t in oracle.make_qkv(1, 1, 128, 64, seed=1, dtype=torch.float16))
    mask = torch.ones(1, 1, 2, 2, dtype=torch.bool, device="cuda")
    with pytest.raises(_lib.BsaError) as err:
        attention_forward_masked(q, k, v, mask, -0.5)
    assert err.value.status == -1


def test_output_rows_on_16_byte_boundaries_only(lib):
    """An output tensor whose rows start on 16-byte but not 32-byte boundaries takes the narrow
    store path of the write-out; same bits as the whole-sector stores."""
    from fa2_custom_mask import attention_forward, build_tile_lists
    B, H, N = 1, 2, 320
    q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=8, dtype=torch.float16))
    lists = build_tile_lists(oracle.make_block_mask(B, H, N // 64, 0.5, seed=8).cuda())
    o_ref, lse_ref, _ = attention_forward(q, k, v, lists, 0.125)
    wide = torch.zeros(B, H, N, 72, dtype=q.dtype, device="cuda")
    o_view = wide[..., 8:]
    assert o_view.data_ptr() % 32 == 16
    lse = torch.empty(B, H, N, dtype=torch.float32, device="cuda")
    attention_forward(q, k, v, lists, 0.125, out=(o_view, lse))
    torch.cuda.synchronize()
    assert torch.equal(o_view, o_ref) and torch.equal(lse, lse_ref)
    assert not wide[..., :8].any()
