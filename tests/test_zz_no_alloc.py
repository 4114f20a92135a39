"""The allocation-free forward entry point against the ordinary two-call path.

bsa_attn_fwd_block_mask_static serves hosts that cannot give the library device buffers at call
time (an engine plugin with a fixed workspace, a process whose device memory is owned by another
pool): the row lists live in a fixed array inside the library instead of caller memory.  Its output
must equal bsa_tile_lists_build + bsa_attn_fwd.  Two calls in a row with different masks check that
nothing of the first call's lists leaks into the second.
"""
import ctypes

import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
O_TOL = 2e-2      # same bound as the forward parity tests
LSE_TOL = 2e-3


def _static_forward(lib, q, k, v, mask, sm_scale):
    from fa2_custom_mask import _lib
    B, H, N, D = q.shape
    m = mask.view(torch.uint8)
    o = torch.empty_like(q)
    lse2 = torch.empty(B, H, N, dtype=torch.float32, device=q.device)
    rc = lib.bsa_attn_fwd_block_mask_static(
        _lib.ptr(q), _lib.strides4(q), _lib.ptr(k), _lib.strides4(k), _lib.ptr(v),
        _lib.strides4(v), _lib.ptr(o), _lib.strides4(o), _lib.ptr(lse2), _lib.ptr(m),
        _lib.strides4(m), m.shape[0], m.shape[1], float(sm_scale), _lib.dtype_code(q.dtype),
        B, H, N, D, _lib.stream_ptr(q.device))
    _lib.check("bsa_attn_fwd_block_mask_static", rc)
    return o, lse2


def test_static_entry_matches_two_call_path_twice_in_a_row(lib):
    from fa2_custom_mask import attention_forward, build_tile_lists
    cases = [
        (2, 2, 2, 2, 512, 0.5, torch.float16, 21, False),   # per-head masks, rows without tiles
        (1, 3, 1, 3, 1024, 0.1, torch.bfloat16, 22, True),  # sparser and larger: shorter lists than call 1
        (2, 3, 2, 1, 512, 0.4, torch.float16, 24, False),   # one mask per batch entry, shared by heads
        (2, 3, 1, 3, 512, 0.4, torch.bfloat16, 25, False),  # one mask per head, shared by the batch
    ]
    for B, H, Bm, Hm, N, p, dtype, seed, diag in cases:
        q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=seed, dtype=dtype))
        mask = oracle.make_block_mask(Bm, Hm, N // 64, p, seed=seed, diagonal=diag).cuda()
        o_s, lse_s = _static_forward(lib, q, k, v, mask, 0.125)
        lists = build_tile_lists(mask, want_csc=False)
        o_r, lse_r, _ = attention_forward(q, k, v, lists, 0.125)
        torch.cuda.synchronize()
        assert (o_s.float() - o_r.float()).abs().max().item() <= O_TOL
        live = torch.isfinite(lse_r)
        assert torch.equal(torch.isfinite(lse_s), live)
        assert (lse_s[live] - lse_r[live]).abs().max().item() <= LSE_TOL
        # and against the oracle itself
        o_ref, _ = oracle.attn_forward(q.cpu(), k.cpu(), v.cpu(),
                                       mask.cpu().expand(B, H, N // 64, N // 64), 0.125)
        assert (o_s.float().cpu() - o_ref).abs().max().item() <= O_TOL


def test_static_entry_general_list_path_allocates_nothing(lib):
    """A mask too large for the one-launch list builder (two heads of 320 x 320 blocks) takes the
    count / scan / fill path through the fixed array.  On the second call, when every lazy
    first-use cost has been paid, the free device memory is the same before and after."""
    from fa2_custom_mask import attention_forward, build_tile_lists
    B, H, N = 1, 2, 20480
    assert lib.bsa_static_warmup() == 0
    q, k, v = (t.cuda() for t in oracle.make_qkv(B, H, N, 64, seed=26, dtype=torch.float16))
    mask = oracle.make_block_mask(1, H, N // 64, 0.05, seed=26).cuda()
    lists = build_tile_lists(mask, want_csc=False)
    o_r, lse_r, _ = attention_forward(q, k, v, lists, 0.125)
    _static_forward(lib, q, k, v, mask, 0.125)
    o = torch.empty_like(q)
    lse2 = torch.empty(B, H, N, dtype=torch.float32, device=q.device)
    m = mask.view(torch.uint8)
    from fa2_custom_mask import _lib
    args = (_lib.ptr(q), _lib.strides4(q), _lib.ptr(k), _lib.strides4(k), _lib.ptr(v),
            _lib.strides4(v), _lib.ptr(o), _lib.strides4(o), _lib.ptr(lse2), _lib.ptr(m),
            _lib.strides4(m), 1, H, 0.125, _lib.dtype_code(q.dtype), B, H, N, 64,
            _lib.stream_ptr(q.device))
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    assert lib.bsa_attn_fwd_block_mask_static(*args) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.equal(o, o_r) and torch.equal(lse2, lse_r)
    # a missing stride array is refused on the host
    bad = list(args)
    bad[10] = None
    assert lib.bsa_attn_fwd_block_mask_static(*bad) == -4


def test_static_entry_shared_mask_and_capacity(lib):
    from fa2_custom_mask import _lib
    q, k, v = (t.cuda() for t in oracle.make_qkv(2, 2, 256, 64, seed=23, dtype=torch.float16))
    shared = oracle.make_block_mask(1, 1, 4, 0.6, seed=23).cuda()
    o_s, _ = _static_forward(lib, q, k, v, shared, 0.125)
    o_ref, _ = oracle.attn_forward(q.cpu(), k.cpu(), v.cpu(), shared.cpu().expand(2, 2, 4, 4), 0.125)
    assert (o_s.float().cpu() - o_ref).abs().max().item() <= O_TOL
    # beyond the fixed capacity the call refuses before touching the GPU
    s4 = (ctypes.c_int64 * 4)(1, 1, 1, 1)
    fake = ctypes.c_void_p(0x1000)
    rc = lib.bsa_attn_fwd_block_mask_static(fake, s4, fake, s4, fake, s4, fake, s4, fake, fake, s4,
                                            1, 64, 0.125, 0, 1, 64, 64 * 512, 64, None)
    assert rc == -8 and b"capacity" in lib.bsa_strerror(rc)
