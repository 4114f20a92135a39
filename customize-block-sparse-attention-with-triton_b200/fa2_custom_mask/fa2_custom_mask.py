"""Host side of the block-sparse attention op: same Python surface as the reference's
fa2_custom_mask/fa2_custom_mask.py, with every device step done by libbsattn (sm_100a CUDA).

    flash_attention_custom_mask(q, k, v, mask, sm_scale)      # torch.autograd.Function.apply
    build_groups_from_block_mask(mask) -> (groups, n_list) | (None, None)

Differences from the reference that a caller can observe (all are supersets):
  * `mask` may be the reference's block mask [B,H,N/64,N/64] (leading dims may be 1 or absent to
    share one mask across batch/heads) or a dense boolean mask whose last two dims are [N,N]; a
    dense mask is reduced to blocks on the GPU (a block is listed when any of its elements is
    kept) and applied element by element inside the blocks that are only partly kept, in forward
    and backward: the result is the reference's naive masked softmax (kernel-test.py:37-40) for
    ANY boolean mask, at the cost of the listed blocks only;
  * `mask=None` attends every block (the reference raises);
  * rows of query blocks with no kept block get O = 0 (the reference leaves them unwritten);
  * the backward is correct for any block mask and works for bf16 (the reference's is not);
  * no host synchronisation happens anywhere in forward or backward.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

BLOCK = 64


@dataclass
class TileLists:
    """Device-resident tile lists of one block mask of shape [Bm,Hm,nb,nb]."""
    Bm: int
    Hm: int
    nb: int
    row_ptr: Optional[torch.Tensor] = None
    col_idx: Optional[torch.Tensor] = None
    col_ptr: Optional[torch.Tensor] = None
    row_idx: Optional[torch.Tensor] = None
    groups: Optional[torch.Tensor] = None
    meta: Optional[torch.Tensor] = None  # int32[8]: nnz, G, then zeros

    def list_strides(self, B: int, H: int):
        """(list_b_stride, list_h_stride) so that head (b,h) uses list b*sb + h*sh."""
        if self.Bm not in (1, B) or self.Hm not in (1, H):
            raise ValueError(f"mask leading dims ({self.Bm},{self.Hm}) do not broadcast to ({B},{H})")
        return (self.Hm if self.Bm > 1 else 0), (1 if self.Hm > 1 else 0)


class _NoSwitch:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_SWITCH = _NoSwitch()


def _on_device(dev):
    """Context that makes `dev` current; free when it already is (the common case)."""
    if torch.cuda.current_device() == dev.index:
        return _NO_SWITCH
    return torch.cuda.device(dev)


def _as_bytes(mask: torch.Tensor) -> torch.Tensor:
    if mask.dtype == torch.bool:
        return mask.view(torch.uint8)
    if mask.dtype == torch.uint8:
        return mask
    raise AssertionError("mask must be a bool tensor")  # fa2_custom_mask.py:20 asserts bool


def _as_4d(mask: torch.Tensor) -> torch.Tensor:
    if mask.dim() > 4 or mask.dim() < 2:
        raise ValueError("mask must have 2 to 4 dims")
    while mask.dim() < 4:
        mask = mask.unsqueeze(0)
    return mask


def _dense_ready(dense: torch.Tensor) -> torch.Tensor:
    """A dense mask as bytes [Bm,Hm,N,N] that the kernels can read: unit inner stride, 16-byte
    aligned base and outer strides (a copy is made otherwise)."""
    d4 = _as_4d(_as_bytes(dense))
    Bm, Hm, N, N2 = d4.shape
    if N != N2 or N % BLOCK:
        raise ValueError("dense mask must be [..., N, N] with N a multiple of 64")
    if not d4.is_cuda:
        raise ValueError("mask must be a CUDA tensor")
    ok = (d4.stride(3) == 1 and d4.stride(2) % 16 == 0 and d4.data_ptr() % 16 == 0
          and all(d4.stride(i) % 16 == 0 for i in (0, 1)))
    return d4 if ok else d4.contiguous()


def reduce_dense_mask(dense: torch.Tensor, return_partial: bool = False,
                      mark_partial: bool = False):
    """Dense boolean mask [..., N, N] -> block mask [..., N/64, N/64] on the GPU.

    By default the result is bool (a block is kept when any of its elements is).  With
    mark_partial=True it is uint8: 0 = nothing kept, 1 = kept, 2 = kept but with masked elements
    inside; the kernels apply the dense mask inside the blocks marked 2.
    With return_partial=True also returns a one-element int32 device tensor counting the tiles
    that are neither fully kept nor fully masked (reading it synchronises; the op never does)."""
    lib = _lib.load()
    d4 = _dense_ready(dense)
    Bm, Hm, N, _ = d4.shape
    nb = N // BLOCK
    block = torch.empty((Bm, Hm, nb, nb), dtype=torch.uint8, device=d4.device)
    partial = torch.empty(1, dtype=torch.int32, device=d4.device) if return_partial else None
    with _on_device(d4.device):
        _lib.check("bsa_mask_reduce", lib.bsa_mask_reduce(
            _lib.ptr(d4), _lib.strides4(d4), Bm, Hm, N, _lib.ptr(block), _lib.ptr(partial),
            1 if mark_partial else 0, _lib.stream_ptr(d4.device)))
    out = block if mark_partial else block.view(torch.bool)
    out = out.reshape(*dense.shape[:-2], nb, nb)
    return (out, partial) if return_partial else out


def build_tile_lists(block_mask: torch.Tensor, want_csr: bool = True, want_groups: bool = False,
                     want_csc: bool = True) -> TileLists:
    """Block mask [..,nb,nb] -> device tile lists (worst-case sized, no host synchronisation).
    want_csr: row lists (forward and dQ kernels); want_csc: column lists (dK/dV kernel);
    want_groups: the reference's groups layout."""
    lib = _lib.load()
    m4 = _as_4d(_as_bytes(block_mask))
    if not m4.is_cuda:
        raise ValueError("mask must be a CUDA tensor")
    Bm, Hm, nb, nb2 = m4.shape
    if nb != nb2:
        raise ValueError("block mask must be square in its last two dims")
    dev = m4.device
    # worst-case sizes, the same numbers bsa_tile_list_sizes reports
    rows = Bm * Hm * nb

    def buf(n):
        return torch.empty(n, dtype=torch.int32, device=dev)

    tl = TileLists(Bm=Bm, Hm=Hm, nb=nb, meta=buf(8))
    want_csr = want_csr or want_groups
    want_csc = want_csc or want_groups
    if want_csr:
        tl.row_ptr, tl.col_idx = buf(rows + 1), buf(rows * nb)
    if want_csc:
        tl.col_ptr, tl.row_idx = buf(rows + 1), buf(rows * nb)
    if want_groups:
        tl.groups = buf(rows * 5)
    with _on_device(dev):
        _lib.check("bsa_tile_lists_build", lib.bsa_tile_lists_build(
            _lib.ptr(m4), _lib.strides4(m4), Bm, Hm, nb,
            _lib.ptr(tl.row_ptr), _lib.ptr(tl.col_idx), _lib.ptr(tl.col_ptr), _lib.ptr(tl.row_idx),
            _lib.ptr(tl.groups), _lib.ptr(tl.meta), _lib.stream_ptr(dev)))
    return tl


def build_groups_from_block_mask(mask: torch.Tensor):
    """Drop-in for the reference's build_groups_from_block_mask
    (fa2_custom_mask/fa2_custom_mask.py:15-38): returns (groups int32 [G,5], n_list int32 [nnz])
    on mask.device, or (None, None) when no block is kept.  Built on the GPU; the only host
    synchronisation is the 8-byte read of (nnz, G) needed to size the returned tensors."""
    assert mask.dtype == torch.bool
    assert mask.dim() == 4
    tl = build_tile_lists(mask, want_groups=True)
    nnz, G = (int(x) for x in tl.meta[:2].tolist())
    if G == 0:
        return None, None
    groups = tl.groups[: 5 * G].reshape(G, 5).clone()
    n_list = tl.col_idx[:nnz].clone()
    return groups.contiguous(), n_list.contiguous()


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """TMA needs a unit inner stride, 16-byte aligned base and outer strides."""
    ok = (t.stride(3) == 1 and t.data_ptr() % 16 == 0
          and all(s > 0 and s % 8 == 0 for s in t.stride()[:3]))
    return t if ok else t.contiguous()


def _block_mask_for(mask, B, H, N, device):
    """The op's `mask` argument as (block mask [..,nb,nb], dense mask bytes [Bm,Hm,N,N] or None) on
    `device`.  With a dense mask the block mask marks the partly kept blocks with 2."""
    nb = N // BLOCK
    if mask is None:
        mask = torch.ones((1, 1, nb, nb), dtype=torch.bool, device=device)
    if mask.device != device:
        raise ValueError("mask must live on the same device as q")
    dense = None
    if mask.shape[-1] == nb and mask.shape[-2] == nb:
        block = mask
    elif mask.shape[-1] == N and mask.shape[-2] == N:
        dense = _dense_ready(mask)
        block = reduce_dense_mask(dense, mark_partial=True)
    else:
        raise ValueError(
            f"mask must be a block mask [..,{nb},{nb}] or a dense mask [..,{N},{N}], got {tuple(mask.shape)}")
    m4 = _as_4d(block)
    if m4.shape[0] not in (1, B) or m4.shape[1] not in (1, H):
        raise ValueError(f"mask leading dims {tuple(m4.shape[:2])} do not broadcast to ({B},{H})")
    return block, dense


def _dense_args(dense, B, H):
    """(pointer, strides) of an optional dense mask [Bm,Hm,N,N], broadcast axes with stride 0."""
    if dense is None:
        return None, None
    d4 = _dense_ready(dense)
    if d4.shape[0] not in (1, B) or d4.shape[1] not in (1, H):
        raise ValueError(f"dense mask leading dims {tuple(d4.shape[:2])} do not broadcast to ({B},{H})")
    st = list(d4.stride())
    if d4.shape[0] == 1:
        st[0] = 0
    if d4.shape[1] == 1:
        st[1] = 0
    return d4, (ctypes.c_int64 * 4)(*st)


def new_status_word(device) -> torch.Tensor:
    """A zeroed int32 device word for the kernels' bounded-wait reports (see check_status)."""
    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor):
    """Synchronises the current stream and raises if a kernel's bounded wait gave up."""
    lib = _lib.load()
    with _on_device(status.device):
        _lib.check("bsa_check_status", lib.bsa_check_status(
            _lib.ptr(status), _lib.stream_ptr(status.device)))


class _StreamState:
    """What the public op keeps per (device, stream): the zeroed work counter of the persistent
    kernels (they leave it at zero, also after a bounded wait gave up), and a status word in
    pinned host memory, which the device can write and the host can read without a
    synchronisation.  The kernels only ever touch the status word when a wait gave up."""

    def __init__(self, device):
        # zeroed on the stream that will use it, so no cross-stream ordering is needed
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32).pin_memory()

    def raise_if_reported(self):
        """Looks at the status word as it is now.  A report means that some earlier call on this
        stream produced incomplete results; it surfaces at the first call after the kernel that
        gave up has ended."""
        code = int(self.status[0])
        if code != 0:
            self.status.zero_()
            raise _lib.BsaError("flash_attention_custom_mask", -9,
                                f"a bounded wait inside an earlier kernel on this stream gave up "
                                f"(role {code}); its results are incomplete")


_stream_states = {}


def _stream_state(device: torch.device, stream: int) -> Optional[_StreamState]:
    key = (device.index, stream)
    st = _stream_states.get(key)
    if st is None:
        if torch.cuda.is_current_stream_capturing():
            return None  # no allocation inside a graph capture: fixed-stride hand-out, no report
        st = _StreamState(device)
        _stream_states[key] = st
    return st


def _row_range(rows, nb):
    if rows is None:
        return 0, nb
    r0, r1 = int(rows[0]), int(rows[1])
    if not (0 <= r0 <= r1 <= nb):
        raise ValueError(f"rows must satisfy 0 <= begin <= end <= {nb}, got {rows}")
    return r0, r1


def _fwd_outputs(q, out, want_rowmax):
    B, H, N, D = q.shape
    if out is None:
        o = torch.empty((B, H, N, D), dtype=q.dtype, device=q.device)
        lse2 = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    else:
        o, lse2 = out
        if o.shape != q.shape or o.dtype != q.dtype or lse2.shape != (B, H, N) or \
                lse2.dtype != torch.float32 or not lse2.is_contiguous():
            raise ValueError("out must be (o like q, contiguous float32 lse2 [B,H,N])")
    rowmax = torch.empty((B, H, N), dtype=torch.float32, device=q.device) if want_rowmax else None
    return o, lse2, rowmax


def attention_forward(q, k, v, lists: TileLists, sm_scale: float, want_rowmax: bool = False,
                      status: Optional[torch.Tensor] = None, rows=None, out=None, dense=None):
    """Runs the forward kernel on prepared tile lists.  Returns (o, lse2, rowmax|None):
    lse2 is the base-2 log-sum-exp of the logits scaled by sm_scale*log2(e).
    rows=(begin, end) restricts the call to that range of query-block rows of every head (the
    other rows of the outputs are left untouched); out=(o, lse2) supplies the output tensors;
    dense = the element-level mask [..,N,N] the lists' block mask was reduced from with
    mark_partial (applied inside the blocks marked 2)."""
    lib = _lib.load()
    B, H, N, D = q.shape
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    o, lse2, rowmax = _fwd_outputs(q, out, want_rowmax)
    sb, sh = lists.list_strides(B, H)
    r0, r1 = _row_range(rows, N // BLOCK)
    d4, dst = _dense_args(dense, B, H)
    with _on_device(q.device):
        stream = _lib.stream_ptr(q.device)
        state = _stream_state(q.device, stream.value or 0)
        _lib.check("bsa_attn_fwd_rows", lib.bsa_attn_fwd_rows(
            _lib.ptr(q), _lib.strides4(q), _lib.ptr(k), _lib.strides4(k), _lib.ptr(v),
            _lib.strides4(v), _lib.ptr(o), _lib.strides4(o), _lib.ptr(lse2), _lib.ptr(rowmax),
            _lib.ptr(lists.row_ptr), _lib.ptr(lists.col_idx), sb, sh, float(sm_scale),
            _lib.dtype_code(q.dtype), B, H, N, D, r0, r1, _lib.ptr(d4), dst,
            _lib.ptr(state.counter if state else None), _lib.ptr(status), stream))
    return o, lse2, rowmax


def attention_forward_masked(q, k, v, block_mask: torch.Tensor, sm_scale: float,
                             want_rowmax: bool = False, status: Optional[torch.Tensor] = None,
                             rows=None, out=None, dense=None):
    """Forward straight from a block mask [..,nb,nb]: every CTA lists its own mask row, no tile
    lists are built.  Returns (o, lse2, rowmax|None); rows, out and dense as in
    attention_forward."""
    lib = _lib.load()
    B, H, N, D = q.shape
    m4 = _as_4d(_as_bytes(block_mask))
    q, k, v = _tma_ready(q), _tma_ready(k), _tma_ready(v)
    o, lse2, rowmax = _fwd_outputs(q, out, want_rowmax)
    r0, r1 = _row_range(rows, N // BLOCK)
    d4, dst = _dense_args(dense, B, H)
    with _on_device(q.device):
        stream = _lib.stream_ptr(q.device)
        state = _stream_state(q.device, stream.value or 0)
        _lib.check("bsa_attn_fwd_block_mask_rows", lib.bsa_attn_fwd_block_mask_rows(
            _lib.ptr(q), _lib.strides4(q), _lib.ptr(k), _lib.strides4(k), _lib.ptr(v),
            _lib.strides4(v), _lib.ptr(o), _lib.strides4(o), _lib.ptr(lse2), _lib.ptr(rowmax),
            _lib.ptr(m4), _lib.strides4(m4), m4.shape[0], m4.shape[1], float(sm_scale),
            _lib.dtype_code(q.dtype), B, H, N, D, r0, r1, _lib.ptr(d4), dst,
            _lib.ptr(state.counter if state else None), _lib.ptr(status), stream))
    return o, lse2, rowmax


def attention_backward(q, k, v, o, lse2, dout, lists: TileLists, sm_scale: float,
                       status: Optional[torch.Tensor] = None, dense=None):
    """delta, then dK/dV over the column lists and dQ over the row lists.  dense: the element-level
    mask the forward was given, if any."""
    lib = _lib.load()
    B, H, N, D = q.shape
    # the three kernels take one stride set for q, k, v, o, dO and the gradients
    same = q.stride() == k.stride() == v.stride() == o.stride() == dout.stride()
    if not same or _tma_ready(q) is not q:
        q, k, v, o, dout = (t.contiguous() for t in (q, k, v, o, dout))
    # the gradients are written with q's strides: allocate them with exactly those (empty_like
    # would hand back a compact tensor for a view with gaps, e.g. a slice of a fused qkv buffer)
    dq, dk, dv = (torch.empty_strided(q.shape, q.stride(), dtype=q.dtype, device=q.device)
                  for _ in range(3))
    delta = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    sb, sh = lists.list_strides(B, H)
    code = _lib.dtype_code(q.dtype)
    st = _lib.strides4(q)
    d4, dst = _dense_args(dense, B, H)
    with _on_device(q.device):
        stream = _lib.stream_ptr(q.device)
        state = _stream_state(q.device, stream.value or 0)
        counter = state.counter if state else None
        _lib.check("bsa_attn_bwd_delta", lib.bsa_attn_bwd_delta(
            _lib.ptr(o), _lib.ptr(dout), st, _lib.ptr(delta), code, B, H, N, D, stream))
        _lib.check("bsa_attn_bwd_dkdv", lib.bsa_attn_bwd_dkdv(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(dout), st, _lib.ptr(lse2),
            _lib.ptr(delta), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(lists.col_ptr),
            _lib.ptr(lists.row_idx), sb, sh, float(sm_scale), code, B, H, N, D, _lib.ptr(d4), dst,
            _lib.ptr(counter), _lib.ptr(status), stream))
        _lib.check("bsa_attn_bwd_dq", lib.bsa_attn_bwd_dq(
            _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(dout), st, _lib.ptr(lse2),
            _lib.ptr(delta), _lib.ptr(dq), _lib.ptr(lists.row_ptr), _lib.ptr(lists.col_idx),
            sb, sh, float(sm_scale), code, B, H, N, D, _lib.ptr(d4), dst, _lib.ptr(counter),
            _lib.ptr(status), stream))
    return dq, dk, dv


def _op_status(device):
    """The status word the public op hands to its kernels on the current stream of `device`, after
    a look at what earlier calls left in it (no synchronisation)."""
    with _on_device(device):
        state = _stream_state(device, _lib.stream_ptr(device).value or 0)
    if state is None:
        return None
    state.raise_if_reported()
    return state.status


class _attention(torch.autograd.Function):
    """Same signature as the reference's _attention (fa2_custom_mask/fa2_custom_mask.py:40-155)."""

    @staticmethod
    def forward(ctx, q, k, v, mask=None, sm_scale=1.3):
        if q.dim() != 4 or k.shape != q.shape or v.shape != q.shape:
            raise AssertionError("q, k, v must share the shape [B, H, N, D]")
        B, H, N, D = q.shape
        assert q.shape[-1] == k.shape[-1] == v.shape[-1]
        assert D in {16, 32, 64, 128, 256}  # the reference's own check (fa2_custom_mask.py:58)
        if D != 64:
            raise NotImplementedError("the kernels are built for head dimension 64 (16 and 32 are "
                                      "zero-padded to it by flash_attention_custom_mask)")
        if N % BLOCK:
            raise AssertionError("sequence length must be a multiple of 64")
        if not q.is_cuda:
            raise RuntimeError("flash_attention_custom_mask needs CUDA tensors; there is no CPU path")
        if not (q.dtype == k.dtype == v.dtype) or q.dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("q, k, v must all be float16 or all bfloat16")
        block, dense = _block_mask_for(mask, B, H, N, q.device)
        status = _op_status(q.device)
        # the forward lists each mask row inside the kernel; only the backward needs lists as data
        o, lse2, _ = attention_forward_masked(q, k, v, block, sm_scale, status=status, dense=dense)
        if any(ctx.needs_input_grad[:3]):
            lists = build_tile_lists(block, want_csr=True, want_csc=True)
            ctx.save_for_backward(q, k, v, o, lse2, lists.row_ptr, lists.col_idx,
                                  lists.col_ptr, lists.row_idx)
            ctx.lists_shape = (lists.Bm, lists.Hm, lists.nb)
            ctx.dense = dense  # the caller's mask (or an aligned copy of it): not to be changed before backward
        ctx.sm_scale = sm_scale
        ctx.HEAD_DIM = D
        ctx.USE_MASK = mask is not None
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse2, rp, ci, cp, ri = ctx.saved_tensors
        Bm, Hm, nb = ctx.lists_shape
        lists = TileLists(Bm=Bm, Hm=Hm, nb=nb, row_ptr=rp, col_idx=ci, col_ptr=cp, row_idx=ri)
        dq, dk, dv = attention_backward(q, k, v, o, lse2, do, lists, ctx.sm_scale,
                                        status=_op_status(q.device), dense=ctx.dense)
        return dq, dk, dv, None, None


def flash_attention_custom_mask(q, k, v, mask=None, sm_scale=1.3):
    """The reference's public op (fa2_custom_mask/fa2_custom_mask.py:157, `_attention.apply`), same
    positional arguments.  Head dimensions 16 and 32 run on the D = 64 kernels with zero columns
    appended to q, k, v (Q K^T is unchanged, the extra columns of P V are zero and are cut off
    again; autograd slices the gradients); 128 and 256, which the reference also lists, are not
    built."""
    D = q.shape[-1] if q.dim() == 4 else 0
    if D in (16, 32) and k.shape == q.shape and v.shape == q.shape:
        pad = (0, 64 - D)
        qp, kp, vp = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
        return _attention.apply(qp, kp, vp, mask, sm_scale)[..., :D].contiguous()
    return _attention.apply(q, k, v, mask, sm_scale)
