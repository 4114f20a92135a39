"""CPU oracle for the block-sparse attention path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, the algorithms of the reference project
`rickyxie2004/Customize-Block-Sparse-Attention-with-Triton` that the CUDA library replaces.  It is
the checker for `tests/`, for the smoke test and for the CPU-baseline leg of the benchmark; the
product never imports it.  Every function cites the reference lines it follows (paths are relative
to the reference project's root).

Pinned against the reference itself: `tests/golden/make_golden.py` runs the reference's own code
(`build_groups_from_block_mask` natively, `_attn_fwd` / `reorder_kernel` / `inv_reorder_kernel`
under the Triton CPU interpreter) on seeded inputs and stores the results under `tests/golden/`;
`tests/test_oracle_golden.py` checks this file against those vectors.  The reference's backward
kernels produce wrong gradients, so gradients (and the log-sum-exp, which the reference never
computes) are pinned only by torch autograd / torch.logsumexp on the fp32 restatement:
"parity unpinned" by the reference for those two quantities.
"""
from __future__ import annotations

import math

import numpy as np
import torch

BLOCK = 64  # tile edge: BLOCK_M = BLOCK_N = 64 in fa2_custom_mask/fa2_fwd.py:13-14
LOG2E = 1.44269504  # the constant used at fa2_custom_mask/fa2_fwd.py:150


# --------------------------------------------------------------------------------------------
# synthetic inputs (shapes and distributions of kernel-test.py:13-19)
# --------------------------------------------------------------------------------------------
def make_block_mask(B, H, nb, density, seed, diagonal=True, causal=False):
    """Bernoulli(density) block mask [B,H,nb,nb] as in kernel-test.py:16-17; `diagonal` forces the
    diagonal blocks on; `causal` keeps only the lower triangle (sampled) plus the diagonal."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    m = torch.rand(B, H, nb, nb, generator=g) < density
    if causal:
        m = torch.tril(m, diagonal=-1)
    if diagonal:
        m = m | torch.eye(nb, dtype=torch.bool)
    return m


def make_qkv(B, H, N, D, seed, dtype=torch.float32, n=3):
    """n tensors ~ N(0,1) of shape [B,H,N,D] (kernel-test.py:13-15), generated in fp32 then cast."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randn(B, H, N, D, generator=g).to(dtype) for _ in range(n)]


def expand_block_mask(block: torch.Tensor) -> torch.Tensor:
    """Block mask -> dense mask, kernel-test.py:18."""
    return block.repeat_interleave(BLOCK, dim=-2).repeat_interleave(BLOCK, dim=-1)


def reduce_dense_mask(dense: torch.Tensor) -> torch.Tensor:
    """Dense mask [..., N, N] -> block mask [..., nb, nb]: a block is kept when any of its 64x64
    elements is kept (the inverse of kernel-test.py:18)."""
    *lead, n0, n1 = dense.shape
    assert n0 % BLOCK == 0 and n1 % BLOCK == 0
    v = dense.reshape(*lead, n0 // BLOCK, BLOCK, n1 // BLOCK, BLOCK)
    return v.ne(0).any(dim=-1).any(dim=-2)


def count_partial_tiles(dense: torch.Tensor) -> int:
    """Number of 64x64 tiles that are neither fully kept nor fully masked."""
    *lead, n0, n1 = dense.shape
    v = dense.reshape(*lead, n0 // BLOCK, BLOCK, n1 // BLOCK, BLOCK).ne(0)
    any_ = v.any(dim=-1).any(dim=-2)
    all_ = v.all(dim=-1).all(dim=-2)
    return int((any_ & ~all_).sum())


# --------------------------------------------------------------------------------------------
# mask preprocessing (fa2_custom_mask/fa2_custom_mask.py:15-38)
# --------------------------------------------------------------------------------------------
def build_groups(mask) -> tuple:
    """Restatement of build_groups_from_block_mask: groups[G,5] = (b,h,m,start,len) for the
    non-empty rows in (b,h,m) order, n_list = their ascending column indices concatenated;
    (None, None) when no block is kept (fa2_custom_mask/fa2_custom_mask.py:34-35)."""
    m = np.asarray(mask).astype(bool)
    B, H, nb, _ = m.shape
    groups, n_list = [], []
    for b in range(B):
        for h in range(H):
            for r in range(nb):
                cols = np.flatnonzero(m[b, h, r])
                if cols.size == 0:
                    continue
                groups.append([b, h, r, len(n_list), cols.size])
                n_list.extend(cols.tolist())
    if not groups:
        return None, None
    return np.asarray(groups, dtype=np.int32), np.asarray(n_list, dtype=np.int32)


def tile_lists(mask) -> dict:
    """All list products of the library's tile-list builder, from a [B,H,nb,nb] block mask:
    CSR (row_ptr, col_idx), transposed CSR (col_ptr, row_idx), and the reference's groups."""
    m = np.asarray(mask).astype(bool)
    B, H, nb, _ = m.shape
    flat = m.reshape(B * H, nb, nb)

    def csr(mat):  # mat [BH, major, minor]
        counts = mat.sum(-1).reshape(-1)
        ptr = np.zeros(counts.size + 1, dtype=np.int32)
        np.cumsum(counts, out=ptr[1:])
        idx = np.nonzero(mat.reshape(-1, mat.shape[-1]))[1].astype(np.int32)
        return ptr, idx

    row_ptr, col_idx = csr(flat)
    col_ptr, row_idx = csr(flat.transpose(0, 2, 1))
    groups, n_list = build_groups(m)
    return dict(row_ptr=row_ptr, col_idx=col_idx, col_ptr=col_ptr, row_idx=row_idx,
                groups=groups, n_list=n_list,
                meta=np.asarray([col_idx.size, 0 if groups is None else groups.shape[0]],
                                dtype=np.int32))


# --------------------------------------------------------------------------------------------
# attention, naive form (kernel-test.py:37-40) — the numeric oracle at every size
# --------------------------------------------------------------------------------------------
def attn_forward_dense(q, k, v, dense_mask, sm_scale):
    """fp32 masked softmax attention exactly as kernel-test.py:37-40 computes it, for an
    element-level boolean mask [.., N, N] (the reference's naive path masks per element; its kernel
    only knows whole blocks, fa2_custom_mask/fa2_fwd.py:57-75 shows the in-tile mask it intended).
    Returns (O, LSE) with LSE = logsumexp of the scaled, masked logits (natural log).
    Rows without any kept element give O = 0 and LSE = -inf (the reference's naive path gives NaN
    there; its kernel leaves rows of empty query blocks unwritten)."""
    qf, kf, vf = q.float(), k.float(), v.float()
    dense = dense_mask.to(torch.bool)
    s = torch.matmul(qf, kf.transpose(-2, -1)) * sm_scale
    s = s.masked_fill(~dense, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    o = torch.matmul(p, vf)
    return o, lse


def attn_forward(q, k, v, block_mask, sm_scale):
    """attn_forward_dense for a 64x64 block mask [.., nb, nb] (expanded as kernel-test.py:18)."""
    return attn_forward_dense(q, k, v, expand_block_mask(block_mask.to(torch.bool)), sm_scale)


def attn_forward_backward_dense(q, k, v, dense_mask, sm_scale, dout):
    """O, LSE and (dQ, dK, dV) by torch autograd through the fp32 naive form above."""
    qf = q.detach().float().requires_grad_(True)
    kf = k.detach().float().requires_grad_(True)
    vf = v.detach().float().requires_grad_(True)
    dense = dense_mask.to(torch.bool)
    s = torch.matmul(qf, kf.transpose(-2, -1)) * sm_scale
    s = s.masked_fill(~dense, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    empty = ~dense.any(dim=-1, keepdim=True)
    p = torch.softmax(s.masked_fill(empty, 0.0), dim=-1).masked_fill(empty, 0.0)
    o = torch.matmul(p, vf)
    o.backward(dout.float())
    return o.detach(), lse.detach(), qf.grad, kf.grad, vf.grad


def attn_forward_backward(q, k, v, block_mask, sm_scale, dout):
    """attn_forward_backward_dense for a 64x64 block mask."""
    return attn_forward_backward_dense(q, k, v, expand_block_mask(block_mask.to(torch.bool)),
                                       sm_scale, dout)


def naive_cpu_forward(q, k, v, dense_mask, sm_scale):
    """The reference's naive path verbatim in arithmetic (kernel-test.py:37-40), used as the timed
    CPU baseline: matmul, masked_fill(-inf), softmax, matmul."""
    attn = torch.matmul(q, k.transpose(-2, -1)) * sm_scale
    attn = attn.masked_fill(~dense_mask, float("-inf"))
    attn = torch.softmax(attn, dim=-1)
    return torch.matmul(attn, v)


# --------------------------------------------------------------------------------------------
# attention, tile loop of the reference kernel (fa2_custom_mask/fa2_fwd.py:122-206)
# --------------------------------------------------------------------------------------------
def attn_forward_tiled(q, k, v, groups, n_list, sm_scale):
    """Restatement of _attn_fwd: for each group (b,h,m,start,len) an online softmax over the
    listed key blocks in list order, exp2 domain with qk_scale = sm_scale * 1.44269504
    (fa2_custom_mask/fa2_fwd.py:150), fp32 accumulation, P rounded to the value dtype before P V
    (fa2_custom_mask/fa2_fwd.py:189).  Returns (O, M) where M is what the reference stores: the
    running row maximum in the exp2 domain (fa2_custom_mask/fa2_fwd.py:193-196), not an LSE.
    Rows that no group covers stay NaN in both outputs (the reference leaves them unwritten)."""
    B, H, N, D = q.shape
    dt = q.dtype
    qn = q.float().numpy()
    kn = k.float().numpy()
    vn = v.float().numpy()
    out = np.full((B, H, N, D), np.nan, dtype=np.float32)
    mrow = np.full((B, H, N), np.nan, dtype=np.float32)
    qk_scale = np.float32(sm_scale * LOG2E)
    for b, h, m, start, length in np.asarray(groups).tolist():
        qt = qn[b, h, m * BLOCK:(m + 1) * BLOCK]
        m_i = np.full(BLOCK, -np.inf, dtype=np.float32)
        l_i = np.ones(BLOCK, dtype=np.float32)
        acc = np.zeros((BLOCK, D), dtype=np.float32)
        for idx in range(length):
            n = int(n_list[start + idx])
            kt = kn[b, h, n * BLOCK:(n + 1) * BLOCK]
            vt = vn[b, h, n * BLOCK:(n + 1) * BLOCK]
            qk = (qt @ kt.T).astype(np.float32)
            m_ij = np.maximum(m_i, qk.max(axis=1) * qk_scale)
            p = np.exp2(qk * qk_scale - m_ij[:, None]).astype(np.float32)
            l_ij = p.sum(axis=1)
            alpha = np.exp2(m_i - m_ij).astype(np.float32)
            l_i = l_i * alpha + l_ij
            acc = acc * alpha[:, None]
            p_cast = torch.from_numpy(p).to(dt).float().numpy()
            acc = acc + p_cast @ vt
            m_i = m_ij
        out[b, h, m * BLOCK:(m + 1) * BLOCK] = acc / l_i[:, None]
        mrow[b, h, m * BLOCK:(m + 1) * BLOCK] = m_i
    return torch.from_numpy(out), torch.from_numpy(mrow)


# --------------------------------------------------------------------------------------------
# head-wise token reorder (fa2_custom_mask/permute.py, fa2_custom_mask/functional.py)
# --------------------------------------------------------------------------------------------
PERMUTATIONS = np.asarray([[0, 1, 2], [0, 2, 1], [1, 2, 0], [1, 0, 2], [2, 1, 0], [2, 0, 1]],
                          dtype=np.int32)  # fa2_custom_mask/functional.py:23-26
PERMUTATIONS_INV = np.asarray([[0, 1, 2], [0, 2, 1], [2, 0, 1], [1, 0, 2], [2, 1, 0], [1, 2, 0]],
                              dtype=np.int32)  # fa2_custom_mask/functional.py:69-76


def _dest_tokens(T, ext, order):
    """new_t for every t, following fa2_custom_mask/permute.py:24-52."""
    t = np.arange(T)
    e0, e1, e2 = ext
    f = t // (e1 * e2)
    r = t % (e1 * e2)
    coords = [f, r // e2, r % e2]
    dims = [e0, e1, e2]
    p0, p1, p2 = (int(x) for x in order)
    return coords[p0] * (dims[p1] * dims[p2]) + coords[p1] * dims[p2] + coords[p2]


def reorder(x: torch.Tensor, orders, F, H, W) -> torch.Tensor:
    """reorder_kernel (fa2_custom_mask/permute.py:5-58): out[b,h,new_t] = in[b,h,t]."""
    out = torch.empty_like(x)
    T = x.shape[2]
    for h in range(x.shape[1]):
        nt = torch.from_numpy(_dest_tokens(T, (F, H, W), np.asarray(orders)[h]))
        out[:, h, nt] = x[:, h]
    return out


def inv_reorder(x: torch.Tensor, orders, inv_orders, F, H, W) -> torch.Tensor:
    """inv_reorder_kernel (fa2_custom_mask/permute.py:60-126): the source grid has the extents
    permuted by `orders` (permute.py:80-90); `inv_orders` lays the coordinates back out."""
    out = torch.empty_like(x)
    T = x.shape[2]
    dims = [F, H, W]
    for h in range(x.shape[1]):
        o = [int(v) for v in np.asarray(orders)[h]]
        ext = (dims[o[0]], dims[o[1]], dims[o[2]])
        nt = torch.from_numpy(_dest_tokens(T, ext, np.asarray(inv_orders)[h]))
        out[:, h, nt] = x[:, h]
    return out


def reorder_by_view(x: torch.Tensor, orders, F, H, W) -> torch.Tensor:
    """The same permutation written with view/permute/reshape: an independent second statement."""
    B, heads, T, D = x.shape
    out = torch.empty_like(x)
    for h in range(heads):
        p = [int(v) for v in np.asarray(orders)[h]]
        g = x[:, h].reshape(B, F, H, W, D).permute(0, 1 + p[0], 1 + p[1], 1 + p[2], 4)
        out[:, h] = g.reshape(B, T, D)
    return out


def active_tile_flops(n_tiles: int, D: int = 64, backward: bool = False) -> float:
    """Algorithmic FLOPs: 4*64*64*D per listed tile forward (two GEMMs), 10*64*64*D backward."""
    return float(n_tiles) * (10 if backward else 4) * BLOCK * BLOCK * D


__all__ = [n for n in dir() if not n.startswith("_")]
