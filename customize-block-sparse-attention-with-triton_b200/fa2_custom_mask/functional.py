"""Head-wise token reorder helpers with the reference's names and argument order
(fa2_custom_mask/functional.py:5-84); the gather kernels run in libbsattn instead of Triton.

A video-DiT attention layer calls  permute_qkv_triton -> flash_attention_custom_mask ->
inv_permute_attn_triton : each head re-lays-out its F x H x W image-token grid in one of six axis
orders so that its attention pattern becomes block-sparse, and the output is laid back.
"""
from __future__ import annotations

import torch

from . import _lib

# axis orders selectable per head, and their inverses (fa2_custom_mask/functional.py:23-26, 69-76)
_PERMUTATIONS = ((0, 1, 2), (0, 2, 1), (1, 2, 0), (1, 0, 2), (2, 1, 0), (2, 0, 1))
_PERMUTATIONS_INV = ((0, 1, 2), (0, 2, 1), (2, 0, 1), (1, 0, 2), (2, 1, 0), (1, 2, 0))
_table_cache = {}


def _tables(device):
    """The two constant tables, created once per device (the reference rebuilds them per call)."""
    key = (device.type, device.index)
    if key not in _table_cache:
        _table_cache[key] = (
            torch.tensor(_PERMUTATIONS, dtype=torch.int32, device=device),
            torch.tensor(_PERMUTATIONS_INV, dtype=torch.int32, device=device))
    return _table_cache[key]


def _check(tensor, F, H, W):
    BS, N_head, N_token, D = tensor.shape
    assert N_token == F * H * W
    if not tensor.is_cuda:
        raise RuntimeError("token reorder needs CUDA tensors; there is no CPU path")
    if tensor.stride(3) != 1:
        tensor = tensor.contiguous()
    return tensor, BS, N_head, N_token, D


def _orders_i32(orders, device):
    return orders.to(device=device, dtype=torch.int32).contiguous()


def _identity_orders(device, n_head):
    key = (device.type, device.index, n_head)
    if key not in _table_cache:
        _table_cache[key] = torch.tensor([[0, 1, 2]], dtype=torch.int32, device=device).repeat(n_head, 1)
    return _table_cache[key]


def _write_back(view, dense, F, H, W):
    """view[...] = dense for a slice `view` of a caller's tensor, through the gather kernel with
    the identity order (it moves 16-byte pieces at the copy bandwidth whatever the strides)."""
    lib = _lib.load()
    BS, N_head, N_token, D = view.shape
    if view.stride(3) != 1 or dense.stride(3) != 1:
        view.copy_(dense)
        return
    with torch.cuda.device(view.device):
        _lib.check("bsa_reorder_strided", lib.bsa_reorder_strided(
            _lib.ptr(dense), _lib.strides4(dense), _lib.ptr(view), _lib.strides4(view),
            _lib.ptr(_identity_orders(view.device, N_head)), BS, N_head, N_token, D, F, H, W,
            view.element_size(), _lib.stream_ptr(view.device)))


def apply_head_wise_reorder(tensor, permute_orders, F, H, W):
    """out[b, h, new_t] = tensor[b, h, t]; new_t re-lays-out t's (f, y, x) grid coordinate in the
    axis order permute_orders[h] (reorder_kernel, fa2_custom_mask/permute.py:5-58)."""
    lib = _lib.load()
    tensor, BS, N_head, N_token, D = _check(tensor, F, H, W)
    # a slice or any other view with unit last stride is read where it lies; the result is dense
    output = torch.empty(tensor.shape, dtype=tensor.dtype, device=tensor.device)
    orders = _orders_i32(permute_orders, tensor.device)
    with torch.cuda.device(tensor.device):
        _lib.check("bsa_reorder_strided", lib.bsa_reorder_strided(
            _lib.ptr(tensor), _lib.strides4(tensor), _lib.ptr(output), _lib.strides4(output),
            _lib.ptr(orders), BS, N_head, N_token, D, F, H, W, tensor.element_size(),
            _lib.stream_ptr(tensor.device)))
    return output


def permute_qkv_triton(query, key, value, permute_plan, i_block, F=13, H=30, W=45, n_text_tokens=226):
    """Reorders the image tokens of q, k, v in place (text tokens stay) and returns the same three
    tensors, like the reference (fa2_custom_mask/functional.py:22-43)."""
    permutations, _ = _tables(query.device)
    idx = permute_plan['permute'][i_block]  # [N_head]
    permute_orders = permutations[idx]      # [N_head, 3]
    for t in (query, key, value):
        image = t[:, :, n_text_tokens:, :]
        _write_back(image, apply_head_wise_reorder(image, permute_orders, F, H, W), F, H, W)
    return query, key, value


def apply_inv_reorder(tensor, permute_orders, inv_permute_orders, F, H, W):
    """Inverse gather (inv_reorder_kernel, fa2_custom_mask/permute.py:60-126): `tensor` is laid out
    in the order permute_orders[h]; inv_permute_orders[h] lays it back to (F, H, W)."""
    lib = _lib.load()
    tensor, BS, N_head, N_token, D = _check(tensor, F, H, W)
    output = torch.empty(tensor.shape, dtype=tensor.dtype, device=tensor.device)
    orders = _orders_i32(permute_orders, tensor.device)
    inv_orders = _orders_i32(inv_permute_orders, tensor.device)
    with torch.cuda.device(tensor.device):
        _lib.check("bsa_inv_reorder_strided", lib.bsa_inv_reorder_strided(
            _lib.ptr(tensor), _lib.strides4(tensor), _lib.ptr(output), _lib.strides4(output),
            _lib.ptr(orders), _lib.ptr(inv_orders), BS, N_head, N_token, D, F, H, W,
            tensor.element_size(), _lib.stream_ptr(tensor.device)))
    return output


def inv_permute_attn_triton(attn_out, permute_plan, i_block, F=13, H=30, W=45, n_text_tokens=226):
    """Lays the image tokens of the attention output back in place and returns attn_out
    (fa2_custom_mask/functional.py:64-84)."""
    permutations, permutations_inv = _tables(attn_out.device)
    idx = permute_plan['permute'][i_block]
    permute_orders = permutations[idx]
    inv_permute_orders = permutations_inv[idx]
    attn_image = attn_out[:, :, n_text_tokens:, :]
    _write_back(attn_image, apply_inv_reorder(attn_image, permute_orders, inv_permute_orders, F, H, W),
                F, H, W)
    return attn_out
