"""fa2_custom_mask — block-sparse FlashAttention-2 for NVIDIA B200, same import names as the
reference package (fa2_custom_mask/__init__.py:1-5) minus its raw Triton kernel objects."""
from .fa2_custom_mask import (  # noqa: F401
    TileLists,
    attention_backward,
    attention_forward,
    attention_forward_masked,
    build_groups_from_block_mask,
    build_tile_lists,
    check_status,
    new_status_word,
    flash_attention_custom_mask,
    reduce_dense_mask,
)
from . import sharding  # noqa: F401
from .functional import (  # noqa: F401
    apply_head_wise_reorder,
    apply_inv_reorder,
    inv_permute_attn_triton,
    permute_qkv_triton,
)
