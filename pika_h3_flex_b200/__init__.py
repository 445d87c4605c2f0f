"""B200-native (sm_100a) attention path for the Pika H3 Flex joint video+audio DiT.

Python here is host-side plumbing over ``libh3attn.so`` (hand-written CUDA behind a C ABI, see
``include/h3attn.h``); there is no CPU or library fallback.
"""
from . import _lib, ops
from ._lib import (
    MODE_BLOCK_SPARSE,
    MODE_DENSE_BF16,
    MODE_FP8_QK,
    H3AError,
)
from .graphs import StepGraph, renoise_sample
from .host_path import HostJointAttention
from .layout import position_grid
from .ops import (
    BlockIndex,
    adaln_norm,
    attn_fwd,
    attn_fwd_sparse_static,
    static_scratch_capacity,
    build_block_index,
    joint_attention,
    proj_fwd,
    qk_prep,
    read_status,
    check_status,
    StatusWord,
    rope_table,
    rope_table_from_cos_sin,
)

__all__ = [
    "_lib", "ops", "H3AError", "MODE_DENSE_BF16", "MODE_FP8_QK", "MODE_BLOCK_SPARSE",
    "BlockIndex", "adaln_norm", "attn_fwd", "attn_fwd_sparse_static", "static_scratch_capacity", "build_block_index", "joint_attention", "proj_fwd", "qk_prep",
    "read_status", "check_status", "StatusWord", "rope_table", "rope_table_from_cos_sin", "position_grid", "HostJointAttention", "StepGraph", "renoise_sample",
]
