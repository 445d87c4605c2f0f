"""GPU: the allocation-free block-sparse entry point (h3a_attn_fwd_sparse_static) against the regular one.

Some hosts hand the whole GPU to their own memory arena when they start and may not call cudaMalloc while
serving; they cannot supply the `workspace` the regular block-sparse call needs, so the library carries a
fixed 1 MiB scratch array for them.  Two calls in a row with different block indices check that the shared
array, which keeps whatever the previous call wrote, never leaks stale plan entries into a later result.
This file sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _case(grid, n_audio, window, H, seed):
    keep = O.neighbourhood_block_mask(grid, n_audio, window)
    rp, ci = O.mask_to_csr(keep)
    L = n_audio + grid[0] * grid[1] * grid[2]
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(L, H, 128, generator=g).bfloat16().cuda() for _ in range(3))
    return q, k, v, (rp, ci), keep


def test_static_scratch_entry_point_matches_regular_one_twice_in_a_row(lib):
    import pika_h3_flex_b200 as h3

    assert torch.cuda.is_available()
    assert h3.static_scratch_capacity() == 262144
    # first a wide index (many plan entries), then a narrow one on a shorter sequence: the second call sees the
    # first call's leftovers in the shared array and must not be affected by them
    # the third and fourth calls pass a logit bound (N(0,1) inputs: |q.k| / sqrt(128) stays far below 12): the fixed-
    # reference kernels, on CTA pairs for the 18-tile sequence, whose merged plan lives in the same array
    cases = [(_case((6, 8, 16), 256, (2, 8, 8), 2, 71), 0.0), (_case((3, 8, 16), 128, (0, 1, 1), 3, 72), 0.0),
             (_case((8, 16, 16), 256, (2, 8, 8), 2, 73), 12.0), (_case((6, 8, 16), 256, (1, 2, 2), 2, 74), 12.0)]
    for (q, k, v, csr, keep), bound in cases:
        bi = h3.BlockIndex.from_csr(csr[0], csr[1], keep.shape[1]).to("cuda")
        want = h3.attn_fwd(q, k, v, h3.MODE_BLOCK_SPARSE, block_index=bi, logit_bound=bound)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = torch.full_like(want, 3.0)
        before = torch.cuda.memory_allocated()
        h3.attn_fwd_sparse_static(q, k, v, bi, out, status_word=status, logit_bound=bound)
        assert torch.cuda.memory_allocated() == before  # the call took nothing from the caching allocator either
        assert h3.read_status(status) == 0
        # same kernels, same plan: bit-identical; the oracle bounds (2e-2 / 2e-3) hold as for the regular call
        assert torch.equal(out, want)
        st = O.error_stats(out.float().cpu(), O.attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), csr=csr))
        assert st["max_abs"] <= 2e-2 and st["mean_abs"] <= 2e-3, st


def test_static_scratch_entry_point_rejects_what_it_cannot_hold(lib):
    from pika_h3_flex_b200 import _lib

    p = _lib.AttnParams()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p.q = p.k = p.v = p.o = buf.data_ptr()
    p.row_ptr = p.col_idx = buf.data_ptr()
    for name in ("q", "k", "v", "o"):
        setattr(p, f"{name}_stride_l", 128)
        setattr(p, f"{name}_stride_h", 128)
    p.Lq = p.Lk = 128 * 600
    p.H, p.d, p.B = 1, 128, 1
    p.mode = _lib.MODE_BLOCK_SPARSE
    p.nnz = 262144  # plus 300 query-tile pairs: one more than fits
    assert lib.h3a_attn_fwd_sparse_static(C.byref(p), None) == _lib.H3A_ERR_STATIC_SCRATCH
    assert "static scratch" in _lib.status_string(_lib.H3A_ERR_STATIC_SCRATCH)
    p.mode = _lib.MODE_DENSE_BF16
    assert lib.h3a_attn_fwd_sparse_static(C.byref(p), None) == _lib.H3A_ERR_ARG
