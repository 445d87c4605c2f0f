"""Host-buffer entry path: the whole hot path driven from pinned HOST tensors.

The reference moves its tensors to the GPU in full before the forward and back afterwards
(``src/pika_h3/core/wrapper.py:164-166``, ``src/pika_h3/pipeline.py:115,128``).  Here the three transfers and the
kernels are pipelined over groups of heads (attention is independent per head): while group g is being
computed, group g+1 is on its way in and group g-1 on its way out, each on its own CUDA stream.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib, ops
from ._lib import check


def _copy_heads(dst: torch.Tensor, src: torch.Tensor, h0: int, h1: int, to_host: bool, stream: torch.cuda.Stream) -> None:
    """Copy heads [h0, h1) of a token-major ``[L, H, 128]`` bf16 tensor between pinned host and device."""
    L, H, d = src.shape
    row = H * d * 2
    off = h0 * d * 2
    check(
        _lib.load().h3a_memcpy2d_async(dst.data_ptr() + off, row, src.data_ptr() + off, row, (h1 - h0) * d * 2, L,
                                      1 if to_host else 0, stream.cuda_stream),
        "h3a_memcpy2d_async",
    )


def default_head_groups(H: int, copy_to_compute: float = 0.75) -> list:
    """Head groups for the pipeline.  Only the first group's copy-in and the last group's copy-out are exposed, so
    both are small; in between a group is as large as its copy-in can be while still finishing before the groups
    ahead of it have been computed.  ``copy_to_compute`` = time to bring one head's Q, K, V in / time to compute
    one head (0.75 measured for dense bf16 at the 480p-like length over PCIe 5 x16); with copy time c per head the
    condition  c * n_g <= c * first + (c / copy_to_compute - c) * heads_before_g  gives the growth rule below."""
    first = max(1, H // 20)
    last = max(1, H // 16) if H > 2 else 0
    if first + last >= H:
        return [H]
    groups, done = [first], first
    gain = max(0.0, 1.0 / max(copy_to_compute, 1e-3) - 1.0)
    while done < H - last:
        n = max(1, min(int(first + gain * done), H - last - done))
        groups.append(n)
        done += n
    if H - done > 0:
        groups.append(H - done)
    return groups


class HostJointAttention:
    """``out_host = HostJointAttention(L, H)(q_host, k_host, v_host, rope, out_host)`` with pinned ``[L, H, 128]``
    bf16 host tensors.  Device staging buffers and streams are created once and reused."""

    def __init__(self, L: int, H: int, mode: int = _lib.MODE_DENSE_BF16, block_index: Optional[ops.BlockIndex] = None,
                 head_groups: Optional[Sequence[int]] = None, device=None, copy_to_compute: float = 0.75):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.L, self.H, self.mode, self.block_index = L, H, mode, block_index
        if head_groups is None:
            head_groups = default_head_groups(H, copy_to_compute)
        if sum(head_groups) != H:
            raise ValueError("head_groups must sum to H")
        self.groups = list(head_groups)
        mk = lambda: torch.empty(L, H, ops.HEAD_DIM, dtype=torch.bfloat16, device=self.device)
        self.dq, self.dk, self.dv, self.do = mk(), mk(), mk(), mk()
        self.s_in, self.s_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rope: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        for t in (q, k, v, out):
            if t.is_cuda or not t.is_pinned() or t.dtype != torch.bfloat16 or tuple(t.shape) != (self.L, self.H, ops.HEAD_DIM) or not t.is_contiguous():
                raise ValueError("host tensors must be pinned, contiguous bf16 [L, H, 128]")
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)   # staging buffers may still be read by earlier work on the caller's stream
        self.s_out.wait_stream(cur)
        fp8 = self.mode == _lib.MODE_FP8_QK
        h0 = 0
        for g in self.groups:
            h1 = h0 + g
            for dst, src in ((self.dq, q), (self.dk, k), (self.dv, v)):
                _copy_heads(dst, src, h0, h1, False, self.s_in)
            ev_in = torch.cuda.Event()
            ev_in.record(self.s_in)
            cur.wait_event(ev_in)
            qp, kp, qs, ks = ops.qk_prep(self.dq[:, h0:h1], self.dk[:, h0:h1], rope, rope, fp8=fp8)
            ops.attn_fwd(qp, kp, self.dv[:, h0:h1], self.mode, qs, ks, self.block_index, out=self.do[:, h0:h1],
                         logit_bound=ops.normed_logit_bound(fp8=fp8))
            ev_c = torch.cuda.Event()
            ev_c.record(cur)
            self.s_out.wait_event(ev_c)
            _copy_heads(out, self.do, h0, h1, True, self.s_out)
            h0 = h1
        cur.wait_stream(self.s_out)  # the result is complete in stream order of the caller's stream
        return out
