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


class HostUlyssesAttention:
    """The host-buffer call under Ulysses sequence parallelism: every rank passes pinned host tensors holding ITS
    ``[L/P, H, 128]`` shard of Q, K, V and gets its shard of the output in a pinned host tensor.

    The pipeline of :class:`HostJointAttention` (copy-in / compute / copy-out over groups of heads) needs each
    group to be a CONTIGUOUS head range, so heads are dealt to ranks round-robin here (head ``h`` is computed by
    rank ``h % P``) instead of in blocks: local head slots ``[j0, j1)`` are then the heads ``[j0 P, j1 P)``.  Per
    group: one 2-D copy per tensor brings the head range in (copy stream), preparation and a pack into per-peer
    blocks run on a preparation stream and start the inbound ``all_to_all``; the caller's stream places the blocks,
    runs the attention and starts the outbound ``all_to_all``; a copy-out stream unpacks into token-major order
    and copies the head range to the host.  Dense bf16 and block-sparse modes (FP8-QK would add a scale exchange).
    """

    def __init__(self, Ls: int, H: int, mode: int = _lib.MODE_DENSE_BF16, block_index: Optional[ops.BlockIndex] = None,
                 group=None, slot_groups: Optional[Sequence[int]] = None, device=None):
        import torch.distributed as dist

        if mode == _lib.MODE_FP8_QK:
            raise NotImplementedError("FP8-QK under the host-buffer Ulysses path is not built")
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.Ls, self.H, self.mode, self.block_index = Ls, H, mode, block_index
        self.hp = (H + self.world - 1) // self.world  # head slots per rank
        if slot_groups is None:  # measured on 2 GPUs: the fine schedule (26.7 ms) beats five coarse groups (28.8 ms)
            slot_groups = default_head_groups(self.hp)
        if sum(slot_groups) != self.hp or min(slot_groups) < 1:
            raise ValueError("slot_groups must be positive and sum to ceil(H / world)")
        self.slot_groups = list(slot_groups)
        mk = lambda: torch.empty(Ls, H, ops.HEAD_DIM, dtype=torch.bfloat16, device=self.device)
        self.dq, self.dk, self.dv, self.do = mk(), mk(), mk(), mk()
        self.s_in, self.s_prep, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self._keep = []

    def _pack(self, x_hm: torch.Tensor, hg: int) -> torch.Tensor:
        """``[n <= hg*P, Ls, C]`` head-major (head ``j*P + p`` at row ``j*P + p``) -> ``[P, hg, Ls, C]`` contiguous: the
        block for peer p holds its heads of this group; missing (padded) heads are zero."""
        P, Ls, Cc = self.world, x_hm.shape[1], x_hm.shape[2]
        if x_hm.shape[0] < hg * P:
            x_hm = torch.cat([x_hm, x_hm.new_zeros(hg * P - x_hm.shape[0], Ls, Cc)], dim=0)
        return x_hm.view(hg, P, Ls, Cc).permute(1, 0, 2, 3).contiguous()

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rope: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        dist, P, Ls, H, Cc = self.dist, self.world, self.Ls, self.H, ops.HEAD_DIM
        for t in (q, k, v, out):
            if t.is_cuda or not t.is_pinned() or t.dtype != torch.bfloat16 or tuple(t.shape) != (Ls, H, Cc) or not t.is_contiguous():
                raise ValueError("host tensors must be pinned, contiguous bf16 [L/P, H, 128] shards")
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_prep, self.s_out):
            s.wait_stream(cur)  # staging buffers may still be in use by earlier work on the caller's stream
        # Temporaries that cross streams (packed blocks read by the exchange, received blocks read on another stream)
        # stay referenced until the NEXT call has made every stream wait for the caller's stream: freed earlier, the
        # caching allocator could hand a block to new work on the stream that allocated it while the exchange,
        # which runs on the communication library's own stream, still reads it.
        self._keep = keep = []
        bound = ops.normed_logit_bound()
        # ---- all copy-ins are queued at once on their stream, one event per group
        ranges, ev_in = [], []
        j0 = 0
        for n in self.slot_groups:
            h0, h1 = j0 * P, min((j0 + n) * P, H)
            ranges.append((j0, n, h0, h1))
            if h1 > h0:
                for dst, src in ((self.dq, q), (self.dk, k), (self.dv, v)):
                    _copy_heads(dst, src, h0, h1, False, self.s_in)
            e = torch.cuda.Event()
            e.record(self.s_in)
            ev_in.append(e)
            j0 += n

        def stage_in(g):
            """Preparation stream: prepare and pack group g, start its inbound exchange."""
            _, n, h0, h1 = ranges[g]
            with torch.cuda.stream(self.s_prep):
                self.s_prep.wait_event(ev_in[g])
                staged, works = [], []
                if h1 > h0:
                    qp, kp, _, _ = ops.qk_prep(self.dq[:, h0:h1], self.dk[:, h0:h1], rope, rope)
                    srcs = [qp.permute(1, 0, 2), kp.permute(1, 0, 2), self.dv[:, h0:h1].permute(1, 0, 2).contiguous()]
                else:  # a group of padded heads only
                    srcs = [torch.zeros(0, Ls, Cc, dtype=torch.bfloat16, device=self.device)] * 3
                for x_hm in srcs:
                    send = self._pack(x_hm, n)
                    recv = torch.empty_like(send)  # [source rank, head slot, token, c]
                    works.append(dist.all_to_all([recv[p] for p in range(P)], [send[p] for p in range(P)], group=self.group, async_op=True))
                    recv.record_stream(cur)
                    staged.append(recv)
                    keep.extend((x_hm, send, recv))
            return staged, works

        def stage_out(g, o_hm, work):
            """Copy-out stream: wait for group g's outbound exchange, restore token-major order, copy to the host."""
            _, n, h0, h1 = ranges[g]
            with torch.cuda.stream(self.s_out):
                work.wait()
                if h1 > h0:
                    heads = o_hm.permute(1, 0, 2, 3).reshape(n * P, Ls, Cc)[: h1 - h0]  # row j*P + p = head h0 + j*P + p
                    keep.append(heads)
                    self.do[:, h0:h1].copy_(heads.permute(1, 0, 2))
                    _copy_heads(out, self.do, h0, h1, True, self.s_out)

        pending = stage_in(0)
        for g, (_, n, h0, h1) in enumerate(ranges):
            staged, works = pending
            for w in works:
                w.wait()  # the caller's stream waits for the exchange
            qh, kh, vh = (s.permute(1, 0, 2, 3).reshape(n, P * Ls, Cc) for s in staged)  # [head slot, all tokens, c]
            oh = torch.empty(n, P * Ls, Cc, dtype=torch.bfloat16, device=self.device)
            ops.attn_fwd(qh.permute(1, 0, 2), kh.permute(1, 0, 2), vh.permute(1, 0, 2), self.mode, None, None, self.block_index,
                         out=oh.permute(1, 0, 2), logit_bound=bound)
            if g + 1 < len(ranges):
                # the next group's preparation and inbound exchange are issued while this group's attention runs (host
                # time hidden behind it) and BEFORE this group's outbound exchange, which has to wait for the attention
                pending = stage_in(g + 1)
            send = oh.view(n, P, Ls, Cc).permute(1, 0, 2, 3).contiguous()  # [destination rank, head slot, its tokens, c]
            recv = torch.empty_like(send)                                  # [owner rank p, head slot j, my tokens, c]
            work = dist.all_to_all([recv[p] for p in range(P)], [send[p] for p in range(P)], group=self.group, async_op=True)
            recv.record_stream(self.s_out)
            keep.extend((qh, kh, vh, oh, send, recv))
            stage_out(g, recv, work)
        cur.wait_stream(self.s_out)  # the result is complete in stream order of the caller's stream
        return out
