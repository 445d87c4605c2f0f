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


def copy_to_compute_estimate(L: int, mode: int = _lib.MODE_DENSE_BF16, density: float = 1.0, link_gbs: float = 50.0) -> float:
    """Time to bring one head's Q, K and V over the host link / time to compute that head, from the shape alone.
    Rates measured on B200 under its power cap: 1.3 PFLOP/s dense bf16, 1.5 FP8-QK, 1.1 on the kept tiles of a
    block-sparse mask; ``link_gbs`` is what one direction of the host link gives this rank (about 50 GB/s alone on
    PCIe 5 x16, half that with four ranks copying at once).  Dense bf16 at the 480p-like length: 0.79 (0.75 measured);
    the literal block-sparse rule at the 720p-like length (7 % of the tiles): 3.6 - the call is bound by the copies,
    whatever the kernel does."""
    rate = {_lib.MODE_DENSE_BF16: 1.3e15, _lib.MODE_FP8_QK: 1.5e15, _lib.MODE_BLOCK_SPARSE: 1.1e15}.get(mode, 1.3e15)
    copy_s = 3.0 * L * ops.HEAD_DIM * 2 / (link_gbs * 1e9)
    compute_s = 4.0 * L * L * ops.HEAD_DIM * max(density, 1e-6) / rate
    return copy_s / compute_s


class HostJointAttention:
    """``out_host = HostJointAttention(L, H)(q_host, k_host, v_host, rope, out_host)`` with pinned ``[L, H, 128]``
    bf16 host tensors.  Device staging buffers and streams are created once and reused.  ``copy_to_compute`` (default:
    estimated from the length, the mode and the block index's density) sizes the head groups of the pipeline;
    ``bound`` says which side the call waits for, "copy" or "compute"."""

    def __init__(self, L: int, H: int, mode: int = _lib.MODE_DENSE_BF16, block_index: Optional[ops.BlockIndex] = None,
                 head_groups: Optional[Sequence[int]] = None, device=None, copy_to_compute: Optional[float] = None,
                 status: Optional[ops.StatusWord] = None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.status = status if status is not None else ops.StatusWord(self.device)
        self.L, self.H, self.mode, self.block_index = L, H, mode, block_index
        if copy_to_compute is None:
            copy_to_compute = copy_to_compute_estimate(L, mode, block_index.density if block_index is not None else 1.0)
        self.copy_to_compute = float(copy_to_compute)
        self.bound = "copy" if self.copy_to_compute >= 1.0 else "compute"
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
                         logit_bound=ops.normed_logit_bound(fp8=fp8), status_word=self.status.tensor())
            ev_c = torch.cuda.Event()
            ev_c.record(cur)
            self.s_out.wait_event(ev_c)
            _copy_heads(out, self.do, h0, h1, True, self.s_out)
            h0 = h1
        cur.wait_stream(self.s_out)  # the result is complete in stream order of the caller's stream
        return out

    def check_status(self) -> None:
        """Synchronise and raise ``H3AError`` when a launch of this object gave up a bounded wait or refused its block
        index: the host buffer then holds an incomplete result."""
        self.status.check("HostJointAttention")


class HostUlyssesAttention:
    """The host-buffer call under Ulysses sequence parallelism: every rank passes pinned host tensors holding ITS
    ``[L/P, H, 128]`` shard of Q, K, V and gets its shard of the output in a pinned host tensor.

    The pipeline of :class:`HostJointAttention` (copy-in / compute / copy-out over groups of heads) needs each
    group to be a CONTIGUOUS head range on the host side, so heads are dealt to ranks round-robin here (head ``h``
    is computed by rank ``h % P`` in its head slot ``h // P``) instead of in blocks: local head slots ``[j0, j1)``
    are then the heads ``[j0 P, j1 P)``.  Per group of slots, on four streams:

      copy-in      one 2-D copy per tensor brings the head range into token-major staging buffers
      scatter      the preparation kernel (RMSNorm + rotation; a plain re-layout for V) stores every row straight
                   into the memory of the rank that owns the row's head (``h3a_qk_prep_scatter``, see ``peer.py``);
                   the ranks then meet
      attention    each rank runs its slots of the group; the kernel stores every output row straight into the
                   token-major output staging buffer of the rank that holds the row's token; the ranks meet again
      copy-out     the head range of the output staging buffer goes to the host

    so a group's copy-in overlaps the previous group's attention and the copy-out of the one before.  FP8-QK:
    the rows travel as bf16 and each owner quantises its heads (block scales need whole 128-token blocks of the
    full sequence).  ``transport="nccl"`` keeps the staged ``all_to_all`` exchange (dense bf16 and block-sparse
    only) for comparison.  ``stage_ms()`` gives the device time of each stage of the last call.
    """

    def __init__(self, Ls: int, H: int, mode: int = _lib.MODE_DENSE_BF16, block_index: Optional[ops.BlockIndex] = None,
                 group=None, slot_groups: Optional[Sequence[int]] = None, device=None, status: Optional[ops.StatusWord] = None,
                 transport: str = "auto"):
        import torch.distributed as dist

        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if transport not in ("auto", "peer", "nccl"):
            raise ValueError("transport must be auto, peer or nccl")
        self.transport = "peer" if transport == "auto" else transport
        self._auto = transport == "auto"
        self.peer_unavailable = None
        if self.transport == "nccl" and mode == _lib.MODE_FP8_QK:
            raise NotImplementedError("FP8-QK under the host-buffer Ulysses path needs the peer transport")
        self.status = status if status is not None else ops.StatusWord(self.device)
        self.Ls, self.H, self.mode, self.block_index = Ls, H, mode, block_index
        P = self.world
        self.hp = (H + P - 1) // P  # head slots per rank
        if block_index is not None:
            nt = (P * Ls + ops.TILE - 1) // ops.TILE
            if block_index.n_q_tiles != nt or block_index.n_k_tiles != nt:
                raise ValueError("block index does not describe the full sequence")
        if slot_groups is None:
            # peer transport: a group costs two meetings of the ranks and nothing else, so small groups hide the most
            # copy time; the staged exchange pays per group and prefers the coarser schedule
            slot_groups = [1] * self.hp if (self.transport == "peer" and self.hp <= 8) else default_head_groups(self.hp)
        if sum(slot_groups) != self.hp or min(slot_groups) < 1:
            raise ValueError("slot_groups must be positive and sum to ceil(H / world)")
        self.slot_groups = list(slot_groups)
        mk = lambda: torch.empty(Ls, H, ops.HEAD_DIM, dtype=torch.bfloat16, device=self.device)
        self.dq, self.dk, self.dv = mk(), mk(), mk()
        self.s_in, self.s_prep, self.s_out = (torch.cuda.Stream(self.device) for _ in range(3))
        self._keep = []
        self._marks = None
        self.arena = None
        if self.transport == "peer":
            from .peer import Carver, PeerArena, PeerUnavailable

            c = Carver()
            L = P * Ls
            nb = self.hp * L * ops.HEAD_DIM * 2
            self._off = {n: c.take(nb) for n in ("q", "k", "v")}
            self._off["o"] = c.take(Ls * H * ops.HEAD_DIM * 2)
            try:
                self.arena = PeerArena(c.size, group, self.device)  # fails on every rank alike
            except PeerUnavailable as exc:
                if not self._auto or mode == _lib.MODE_FP8_QK:
                    raise
                self.transport, self.peer_unavailable = "nccl", str(exc)
                if slot_groups is None:
                    self.slot_groups = default_head_groups(self.hp)
        if self.transport == "peer":
            self.qh, self.kh, self.vh = (self.arena.tensor(self._off[n], (self.hp, L, ops.HEAD_DIM), torch.bfloat16) for n in ("q", "k", "v"))
            self.do = self.arena.tensor(self._off["o"], (Ls, H, ops.HEAD_DIM), torch.bfloat16)
        else:
            self.do = mk()

    def close(self) -> None:
        if self.arena is not None:
            self.arena.close()
            self.arena = None

    def check_status(self) -> None:
        self.status.check("HostUlyssesAttention")

    def stage_ms(self):
        """Device time of each stage of the last call on this rank (sums over the groups; the stages overlap, so the
        sums add up to more than the call): host->device copies, preparation + scatter, attention, device->host
        copies, and the span of the whole call."""
        if not self._marks:
            return None
        torch.cuda.synchronize(self.device)
        out = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self._marks.items() if k != "span"}
        a, b = self._marks["span"]
        out["call"] = a.elapsed_time(b)
        return out

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rope: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        Ls, H, Cc = self.Ls, self.H, ops.HEAD_DIM
        for t in (q, k, v, out):
            if t.is_cuda or not t.is_pinned() or t.dtype != torch.bfloat16 or tuple(t.shape) != (Ls, H, Cc) or not t.is_contiguous():
                raise ValueError("host tensors must be pinned, contiguous bf16 [L/P, H, 128] shards")
        return self._call_peer(q, k, v, rope, out) if self.transport == "peer" else self._call_nccl(q, k, v, rope, out)

    def _call_peer(self, q, k, v, rope, out):
        P, Ls, H, Cc, rank = self.world, self.Ls, self.H, ops.HEAD_DIM, self.rank
        L = P * Ls
        fp8 = self.mode == _lib.MODE_FP8_QK
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_prep, self.s_out):
            s.wait_stream(cur)  # staging buffers may still be in use by earlier work on the caller's stream
        bound = ops.normed_logit_bound(fp8=fp8)
        ev = lambda: torch.cuda.Event(enable_timing=True)
        marks = {"h2d": [], "prep_scatter": [], "attention": [], "d2h": []}
        span0 = ev()
        span0.record(cur)
        ranges, ev_in = [], []
        j0 = 0
        for n in self.slot_groups:
            h0, h1 = j0 * P, min((j0 + n) * P, H)
            ranges.append((j0, n, h0, h1))
            a, b = ev(), ev()
            a.record(self.s_in)
            if h1 > h0:
                for dst, src in ((self.dq, q), (self.dk, k), (self.dv, v)):
                    _copy_heads(dst, src, h0, h1, False, self.s_in)
            b.record(self.s_in)
            marks["h2d"].append((a, b))
            ev_in.append(b)
            j0 += n

        def owners(name, h0):
            # round robin: consecutive heads already go to consecutive ranks; each rank starts one head further
            return ops.HeadOwners([self.arena.addr(p, self._off[name]) for p in range(P)], self.hp, True, rank * Ls, L, head0=h0,
                                  start_head=rank + 1)

        def stage_in(g):
            """Scatter stream: prepare group g's heads of this rank's tokens into their owners' memory, then meet."""
            _, n, h0, h1 = ranges[g]
            with torch.cuda.stream(self.s_prep):
                self.s_prep.wait_event(ev_in[g])
                a, b = ev(), ev()
                a.record(self.s_prep)
                if h1 > h0:
                    ops.prep_scatter(self.dq[:, h0:h1], owners("q", h0), rope)
                    ops.prep_scatter(self.dk[:, h0:h1], owners("k", h0), rope)
                    ops.prep_scatter(self.dv[:, h0:h1], owners("v", h0), no_norm=True)
                b.record(self.s_prep)
                marks["prep_scatter"].append((a, b))
                self.arena.barrier()
                done = torch.cuda.Event()
                done.record(self.s_prep)
            return done

        pending = stage_in(0)
        for g, (j0, n, h0, h1) in enumerate(ranges):
            cur.wait_event(pending)
            n_real = sum(1 for j in range(j0, j0 + n) if j * P + rank < H)  # this rank's real heads among the group's slots
            if n_real > 0:
                a, b = ev(), ev()
                a.record(cur)
                qg, kg, vg = (t[j0 : j0 + n_real].permute(1, 0, 2) for t in (self.qh, self.kh, self.vh))
                qs = ks = None
                if fp8:
                    qg, kg, qs, ks = ops.qk_prep(qg, kg, fp8=True, no_norm=True)
                head = j0 * P + rank  # first head of the launch; the next slot's head is P heads further
                to = ops.RankOutputs([self.arena.addr(t, self._off["o"]) + head * Cc * 2 for t in range(P)], Ls, H * Cc, P * Cc)
                ops.attn_fwd(qg, kg, vg, self.mode, qs, ks, self.block_index, out_ranks=to, logit_bound=bound,
                             status_word=self.status.tensor())
                b.record(cur)
                marks["attention"].append((a, b))
            if g + 1 < len(ranges):
                pending = stage_in(g + 1)  # issued while this group's attention runs
            self.arena.barrier()  # every rank's output rows of this group have landed
            landed = torch.cuda.Event()
            landed.record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(landed)
                a, b = ev(), ev()
                a.record(self.s_out)
                if h1 > h0:
                    _copy_heads(out, self.do, h0, h1, True, self.s_out)
                b.record(self.s_out)
                marks["d2h"].append((a, b))
        cur.wait_stream(self.s_out)  # the result is complete in stream order of the caller's stream
        span1 = ev()
        span1.record(cur)
        marks["span"] = (span0, span1)
        self._marks = marks
        return out

    def _pack(self, x_hm: torch.Tensor, hg: int) -> torch.Tensor:
        """``[n <= hg*P, Ls, C]`` head-major (head ``j*P + p`` at row ``j*P + p``) -> ``[P, hg, Ls, C]`` contiguous: the
        block for peer p holds its heads of this group; missing (padded) heads are zero."""
        P, Ls, Cc = self.world, x_hm.shape[1], x_hm.shape[2]
        if x_hm.shape[0] < hg * P:
            x_hm = torch.cat([x_hm, x_hm.new_zeros(hg * P - x_hm.shape[0], Ls, Cc)], dim=0)
        return x_hm.view(hg, P, Ls, Cc).permute(1, 0, 2, 3).contiguous()

    def _call_nccl(self, q, k, v, rope, out):
        """The staged form: per group, pack per peer, ``all_to_all``, place, attention, pack, ``all_to_all``, unpack."""
        dist, P, Ls, H, Cc = self.dist, self.world, self.Ls, self.H, ops.HEAD_DIM
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
                         out=oh.permute(1, 0, 2), logit_bound=bound, status_word=self.status.tensor())
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
