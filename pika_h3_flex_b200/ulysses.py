"""Ulysses sequence parallelism around the attention path: sequence shards -> head shards -> attention
-> sequence shards, one process per GPU, exchanges over NCCL (NVLink / NVSwitch).

The reference runs one request on one GPU ("Multi-GPU inference within one request is not implemented",
reference ``README.md:115``); this wrapper is what lets the same processor call run with the packed
sequence split across ranks.  Rank r holds tokens ``[r*L/P, (r+1)*L/P)`` of every head.  Normalisation,
rotation and (in FP8 mode) quantisation are token-local, so they run BEFORE the exchange and the wire
carries final operands in head-major layout ``[H, L/P, 128]``: the block that goes to rank p (its
``H/P`` heads) is contiguous, and each received ``[L/P, 128]`` block lands directly at its final place in
``[H/P, L, 128]``, so neither side needs a pack or unpack pass.

Transports, same results.  ``peer`` (the default on NCCL groups of more than one GPU): no exchange step at all. The
preparation kernels store each prepared row straight into the memory of the rank that owns the row's head
(``h3a_qk_prep_scatter``, plain stores over NVLink into buffers opened through CUDA's inter-process handles, see
``peer.py``), the attention kernel stores each output row straight into the memory of the rank that owns the row's
token (``h3a_attn_params.o_rank_base``), and the ranks meet twice per call (before the owners read, after the
outputs have landed).  Peer memory is a store target only; every load and every tensor map covers local memory.
``nccl``: on NCCL each exchange is ONE list-form ``all_to_all`` per tensor (grouped
ncclSend/ncclRecv inside the library): the block for a peer is contiguous on the sending side, arrives as one
contiguous ``[heads, L/P, 128]`` block per peer, and a single strided copy puts the blocks at their final place
(the return trip packs instead).  That costs one extra pass over the exchanged tensor (well under 2 % of the
step) and replaces hundreds of per-(peer, head) point-to-point operations per step, whose host-side issue time
(about 10 us each) had become the largest overhead at 8 GPUs.  Other backends (gloo in the CPU tests) use batched
point-to-point operations whose blocks land directly at their final place.  Peers' data always lands in local
memory through the collective before a kernel reads it.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _lib, ops
from .peer import PeerUnavailable


def padded_heads(n_heads: int, world: int) -> int:
    """Heads padded up to a multiple of the world size."""
    return (n_heads + world - 1) // world * world


def _exchange(send_blocks: List[Optional[torch.Tensor]], recv_blocks: List[Optional[torch.Tensor]], group, async_op: bool):
    """Send ``send_blocks[p]`` to rank p and receive ``recv_blocks[p]`` from rank p (lists of lists of
    contiguous tensors); the local block is copied.  Returns the list of outstanding requests."""
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    ops_list = []
    for off in range(1, world):
        dst = (rank + off) % world
        src = (rank - off) % world
        for t in send_blocks[dst]:
            ops_list.append(dist.P2POp(dist.isend, t, dist.get_global_rank(group, dst) if group is not None else dst, group))
        for t in recv_blocks[src]:
            ops_list.append(dist.P2POp(dist.irecv, t, dist.get_global_rank(group, src) if group is not None else src, group))
    for s, r in zip(send_blocks[rank], recv_blocks[rank]):
        r.copy_(s)
    reqs = dist.batch_isend_irecv(ops_list) if ops_list else []
    if not async_op:
        for r in reqs:
            r.wait()
        return []
    return reqs


class _Pending:
    """Outstanding requests of one exchange plus the work left to do once they have completed."""

    def __init__(self, reqs, after: Optional[Callable] = None):
        self.reqs = list(reqs)
        self.after = after

    def wait(self):
        for r in self.reqs:
            r.wait()
        self.reqs = []
        if self.after is not None:
            self.after()
            self.after = None


def _use_all_to_all(x: torch.Tensor, group) -> bool:
    return x.is_cuda and dist.get_backend(group) == "nccl"


def _contiguous_range(slots) -> Optional[range]:
    slots = list(slots)
    if slots and slots == list(range(slots[0], slots[-1] + 1)):
        return range(slots[0], slots[-1] + 1)
    return None


def seq_to_head(x_hm: torch.Tensor, group=None, async_op: bool = False, out: Optional[torch.Tensor] = None,
                slots: Optional[Sequence[int]] = None):
    """``x_hm [Hp, Ls, C]`` head-major local shard (all padded heads, local tokens) ->
    ``[Hp/P, P*Ls, C]`` (local heads, every token).  ``slots`` restricts the exchange to some of the ``Hp/P``
    local head slots (the rest of ``out`` is left alone).  Returns ``(out, requests)``."""
    world = dist.get_world_size(group)
    Hp, Ls, Cc = x_hm.shape
    if Hp % world:
        raise ValueError(f"heads {Hp} not a multiple of world size {world}; pad first")
    hp = Hp // world
    if out is None:
        out = torch.empty(hp, world * Ls, Cc, dtype=x_hm.dtype, device=x_hm.device)
    slots = range(hp) if slots is None else slots
    rng = _contiguous_range(slots)
    if rng is not None and _use_all_to_all(x_hm, group):
        j0, j1, n = rng.start, rng.stop, len(rng)
        staged = torch.empty(world, n, Ls, Cc, dtype=x_hm.dtype, device=x_hm.device)
        work = dist.all_to_all([staged[p] for p in range(world)], [x_hm[p * hp + j0 : p * hp + j1] for p in range(world)],
                               group=group, async_op=True)

        def place():  # [peer, head, token] -> [head, peer * Ls + token]
            out[j0:j1].view(n, world, Ls, Cc).copy_(staged.permute(1, 0, 2, 3))

        pend = _Pending([work], place)
        if not async_op:
            pend.wait()
            return out, []
        return out, [pend]
    send = [[x_hm[p * hp + j] for j in slots] for p in range(world)]
    recv = [[out[j, p * Ls : (p + 1) * Ls] for j in slots] for p in range(world)]
    return out, _exchange(send, recv, group, async_op)


def head_to_seq(o_hm: torch.Tensor, group=None, async_op: bool = False, out: Optional[torch.Tensor] = None,
                slots: Optional[Sequence[int]] = None, hp: Optional[int] = None):
    """Inverse of :func:`seq_to_head`: ``o_hm [n, P*Ls, C]`` (the local head slots ``slots``, ``n = len(slots)``,
    of ``hp`` in total) -> rows ``p*hp + slot`` of ``out [hp*P, Ls, C]``."""
    world = dist.get_world_size(group)
    n, L, Cc = o_hm.shape
    if L % world:
        raise ValueError("sequence length not a multiple of world size")
    Ls = L // world
    hp = n if hp is None else hp
    slots = list(range(n)) if slots is None else list(slots)
    if len(slots) != n:
        raise ValueError("o_hm must hold exactly the listed head slots")
    if out is None:
        out = torch.empty(hp * world, Ls, Cc, dtype=o_hm.dtype, device=o_hm.device)
    rng = _contiguous_range(slots)
    if rng is not None and _use_all_to_all(o_hm, group):
        j0, j1 = rng.start, rng.stop
        packed = o_hm.view(n, world, Ls, Cc).permute(1, 0, 2, 3).contiguous()  # [peer, head, token]
        work = dist.all_to_all([out[p * hp + j0 : p * hp + j1] for p in range(world)], [packed[p] for p in range(world)],
                               group=group, async_op=True)
        pend = _Pending([work])
        if not async_op:
            pend.wait()
            return out, []
        return out, [pend]
    send = [[o_hm[i, p * Ls : (p + 1) * Ls] for i in range(n)] for p in range(world)]
    recv = [[out[p * hp + j] for j in slots] for p in range(world)]
    return out, _exchange(send, recv, group, async_op)


def scales_seq_to_head(s: torch.Tensor, group=None, async_op: bool = False):
    """FP8 block scales ``[Hp, nb_local]`` -> ``[Hp/P, P*nb_local]`` (needs Ls % 128 == 0 so that blocks do
    not straddle ranks).  With ``async_op`` returns ``(fetch, requests)``: call ``fetch()`` after waiting."""
    out, reqs = seq_to_head(s[:, :, None].contiguous(), group, async_op)
    fetch = lambda: out[:, :, 0].contiguous()
    return (fetch, reqs) if async_op else fetch()


def _pad_heads_hm(x_hm: torch.Tensor, Hp: int) -> torch.Tensor:
    if x_hm.shape[0] == Hp:
        return x_hm
    pad = x_hm.new_zeros(Hp - x_hm.shape[0], *x_hm.shape[1:])
    return torch.cat([x_hm, pad], dim=0)


class UlyssesAttention:
    """Sequence-parallel joint attention.  ``__call__(q, k, v, rope)`` takes this rank's ``[L/P, H, 128]``
    bf16 projections and rotary table rows and returns this rank's ``[L/P, H, 128]`` output.  ``run`` takes the
    three projections as callables instead and starts each tensor's exchange as soon as that tensor exists, so the
    exchange of Q runs under the K projection and the exchange of K under the V projection.

    ``prep_fn(q, k, q_rope, k_rope, fp8) -> (q', k', q_scale, k_scale)`` (either of q, k may be None) and
    ``attn_fn(q, k, v, mode, q_scale, k_scale, block_index)`` default to the CUDA library; the CPU tests
    inject host stand-ins to exercise the reshard logic with gloo ranks.  ``head_groups``: 1 = one attention
    launch, 2 = up to two groups chosen by the wave model (default), or an explicit list of group sizes.

    Every rank must bring the same shard shape.  That is checked on the host, once per shape, by one small
    ``all_gather_object`` on the group before the first exchange of that shape: a mismatch raises ``ValueError`` on
    every rank instead of leaving the ranks blocked in an exchange whose sizes disagree.  Exchanges themselves have
    no deadline of their own: create the process group with a finite ``timeout`` (``init_process_group(...,
    timeout=...)``) so that a rank that never arrives ends the collective with an error.  ``status`` is the
    ``ops.StatusWord`` handed to the attention launches (bounded device-side waits); ``check_status()`` reads it.
    """

    def __init__(self, group=None, mode: int = _lib.MODE_DENSE_BF16, block_index: Optional[ops.BlockIndex] = None,
                 prep_fn: Optional[Callable] = None, attn_fn: Optional[Callable] = None,
                 to_head_major: Optional[Callable] = None, head_groups: int = 2, status: Optional[ops.StatusWord] = None,
                 transport: str = "auto"):
        if transport not in ("auto", "peer", "nccl"):
            raise ValueError("transport must be auto, peer or nccl")
        self._transport_arg = transport
        self.peer_unavailable = None  # why the automatic choice fell back from the peer transport, if it did
        self.transport = None  # resolved at the first call: "peer" or "nccl" (which also names the gloo path of the CPU tests)
        self._peer = {}
        self.group = group
        self.status = status if status is not None else ops.StatusWord()
        self._validated = set()
        # set to a list to have every call append {"prep": [(start, end) CUDA events ...], "attention": [...]}:
        # the token-local preparation passes and the attention launches of that call on this rank's stream
        self.timeline = None
        self.head_groups = head_groups
        self.mode = mode
        self.block_index = block_index
        self.prep_fn = prep_fn
        self.attn_fn = attn_fn
        self.to_head_major = to_head_major or (lambda v: v.permute(1, 0, 2).contiguous())

    def check_status(self) -> None:
        self.status.check("UlyssesAttention")

    def close(self) -> None:
        """Release the buffers shared with the other ranks (every rank must call it; needed before the process group
        is destroyed when the peer transport was used)."""
        for st in self._peer.values():
            st.arena.close()
        self._peer = {}

    def _resolve_transport(self, like: torch.Tensor) -> str:
        if self.transport is None:
            t = self._transport_arg
            if t == "auto":
                own = self.prep_fn is None and self.attn_fn is None
                t = "peer" if (own and like.is_cuda and dist.get_backend(self.group) == "nccl" and dist.get_world_size(self.group) > 1) else "nccl"
            if t == "peer" and (self.prep_fn is not None or self.attn_fn is not None or not like.is_cuda):
                raise ValueError("the peer transport runs the library's own kernels on CUDA tensors")
            self.transport = t
        return self.transport

    def launches_per_step(self, Ls: int, H: int) -> int:
        """Kernels of this library one call launches on this rank (for the benchmark's launch count)."""
        fp8 = self.mode == _lib.MODE_FP8_QK
        n = 3 + 1  # Q, K (and, on the peer transport, V) preparation / re-layout + attention
        if self.transport != "peer":
            n -= 1  # V's head-major copy is a torch kernel there
        if self.block_index is not None:
            n += 1
        if fp8 and self.transport == "peer":
            n += 2
        return n

    class _PeerState:
        pass

    def peer_ready(self, Ls: int, H: int, like: torch.Tensor) -> bool:
        """True when calls of this shard shape go over the peer transport: resolves the transport and, the first time,
        builds the shared buffers (a collective step).  When the ranks cannot share memory every rank learns so here:
        an explicit ``transport="peer"`` raises ``PeerUnavailable``, the automatic choice falls back to ``nccl``."""
        if self._resolve_transport(like) != "peer":
            return False
        try:
            self._peer_state(Ls, H, like.device)
        except PeerUnavailable as exc:
            if self._transport_arg == "peer":
                raise
            self.transport = "nccl"
            self.peer_unavailable = str(exc)
            return False
        return True

    def _peer_state(self, Ls: int, H: int, device) -> "_PeerState":
        """Buffers of one shard shape, shared with the other ranks: this rank's heads of Q, K, V over ALL tokens
        (written by every rank's preparation kernels) and this rank's tokens of the output for all heads (written by
        every rank's attention kernel)."""
        from .peer import Carver, PeerArena

        key = (Ls, H)
        st = self._peer.get(key)
        if st is None:
            world = dist.get_world_size(self.group)
            rank = dist.get_rank(self.group)
            st = self._PeerState()
            st.hp = padded_heads(H, world) // world
            st.L = world * Ls
            st.n_local = max(0, min(st.hp, H - rank * st.hp))
            c = Carver()
            nb = st.hp * st.L * ops.HEAD_DIM * 2
            st.off = {n: c.take(nb) for n in ("q", "k", "v")}
            st.off["o"] = c.take(Ls * H * ops.HEAD_DIM * 2)
            st.arena = PeerArena(c.size, self.group, device)  # raises PeerUnavailable on EVERY rank when any rank cannot share
            for n in ("q", "k", "v"):
                setattr(st, n, st.arena.tensor(st.off[n], (st.hp, st.L, ops.HEAD_DIM), torch.bfloat16))
            st.o = st.arena.tensor(st.off["o"], (Ls, H, ops.HEAD_DIM), torch.bfloat16)
            # every rank starts with the heads of the rank after it and ends with its own: at any moment the ranks
            # store to different owners instead of all to the same one
            start = ((rank + 1) % world) * st.hp % H
            st.owners = {n: ops.HeadOwners([st.arena.addr(p, st.off[n]) for p in range(world)], st.hp, False, rank * Ls, st.L,
                                           start_head=start)
                         for n in ("q", "k", "v")}
            # output rows of this rank's heads (global heads rank * hp ...) go to the rank that holds the token
            st.out_ranks = ops.RankOutputs([st.arena.addr(t, st.off["o"]) + rank * st.hp * ops.HEAD_DIM * 2 for t in range(world)],
                                           Ls, H * ops.HEAD_DIM, ops.HEAD_DIM)
            self._peer[key] = st
        return st

    def _run_peer(self, q, k_fn, v_fn, rope, q_weight, k_weight, eps, rope_half, logit_bound, prepared, marks):
        """One call on the peer transport (see the module docstring).  The result is a view of this rank's output
        buffer, which the next call of the same shape overwrites."""
        Ls, H, _ = q.shape

        def producer(name, x_fn):
            def scatter(owners):
                x = x_fn()
                if tuple(x.shape) != (Ls, H, ops.HEAD_DIM):
                    raise ValueError("q, k, v must be [L/P, H, 128] shards of the same shape")
                if name == "v" or prepared:
                    ops.prep_scatter(x, owners, no_norm=True)
                else:
                    ops.prep_scatter(x, owners, rope, q_weight if name == "q" else k_weight, eps, rope_half)
            return scatter

        return self.run_scattered(Ls, H, q.device, producer("q", lambda: q), producer("k", k_fn), producer("v", v_fn),
                                  logit_bound, marks)

    def run_scattered(self, Ls: int, H: int, device, q_to: Callable, k_to: Callable, v_to: Callable, logit_bound: float,
                      marks=None) -> torch.Tensor:
        """The peer transport with the caller's own producers: ``q_to(owners)``, ``k_to(owners)``, ``v_to(owners)`` are
        called in that order and must store this rank's ``Ls`` tokens of all ``H`` heads, prepared (normalised and
        rotated; V as it is), at the heads' owners described by ``owners`` (an ``ops.HeadOwners``): for example
        ``ops.proj_fwd(..., out_to=owners)``, whose epilogue then IS the outbound trip of the reshard and overlaps it
        with the projection's own math.  Returns this rank's ``[Ls, H, 128]`` output (a view of a buffer that the next
        call of the same shape overwrites)."""
        fp8 = self.mode == _lib.MODE_FP8_QK
        self._validate(Ls, H)
        if not self.peer_ready(Ls, H, torch.empty(0, device=device)):
            raise ValueError("run_scattered needs the peer transport (see peer_ready)")
        st = self._peer_state(Ls, H, device)
        own_marks = marks is None and self.timeline is not None
        if own_marks:
            marks = {"prep": [], "attention": []}

        def timed(kind, fn):
            if marks is None:
                return fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn()
            e1.record()
            marks[kind].append((e0, e1))
            return r

        for name, fn in (("q", q_to), ("k", k_to), ("v", v_to)):
            timed("prep", lambda: fn(st.owners[name]))
        st.arena.barrier()  # every rank's rows have landed before an owner reads
        if st.n_local > 0:
            n = st.n_local
            qg, kg, vg = (getattr(st, name)[:n].permute(1, 0, 2) for name in ("q", "k", "v"))
            qs = ks = None
            if fp8:  # block scales need whole 128-token blocks of the FULL sequence: quantise here, at the owner
                qg, kg, qs, ks = timed("prep", lambda: ops.qk_prep(qg, kg, fp8=True, no_norm=True))
            timed("attention", lambda: ops.attn_fwd(qg, kg, vg, self.mode, qs, ks, self.block_index, out_ranks=st.out_ranks,
                                                    logit_bound=logit_bound, status_word=self.status.tensor(st.o)))
        st.arena.barrier()  # every rank's output rows have landed
        if own_marks:
            self.timeline.append(marks)
        return st.o

    def _validate(self, Ls: int, H: int) -> None:
        """All ranks must hold shards of one shape, and the block index must describe the whole sequence."""
        world = dist.get_world_size(self.group)
        if self.block_index is not None:
            nt = (world * Ls + ops.TILE - 1) // ops.TILE
            if self.block_index.n_q_tiles != nt or self.block_index.n_k_tiles != nt:
                raise ValueError(f"block index is {self.block_index.n_q_tiles} x {self.block_index.n_k_tiles} tiles, "
                                 f"the sequence of {world} x {Ls} tokens has {nt}")
        key = (Ls, H)
        if key in self._validated:
            return
        shapes = [None] * world
        dist.all_gather_object(shapes, key, group=self.group)
        if any(tuple(x) != key for x in shapes):
            raise ValueError(f"ranks disagree on the shard shape (tokens per rank, heads): {shapes}")
        self._validated.add(key)

    @staticmethod
    def _waves(n_heads: int, L: int, sms: int) -> float:
        """Estimated duration of one dense attention launch over ``n_heads`` heads, in units of one CTA pair's full
        walk over the keys: whole waves of pairs (one pair per two SMs) plus the last, partly filled wave, which the
        library shortens by splitting the key range (same model as the library's own choice of the split)."""
        wave = max(1, sms // 2)
        total = (L + 511) // 512 * n_heads
        n_kv = (L + 127) // 128
        full, rest = divmod(total, wave)
        if rest == 0:
            return float(full)
        eps = 4.5 / n_kv
        tail = 1.0 + eps
        s = 2
        while s <= 16 and s * 4 <= n_kv and rest * s <= 4 * wave:
            tail = min(tail, -(-rest * s // wave) * (1.0 / s + eps))
            s += 1
        return full + tail

    def _head_slot_groups(self, hp: int, L: int, like: torch.Tensor):
        """Split the ``hp`` local head slots into at most two groups, so that one group's exchanges overlap the
        other's attention.  On a GPU the cut is placed where the two attention launches together are estimated to
        take no longer (within 2 %) than a single launch would; if no cut achieves that, one group is used."""
        if not isinstance(self.head_groups, int):  # explicit group sizes
            sizes = list(self.head_groups)
            if sum(sizes) != hp or min(sizes) < 1:
                raise ValueError(f"head_groups {sizes} must be positive and sum to the {hp} local head slots")
            cuts = [sum(sizes[:i]) for i in range(len(sizes) + 1)]
            return [range(a, b) for a, b in zip(cuts[:-1], cuts[1:])]
        if self.head_groups < 2 or hp < 2:
            return [range(hp)]
        if like.is_cuda and hp < 8:
            return [range(hp)]  # measured at 5 heads per rank (8 GPUs): a second launch costs more than the overlap gains
        if not like.is_cuda:
            return [range(0, hp // 2), range(hp // 2, hp)]
        sms = torch.cuda.get_device_properties(like.device).multi_processor_count
        cost = lambda c: self._waves(c, L, sms) + self._waves(hp - c, L, sms)
        best = min(range(1, hp), key=lambda c: (round(cost(c), 3), abs(c - hp // 2)))
        if cost(best) > 1.02 * self._waves(hp, L, sms):
            return [range(hp)]
        return [range(0, best), range(best, hp)]

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rope: Optional[torch.Tensor], **kw) -> torch.Tensor:
        return self.run(lambda: q, lambda: k, lambda: v, rope, **kw)

    def run(self, q_fn: Callable, k_fn: Callable, v_fn: Callable, rope: Optional[torch.Tensor],
            q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
            rope_half: bool = False, logit_bound: Optional[float] = None, prepared: bool = False) -> torch.Tensor:
        """``q_fn() / k_fn() / v_fn()`` return this rank's ``[L/P, H, 128]`` bf16 projections; they are called in
        that order, each after the previous tensor's exchange has been started.  ``prepared``: Q and K arrive
        normalised and rotated already (the fused projection does that in its epilogue); in FP8-QK mode the two
        callables return ``(e4m3 bytes, block scales)``."""
        world = dist.get_world_size(self.group)
        fp8 = self.mode == _lib.MODE_FP8_QK
        marks = {"prep": [], "attention": []} if self.timeline is not None else None

        def timed(kind, fn):
            if marks is None:
                return fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn()
            e1.record()
            marks[kind].append((e0, e1))
            return r

        def prep(x, which):  # token-local work first: the wire then carries final operands
            if prepared:  # FP8-QK: the callable returned (e4m3 bytes, block scales)
                xp, xs = x if isinstance(x, tuple) else (x, None)
                if fp8 and xs is None:
                    raise ValueError("prepared FP8-QK operands come with their block scales")
                return xp, xs
            a, b = (x, None) if which == 0 else (None, x)
            ra, rb = (rope, None) if which == 0 else (None, rope)
            if self.prep_fn is not None:
                r = self.prep_fn(a, b, ra, rb, fp8)
            else:
                r = ops.qk_prep(a, b, ra, rb, q_weight, k_weight, eps, fp8, rope_half)
            return (r[0], r[2]) if which == 0 else (r[1], r[3])

        q = q_fn()
        Ls, H, _ = (q[0] if isinstance(q, tuple) else q).shape
        self._validate(Ls, H)
        # prepared e4m3 operands carry per-shard scales: they are exchanged below, whatever the transport
        if not (prepared and fp8) and self.peer_ready(Ls, H, q[0] if isinstance(q, tuple) else q):
            if logit_bound is None:
                logit_bound = ops.normed_logit_bound(q_weight, k_weight, 0.0, fp8)
            out = self._run_peer(q, k_fn, v_fn, rope, q_weight, k_weight, eps, rope_half, logit_bound, prepared, marks)
            if marks is not None:
                self.timeline.append(marks)
            return out
        if fp8 and Ls % ops.TILE:
            raise ValueError("FP8 mode under Ulysses needs the local sequence length to be a multiple of 128")
        Hp = padded_heads(H, world)
        hp = Hp // world
        # The local head slots are handled in groups: while one group is in attention the next group's operands
        # are arriving and the previous group's output is leaving.
        groups = self._head_slot_groups(hp, world * Ls, q[0] if isinstance(q, tuple) else q)
        inbound = [[] for _ in groups]
        scale_fetch = [None, None]
        heads = [None, None, None]
        for which, fn in enumerate((None, k_fn, v_fn)):
            x = q if which == 0 else fn()
            if tuple((x[0] if isinstance(x, tuple) else x).shape) != (Ls, H, ops.HEAD_DIM):
                raise ValueError("q, k, v must be [L/P, H, 128] shards of the same shape")
            if which < 2:
                xp, xs = timed("prep", lambda: prep(x, which))
                x_hm = _pad_heads_hm(xp.permute(1, 0, 2).contiguous(), Hp)  # prepared tensors are views of head-major storage
            else:
                xs = None
                x_hm = _pad_heads_hm(timed("prep", lambda: self.to_head_major(x)), Hp)
            for gi, sl in enumerate(groups):
                heads[which], r = seq_to_head(x_hm, self.group, True, heads[which], sl)
                inbound[gi] += r
            if fp8 and which < 2:
                scale_fetch[which], r = scales_seq_to_head(_pad_heads_hm(xs, Hp), self.group, True)
                inbound[0] += r
        qh, kh, vh = heads
        qsh = ksh = None
        if logit_bound is None and self.attn_fn is None:
            logit_bound = ops.normed_logit_bound(q_weight, k_weight, 0.0, fp8)
        o_hm = None
        outbound = []
        for gi, (sl, reqs) in enumerate(zip(groups, inbound)):
            for r in reqs:
                r.wait()
            if fp8 and gi == 0:
                qsh, ksh = scale_fetch[0](), scale_fetch[1]()
            j0, j1 = sl.start, sl.stop
            qg, kg, vg = (t[j0:j1].permute(1, 0, 2) for t in (qh, kh, vh))
            sq = None if qsh is None else qsh[j0:j1].contiguous()
            sk = None if ksh is None else ksh[j0:j1].contiguous()
            if self.attn_fn is not None:
                oh = self.attn_fn(qg, kg, vg, self.mode, sq, sk, self.block_index)
            else:
                # head-major output so that the return exchange sends contiguous blocks without a copy
                oh = torch.empty(j1 - j0, qg.shape[0], ops.HEAD_DIM, dtype=torch.bfloat16, device=qg.device).permute(1, 0, 2)
                timed("attention", lambda: ops.attn_fwd(qg, kg, vg, self.mode, sq, sk, self.block_index, out=oh, logit_bound=logit_bound,
                                                        status_word=self.status.tensor(qg)))
            o_hm, r = head_to_seq(oh.permute(1, 0, 2).contiguous(), self.group, True, o_hm, sl, hp)
            outbound += r
        for r in outbound:
            r.wait()
        if marks is not None:
            self.timeline.append(marks)
        return o_hm[:H].permute(1, 0, 2)
