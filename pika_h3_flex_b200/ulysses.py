"""Ulysses sequence parallelism around the attention path: sequence shards -> head shards -> attention
-> sequence shards, one process per GPU, exchanges over NCCL (NVLink / NVSwitch).

The reference runs one request on one GPU ("Multi-GPU inference within one request is not implemented",
reference ``README.md:115``); this wrapper is what lets the same processor call run with the packed
sequence split across ranks.  Rank r holds tokens ``[r*L/P, (r+1)*L/P)`` of every head.  Normalisation,
rotation and (in FP8 mode) quantisation are token-local, so they run BEFORE the exchange and the wire
carries final operands in head-major layout ``[H, L/P, 128]``: the block that goes to rank p (its
``H/P`` heads) is contiguous, and each received ``[L/P, 128]`` block lands directly at its final place in
``[H/P, L, 128]``, so neither side needs a pack or unpack pass.

Two transports, same results.  On NCCL each exchange is ONE list-form ``all_to_all`` per tensor (grouped
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
    """

    def __init__(self, group=None, mode: int = _lib.MODE_DENSE_BF16, block_index: Optional[ops.BlockIndex] = None,
                 prep_fn: Optional[Callable] = None, attn_fn: Optional[Callable] = None,
                 to_head_major: Optional[Callable] = None, head_groups: int = 2):
        self.group = group
        self.head_groups = head_groups
        self.mode = mode
        self.block_index = block_index
        self.prep_fn = prep_fn
        self.attn_fn = attn_fn
        self.to_head_major = to_head_major or (lambda v: v.permute(1, 0, 2).contiguous())

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
                xp, xs = prep(x, which)
                x_hm = _pad_heads_hm(xp.permute(1, 0, 2).contiguous(), Hp)  # prepared tensors are views of head-major storage
            else:
                xs = None
                x_hm = _pad_heads_hm(self.to_head_major(x), Hp)
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
                ops.attn_fwd(qg, kg, vg, self.mode, sq, sk, self.block_index, out=oh, logit_bound=logit_bound)
            o_hm, r = head_to_seq(oh.permute(1, 0, 2).contiguous(), self.group, True, o_hm, sl, hp)
            outbound += r
        for r in outbound:
            r.wait()
        return o_hm[:H].permute(1, 0, 2)
