"""Attention processor with the call shape of a diffusers attention processor.

The reference project drives its DiT through ``self.model(**model_inputs)``
(``src/pika_h3/core/wrapper.py:248``); inside each transformer block the attention module owns the
projections ``to_q``, ``to_k``, ``to_v`` and ``to_out[0]`` (names fixed by ``DEFAULT_LORA_TARGETS`` in
``src/pika_h3/core/loader.py:9``; they are PEFT LoRA-wrapped Linears after ``apply_lora``,
``src/pika_h3/core/loader.py:20-49``) and delegates the arithmetic between them to a *processor*
object.  ``B200AttnProcessor`` is that object: the projections stay PyTorch modules (LoRA intact),
everything between them runs in ``libh3attn.so``.

The model file that defines the stock processor lives in the un-vendored ``diffusers`` build pinned
at ``pyproject.toml:12``, so the keyword names below follow the public diffusers convention
(``attn, hidden_states, encoder_hidden_states, attention_mask, image_rotary_emb``); unknown keywords
are accepted and the ones that can carry rotary information (``position_ids``, ``rotary_emb``) are
used.  The reference packs one document per forward (``src/pika_h3/core/wrapper.py:231-232``), so the
batch dimension must be 1.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import torch

from . import _lib, ops

MODES = {"dense_bf16": _lib.MODE_DENSE_BF16, "fp8_qk": _lib.MODE_FP8_QK, "block_sparse": _lib.MODE_BLOCK_SPARSE}


class RopeCache:
    """(cos, sin) tables per position grid, like the reference's per-geometry layout cache
    (``src/pika_h3/core/wrapper.py:71-78``).  The reference re-creates the device copy of its layout on every
    forward (``layout.to(device)``, ``src/pika_h3/core/wrapper.py:164-166``), so a grid is recognised by its
    CONTENT: the cache keeps its own device copy of each grid it has built a table for (``size`` of them, a
    few hundred KB each) and compares a new tensor with them (one device-side comparison, i.e. one
    synchronisation per forward).  All blocks of one forward pass the same tensor object; that is recognised
    by identity first, through a weak reference, so the comparison runs once per forward and no caller tensor
    is kept alive."""

    def __init__(self, size: int = 2):
        self.size = size
        self._tables: "OrderedDict[int, tuple]" = OrderedDict()  # serial -> (own copy of the grid, split, theta, table)
        self._seen: "OrderedDict[tuple, tuple]" = OrderedDict()   # identity of a caller tensor -> (weakref, serial)
        self._serial = 0
        self.hits = self.content_hits = self.misses = 0

    def __len__(self) -> int:
        return len(self._tables)

    def get(self, pos: torch.Tensor, split, theta) -> torch.Tensor:
        split, theta = tuple(split), float(theta)
        ident = (id(pos), pos.data_ptr(), pos._version, tuple(pos.shape), pos.dtype, str(pos.device), split, theta)
        seen = self._seen.get(ident)
        if seen is not None and seen[0]() is pos and seen[1] in self._tables:
            self._tables.move_to_end(seen[1])
            self.hits += 1
            return self._tables[seen[1]][3]
        dev = _cuda_device(pos)
        p32 = pos.to(device=dev, dtype=torch.float32)
        serial = None
        for sn, (own, sp, th, _) in self._tables.items():
            if sp == split and th == theta and own.shape == p32.shape and own.device == p32.device and torch.equal(own, p32):
                serial = sn
                self.content_hits += 1
                break
        if serial is None:
            self.misses += 1
            tab = ops.rope_table(p32, split, theta)
            if len(self._tables) >= self.size:
                self._tables.popitem(last=False)
            self._serial += 1
            serial = self._serial
            own = p32 if p32.data_ptr() != pos.data_ptr() else p32.clone()
            self._tables[serial] = (own, split, theta, tab)
        self._tables.move_to_end(serial)
        import weakref

        while len(self._seen) >= 8:
            self._seen.popitem(last=False)
        self._seen[ident] = (weakref.ref(pos), serial)
        return self._tables[serial][3]


def _cuda_device(t: torch.Tensor):
    return t.device if t.is_cuda else torch.device("cuda", torch.cuda.current_device())


def _norm_params(mod, name: str = "norm"):
    """``(weight, eps)`` of a per-head RMSNorm module, or ``(None, None)`` for no module.  The library normalises
    each head's 128 values by their own root mean square and multiplies by ONE weight vector of 128 entries shared
    by all heads; anything that computes something else (a norm across all heads with a ``[heads * 128]`` weight, a
    LayerNorm with a bias or with mean subtraction) is refused here instead of being silently replaced."""
    if mod is None:
        return None, None
    if isinstance(mod, torch.nn.LayerNorm):
        raise NotImplementedError(f"{name} is a LayerNorm (mean subtraction); the library's Q/K preparation is a per-head RMSNorm")
    if getattr(mod, "bias", None) is not None:
        raise NotImplementedError(f"{name} has a bias; the library's Q/K preparation is a bias-free per-head RMSNorm")
    w = getattr(mod, "weight", None)
    if w is not None and w.numel() != ops.HEAD_DIM:
        raise NotImplementedError(
            f"{name}.weight has {w.numel()} entries: only a per-head RMSNorm over the 128 head dims (one [128] weight shared "
            "by all heads) is implemented, not a norm across heads")
    eps = getattr(mod, "eps", None)
    if eps is None:
        eps = getattr(mod, "variance_epsilon", None)
    return w, eps


def _linear_parts(mod):
    """``(weight, bias, lora_a, lora_b, scale)`` of a plain ``nn.Linear`` or of a LoRA-wrapped one, or None when
    the module is not one this function can take apart (the processor then simply calls the module).  Recognised
    wrappers: PEFT's ``lora.Linear`` (``base_layer`` + ``lora_A`` / ``lora_B`` ModuleDicts + ``scaling``, one
    active adapter, not merged, no dropout in effect) as the reference's ``apply_lora`` builds them
    (src/pika_h3/core/loader.py:20-49), and a bare ``base`` + ``A`` + ``B`` triple of Linears."""
    nn = torch.nn
    if isinstance(mod, nn.Linear):
        return mod.weight, mod.bias, None, None, 1.0
    base = getattr(mod, "base_layer", None)
    if isinstance(base, nn.Linear) and hasattr(mod, "lora_A") and hasattr(mod, "lora_B"):
        if getattr(mod, "merged", False):
            return base.weight, base.bias, None, None, 1.0
        if getattr(mod, "disable_adapters", False):
            return base.weight, base.bias, None, None, 1.0
        names = list(getattr(mod, "active_adapters", None) or mod.lora_A.keys())
        names = [n for n in names if n in mod.lora_A]
        if len(names) != 1:
            return None
        n = names[0]
        drop = getattr(mod, "lora_dropout", {})
        d = drop[n] if n in drop else None
        if d is not None and not isinstance(d, nn.Identity) and (mod.training and getattr(d, "p", 0.0) > 0):
            return None
        a, b = mod.lora_A[n], mod.lora_B[n]
        if not isinstance(a, nn.Linear) or not isinstance(b, nn.Linear) or a.bias is not None or b.bias is not None:
            return None
        return base.weight, base.bias, a.weight, b.weight, float(mod.scaling[n])
    base = getattr(mod, "base", None)
    a, b = getattr(mod, "A", None), getattr(mod, "B", None)
    if isinstance(base, nn.Linear) and isinstance(a, nn.Linear) and isinstance(b, nn.Linear) and a.bias is None and b.bias is None:
        return base.weight, base.bias, a.weight, b.weight, float(getattr(mod, "scale", 1.0))
    return None


class B200AttnProcessor:
    """Drop-in processor: ``processor(attn, hidden_states, encoder_hidden_states=None, ...)``.

    mode          ``dense_bf16`` | ``fp8_qk`` | ``block_sparse``
    block_index   ``ops.BlockIndex`` on the device (``block_sparse`` only; self-attention only)
    rope_half     rotary pairs ``(j, j+64)`` instead of ``(2j, 2j+1)``
    qk_norm       what to do with a module that has NO ``norm_q`` / ``norm_k``: ``True`` applies the per-head RMSNorm
                  with unit weights all the same (BASELINE's configs), ``None`` (default) refuses such a module, so
                  that a norm-free model is never normalised by accident.  Modules WITH ``norm_q`` / ``norm_k`` must
                  carry a per-head RMSNorm (one ``[128]`` weight, no bias); anything else raises.
    softmax       ``"auto"`` (default): the logit bound that follows from the QK-RMSNorm weights selects the fixed softmax
                  reference whenever it is at most 110 (every row served up to 64, beyond that rows whose keys are ALL
                  strongly anti-aligned with the query are reported through the status word), else the online softmax;
                  ``"online"``: always the online softmax with a running row maximum (no bound used).
    status        ``ops.StatusWord`` shared by every launch of this processor (default: its own).  A kernel whose
                  bounded wait runs out, or that finds a malformed block index, records it there and every later
                  launch does nothing; :meth:`check_status` (one synchronisation: call it once per forward or per
                  sampler step) raises ``H3AError`` then.  ``check_every_call=True`` does that after each call.
    group         a ``torch.distributed`` process group (NCCL, one process per GPU): Ulysses sequence parallelism.
                  ``hidden_states`` is then this rank's shard ``[1, S/P, D]`` of the packed sequence (rank r holds
                  tokens ``[r*S/P, (r+1)*S/P)``; rotary inputs are the rows of the same shard) and so is the result.
                  The projections stay token-local; the exchange of Q runs under the K projection and that of K
                  under the V projection.  Cross-attention needs no exchange (keys and values are replicated).
    fused_projection  run to_q / to_k / to_v (and to_out.0) through the library's own GEMM with the norm + rotation
                  (+ e4m3 quantisation in FP8-QK mode) in its epilogue: plain or LoRA-wrapped Linears that
                  ``_linear_parts`` recognises, bf16 weights and activations.  Anything else goes through the module
                  call and the separate preparation kernel.
    merge_lora    (with ``fused_projection``) fold a LoRA update into a copy of the base weight once per module,
                  ``W' = bf16(W + (alpha / r) B A)``, so that a projection is ONE launch with no LoRA term left (the
                  default keeps the update apart, as the reference's un-merged PEFT wrappers do: ``x A^T`` as a thin
                  matmul in front, 128 more columns of the contraction inside the GEMM).  The merged weight is rounded
                  to bf16, so results differ from the un-merged form by that rounding; it costs one more copy of each
                  wrapped weight in device memory.  Weights are taken as static (inference): re-create the processor,
                  or call :meth:`forget_merged`, after changing them.
    """

    def __init__(self, mode: str = "dense_bf16", block_index: Optional[ops.BlockIndex] = None, rope_half: bool = False,
                 rope_split=ops.ROPE_SPLIT, rope_theta: float = 10000.0, qk_norm: Optional[bool] = None, eps: float = 1e-6,
                 group=None, sequence_parallel: bool = False, fused_projection: bool = False,
                 status: Optional[ops.StatusWord] = None, check_every_call: bool = False, softmax: str = "auto",
                 merge_lora: bool = False):
        if mode not in MODES:
            raise ValueError(f"mode must be one of {sorted(MODES)}")
        if mode == "block_sparse" and block_index is None:
            raise ValueError("block_sparse needs a block index")
        _lib.load()  # fail here, loudly, when the CUDA library is missing
        self.mode = mode
        self.block_index = block_index
        self.rope_half = rope_half
        self.rope_split = tuple(rope_split)
        self.rope_theta = rope_theta
        self.qk_norm = qk_norm
        self.eps = eps
        self._rope_cache = RopeCache()
        self._bounds = {}
        self.fused_projection = fused_projection
        self.merge_lora = merge_lora
        self._scaled_b = {}
        self._merged_w = {}
        if softmax not in ("auto", "online"):
            raise ValueError("softmax must be auto or online")
        self.softmax = softmax
        self.status = status if status is not None else ops.StatusWord()
        self.check_every_call = check_every_call
        self._ulysses = None
        if group is not None or sequence_parallel:  # sequence_parallel=True with group=None: the default group
            from .ulysses import UlyssesAttention

            self._ulysses = UlyssesAttention(group, MODES[mode], block_index, status=self.status)

    def close(self) -> None:
        """Release what the sequence-parallel mode shares with the other ranks (call on every rank before the process
        group is destroyed); nothing to do on one GPU."""
        if self._ulysses is not None:
            self._ulysses.close()

    def check_status(self) -> None:
        """Synchronise and raise ``H3AError`` if any launch of this processor gave up a bounded wait (``H3A_ERR_TIMEOUT``)
        or found a malformed block index (``H3A_ERR_INDEX``) since the status word was last zeroed."""
        self.status.check("B200AttnProcessor")

    # ---- rotary information from whatever the caller passes
    def _rope(self, S: int, image_rotary_emb, kwargs) -> Optional[torch.Tensor]:
        emb = image_rotary_emb if image_rotary_emb is not None else kwargs.get("rotary_emb")
        if emb is not None:
            if isinstance(emb, torch.Tensor) and emb.shape[-2:] == (64, 2):
                return emb.reshape(S, 64, 2).to(torch.float32).contiguous()
            cos, sin = emb
            cos, sin = cos.reshape(S, -1), sin.reshape(S, -1)
            if cos.shape[-1] == ops.HEAD_DIM:  # each frequency repeated for both dims of its pair
                sl = slice(0, None, 2) if not self.rope_half else slice(0, 64)
                cos, sin = cos[:, sl], sin[:, sl]
            return ops.rope_table_from_cos_sin(cos, sin)
        pos = kwargs.get("position_ids")
        if pos is not None:
            if pos.dim() != 2 or pos.shape != (S, 3):
                raise ValueError(f"position_ids must be [S, 3], got {tuple(pos.shape)}")
            return self._rope_cache.get(pos, self.rope_split, self.rope_theta)
        return None

    def project(self, attn, hidden_states, encoder_hidden_states):
        """Q/K/V projections through the module's own (possibly LoRA-wrapped) Linears."""
        ctx = hidden_states if encoder_hidden_states is None else encoder_hidden_states
        H = attn.heads
        q = attn.to_q(hidden_states)
        k = attn.to_k(ctx)
        v = attn.to_v(ctx)
        if q.shape[-1] != H * ops.HEAD_DIM:
            raise ValueError(f"inner dim {q.shape[-1]} != heads {H} x 128")
        to = dict(dtype=torch.bfloat16)
        return (q.to(**to).view(-1, H, ops.HEAD_DIM), k.to(**to).view(-1, H, ops.HEAD_DIM), v.to(**to).view(-1, H, ops.HEAD_DIM))

    def _norm_and_bound(self, attn, mode):
        nq, nk = getattr(attn, "norm_q", None), getattr(attn, "norm_k", None)
        if (nq is None) != (nk is None):
            raise NotImplementedError("norm_q and norm_k must both be present or both be absent")
        if nq is None and self.qk_norm is not True:
            raise NotImplementedError(
                "the attention module has no norm_q / norm_k and the library's Q/K preparation always normalises: pass "
                "qk_norm=True to apply the unit-weight per-head RMSNorm on purpose")
        qw, qeps = _norm_params(nq, "norm_q")
        kw, keps = _norm_params(nk, "norm_k")
        eps = qeps or keps or self.eps
        # the logit bound depends only on the (static) norm weights: read them once per module
        key = (id(attn), mode == _lib.MODE_FP8_QK)
        bound = self._bounds.get(key)
        if bound is None:
            bound = self._bounds[key] = ops.normed_logit_bound(qw, kw, 0.0, mode == _lib.MODE_FP8_QK)
        return qw, kw, eps, (0.0 if self.softmax == "online" else bound)

    def attention(self, attn, q, k, v, rope, cross: bool):
        """Norm + rotation + attention on ``[L, H, 128]`` projections (one GPU)."""
        mode = MODES[self.mode]
        bi = self.block_index
        if cross and mode == _lib.MODE_BLOCK_SPARSE:
            mode, bi = _lib.MODE_DENSE_BF16, None  # the block index describes the joint self-attention only
        qw, kw, eps, bound = self._norm_and_bound(attn, mode)
        return ops.joint_attention(q, k, v, None if cross else rope, mode, bi, qw, kw, eps, self.rope_half, logit_bound=bound,
                                   status_word=self.status.tensor(q))

    # ---- fused projections
    def _fusable(self, attn, x, ctx):
        if not self.fused_projection:
            return None
        if x.dtype != torch.bfloat16 or ctx.dtype != torch.bfloat16:
            return None
        parts = [_linear_parts(m) for m in (attn.to_q, attn.to_k, attn.to_v)]
        if any(p is None or p[0].dtype != torch.bfloat16 for p in parts):
            return None
        return parts

    def _lora_operands(self, mod, parts, x2d):
        """``(weight, bias, x A^T or None, scaled B or None)`` for ``ops.proj_fwd``: the LoRA update either merged into
        a bf16 copy of the weight (``merge_lora``) or kept apart with ``(alpha / rank) B`` scaled once per module."""
        w, bias, a, b, scale = parts
        if a is None:
            return w, bias, None, None
        if self.merge_lora:
            key = (id(mod), w.data_ptr(), a.data_ptr(), b.data_ptr(), scale)
            wm = self._merged_w.get(key)
            if wm is None:  # W + (alpha / rank) B A in fp32, rounded once
                wm = self._merged_w[key] = torch.addmm(w.float(), b.float() * scale, a.float()).to(torch.bfloat16).contiguous()
            return wm, bias, None, None
        t = torch.nn.functional.linear(x2d, a.to(torch.bfloat16))
        key = (id(mod), b.data_ptr(), scale)
        bs = self._scaled_b.get(key)
        if bs is None:  # static at inference
            bs = self._scaled_b[key] = (b.float() * scale).to(torch.bfloat16).contiguous()
        return w, bias, t, bs

    def _fused(self, mod, parts, x2d, prep, rope, norm_w, eps, fp8=False, out_to=None):
        """One projection through the library's GEMM; the thin LoRA product ``x A^T`` stays a torch matmul.
        ``fp8``: returns ``(e4m3 bytes, block scales)``.  ``out_to``: the rows go straight to the heads' owning ranks."""
        w, bias, t, bs = self._lora_operands(mod, parts, x2d)
        return ops.proj_fwd(x2d, w, bias, t, bs, prep=prep, rope=rope, norm_weight=norm_w, eps=eps, rope_half=self.rope_half, fp8=fp8,
                            status_word=self.status.tensor(x2d), out_to=out_to)

    def forget_merged(self) -> None:
        """Drop the merged and scaled LoRA weights this processor keeps (call after the wrapped weights changed)."""
        self._merged_w.clear()
        self._scaled_b.clear()

    def attention_fused(self, attn, parts, hidden_states, ctx, rope, cross: bool):
        """Projections with the preparation in their epilogue, then attention (one GPU)."""
        mode = MODES[self.mode]
        bi = self.block_index
        if cross and mode == _lib.MODE_BLOCK_SPARSE:
            mode, bi = _lib.MODE_DENSE_BF16, None
        qw, kw, eps, bound = self._norm_and_bound(attn, mode)
        x2d, c2d = hidden_states[0], ctx[0]
        fp8 = mode == _lib.MODE_FP8_QK
        q = self._fused(attn.to_q, parts[0], x2d, True, None if cross else rope, qw, eps, fp8)
        k = self._fused(attn.to_k, parts[1], c2d, True, None if cross else rope, kw, eps, fp8)
        v = self._fused(attn.to_v, parts[2], c2d, False, None, None, eps)
        (q, qs), (k, ks) = (q, k) if fp8 else ((q, None), (k, None))
        return ops.attn_fwd(q, k, v, mode, qs, ks, bi, logit_bound=bound, status_word=self.status.tensor(v))

    def attention_sequence_parallel(self, attn, hidden_states, rope):
        """Self-attention with the sequence sharded over the group: each projection is computed when the previous
        tensor's exchange is already on its way."""
        H = attn.heads
        qw, kw, eps, bound = self._norm_and_bound(attn, MODES[self.mode])
        parts = self._fusable(attn, hidden_states, hidden_states)
        if parts is not None:
            x2d = hidden_states[0]
            fp8 = MODES[self.mode] == _lib.MODE_FP8_QK
            if self._ulysses.peer_ready(x2d.shape[0], H, x2d):
                # the projections' epilogues store every prepared row at its head's owning rank: the outbound trip of
                # the reshard costs no pass of its own and overlaps the GEMMs (FP8-QK: the owner quantises)
                return self._ulysses.run_scattered(
                    x2d.shape[0], H, x2d.device,
                    lambda to: self._fused(attn.to_q, parts[0], x2d, True, rope, qw, eps, out_to=to),
                    lambda to: self._fused(attn.to_k, parts[1], x2d, True, rope, kw, eps, out_to=to),
                    lambda to: self._fused(attn.to_v, parts[2], x2d, False, None, None, eps, out_to=to),
                    bound)
            return self._ulysses.run(
                lambda: self._fused(attn.to_q, parts[0], x2d, True, rope, qw, eps, fp8),
                lambda: self._fused(attn.to_k, parts[1], x2d, True, rope, kw, eps, fp8),
                lambda: self._fused(attn.to_v, parts[2], x2d, False, None, None, eps),
                None, logit_bound=bound, prepared=True)

        def proj(lin):
            def f():
                y = lin(hidden_states)
                if y.shape[-1] != H * ops.HEAD_DIM:
                    raise ValueError(f"inner dim {y.shape[-1]} != heads {H} x 128")
                return y.to(torch.bfloat16).view(-1, H, ops.HEAD_DIM)
            return f

        return self._ulysses.run(proj(attn.to_q), proj(attn.to_k), proj(attn.to_v), rope, qw, kw, eps, self.rope_half, bound)

    def __call__(self, attn, hidden_states: torch.Tensor, encoder_hidden_states: Optional[torch.Tensor] = None,
                 attention_mask: Optional[torch.Tensor] = None, image_rotary_emb=None, **kwargs) -> torch.Tensor:
        if attention_mask is not None:
            raise NotImplementedError("the joint DiT attention is unmasked; pass a block index for sparsity")
        if hidden_states.dim() != 3 or hidden_states.shape[0] != 1:
            raise ValueError("one document per forward: hidden_states must be [1, S, D]")
        if not hidden_states.is_cuda:
            raise RuntimeError("B200AttnProcessor needs CUDA tensors (there is no CPU path)")
        S = hidden_states.shape[1]
        cross = encoder_hidden_states is not None
        rope = None if cross else self._rope(S, image_rotary_emb, kwargs)
        ctx = hidden_states if encoder_hidden_states is None else encoder_hidden_states
        parts = None if (self._ulysses is not None and not cross) else self._fusable(attn, hidden_states, ctx)
        if self._ulysses is not None and not cross:
            o = self.attention_sequence_parallel(attn, hidden_states, rope)
        elif parts is not None:
            if ctx.dim() != 3 or ctx.shape[0] != 1:
                raise ValueError("encoder_hidden_states must be [1, T, D]")
            o = self.attention_fused(attn, parts, hidden_states, ctx, rope, cross)
        else:
            q, k, v = self.project(attn, hidden_states, encoder_hidden_states)
            o = self.attention(attn, q, k, v, rope, cross)
        o = o.reshape(1, S, -1).to(hidden_states.dtype)
        to_out = attn.to_out
        out_parts = _linear_parts(to_out[0]) if (self.fused_projection and o.dtype == torch.bfloat16) else None
        if out_parts is not None and out_parts[0].dtype == torch.bfloat16 and out_parts[0].shape[0] % ops.HEAD_DIM == 0:
            # the output projection through the same GEMM (plain epilogue, token-major rows)
            o2d = o[0].contiguous()
            w, bias, t, bs = self._lora_operands(to_out[0], out_parts, o2d)
            o = ops.proj_fwd(o2d, w, bias, t, bs, token_major=True, status_word=self.status.tensor(o))[None]
        else:
            o = to_out[0](o)
        if len(to_out) > 1:
            o = to_out[1](o)
        if self.check_every_call:
            self.check_status()
        return o
