"""CPU oracle for the joint video+audio DiT attention path.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke check and the
benchmark's CPU-baseline leg may import it.  The shipped path is the CUDA library and it refuses
to run without it.

PARITY UNPINNED.  The reference project (Pika-Labs/Pika-H3-Flex) keeps its attention arithmetic
in a third-party dependency that is not vendored: Hugging Face ``diffusers`` pinned at git SHA
3a2f35d4efa4c059c8bfb3bc0d6c906264895c81 (reference ``pyproject.toml:12``, ``requirements.txt:13``),
file ``models/transformers/transformer_minimax_h3.py`` (imported at
``src/pika_h3/core/loader.py:12``, hash-pinned at ``src/pika_h3/runtime.py:9``).  That package is
not installed here and the reference ships no test, golden vector or fixture for this path
(its only test is ``tests/test_text_encoder_truncation.py``).  The functions below therefore restate
the *published* algorithms (RMSNorm, rotary position embedding, softmax attention, e4m3 block
quantisation) under the contracts the reference does pin:

* token order of video rows is frame-major, then row, then column
  (``src/pika_h3/core/packing.py:49-54`` and ``:65-69``);
* rotary positions are a *float* ``[S, 3]`` grid built on the host in float64 and handed to the
  model as data (``src/pika_h3/core/packing.py:126-133`` and ``:166``), so every function here
  takes positions as an argument instead of deriving them from indices;
* one document per forward, batch size 1 (``src/pika_h3/core/wrapper.py:60-66``);
* true fp32 matmuls, TF32 off (``src/pika_h3/core/numerics.py:24-42``).

Choices the reference leaves open (its model file is absent) and this oracle fixes:
per-head RMSNorm over d (eps 1e-6), applied before the rotation; interleaved rotary pairs
``(2i, 2i+1)`` by default (``half`` pairs ``(i, i+d/2)`` selectable); head dim split
``[32, 48, 48]`` over the (t, h, w) axes with base 10000; audio tokens carry positions
``(a, 0, 0)`` so they rotate only the first 32 dims (1-D rotary embedding); softmax scale 1/sqrt(d).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch

ROPE_SPLIT = (32, 48, 48)
ROPE_THETA = 10000.0
RMS_EPS = 1e-6
E4M3_MAX = 448.0
TILE = 128


# --------------------------------------------------------------------------------------------
# positions and rotary tables
# --------------------------------------------------------------------------------------------
def make_positions(grid: Tuple[int, int, int], n_audio: int = 0, dtype=torch.float64) -> torch.Tensor:
    """Position grid ``[L, 3]`` for ``n_audio`` audio tokens followed by a ``(T, Hg, Wg)`` video grid.

    Video token n maps to ``(t, h, w) = (n // (Hg*Wg), (n // Wg) % Hg, n % Wg)``: the frame-major,
    row-major order of reference ``src/pika_h3/core/packing.py:49-54``.  Audio token a maps to
    ``(a, 0, 0)``.  Audio rows come first, matching the order in which the reference counts them
    (``src/pika_h3/core/geometry.py:82-113`` lists audio before video).
    """
    T, Hg, Wg = grid
    n = torch.arange(T * Hg * Wg, dtype=torch.int64)
    vid = torch.stack([n // (Hg * Wg), (n // Wg) % Hg, n % Wg], dim=1).to(dtype)
    aud = torch.zeros(n_audio, 3, dtype=dtype)
    aud[:, 0] = torch.arange(n_audio, dtype=dtype)
    return torch.cat([aud, vid], dim=0)


def rope_table(pos: torch.Tensor, split: Sequence[int] = ROPE_SPLIT, theta: float = ROPE_THETA):
    """``cos, sin`` tables ``[L, d/2]`` in float64 from a float position grid ``[L, 3]``.

    Pair j of axis a (a block of ``split[a]`` dims) turns by ``pos[:, a] * theta**(-2j/split[a])``.
    """
    pos = pos.to(torch.float64)
    cols = []
    for a, da in enumerate(split):
        j = torch.arange(da // 2, dtype=torch.float64)
        inv = theta ** (-2.0 * j / da)
        cols.append(pos[:, a : a + 1] * inv[None, :])
    ang = torch.cat(cols, dim=1)
    return torch.cos(ang), torch.sin(ang)


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = RMS_EPS) -> torch.Tensor:
    """Per-head RMSNorm over the last dim: ``x * rsqrt(mean(x^2) + eps) * w``."""
    y = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool = True) -> torch.Tensor:
    """Rotate ``x [L, H, d]`` by tables ``[L, d/2]``.  Pair j is ``(2j, 2j+1)`` or ``(j, j+d/2)``."""
    c = cos.to(x.dtype)[:, None, :]
    s = sin.to(x.dtype)[:, None, :]
    if interleaved:
        a, b = x[..., 0::2], x[..., 1::2]
        out = torch.empty_like(x)
        out[..., 0::2] = a * c - b * s
        out[..., 1::2] = a * s + b * c
        return out
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def qk_prep(q, k, cos, sin, q_weight=None, k_weight=None, eps: float = RMS_EPS, interleaved: bool = True):
    """RMSNorm then rotation on ``q`` and ``k`` ``[L, H, d]``; math in the dtype of ``q``."""
    return (
        apply_rope(rms_norm(q, q_weight, eps), cos, sin, interleaved),
        apply_rope(rms_norm(k, k_weight, eps), cos, sin, interleaved),
    )


# --------------------------------------------------------------------------------------------
# e4m3 block quantisation
# --------------------------------------------------------------------------------------------
def quantize_e4m3_blocks(x: torch.Tensor, block: int = TILE):
    """Quantise ``x [L, H, d]`` to e4m3 with one absmax scale per (head, ``block`` tokens).

    Returns ``(xq, scale)``: ``xq`` float32 holding the e4m3 values (not yet multiplied back) and
    ``scale [H, ceil(L/block)]`` float32 with ``scale = absmax / 448`` (1.0 for an all-zero block),
    so that ``x ~= xq * scale``.
    """
    L, H, d = x.shape
    nb = (L + block - 1) // block
    xf = x.to(torch.float32)
    pad = nb * block - L
    xp = torch.cat([xf, xf.new_zeros(pad, H, d)], dim=0) if pad else xf
    xb = xp.view(nb, block, H, d)
    amax = xb.abs().amax(dim=(1, 3))  # [nb, H]
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    inv = (1.0 / scale).to(torch.float32)
    y = (xb * inv[:, None, :, None]).clamp_(-E4M3_MAX, E4M3_MAX)
    yq = y.to(torch.float8_e4m3fn).to(torch.float32)
    return yq.view(nb * block, H, d)[:L].contiguous(), scale.t().contiguous()


def dequantize_blocks(xq: torch.Tensor, scale: torch.Tensor, block: int = TILE) -> torch.Tensor:
    L = xq.shape[0]
    s = scale.t().repeat_interleave(block, dim=0)[:L]  # [L, H]
    return xq * s[:, :, None]


# --------------------------------------------------------------------------------------------
# block mask
# --------------------------------------------------------------------------------------------
def neighbourhood_block_mask(
    grid: Tuple[int, int, int],
    n_audio: int,
    window: Tuple[int, int, int] = (2, 8, 8),
    block: int = TILE,
    audio_rows_dense: bool = True,
) -> np.ndarray:
    """Boolean tile mask ``[nQB, nKB]`` for audio-first, frame-major token order.

    A video-video tile is kept when some query token of the row tile and some key token of the column
    tile lie within ``window`` = (|dt|, |dh|, |dw|) of each other; every audio column tile is kept for
    every row; audio row tiles keep every column when ``audio_rows_dense``.  Tiles that straddle the
    audio/video border count for both regions.
    """
    T, Hg, Wg = grid
    L = n_audio + T * Hg * Wg
    nb = (L + block - 1) // block
    pos = make_positions(grid, n_audio, dtype=torch.int64).numpy()
    is_video = np.arange(L) >= n_audio
    keep = np.zeros((nb, nb), dtype=bool)
    # bounding intervals are not enough (a tile wraps rows/frames): compare token sets per axis.
    tok_blocks = [np.arange(b * block, min(L, (b + 1) * block)) for b in range(nb)]
    has_audio = np.array([(~is_video[t]).any() for t in tok_blocks])
    vid_tok = [t[is_video[t]] for t in tok_blocks]
    wt, wh, ww = window
    for qb in range(nb):
        q = pos[vid_tok[qb]]
        if has_audio[qb] and audio_rows_dense:
            keep[qb, :] = True
            continue
        for kb in range(nb):
            if has_audio[kb]:
                keep[qb, kb] = True
                continue
            kk = pos[vid_tok[kb]]
            if q.size == 0 or kk.size == 0:
                continue
            # cheap reject on frame range first
            if kk[:, 0].min() - q[:, 0].max() > wt or q[:, 0].min() - kk[:, 0].max() > wt:
                continue
            d = np.abs(q[:, None, :] - kk[None, :, :])
            keep[qb, kb] = bool(((d[..., 0] <= wt) & (d[..., 1] <= wh) & (d[..., 2] <= ww)).any())
    return keep


def mask_to_csr(keep: np.ndarray):
    """Tile mask -> CSR ``(row_ptr int32 [nQB+1], col_idx int32 [nnz])``, columns ascending per row."""
    row_ptr = np.zeros(keep.shape[0] + 1, dtype=np.int32)
    row_ptr[1:] = np.cumsum(keep.sum(axis=1))
    col_idx = np.nonzero(keep)[1].astype(np.int32)
    return row_ptr, col_idx


def csr_to_token_mask(row_ptr, col_idx, Lq: int, Lk: int, block: int = TILE) -> torch.Tensor:
    nqb = len(row_ptr) - 1
    nkb = (Lk + block - 1) // block
    keep = np.zeros((nqb, nkb), dtype=bool)
    for r in range(nqb):
        keep[r, col_idx[row_ptr[r] : row_ptr[r + 1]]] = True
    m = torch.from_numpy(keep).repeat_interleave(block, 0).repeat_interleave(block, 1)
    return m[:Lq, :Lk]


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    scale: Optional[float] = None,
    csr: Optional[Tuple[np.ndarray, np.ndarray]] = None,
    q_rows: Optional[torch.Tensor] = None,
    chunk: int = 1024,
    return_lse: bool = False,
):
    """Exact softmax attention ``O = softmax(q k^T * scale) v`` per head, non-causal.

    ``q [Lq, H, d]``, ``k, v [Lk, H, d]``; math in the dtype of ``q`` (fp32 or fp64), queries processed
    ``chunk`` rows at a time with the full key range (no online-softmax tricks).  ``csr`` restricts each
    128-row query tile to the listed 128-column key tiles.  ``q_rows`` selects a subset of query rows
    (their global indices, needed to look up the mask); the output then has ``len(q_rows)`` rows.
    """
    Lq_full, H, d = q.shape
    Lk = k.shape[0]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    rows = torch.arange(Lq_full) if q_rows is None else q_rows.to(torch.int64)
    kt = k.permute(1, 2, 0).contiguous()  # [H, d, Lk]
    vh = v.permute(1, 0, 2).contiguous()  # [H, Lk, d]
    tok_mask = None
    if csr is not None:
        nkb = (Lk + TILE - 1) // TILE
        keep = np.zeros((len(csr[0]) - 1, nkb), dtype=bool)
        for r in range(keep.shape[0]):
            keep[r, csr[1][csr[0][r] : csr[0][r + 1]]] = True
        tok_mask = torch.from_numpy(keep)
    out = torch.empty(len(rows), H, d, dtype=q.dtype)
    lse = torch.empty(len(rows), H, dtype=q.dtype)
    for s in range(0, len(rows), chunk):
        r = rows[s : s + chunk]
        qc = q[r].permute(1, 0, 2)  # [H, c, d]
        sc = torch.matmul(qc, kt) * scale  # [H, c, Lk]
        if tok_mask is not None:
            m = tok_mask[r // TILE].repeat_interleave(TILE, dim=1)[:, :Lk]  # [c, Lk]
            sc = sc.masked_fill(~m[None], float("-inf"))
        mx = sc.amax(dim=-1, keepdim=True)
        p = torch.exp(sc - mx)
        den = p.sum(dim=-1, keepdim=True)
        out[s : s + chunk] = torch.matmul(p / den, vh).permute(1, 0, 2)
        lse[s : s + chunk] = (mx + den.log()).squeeze(-1).t()
    return (out, lse) if return_lse else out


def attention_fp8_qk(q, k, v, scale=None, csr=None, q_rows=None, chunk: int = 1024):
    """Attention with q, k replaced by their per-(head, 128-token) e4m3 quantisation; v untouched."""
    qq, sq = quantize_e4m3_blocks(q)
    kq, sk = quantize_e4m3_blocks(k)
    return attention(
        dequantize_blocks(qq, sq).to(q.dtype), dequantize_blocks(kq, sk).to(q.dtype), v, scale, csr, q_rows, chunk
    )


def joint_attention(q, k, v, pos, mode: str = "dense", csr=None, q_rows=None, interleaved: bool = True,
                    q_weight=None, k_weight=None, chunk: int = 1024):
    """Whole hot path on one rank: RMSNorm + rotation on q, k, then attention in ``mode``
    (``dense`` | ``fp8_qk`` | ``block_sparse``).  Inputs ``[L, H, d]``; positions ``[L, 3]``."""
    cos, sin = rope_table(pos)
    qp, kp = qk_prep(q, k, cos, sin, q_weight, k_weight, interleaved=interleaved)
    if mode == "fp8_qk":
        return attention_fp8_qk(qp, kp, v, csr=csr, q_rows=q_rows, chunk=chunk)
    if mode == "block_sparse" and csr is None:
        raise ValueError("block_sparse needs a CSR block index")
    return attention(qp, kp, v, csr=csr if mode == "block_sparse" else None, q_rows=q_rows, chunk=chunk)


# --------------------------------------------------------------------------------------------
# Ulysses reshard, simulated on one process
# --------------------------------------------------------------------------------------------
def lora_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                lora_a: Optional[torch.Tensor] = None, lora_b: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """``y = x W^T + scale * (x A^T) B^T + bias`` in fp32: the LoRA-wrapped Linear the reference puts on
    to_q / to_k / to_v / to_out.0 (src/pika_h3/core/loader.py:9, :20-49; rank = alpha = 128, src/pika_h3/pipeline.py:34,
    so scale = alpha / rank = 1).  ``x [L, K]``, ``weight [N, K]``, ``lora_a [R, K]``, ``lora_b [N, R]``."""
    y = x.float() @ weight.float().t()
    if lora_a is not None:
        y = y + scale * ((x.float() @ lora_a.float().t()) @ lora_b.float().t())
    if bias is not None:
        y = y + bias.float()
    return y


def project_and_prepare(x, weight, heads: int, bias=None, lora_a=None, lora_b=None, scale: float = 1.0,
                        cos=None, sin=None, norm_weight=None, eps: float = 1e-6, interleaved: bool = True) -> torch.Tensor:
    """Projection followed by the per-head RMSNorm and rotation: what the fused projection kernel produces for
    Q and K (``[L, heads, 128]`` fp32)."""
    y = lora_linear(x, weight, bias, lora_a, lora_b, scale).view(x.shape[0], heads, 128)
    y = rms_norm(y, norm_weight, eps)
    if cos is not None:
        y = apply_rope(y, cos, sin, interleaved)
    return y


def adaln_modulate(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, idx: Optional[torch.Tensor] = None,
                   eps: float = 1e-6, rms: bool = False, weight: Optional[torch.Tensor] = None,
                   bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``norm(x) * (1 + scale[idx]) + shift[idx]`` in fp32: the reference's patched adaptive layer norm
    (patches/0001-h3-adaln-fp32.patch:36-40: ``self.norm(hidden_states)`` then the modulation with
    ``index_select(0, timestep_indices)``).  ``x [L, D]``, ``scale`` / ``shift`` ``[T, D]``, ``idx [L]``."""
    x = x.float()
    if rms:
        n = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    else:
        mu = x.mean(-1, keepdim=True)
        n = (x - mu) * torch.rsqrt((x - mu).pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        n = n * weight.float()
    if bias is not None:
        n = n + bias.float()
    if idx is None:
        idx = torch.zeros(x.shape[0], dtype=torch.long)
    return n * (1.0 + scale.float().index_select(0, idx)) + shift.float().index_select(0, idx)


def ulysses_simulate(q_shards, k_shards, v_shards, attn_fn, n_heads: int):
    """Sequence-parallel attention over ``P = len(q_shards)`` simulated ranks.

    Rank r holds tokens ``[r*L/P, (r+1)*L/P)`` of every head.  Heads are padded to a multiple of P,
    resharded so each rank holds every token of ``Hp/P`` heads, ``attn_fn(q, k, v)`` runs per rank,
    and the inverse reshard restores sequence shards.  Returns the list of per-rank outputs.
    """
    P = len(q_shards)
    Hp = (n_heads + P - 1) // P * P

    def pad(x):
        return x if Hp == n_heads else torch.cat([x, x.new_zeros(x.shape[0], Hp - n_heads, x.shape[2])], dim=1)

    def seq_to_head(shards):
        shards = [pad(s) for s in shards]
        hp = Hp // P
        return [torch.cat([s[:, r * hp : (r + 1) * hp] for s in shards], dim=0) for r in range(P)]

    qh, kh, vh = seq_to_head(q_shards), seq_to_head(k_shards), seq_to_head(v_shards)
    oh = [attn_fn(qh[r], kh[r], vh[r]) for r in range(P)]
    lq = q_shards[0].shape[0]
    outs = []
    for r in range(P):
        o = torch.cat([oh[p][r * lq : (r + 1) * lq] for p in range(P)], dim=1)
        outs.append(o[:, :n_heads].contiguous())
    return outs


# --------------------------------------------------------------------------------------------
# seeded workloads named by the benchmark configs
# --------------------------------------------------------------------------------------------
CONFIGS = {
    # name: (grid, n_audio, heads, seed)
    "cfg0": ((4, 32, 32), 0, 8, 1000),
    "cfg1": ((31, 30, 52), 1024, 40, 1001),
    "cfg3": ((31, 48, 84), 1024, 40, 1003),
}


def seeded_qkv(L: int, H: int, d: int = 128, seed: int = 0, dtype=torch.float32):
    """Q, K, V ~ N(0,1) drawn in that order from one CPU generator, shape ``[L, H, d]``."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(L, H, d, generator=g, dtype=torch.float32)
    k = torch.randn(L, H, d, generator=g, dtype=torch.float32)
    v = torch.randn(L, H, d, generator=g, dtype=torch.float32)
    return q.to(dtype), k.to(dtype), v.to(dtype)


def error_stats(out: torch.Tensor, ref: torch.Tensor) -> dict:
    o, r = out.to(torch.float64), ref.to(torch.float64)
    diff = (o - r).abs()
    return {
        "max_abs": float(diff.max()),
        "mean_abs": float(diff.mean()),
        "rel_l2": float((o - r).norm() / r.norm().clamp_min(1e-30)),
    }
