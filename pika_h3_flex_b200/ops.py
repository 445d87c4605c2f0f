"""Torch-facing wrappers over the C ABI.  Tensors are device memory handles only: every function hands
``data_ptr()``, element strides and the current CUDA stream to ``libh3attn.so``.

All sequence tensors have *logical* shape ``[L, H, 128]`` with the last dim contiguous; any L/H strides
(so ``[H, L, 128]`` storage viewed through ``permute(1, 0, 2)`` is fine and is what ``qk_prep`` returns).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import AttnParams, PrepParams, check

TILE = 128
HEAD_DIM = 128
ROPE_SPLIT = (32, 48, 48)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("h3attn runs on CUDA tensors only (there is no CPU path)")


def _lhd(t: torch.Tensor, name: str, dtypes) -> Tuple[int, int, int, int]:
    if t.dim() != 3 or t.shape[2] != HEAD_DIM or t.stride(2) != 1:
        raise ValueError(f"{name}: expected logical [L, H, 128] with a contiguous last dim, got {tuple(t.shape)} / {t.stride()}")
    if t.dtype not in dtypes:
        raise TypeError(f"{name}: dtype {t.dtype} not in {dtypes}")
    return t.shape[0], t.shape[1], t.stride(0), t.stride(1)


@dataclass
class RankOutputs:
    """Where the attention output goes under sequence parallelism: query row ``g`` is stored at row ``g % rows`` of
    the buffer at device address ``bases[g // rows]`` (this process's memory or a peer GPU's, see ``peer.py``), head
    ``j`` of the launch at ``j * stride_h`` elements, rows ``stride_l`` elements apart; each base already points at
    the launch's first head."""

    bases: list
    rows: int
    stride_l: int
    stride_h: int


@dataclass
class HeadOwners:
    """Where prepared rows go under sequence parallelism (``h3a_head_scatter``): ``bases[p]`` is the device address of
    rank p's ``[heads_per_rank, L_total, 128]`` bf16 buffer; head ``head0 + h`` of the input belongs to rank
    ``// heads_per_rank`` (blocks) or ``% n_ranks`` (``round_robin``); this shard's token l is row ``row_offset + l``."""

    bases: list
    heads_per_rank: int
    round_robin: bool
    row_offset: int
    L_total: int
    head0: int = 0
    start_head: int = 0  # order in which the launch walks the heads (see h3a_head_scatter.start_head): differs per rank

    def c_struct(self):
        s = _lib.HeadScatter()
        for r, b in enumerate(self.bases):
            s.base[r] = b
        s.n_ranks, s.heads_per_rank, s.round_robin = len(self.bases), int(self.heads_per_rank), int(bool(self.round_robin))
        s.head0, s.row_offset, s.L_total = int(self.head0), int(self.row_offset), int(self.L_total)
        s.start_head = int(self.start_head)
        return s


def prep_scatter(x: torch.Tensor, to: HeadOwners, rope: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None,
                 eps: float = 1e-6, rope_half: bool = False, no_norm: bool = False) -> None:
    """``h3a_qk_prep_scatter`` for one tensor: prepare this rank's ``x [Ls, H, 128]`` bf16 rows (RMSNorm x ``weight``,
    rotation by ``rope``; ``no_norm`` with no table = the plain re-layout V needs) and store each row at its head's
    owning rank.  Returns nothing: the rows are in the owners' buffers once every rank's kernel has finished."""
    _require_cuda(x)
    L, H, sl, sh = _lhd(x, "x", (torch.bfloat16,))
    p = PrepParams()
    p.d, p.H, p.eps = HEAD_DIM, H, float(eps)
    p.rope_mode = _lib.ROPE_HALF if rope_half else _lib.ROPE_INTERLEAVED
    p.flags = _lib.PREP_NO_NORM if no_norm else 0
    p.q_in, p.q_stride_l, p.q_stride_h, p.Lq = x.data_ptr(), sl, sh, L
    if rope is not None:
        if rope.shape != (L, 64, 2) or rope.dtype != torch.float32 or not rope.is_contiguous():
            raise ValueError("rope must be a contiguous fp32 [L, 64, 2] table")
        p.q_rope = rope.data_ptr()
    if weight is not None:
        weight = weight.to(torch.float32).contiguous()
        p.q_weight = weight.data_ptr()
    st = to.c_struct()
    check(_lib.load().h3a_qk_prep_scatter(C.byref(p), C.byref(st), None, _stream()), "h3a_qk_prep_scatter")


@dataclass
class BlockIndex:
    """CSR index over 128x128 tiles: ``row_ptr [nQB+1]``, ``col_idx [nnz]`` (int32, columns ascending)."""

    row_ptr: torch.Tensor
    col_idx: torch.Tensor
    nnz: int
    n_q_tiles: int
    n_k_tiles: int
    heavy_pairs: int = 0  # scheduling hint: leading query-tile pairs with far longer key lists than the rest

    @property
    def density(self) -> float:
        return self.nnz / float(self.n_q_tiles * self.n_k_tiles)

    def to(self, device) -> "BlockIndex":
        return BlockIndex(self.row_ptr.to(device), self.col_idx.to(device), self.nnz, self.n_q_tiles, self.n_k_tiles,
                          self.heavy_pairs)

    @staticmethod
    def from_csr(row_ptr, col_idx, n_k_tiles: int) -> "BlockIndex":
        rp = torch.as_tensor(np.asarray(row_ptr), dtype=torch.int32)
        ci = torch.as_tensor(np.asarray(col_idx), dtype=torch.int32)
        return BlockIndex(rp, ci, int(ci.numel()), int(rp.numel() - 1), int(n_k_tiles), _leading_heavy_pairs(rp.numpy()))


def _leading_heavy_pairs(row_ptr: np.ndarray) -> int:
    """Number of leading pairs of query tiles whose key lists are more than 4x the median pair's (the dense
    audio rows at the head of the joint sequence); 0 when there is no such prefix."""
    per_row = np.diff(row_ptr.astype(np.int64))
    if per_row.size < 4:
        return 0
    if per_row.size % 2:
        per_row = np.append(per_row, 0)
    per_pair = per_row[0::2] + per_row[1::2]
    thresh = 4 * max(1.0, float(np.median(per_pair)))
    n = 0
    while n < per_pair.size and per_pair[n] > thresh:
        n += 1
    return n if n < per_pair.size else 0


def build_block_index(grid: Tuple[int, int, int], n_audio: int, window: Tuple[int, int, int] = (2, 8, 8)) -> BlockIndex:
    """Spatiotemporal-neighbourhood block index (host memory) via ``h3a_build_block_index``."""
    lib = _lib.load()
    T, Hg, Wg = (int(x) for x in grid)
    L = n_audio + T * Hg * Wg
    nb = (L + TILE - 1) // TILE
    nnz = C.c_int64(0)
    args = [T, Hg, Wg, int(n_audio), int(window[0]), int(window[1]), int(window[2])]
    check(lib.h3a_build_block_index(*args, None, None, C.byref(nnz)), "h3a_build_block_index(size)")
    row_ptr = np.zeros(nb + 1, dtype=np.int32)
    col_idx = np.zeros(max(1, nnz.value), dtype=np.int32)
    check(
        lib.h3a_build_block_index(*args, row_ptr.ctypes.data, col_idx.ctypes.data, C.byref(nnz)),
        "h3a_build_block_index(fill)",
    )
    return BlockIndex(torch.from_numpy(row_ptr), torch.from_numpy(col_idx[: nnz.value].copy()), int(nnz.value), nb, nb,
                      _leading_heavy_pairs(row_ptr))


def rope_table(pos: torch.Tensor, split=ROPE_SPLIT, theta: float = 10000.0) -> torch.Tensor:
    """(cos, sin) table ``[L, 64, 2]`` fp32 on the device from a position grid ``[L, 3]``."""
    _require_cuda(pos)
    lib = _lib.load()
    p = pos.to(torch.float32).contiguous()
    L = p.shape[0]
    table = torch.empty(L, 64, 2, dtype=torch.float32, device=p.device)
    sp = (C.c_int32 * 3)(*[int(s) for s in split])
    check(lib.h3a_rope_table(p.data_ptr(), L, sp, float(theta), table.data_ptr(), _stream()), "h3a_rope_table")
    return table


def rope_table_from_cos_sin(cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Pack caller-supplied ``cos, sin [L, 64]`` into the ``[L, 64, 2]`` fp32 table layout."""
    return torch.stack([cos.to(torch.float32), sin.to(torch.float32)], dim=-1).contiguous()


def qk_prep(
    q: Optional[torch.Tensor],
    k: Optional[torch.Tensor],
    q_rope: Optional[torch.Tensor] = None,
    k_rope: Optional[torch.Tensor] = None,
    q_weight: Optional[torch.Tensor] = None,
    k_weight: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
    fp8: bool = False,
    rope_half: bool = False,
    no_norm: bool = False,
):
    """RMSNorm + rotation (+ e4m3 quantisation).  Returns ``(q', k', q_scale, k_scale)``; the prepared
    tensors are logical ``[L, H, 128]`` views of head-major storage; scales are ``[H, ceil(L/128)]`` or None.
    ``no_norm`` skips the RMSNorm: with no rotation table the call only re-lays rows out head-major, or (``fp8``)
    quantises rows that are prepared already."""
    _require_cuda(q, k)
    lib = _lib.load()
    p = PrepParams()
    p.d = HEAD_DIM
    p.eps = float(eps)
    p.rope_mode = _lib.ROPE_HALF if rope_half else _lib.ROPE_INTERLEAVED
    p.flags = (_lib.PREP_FP8 if fp8 else 0) | (_lib.PREP_NO_NORM if no_norm else 0)
    outs = {}
    keep = []
    H = None
    for name, x, rope, w in (("q", q, q_rope, q_weight), ("k", k, k_rope, k_weight)):
        if x is None:
            outs[name] = (None, None)
            continue
        L, h, sl, sh = _lhd(x, name, (torch.bfloat16,))
        if H is not None and h != H:
            raise ValueError("q and k must have the same number of heads")
        H = h
        out = torch.empty(h, L, HEAD_DIM, dtype=torch.uint8 if fp8 else torch.bfloat16, device=x.device)
        scale = torch.empty(h, (L + TILE - 1) // TILE, dtype=torch.float32, device=x.device) if fp8 else None
        setattr(p, f"{name}_in", x.data_ptr())
        setattr(p, f"{name}_out", out.data_ptr())
        setattr(p, f"{name}_scale", scale.data_ptr() if fp8 else None)
        setattr(p, f"{name}_stride_l", sl)
        setattr(p, f"{name}_stride_h", sh)
        setattr(p, f"L{name}", L)
        if rope is not None:
            if rope.shape != (L, 64, 2) or rope.dtype != torch.float32 or not rope.is_contiguous():
                raise ValueError(f"{name}_rope must be a contiguous fp32 [L, 64, 2] table")
            setattr(p, f"{name}_rope", rope.data_ptr())
        if w is not None:
            w = w.to(torch.float32).contiguous()
            keep.append(w)
            setattr(p, f"{name}_weight", w.data_ptr())
        outs[name] = (out.permute(1, 0, 2), scale)
    if H is None:
        raise ValueError("nothing to prepare")
    p.H = H
    check(lib.h3a_qk_prep(C.byref(p), _stream()), "h3a_qk_prep")
    return outs["q"][0], outs["k"][0], outs["q"][1], outs["k"][1]


def attn_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mode: int = _lib.MODE_DENSE_BF16,
    q_scale: Optional[torch.Tensor] = None,
    k_scale: Optional[torch.Tensor] = None,
    block_index: Optional[BlockIndex] = None,
    softmax_scale: float = 0.0,
    out: Optional[torch.Tensor] = None,
    return_lse: bool = False,
    status_word: Optional[torch.Tensor] = None,
    wait_limit_ns: int = 0,
    workspace: Optional[torch.Tensor] = None,
    logit_bound: float = 0.0,
    out_ranks: Optional["RankOutputs"] = None,
):
    """Forward attention through ``h3a_attn_fwd``.  Returns ``out [Lq, H, 128]`` bf16 (and ``lse [H, Lq]``).
    ``out_ranks`` (sequence parallelism): the rows are stored where their token lives, in the buffers it names,
    instead of in ``out``; the call then returns None for the output."""
    _require_cuda(q, k, v)
    lib = _lib.load()
    fp8 = mode == _lib.MODE_FP8_QK
    qk_types = (torch.uint8, torch.float8_e4m3fn) if fp8 else (torch.bfloat16,)
    Lq, H, qsl, qsh = _lhd(q, "q", qk_types)
    Lk, Hk, ksl, ksh = _lhd(k, "k", qk_types)
    Lv, Hv, vsl, vsh = _lhd(v, "v", (torch.bfloat16,))
    if Hk != H or Hv != H or Lv != Lk:
        raise ValueError("q, k, v disagree on heads or key length")
    p = AttnParams()
    if out_ranks is not None:
        if out is not None:
            raise ValueError("out and out_ranks exclude each other")
        if len(out_ranks.bases) * out_ranks.rows < Lq or not 1 <= len(out_ranks.bases) <= _lib.MAX_RANKS:
            raise ValueError("out_ranks does not cover the query rows")
        osl, osh = int(out_ranks.stride_l), int(out_ranks.stride_h)
        p.o = out_ranks.bases[0]
        for r, b in enumerate(out_ranks.bases):
            p.o_rank_base[r] = b
        p.o_n_ranks, p.o_rank_rows = len(out_ranks.bases), int(out_ranks.rows)
    else:
        if out is None:
            out = torch.empty(Lq, H, HEAD_DIM, dtype=torch.bfloat16, device=q.device)
        _, _, osl, osh = _lhd(out, "out", (torch.bfloat16,))
        p.o = out.data_ptr()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.q_stride_l, p.q_stride_h = qsl, qsh
    p.k_stride_l, p.k_stride_h = ksl, ksh
    p.v_stride_l, p.v_stride_h = vsl, vsh
    p.o_stride_l, p.o_stride_h = osl, osh
    p.Lq, p.Lk, p.H, p.d, p.B = Lq, Lk, H, HEAD_DIM, 1
    p.mode = int(mode)
    p.softmax_scale = float(softmax_scale)
    if fp8:
        nqb, nkb = (Lq + TILE - 1) // TILE, (Lk + TILE - 1) // TILE
        if q_scale is None or k_scale is None:
            raise ValueError("FP8_QK mode needs q_scale and k_scale")
        if tuple(q_scale.shape) != (H, nqb) or tuple(k_scale.shape) != (H, nkb):
            raise ValueError("scale tensors must be [H, ceil(L/128)]")
        q_scale, k_scale = q_scale.contiguous(), k_scale.contiguous()
        p.q_scale, p.k_scale = q_scale.data_ptr(), k_scale.data_ptr()
    if mode == _lib.MODE_BLOCK_SPARSE:
        if block_index is None:
            raise ValueError("BLOCK_SPARSE mode needs a block index")
        if block_index.n_q_tiles != (Lq + TILE - 1) // TILE or block_index.n_k_tiles != (Lk + TILE - 1) // TILE:
            raise ValueError("block index does not match Lq / Lk")
        if not block_index.row_ptr.is_cuda:
            raise ValueError("block index must be on the device (BlockIndex.to(device))")
        p.row_ptr, p.col_idx, p.nnz = block_index.row_ptr.data_ptr(), block_index.col_idx.data_ptr(), block_index.nnz
        p.sparse_heavy_pairs = block_index.heavy_pairs
        need = C.c_size_t(0)
        check(lib.h3a_attn_workspace_bytes(C.byref(p), C.byref(need)), "h3a_attn_workspace_bytes")
        if workspace is None or workspace.numel() * workspace.element_size() < need.value:
            workspace = torch.empty(max(16, need.value), dtype=torch.uint8, device=q.device)
        p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    lse = None
    if return_lse:
        lse = torch.empty(H, Lq, dtype=torch.float32, device=q.device)
        p.lse = lse.data_ptr()
    if status_word is not None:
        p.status_word = status_word.data_ptr()
    p.wait_limit_ns = int(wait_limit_ns)
    p.logit_bound = float(logit_bound)
    if mode != _lib.MODE_BLOCK_SPARSE:
        # optional scratch: lets the launch split the key range for the CTAs of its last, partly filled wave (with a logit
        # bound), or run the online softmax as two launches (without one)
        need = C.c_size_t(0)
        check(lib.h3a_attn_workspace_bytes(C.byref(p), C.byref(need)), "h3a_attn_workspace_bytes")
        if need.value:
            if workspace is None:  # a caller's own workspace is passed as it is: one that is too small means "do not split"
                workspace = torch.empty(need.value, dtype=torch.uint8, device=q.device)
            p.workspace, p.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    check(lib.h3a_attn_fwd(C.byref(p), _stream()), "h3a_attn_fwd")
    return (out, lse) if return_lse else out


def split_workspace_bytes(Lq: int, Lk: int, H: int, mode: int = _lib.MODE_DENSE_BF16, logit_bound: float = 0.0) -> int:
    """Bytes of optional scratch for a dense / FP8-QK launch of this shape on the current device: with a logit bound,
    what lets it split the key range for the CTA pairs of its last, partly filled wave; without one, the redo list of
    the two-launch online softmax (0: neither applies).  ``attn_fwd`` allocates it per call when no ``workspace`` is
    given; callers in a loop can allocate it once."""
    if mode == _lib.MODE_BLOCK_SPARSE:
        return 0
    p = AttnParams()
    p.Lq, p.Lk, p.H, p.d, p.B, p.mode, p.logit_bound = int(Lq), int(Lk), int(H), HEAD_DIM, 1, int(mode), float(logit_bound)
    need = C.c_size_t(0)
    check(_lib.load().h3a_attn_workspace_bytes(C.byref(p), C.byref(need)), "h3a_attn_workspace_bytes")
    return int(need.value)


def kernel_choice(Lq: int, Lk: int, H: int, mode: int = _lib.MODE_DENSE_BF16, logit_bound: float = 0.0, nnz: int = 0,
                  workspace_bytes: int = 0) -> dict:
    """Which attention kernel the library launches for this shape on the current device (``h3a_attn_kernel_choice``):
    ``{"kernel", "cta_pairs", "fixed_reference", "split_last_wave", "online_two_launch", "persistent"}``."""
    p = AttnParams()
    p.Lq, p.Lk, p.H, p.d, p.B, p.mode, p.logit_bound, p.nnz = int(Lq), int(Lk), int(H), HEAD_DIM, 1, int(mode), float(logit_bound), int(nnz)
    if workspace_bytes:
        p.workspace, p.workspace_bytes = 16, int(workspace_bytes)  # only looked at, never dereferenced
    c = C.c_int32(0)
    check(_lib.load().h3a_attn_kernel_choice(C.byref(p), C.byref(c)), "h3a_attn_kernel_choice")
    pairs = bool(c.value & _lib.KERNEL_CTA_PAIRS)
    return {"kernel": "attn_fwd_pair_kernel" if pairs else "attn_fwd_kernel", "cta_pairs": pairs,
            "fixed_reference": bool(c.value & _lib.KERNEL_FIXED_REFERENCE), "split_last_wave": bool(c.value & _lib.KERNEL_SPLIT_LAST_WAVE),
            "online_two_launch": bool(c.value & _lib.KERNEL_ONLINE_TWO_LAUNCH), "persistent": bool(c.value & _lib.KERNEL_PERSISTENT)}


def proj_fwd(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    lora_t: Optional[torch.Tensor] = None,
    lora_bs: Optional[torch.Tensor] = None,
    prep: bool = False,
    rope: Optional[torch.Tensor] = None,
    norm_weight: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
    rope_half: bool = False,
    status_word: Optional[torch.Tensor] = None,
    wait_limit_ns: int = 0,
    token_major: bool = False,
    fp8: bool = False,
    out_to: Optional[HeadOwners] = None,
):
    """One of the Q / K / V (or, with ``token_major``, the output) projections through ``h3a_proj_fwd``: ``x [L, K]`` bf16 times ``weight [N, K]`` bf16
    (``nn.Linear`` layout, N = heads x 128), plus ``lora_t [L, R] @ lora_bs [N, R]^T`` and ``bias [N]`` when given;
    with ``prep`` the per-head RMSNorm (x ``norm_weight``) and the rotation by ``rope [L, 64, 2]`` run in the
    epilogue.  Returns a logical ``[L, heads, 128]`` bf16 view of head-major storage, like :func:`qk_prep`; with
    ``token_major`` a plain contiguous ``[L, N]`` tensor (what ``to_out`` produces).  ``fp8`` (with ``prep``):
    e4m3 bytes plus per-(head, 128-token block) scales, returned as ``(out_uint8, scale [heads, ceil(L/128)])``.
    ``out_to`` (sequence parallelism, bf16 head-major epilogues): the rows go straight to the rank that computes their
    head (as :func:`prep_scatter` does) and the call returns None."""
    _require_cuda(x, weight)
    lib = _lib.load()
    if x.dim() != 2 or weight.dim() != 2 or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise ValueError("x [L, K] and weight [N, K] must be 2-D bf16")
    L, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K or N % HEAD_DIM or x.stride(1) != 1 or weight.stride(1) != 1:
        raise ValueError("weight must be [N, K] with N a multiple of 128; K must be contiguous in both")
    p = _lib.ProjParams()
    keep = []
    p.x, p.w = x.data_ptr(), weight.data_ptr()
    p.x_stride_l, p.w_stride_n = x.stride(0), weight.stride(0)
    p.L, p.K, p.N = L, K, N
    if (lora_t is None) != (lora_bs is None):
        raise ValueError("lora_t and lora_bs go together")
    if lora_t is not None:
        if lora_t.shape[0] != L or lora_bs.shape[0] != N or lora_t.shape[1] != lora_bs.shape[1]:
            raise ValueError("lora_t must be [L, R] and lora_bs [N, R]")
        lora_t, lora_bs = lora_t.to(torch.bfloat16).contiguous(), lora_bs.to(torch.bfloat16).contiguous()
        keep += [lora_t, lora_bs]
        p.lora_t, p.lora_bs, p.R = lora_t.data_ptr(), lora_bs.data_ptr(), lora_t.shape[1]
        p.lora_t_stride_l, p.lora_bs_stride_n = lora_t.stride(0), lora_bs.stride(0)
    if bias is not None:
        bias = bias.to(torch.float32).contiguous()
        keep.append(bias)
        p.bias = bias.data_ptr()
    if fp8 and (not prep or token_major):
        raise ValueError("fp8 output is the quantised preparation: needs prep=True and head-major output")
    p.epilogue = (_lib.PROJ_PREP_FP8 if fp8 else _lib.PROJ_PREP) if prep else _lib.PROJ_STORE
    if prep:
        if rope is not None:
            if rope.shape != (L, 64, 2) or rope.dtype != torch.float32 or not rope.is_contiguous():
                raise ValueError("rope must be a contiguous fp32 [L, 64, 2] table")
            p.rope = rope.data_ptr()
        if norm_weight is not None:
            norm_weight = norm_weight.to(torch.float32).contiguous()
            keep.append(norm_weight)
            p.norm_weight = norm_weight.data_ptr()
    p.eps = float(eps)
    p.rope_mode = _lib.ROPE_HALF if rope_half else _lib.ROPE_INTERLEAVED
    H = N // HEAD_DIM
    st_to = None
    if out_to is not None:
        if fp8 or token_major:
            raise ValueError("out_to needs the bf16 head-major epilogue")
        st_to = out_to.c_struct()
        keep.append(st_to)
        p.out_to = C.addressof(st_to)
        out = None
    elif token_major:
        out = torch.empty(L, N, dtype=torch.bfloat16, device=x.device)
        p.out, p.out_stride_l, p.out_stride_h = out.data_ptr(), N, HEAD_DIM
    else:
        out = torch.empty(H, L, HEAD_DIM, dtype=torch.uint8 if fp8 else torch.bfloat16, device=x.device)
        p.out, p.out_stride_l, p.out_stride_h = out.data_ptr(), HEAD_DIM, L * HEAD_DIM
    scale = None
    if fp8:
        scale = torch.empty(H, (L + TILE - 1) // TILE, dtype=torch.float32, device=x.device)
        p.out_scale = scale.data_ptr()
    if status_word is not None:
        p.status_word = status_word.data_ptr()
    p.wait_limit_ns = int(wait_limit_ns)
    check(lib.h3a_proj_fwd(C.byref(p), _stream()), "h3a_proj_fwd")
    if out_to is not None:
        return None
    if fp8:
        return out.permute(1, 0, 2), scale
    return out if token_major else out.permute(1, 0, 2)


def adaln_norm(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, idx: Optional[torch.Tensor] = None,
               eps: float = 1e-6, rms: bool = False, weight: Optional[torch.Tensor] = None,
               bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``norm(x) * (1 + scale[idx]) + shift[idx]`` per token row through ``h3a_adaln_norm``: ``x [L, D]`` bf16,
    ``scale`` / ``shift`` ``[T, D]`` bf16 (views with their own row stride are fine, e.g. the two chunks of one
    ``[T, 2 D]`` projection), ``idx [L]`` int64 table row per token (None: row 0 for every token)."""
    _require_cuda(x, scale, shift)
    if x.dim() != 2 or scale.dim() != 2 or shift.dim() != 2 or x.dtype != torch.bfloat16 or scale.dtype != torch.bfloat16 or shift.dtype != torch.bfloat16:
        raise ValueError("x [L, D], scale [T, D] and shift [T, D] must be 2-D bf16")
    L, D = x.shape
    if scale.shape != shift.shape or scale.shape[1] != D or x.stride(1) != 1 or scale.stride(1) != 1 or shift.stride(1) != 1:
        raise ValueError("scale and shift must be [T, D] with contiguous rows")
    p = _lib.AdaLnParams()
    keep = []
    if out is None:
        out = torch.empty(L, D, dtype=torch.bfloat16, device=x.device)
    p.x, p.y, p.scale, p.shift = x.data_ptr(), out.data_ptr(), scale.data_ptr(), shift.data_ptr()
    p.x_stride, p.y_stride, p.scale_stride, p.shift_stride = x.stride(0), out.stride(0), scale.stride(0), shift.stride(0)
    p.L, p.D, p.T = L, D, scale.shape[0]
    if idx is not None:
        if idx.shape != (L,) or idx.dtype != torch.int64 or not idx.is_cuda:
            raise ValueError("idx must be an int64 [L] device tensor")
        idx = idx.contiguous()
        keep.append(idx)
        p.idx = idx.data_ptr()
    for name, t in (("weight", weight), ("bias", bias)):
        if t is not None:
            t = t.to(torch.float32).contiguous()
            keep.append(t)
            setattr(p, name, t.data_ptr())
    p.rms, p.eps = int(bool(rms)), float(eps)
    check(_lib.load().h3a_adaln_norm(C.byref(p), _stream()), "h3a_adaln_norm")
    return out


def static_scratch_capacity() -> int:
    """Plan entries (int32) the library's built-in scratch holds: the limit on ``nnz + ceil(Lq/256)`` for
    :func:`attn_fwd_sparse_static`."""
    n = C.c_size_t(0)
    check(_lib.load().h3a_static_scratch_capacity(C.byref(n)), "h3a_static_scratch_capacity")
    return int(n.value)


def attn_fwd_sparse_static(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_index: BlockIndex,
                           out: torch.Tensor, softmax_scale: float = 0.0, status_word: Optional[torch.Tensor] = None,
                           logit_bound: float = 0.0):
    """Block-sparse attention through ``h3a_attn_fwd_sparse_static``: for hosts that may not allocate device
    memory once they are running, so the tile-plan scratch is the 1 MiB array inside the library and ``out``
    must be supplied.  This wrapper itself creates no tensor.  Calls on one device share that scratch: do not
    let two of them overlap on the GPU; make the first call on a device before any stream capture there."""
    _require_cuda(q, k, v, out)
    lib = _lib.load()
    Lq, H, qsl, qsh = _lhd(q, "q", (torch.bfloat16,))
    Lk, Hk, ksl, ksh = _lhd(k, "k", (torch.bfloat16,))
    Lv, Hv, vsl, vsh = _lhd(v, "v", (torch.bfloat16,))
    Lo, Ho, osl, osh = _lhd(out, "out", (torch.bfloat16,))
    if Hk != H or Hv != H or Ho != H or Lv != Lk or Lo != Lq:
        raise ValueError("q, k, v, out disagree on heads or lengths")
    if block_index.n_q_tiles != (Lq + TILE - 1) // TILE or block_index.n_k_tiles != (Lk + TILE - 1) // TILE:
        raise ValueError("block index does not match Lq / Lk")
    if not block_index.row_ptr.is_cuda:
        raise ValueError("block index must be on the device (BlockIndex.to(device))")
    p = AttnParams()
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.q_stride_l, p.q_stride_h = qsl, qsh
    p.k_stride_l, p.k_stride_h = ksl, ksh
    p.v_stride_l, p.v_stride_h = vsl, vsh
    p.o_stride_l, p.o_stride_h = osl, osh
    p.Lq, p.Lk, p.H, p.d, p.B = Lq, Lk, H, HEAD_DIM, 1
    p.mode = _lib.MODE_BLOCK_SPARSE
    p.softmax_scale = float(softmax_scale)
    p.row_ptr, p.col_idx, p.nnz = block_index.row_ptr.data_ptr(), block_index.col_idx.data_ptr(), block_index.nnz
    p.sparse_heavy_pairs = block_index.heavy_pairs
    p.logit_bound = float(logit_bound)
    if status_word is not None:
        p.status_word = status_word.data_ptr()
    check(lib.h3a_attn_fwd_sparse_static(C.byref(p), _stream()), "h3a_attn_fwd_sparse_static")
    return out


def read_status(status_word: torch.Tensor) -> int:
    """Synchronise the current stream and return the raw device status word (0 = no wait gave up and no block
    index failed its check)."""
    raw = C.c_int32(0)
    rc = _lib.load().h3a_read_device_status(status_word.data_ptr(), _stream(), C.byref(raw))
    if rc not in (_lib.H3A_OK, _lib.H3A_ERR_TIMEOUT, _lib.H3A_ERR_INDEX, _lib.H3A_ERR_BOUND):
        check(rc, "h3a_read_device_status")
    return raw.value


def check_status(status_word: torch.Tensor, where: str = "h3attn") -> None:
    """Synchronise the current stream and raise :class:`H3AError` (``H3A_ERR_TIMEOUT`` / ``H3A_ERR_INDEX``) when a
    kernel that was given this status word gave up a bounded wait or found a malformed block index.  The word stays
    set (every later launch given it does nothing) until the caller zeroes it."""
    raw = C.c_int32(0)
    rc = _lib.load().h3a_read_device_status(status_word.data_ptr(), _stream(), C.byref(raw))
    if rc != _lib.H3A_OK:
        raise _lib.H3AError(rc, f"{where} (device status word 0x{raw.value & 0xFFFFFFFF:x})")


class StatusWord:
    """One persistent device ``int32`` shared by all the launches of an object (a processor, a sequence-parallel
    wrapper, a host-buffer pipeline): zeroed once, handed to every kernel that has bounded waits, read with
    :meth:`check` at a point where the caller synchronises anyway (once per forward or per sampler step)."""

    def __init__(self, device=None):
        self.device = device
        self._t: Optional[torch.Tensor] = None

    def tensor(self, like: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._t is None:
            dev = self.device if self.device is not None else (like.device if like is not None else torch.device("cuda", torch.cuda.current_device()))
            self._t = torch.zeros(1, dtype=torch.int32, device=dev)
        return self._t

    def check(self, where: str = "h3attn") -> None:
        if self._t is not None:
            with torch.cuda.device(self._t.device):
                check_status(self._t, where)

    def reset(self) -> None:
        if self._t is not None:
            self._t.zero_()


def normed_logit_bound(q_weight=None, k_weight=None, softmax_scale: float = 0.0, fp8: bool = False) -> float:
    """Upper bound of ``|q.k| * scale`` after per-head RMSNorm: each prepared row has norm at most
    ``sqrt(128) * max|w|`` (Cauchy-Schwarz), so ``|q.k| <= 128 * max|w_q| * max|w_k|``.  A 2 % margin covers the
    bf16 rounding of the prepared rows, 13 % more the e4m3 rounding in FP8 mode.  Reads the weights once (a device
    synchronisation): cache the result per module."""
    wq = 1.0 if q_weight is None else float(q_weight.detach().abs().max())
    wk = 1.0 if k_weight is None else float(k_weight.detach().abs().max())
    scale = softmax_scale if softmax_scale > 0 else HEAD_DIM ** -0.5
    return HEAD_DIM * wq * wk * scale * (1.15 if fp8 else 1.02)


def joint_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    rope: Optional[torch.Tensor],
    mode: int = _lib.MODE_DENSE_BF16,
    block_index: Optional[BlockIndex] = None,
    q_weight=None,
    k_weight=None,
    eps: float = 1e-6,
    rope_half: bool = False,
    k_rope: Optional[torch.Tensor] = None,
    logit_bound: Optional[float] = None,
    **kw,
):
    """The whole hot path on one GPU: prepare Q/K (norm, rotation, optional e4m3) then attention.
    ``logit_bound`` None derives the bound from the RMSNorm weights (unit weights need no device read); pass a
    cached value to avoid the read, or 0 to force the running-maximum kernel."""
    fp8 = mode == _lib.MODE_FP8_QK
    if logit_bound is None:
        logit_bound = normed_logit_bound(q_weight, k_weight, kw.get("softmax_scale", 0.0), fp8)
    qp, kp, qs, ks = qk_prep(q, k, rope, rope if k_rope is None else k_rope, q_weight, k_weight, eps, fp8, rope_half)
    return attn_fwd(qp, kp, v, mode, qs, ks, block_index, logit_bound=logit_bound, **kw)
