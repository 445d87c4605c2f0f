"""CPU: the C-ABI library loads, exports what include/h3attn.h declares, validates arguments before
touching a device, and its host-side block-index builder agrees with the oracle."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import oracle as O
from pika_h3_flex_b200 import _lib, ops

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "h3attn.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(h3a_[a-z0-9_]+)\s*\(", src)))


def test_header_and_library_agree(lib):
    names = declared_functions()
    assert set(names) >= set(_lib.EXPORTS)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/h3attn.h but not exported"


def test_version_and_status_strings(lib):
    assert _lib.version() == (0, 2)
    seen = set()
    for code in range(0, -12, -1):
        s = _lib.status_string(code)
        assert s and s != "unknown status" and s not in seen
        seen.add(s)
    assert _lib.status_string(-99) == "unknown status"


def test_struct_sizes_match_header(lib):
    # natural-alignment sizes of the two parameter structs as a C compiler lays them out
    assert C.sizeof(_lib.AttnParams) == 216 + 8 * 8 + 8  # + the per-rank output bases of the sequence-parallel return trip
    assert C.sizeof(_lib.HeadScatter) == 8 * 8 + 8 * 4  # seven int32 fields, padded to the pointers' alignment
    assert C.sizeof(_lib.PrepParams) == 144
    assert C.sizeof(_lib.ProjParams) == 176
    assert C.sizeof(_lib.AdaLnParams) == 112


def test_struct_sizes_match_a_c_compiler(tmp_path):
    """The same three sizes from the header itself, through gcc."""
    import os
    import shutil
    import subprocess

    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "h3attn.h"\nint main(void) { printf("%zu %zu %zu %zu %zu\\n", sizeof(h3a_attn_params), '
                   'sizeof(h3a_prep_params), sizeof(h3a_proj_params), sizeof(h3a_adaln_params), sizeof(h3a_head_scatter)); return 0; }\n')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", os.path.join(root, "include"), "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()
    assert [int(v) for v in out] == [C.sizeof(_lib.AttnParams), C.sizeof(_lib.PrepParams), C.sizeof(_lib.ProjParams),
                                     C.sizeof(_lib.AdaLnParams), C.sizeof(_lib.HeadScatter)]


def test_proj_argument_validation_without_a_device(lib):
    p = _lib.ProjParams()
    assert lib.h3a_proj_fwd(C.byref(p), None) == _lib.H3A_ERR_ARG  # null pointers
    buf = (C.c_char * 4096)()
    base = (C.addressof(buf) + 255) & ~255
    p.x = p.w = p.out = base
    p.L, p.K, p.N = 128, 64, 130
    assert lib.h3a_proj_fwd(C.byref(p), None) == _lib.H3A_ERR_SHAPE  # N not a multiple of 128
    p.N, p.epilogue = 128, 5
    assert lib.h3a_proj_fwd(C.byref(p), None) == _lib.H3A_ERR_ARG  # epilogue
    p.epilogue, p.R = _lib.PROJ_STORE, 64
    assert lib.h3a_proj_fwd(C.byref(p), None) == _lib.H3A_ERR_ARG  # LoRA operands missing
    p.R = 0
    p.out_stride_l, p.out_stride_h = 100, 128
    assert lib.h3a_proj_fwd(C.byref(p), None) == _lib.H3A_ERR_ALIGN  # output stride


def test_attn_argument_validation_without_a_device(lib):
    p = _lib.AttnParams()
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_ARG  # null pointers
    buf = (C.c_char * 4096)()
    base = (C.addressof(buf) + 255) & ~255
    p.q = p.k = p.v = p.o = base
    p.Lq, p.Lk, p.H, p.d, p.B = 128, 128, 1, 64, 1
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_SHAPE  # head dim
    p.d, p.B = 128, 2
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_SHAPE  # batch
    p.B, p.mode = 1, 7
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_ARG  # mode
    p.mode = _lib.MODE_FP8_QK
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_ARG  # scales missing
    p.mode = _lib.MODE_BLOCK_SPARSE
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_ARG  # block index missing
    p.mode = _lib.MODE_DENSE_BF16
    p.o = base + 2
    p.o_stride_l = p.o_stride_h = 128
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_ALIGN
    p.o, p.o_stride_l = base, 100
    assert lib.h3a_attn_fwd(C.byref(p), None) == _lib.H3A_ERR_ALIGN
    # workspace query
    need = C.c_size_t(123)
    assert lib.h3a_attn_workspace_bytes(C.byref(p), C.byref(need)) == 0 and need.value == 0
    p.mode, p.nnz, p.Lq = _lib.MODE_BLOCK_SPARSE, 1000, 1024
    assert lib.h3a_attn_workspace_bytes(C.byref(p), C.byref(need)) == 0 and need.value == (1000 + 4) * 4


def test_prep_and_rope_argument_validation(lib):
    assert lib.h3a_qk_prep(None, None) == _lib.H3A_ERR_ARG
    p = _lib.PrepParams()
    p.d, p.H = 64, 1
    assert lib.h3a_qk_prep(C.byref(p), None) == _lib.H3A_ERR_SHAPE
    p.d, p.rope_mode = 128, 5
    assert lib.h3a_qk_prep(C.byref(p), None) == _lib.H3A_ERR_ARG
    p.rope_mode, p.flags = 0, 8
    assert lib.h3a_qk_prep(C.byref(p), None) == _lib.H3A_ERR_ARG
    split = (C.c_int32 * 3)(32, 48, 40)
    buf = (C.c_char * 256)()
    assert lib.h3a_rope_table(C.addressof(buf), 4, split, 10000.0, C.addressof(buf), None) == _lib.H3A_ERR_SHAPE
    assert lib.h3a_rope_table(None, 4, split, 10000.0, C.addressof(buf), None) == _lib.H3A_ERR_ARG


def test_torch_wrappers_refuse_cpu_tensors(lib):
    import torch

    x = torch.zeros(128, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.attn_fwd(x, x, x)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.qk_prep(x, x)


@pytest.mark.parametrize(
    "grid,n_audio,window",
    [((3, 8, 12), 0, (1, 2, 3)), ((4, 10, 20), 128, (1, 2, 3)), ((5, 8, 16), 100, (2, 8, 8)), ((6, 7, 9), 300, (0, 1, 1)),
     ((2, 16, 16), 130, (1, 0, 0))],
)
def test_block_index_builder_matches_oracle_mask(lib, grid, n_audio, window):
    keep = O.neighbourhood_block_mask(grid, n_audio, window)
    rp, ci = O.mask_to_csr(keep)
    bi = ops.build_block_index(grid, n_audio, window)
    assert np.array_equal(bi.row_ptr.numpy(), rp)
    assert np.array_equal(bi.col_idx.numpy(), ci)
    assert abs(bi.density - keep.mean()) < 1e-12


def test_block_index_at_768p_shape(lib):
    bi = ops.build_block_index((31, 48, 84), 1024, (2, 8, 8))
    assert bi.n_q_tiles == 985 and bi.nnz == int(bi.row_ptr[-1])
    assert 0.07 < bi.density < 0.075  # the literal +-2 frames, +-8 rows/cols rule
    per_row = np.diff(bi.row_ptr.numpy())
    assert per_row[:8].min() == 985 and per_row[8:].min() >= 28 and per_row[8:].max() <= 8 + 71
    # columns ascending inside each row, audio tiles in every row
    ci, rp = bi.col_idx.numpy(), bi.row_ptr.numpy()
    for r in (0, 8, 500, 984):
        row = ci[rp[r] : rp[r + 1]]
        assert (np.diff(row) > 0).all() and (row[:8] == np.arange(8)).all()
    wide = ops.build_block_index((31, 48, 84), 1024, (3, 48, 84))
    assert 0.2 < wide.density < 0.25  # the ~20 % regime: +-3 frames, whole frame spatially


def test_block_index_rejects_bad_arguments(lib):
    n = C.c_int64(0)
    assert lib.h3a_build_block_index(0, 4, 4, 0, 1, 1, 1, None, None, C.byref(n)) == _lib.H3A_ERR_SHAPE
    assert lib.h3a_build_block_index(2, 4, 4, 0, 1, 1, 1, None, None, None) == _lib.H3A_ERR_ARG
    # capacity too small on the fill call
    rp = np.zeros(2, dtype=np.int32)
    ci = np.zeros(1, dtype=np.int32)
    n = C.c_int64(0)
    assert lib.h3a_build_block_index(2, 8, 16, 0, 1, 1, 1, rp.ctypes.data, ci.ctypes.data, C.byref(n)) == _lib.H3A_ERR_WORKSPACE


def test_memcpy2d_argument_validation(lib):
    buf = (C.c_char * 64)()
    a = C.addressof(buf)
    assert lib.h3a_memcpy2d_async(None, 16, a, 16, 16, 1, 0, None) == _lib.H3A_ERR_ARG
    assert lib.h3a_memcpy2d_async(a, 8, a, 16, 16, 1, 0, None) == _lib.H3A_ERR_ARG  # width beyond the pitch
    assert lib.h3a_memcpy2d_async(a, 16, a, 16, 0, 1, 0, None) == _lib.H3A_ERR_ARG


def test_host_buffer_path_knows_when_the_copies_bound_it(lib):
    """Head groups of the host-buffer pipeline follow the ratio of copy time to compute time per head, estimated from
    the length, the mode and the mask's density: dense bf16 at the 480p-like length is bound by the kernel (0.79; 0.75
    measured), the literal block-sparse rule at the 720p-like length (7 % of the tiles) by the copies."""
    from pika_h3_flex_b200.host_path import copy_to_compute_estimate, default_head_groups

    dense = copy_to_compute_estimate(49384)
    assert 0.7 < dense < 0.9
    bi = ops.build_block_index((31, 48, 84), 1024, (2, 8, 8))
    sparse = copy_to_compute_estimate(31 * 48 * 84 + 1024, _lib.MODE_BLOCK_SPARSE, bi.density)
    assert sparse > 3.0
    assert copy_to_compute_estimate(49384, link_gbs=25.0) > 1.5  # four ranks sharing the host link
    for ratio in (dense, sparse):
        groups = default_head_groups(40, ratio)
        assert sum(groups) == 40 and min(groups) >= 1
    # bound by the copies: nothing to hide a long copy behind, so the groups stay small
    assert max(default_head_groups(40, sparse)) <= 4
