"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs.

Tolerances (bf16 modes, vs the fp32 oracle on the same bf16-rounded inputs): max-abs <= 2e-2,
mean-abs <= 2e-3, and additionally rel-L2 <= 1e-2.  FP8-QK vs the fp32 dense result: max-abs <= 3e-2,
mean-abs <= 3e-3, rel-L2 <= 6e-2 at L >= 4096; vs the oracle run on the SAME quantised operands the bf16
bounds apply.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

BF16_MAX, BF16_MEAN, BF16_REL = 2e-2, 2e-3, 1e-2
FP8_MAX, FP8_MEAN, FP8_REL = 3e-2, 3e-3, 6e-2


@pytest.fixture(scope="module")
def h(lib):
    import pika_h3_flex_b200 as pkg

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.backends.cuda.matmul.allow_tf32 = False
    return pkg


def dev(x):
    return x.to("cuda")


def check(out, ref, mx=BF16_MAX, mean=BF16_MEAN, rel=BF16_REL):
    o = out.float().cpu()
    bad = ~torch.isfinite(o)
    assert not bool(bad.any()), f"{int(bad.sum())} non-finite outputs, first at {bad.nonzero()[:4].tolist()}"
    st = O.error_stats(o, ref)
    assert st["max_abs"] <= mx and st["mean_abs"] <= mean and st["rel_l2"] <= rel, st
    return st


def bf16_inputs(L, H, seed, Lk=None):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(L, H, 128, generator=g).bfloat16()
    k = torch.randn(Lk or L, H, 128, generator=g).bfloat16()
    v = torch.randn(Lk or L, H, 128, generator=g).bfloat16()
    return q, k, v


# ------------------------------------------------------------------------------------------ preparation
def test_rope_table_matches_oracle(h):
    pos = O.make_positions((5, 6, 7), 300)
    tab = h.rope_table(dev(pos)).cpu().double()
    cos, sin = O.rope_table(pos)
    assert float((tab[..., 0] - cos).abs().max()) < 2e-7 and float((tab[..., 1] - sin).abs().max()) < 2e-7


@pytest.mark.parametrize("L,H,half,weights", [(70, 2, False, False), (300, 3, False, True), (300, 3, True, False), (129, 1, True, True)])
def test_qk_prep_bf16(h, L, H, half, weights):
    q, k, _ = bf16_inputs(L, H, 21)
    pos = O.make_positions((L // 35, 5, 7), L - (L // 35) * 35)
    cos, sin = O.rope_table(pos)
    g = torch.Generator().manual_seed(5)
    qw = (1 + 0.1 * torch.randn(128, generator=g)) if weights else None
    kw = (1 + 0.1 * torch.randn(128, generator=g)) if weights else None
    qo, ko = O.qk_prep(q.float(), k.float(), cos, sin, qw, kw, interleaved=not half)
    tab = h.rope_table(dev(pos))
    qp, kp, qs, ks = h.qk_prep(dev(q), dev(k), tab, tab, None if qw is None else dev(qw), None if kw is None else dev(kw), rope_half=half)
    assert qs is None and ks is None and qp.shape == q.shape
    # outputs are the bf16 rounding of the fp32 oracle (values up to ~4: half an ulp is 0.0078)
    for got, want in ((qp, qo), (kp, ko)):
        d = (got.float().cpu() - want).abs()
        assert float(d.max()) <= 1.6e-2 and float(d.mean()) <= 2e-3
        assert float((got.float().cpu() != want.bfloat16().float()).float().mean()) < 0.02  # rounding ties only


def test_qk_prep_strided_input_and_no_rope(h):
    L, H = 200, 4
    q, k, _ = bf16_inputs(L, H, 22)
    qkv = torch.randn(L, 3, H, 128).bfloat16()
    qkv[:, 0], qkv[:, 1] = q, k
    qkv_d = dev(qkv)
    qp, kp, _, _ = h.qk_prep(qkv_d[:, 0], qkv_d[:, 1])  # views into a fused QKV buffer, no rotation
    assert float((qp.float().cpu() - O.rms_norm(q.float())).abs().max()) <= 1.6e-2
    assert float((kp.float().cpu() - O.rms_norm(k.float())).abs().max()) <= 1.6e-2


def test_qk_prep_fp8(h):
    L, H = 300, 3
    q, k, _ = bf16_inputs(L, H, 23)
    pos = O.make_positions((8, 5, 7), 20)
    cos, sin = O.rope_table(pos)
    qo, ko = O.qk_prep(q.float(), k.float(), cos, sin)
    tab = h.rope_table(dev(pos))
    qp, kp, qs, ks = h.qk_prep(dev(q), dev(k), tab, tab, fp8=True)
    for got, sc, want in ((qp, qs, qo), (kp, ks, ko)):
        wq, ws = O.quantize_e4m3_blocks(want)
        assert float((sc.cpu() - ws).abs().max() / ws.max()) < 1e-5
        codes = got.view(torch.float8_e4m3fn).float().cpu()
        assert float((codes != wq).float().mean()) < 5e-3  # fp32 rounding of the pre-quantisation value
        assert float((codes - wq).abs().max()) <= 32.0      # never more than one code step


# ------------------------------------------------------------------------------------------ attention
@pytest.mark.parametrize(
    "L,Lk,H",
    [(128, 128, 1), (1, 1, 1), (100, 37, 2), (256, 256, 1), (300, 300, 2), (512, 512, 2), (1000, 1500, 3), (385, 129, 2), (257, 1024, 1)],
)
def test_dense_attention_shapes(h, L, Lk, H):
    q, k, v = bf16_inputs(L, H, 100 + L + Lk, Lk)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = h.attn_fwd(dev(q), dev(k), dev(v), return_lse=True, status_word=status)
    ref, ref_lse = O.attention(q.float(), k.float(), v.float(), return_lse=True)
    assert h.read_status(status) == 0
    check(out, ref, mx=3e-2 if Lk < 256 else BF16_MAX, mean=4e-3 if Lk < 256 else BF16_MEAN)
    assert float((lse.cpu().t() - ref_lse).abs().max()) < 2e-3


def test_dense_attention_head_major_views_and_out_buffer(h):
    L, H = 640, 3
    q, k, v = bf16_inputs(L, H, 31)
    qd = dev(q.permute(1, 0, 2).contiguous()).permute(1, 0, 2)
    kd = dev(k.permute(1, 0, 2).contiguous()).permute(1, 0, 2)
    out = torch.full((H, L + 2, 128), 7.0, dtype=torch.bfloat16, device="cuda")  # canary rows around the output
    h.attn_fwd(qd, kd, dev(v), out=out[:, 1 : L + 1].permute(1, 0, 2))
    check(out[:, 1 : L + 1].permute(1, 0, 2), O.attention(q.float(), k.float(), v.float()))
    assert float((out[:, 0].float() - 7).abs().max()) == 0 and float((out[:, L + 1].float() - 7).abs().max()) == 0


def test_dense_attention_large_logits_trigger_rescale(h):
    # keys ordered so that the running maximum keeps growing tile after tile
    L, H = 1024, 1
    q, k, v = bf16_inputs(L, H, 33)
    k = (k.float() * torch.linspace(0.2, 6.0, L)[:, None, None]).bfloat16()
    out = h.attn_fwd(dev(q), dev(k), dev(v))
    check(out, O.attention(q.float(), k.float(), v.float()), mx=6e-2, mean=6e-3, rel=2e-2)


def test_softmax_scale_argument(h):
    q, k, v = bf16_inputs(256, 2, 34)
    out = h.attn_fwd(dev(q), dev(k), dev(v), softmax_scale=0.05)
    check(out, O.attention(q.float(), k.float(), v.float(), scale=0.05))


@pytest.mark.parametrize("L,H", [(512, 2), (1000, 2), (130, 1)])
def test_fp8_attention_on_quantised_operands(h, L, H):
    q, k, v = bf16_inputs(L, H, 40 + L)
    qq, sq = O.quantize_e4m3_blocks(q.float())
    kq, sk = O.quantize_e4m3_blocks(k.float())
    ref = O.attention(O.dequantize_blocks(qq, sq), O.dequantize_blocks(kq, sk), v.float())
    qd = dev(qq.to(torch.float8_e4m3fn).view(torch.uint8).permute(1, 0, 2).contiguous()).permute(1, 0, 2)
    kd = dev(kq.to(torch.float8_e4m3fn).view(torch.uint8).permute(1, 0, 2).contiguous()).permute(1, 0, 2)
    out = h.attn_fwd(qd, kd, dev(v), h.MODE_FP8_QK, dev(sq), dev(sk))
    check(out, ref)


def sparse_case(grid, n_audio, window, H, seed):
    keep = O.neighbourhood_block_mask(grid, n_audio, window)
    csr = O.mask_to_csr(keep)
    L = n_audio + grid[0] * grid[1] * grid[2]
    q, k, v = bf16_inputs(L, H, seed)
    return q, k, v, csr, keep


@pytest.mark.parametrize("grid,n_audio,window", [((4, 10, 20), 128, (1, 2, 3)), ((6, 8, 16), 256, (1, 1, 2)), ((5, 9, 14), 100, (0, 2, 2))])
def test_block_sparse_attention(h, grid, n_audio, window):
    q, k, v, csr, keep = sparse_case(grid, n_audio, window, 2, 50)
    bi = h.BlockIndex.from_csr(csr[0], csr[1], keep.shape[1]).to("cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = h.attn_fwd(dev(q), dev(k), dev(v), h.MODE_BLOCK_SPARSE, block_index=bi, status_word=status)
    assert h.read_status(status) == 0
    check(out, O.attention(q.float(), k.float(), v.float(), csr=csr))
    # the library's own builder gives the same index
    bi2 = h.build_block_index(grid, n_audio, window)
    assert torch.equal(bi2.row_ptr, bi.row_ptr.cpu()) and torch.equal(bi2.col_idx, bi.col_idx.cpu())


def test_block_sparse_rows_with_disjoint_lists_and_empty_row(h):
    # hand-made index: neighbouring query tiles with different key lists, one query tile with none
    L = 5 * 128
    q, k, v = bf16_inputs(L, 1, 51)
    rows = [[0, 1, 2, 3, 4], [1], [], [0, 4], [2, 3]]
    rp = np.cumsum([0] + [len(r) for r in rows]).astype(np.int32)
    ci = np.array([c for r in rows for c in r], dtype=np.int32)
    bi = h.BlockIndex.from_csr(rp, ci, 5).to("cuda")
    out = h.attn_fwd(dev(q), dev(k), dev(v), h.MODE_BLOCK_SPARSE, block_index=bi).float().cpu()
    ref = O.attention(q.float(), k.float(), v.float(), csr=(rp, ci))
    assert float(out[256:384].abs().max()) == 0.0  # no key tile listed -> zero rows
    keep_rows = torch.cat([torch.arange(0, 256), torch.arange(384, L)])
    check(out[keep_rows], ref[keep_rows])


# ------------------------------------------------------------------------------------------ whole path
def test_joint_path_on_golden_fixture(h, golden_dir):
    g = dict(np.load(os.path.join(golden_dir, "small_joint.npz")))
    q, k, v = (torch.from_numpy(g[n]).bfloat16() for n in "qkv")
    tab = h.rope_table(dev(torch.from_numpy(g["pos"])))
    for tag, half in (("inter", False), ("half", True)):
        out = h.joint_attention(dev(q), dev(k), dev(v), tab, rope_half=half)
        check(out, torch.from_numpy(g[f"dense_{tag}"]), mx=4e-2, mean=5e-3, rel=1.5e-2)  # 96 keys: outputs ~10x larger
    out8 = h.joint_attention(dev(q), dev(k), dev(v), tab, h.MODE_FP8_QK)
    st = O.error_stats(out8.float().cpu(), torch.from_numpy(g["dense_inter"]))
    assert st["rel_l2"] <= FP8_REL


@pytest.fixture(scope="module")
def cfg0():
    grid, n_audio, H, seed = O.CONFIGS["cfg0"]
    L = n_audio + grid[0] * grid[1] * grid[2]
    q, k, v = O.seeded_qkv(L, H, seed=seed)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    pos = O.make_positions(grid, n_audio)
    ref = O.joint_attention(q.float(), k.float(), v.float(), pos, "dense")
    return q, k, v, pos, ref


def test_config0_dense(h, cfg0):
    q, k, v, pos, ref = cfg0
    out = h.joint_attention(dev(q), dev(k), dev(v), h.rope_table(dev(pos)))
    st = check(out, ref)
    assert st["rel_l2"] < 5e-3


def test_config0_fp8_within_stated_bounds(h, cfg0):
    q, k, v, pos, ref = cfg0
    out = h.joint_attention(dev(q), dev(k), dev(v), h.rope_table(dev(pos)), h.MODE_FP8_QK)
    check(out, ref, FP8_MAX, FP8_MEAN, FP8_REL)
    ref8 = O.joint_attention(q.float(), k.float(), v.float(), pos, "fp8_qk")
    check(out, ref8)  # against the oracle on quantised operands: bf16 bounds


def test_config0_block_sparse(h, cfg0):
    q, k, v, pos, _ = cfg0
    grid = O.CONFIGS["cfg0"][0]
    bi = h.build_block_index(grid, 0, (1, 8, 8))
    csr = (bi.row_ptr.numpy(), bi.col_idx.numpy())
    assert 0.3 < bi.density < 1.0
    out = h.joint_attention(dev(q), dev(k), dev(v), h.rope_table(dev(pos)), h.MODE_BLOCK_SPARSE, bi.to("cuda"))
    check(out, O.joint_attention(q.float(), k.float(), v.float(), pos, "block_sparse", csr=csr))


# ------------------------------------------------------------------------------------------ full-size properties
def _full_inputs(name, H):
    grid, n_audio, _, seed = O.CONFIGS[name]
    L = n_audio + grid[0] * grid[1] * grid[2]
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(L, H, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(L, H, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(L, H, 128, device="cuda", generator=g).bfloat16()
    return grid, n_audio, L, q, k, v


@pytest.mark.parametrize("bounded", [False, True])
def test_config1_full_length_properties(h, bounded):
    """480p-like length (49,384 tokens, tail tile of 104), 8 of the 40 heads to bound host time: with the running
    maximum (single-CTA kernel) and with the logit bound of the normalised operands (CTA pairs, split last wave)."""
    from pika_h3_flex_b200.ops import normed_logit_bound

    H = 8
    bound = normed_logit_bound() if bounded else 0.0
    grid, n_audio, L, q, k, v = _full_inputs("cfg1", H)
    pos = O.make_positions(grid, n_audio)
    tab = h.rope_table(dev(pos))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    qp, kp, _, _ = h.qk_prep(q, k, tab, tab)
    out, lse = h.attn_fwd(qp, kp, v, return_lse=True, status_word=status, logit_bound=bound)
    assert h.read_status(status) == 0
    # (1) sampled query rows against the fp64 oracle
    rows = torch.cat([torch.arange(0, L, 997), torch.tensor([L - 1, L - 104, L - 105, 1023, 1024])])
    hs = [0, H - 1]
    qo, ko = O.qk_prep(q[:, hs].cpu().double(), k[:, hs].cpu().double(), *O.rope_table(pos))
    ref = O.attention(qo, ko, v[:, hs].cpu().double(), q_rows=rows)
    check(out[rows][:, hs], ref.float())
    # (2) softmax rows sum to one: with V = 1 every output element is 1
    ones = torch.ones_like(v)
    o1 = h.attn_fwd(qp, kp, ones, logit_bound=bound)
    assert float((o1.float() - 1).abs().max()) <= 8e-3
    # (3) key order does not matter: permute K and V rows together
    perm = torch.randperm(L, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    kperm = kp.permute(1, 0, 2)[:, perm].contiguous().permute(1, 0, 2)
    o2, lse2 = h.attn_fwd(qp, kperm, v[perm].contiguous(), return_lse=True, logit_bound=bound)
    assert float((o2.float() - out.float()).abs().max()) <= 4e-3
    assert float((lse2 - lse).abs().max()) <= 1e-3
    # (4) linear in V
    o3 = h.attn_fwd(qp, kp, (2 * v).contiguous(), logit_bound=bound)
    assert float((o3.float() - 2 * out.float()).abs().max()) <= 8e-3


def test_config2_full_length_fp8(h):
    """Config 2 at its own shape: FP8-QK at the 480p-like length (49,384 tokens: 386 key tiles, tail tile of 104,
    block scales [H, 386]), 8 of the 40 heads, through joint_attention on CTA pairs with the split last wave.
    Sampled rows against (a) the fp64 oracle on the SAME e4m3-quantised operands, bf16 bounds, and (b) the fp32
    dense result of config 1, the looser FP8 bounds; V = 1 must give O = 1."""
    from pika_h3_flex_b200.ops import normed_logit_bound, split_workspace_bytes

    H = 8
    grid, n_audio, L, q, k, v = _full_inputs("cfg1", H)  # config 2 = the inputs of config 1
    assert L == 49384
    pos = O.make_positions(grid, n_audio)
    tab = h.rope_table(dev(pos))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bound = normed_logit_bound(fp8=True)
    assert split_workspace_bytes(L, L, H, h.MODE_FP8_QK, bound) > 0  # this launch splits its last wave
    out = h.joint_attention(q, k, v, tab, h.MODE_FP8_QK, status_word=status)
    assert h.read_status(status) == 0
    rows = torch.cat([torch.arange(0, L, 997), torch.tensor([L - 1, L - 104, L - 105, 1023, 1024])])
    hs = [0, H - 1]
    qo, ko = O.qk_prep(q[:, hs].cpu().double(), k[:, hs].cpu().double(), *O.rope_table(pos))
    # (a) same quantised operands: quantise the full prepared tensors (block scales need whole 128-token blocks)
    qq, sq = O.quantize_e4m3_blocks(qo.float())
    kq, sk = O.quantize_e4m3_blocks(ko.float())
    ref_q = O.attention(O.dequantize_blocks(qq, sq).double(), O.dequantize_blocks(kq, sk).double(), v[:, hs].cpu().double(), q_rows=rows)
    check(out[rows][:, hs], ref_q.float())
    # (b) the fp32 / fp64 dense result on unquantised operands
    ref_d = O.attention(qo, ko, v[:, hs].cpu().double(), q_rows=rows)
    check(out[rows][:, hs], ref_d.float(), FP8_MAX, FP8_MEAN, FP8_REL)
    # the library's own quantisation equals the oracle's on these operands (scales to fp32 rounding)
    qp, kp, qs, ks = h.qk_prep(q[:, hs].contiguous(), k[:, hs].contiguous(), tab, tab, fp8=True)
    assert tuple(qs.shape) == (2, 386) and tuple(ks.shape) == (2, 386)
    np.testing.assert_allclose(ks.cpu().numpy(), sk.numpy(), rtol=2e-2)
    o1 = h.joint_attention(q, k, torch.ones_like(v), tab, h.MODE_FP8_QK)
    assert float((o1.float() - 1).abs().max()) <= 8e-3


def test_config1_all_forty_heads(h):
    """Config 1 with all 40 heads, once: the real schedule (3,880 CTA pairs = 52.4 waves of 74, head-major order,
    split last wave at the real pair count).  Sampled rows of the first, a middle and the last head (the last head's
    query tiles are the ones the split wave covers) against the fp64 oracle; V = 1 gives O = 1 for every head."""
    H = 40
    grid, n_audio, L, q, k, v = _full_inputs("cfg1", H)
    pos = O.make_positions(grid, n_audio)
    tab = h.rope_table(dev(pos))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = h.joint_attention(q, k, v, tab, status_word=status)
    assert h.read_status(status) == 0
    rows = torch.cat([torch.arange(0, L, 1999), torch.tensor([L - 1, L - 104, L - 105, L - 513, 1023, 1024])])
    hs = [0, 17, H - 1]
    qo, ko = O.qk_prep(q[:, hs].cpu().double(), k[:, hs].cpu().double(), *O.rope_table(pos))
    ref = O.attention(qo, ko, v[:, hs].cpu().double(), q_rows=rows)
    check(out[rows][:, hs], ref.float())
    o1 = h.joint_attention(q, k, torch.ones_like(v), tab)
    assert float((o1.float() - 1).abs().max()) <= 8e-3


@pytest.mark.parametrize("L,bound", [(1024, 0.0), (1024, 12.0), (2304, 12.0)])
def test_malformed_block_index_is_reported_and_never_overruns(h, L, bound):
    """The plan kernels check the caller's index: an out-of-range column, a descending list, row pointers beyond
    nnz.  Nothing is written outside the workspace (canary words after it stay intact), the status word receives the
    index code (H3A_ERR_INDEX) and the attention launch does nothing."""
    from pika_h3_flex_b200 import _lib

    H = 1
    q, k, v = (dev(x) for x in bf16_inputs(L, H, 81))
    nb = L // 128
    good_rp = np.arange(nb + 1, dtype=np.int32) * nb
    good_ci = np.tile(np.arange(nb, dtype=np.int32), nb)
    cases = []
    ci = good_ci.copy(); ci[5] = nb + 7           # column beyond the key tiles
    cases.append((good_rp, ci))
    ci = good_ci.copy(); ci[[2, 3]] = ci[[3, 2]]   # not ascending
    cases.append((good_rp, ci))
    rp = good_rp.copy(); rp[-1] = nb * nb + 4096   # row pointer beyond nnz
    cases.append((rp, good_ci))
    rp = good_rp.copy(); rp[3] = rp[2] - 1         # decreasing row pointers
    cases.append((rp, good_ci))
    for rp, ci in cases:
        bi = h.BlockIndex(torch.from_numpy(rp).cuda(), torch.from_numpy(ci).cuda(), int(ci.size), nb, nb)
        need = (int(ci.size) + (L + 255) // 256) * 4
        ws = torch.full((need + 4096,), 0x5A, dtype=torch.uint8, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = torch.full((L, H, 128), 7.0, dtype=torch.bfloat16, device="cuda")
        h.attn_fwd(q, k, v, h.MODE_BLOCK_SPARSE, block_index=bi, out=out, status_word=status, workspace=ws[:need], logit_bound=bound)
        raw = h.read_status(status)
        assert raw & 0xFF == 10, hex(raw)
        assert h._lib.load().h3a_read_device_status(status.data_ptr(), torch.cuda.current_stream().cuda_stream, None) == _lib.H3A_ERR_INDEX
        with pytest.raises(h.H3AError):
            h.check_status(status)
        assert bool((ws[need:] == 0x5A).all())       # nothing written past the workspace
        assert bool((out == 7.0).all())              # the attention launch did nothing
    # the well-formed index still runs and the status word stays clear
    bi = h.BlockIndex(torch.from_numpy(good_rp).cuda(), torch.from_numpy(good_ci).cuda(), int(good_ci.size), nb, nb)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = h.attn_fwd(q, k, v, h.MODE_BLOCK_SPARSE, block_index=bi, status_word=status, logit_bound=bound)
    assert h.read_status(status) == 0
    check(out, O.attention(q.float().cpu(), k.float().cpu(), v.float().cpu()))


@pytest.mark.parametrize("window,bounded", [((2, 8, 8), False), ((2, 8, 8), True), ((3, 48, 84), True)])
def test_config3_full_length_block_sparse_properties(h, window, bounded):
    """768p-like length (126,016 tokens), 2 heads: the literal neighbourhood rule (7.2 % of tiles) with the running
    maximum and with the logit bound (single-CTA kernels), and the +-3 frames x whole frame rule (22.7 %) with the
    bound (CTA pairs, merged plans per four query tiles)."""
    from pika_h3_flex_b200.ops import normed_logit_bound

    H = 2
    bound = normed_logit_bound() if bounded else 0.0
    grid, n_audio, L, q, k, v = _full_inputs("cfg3", H)
    bi = h.build_block_index(grid, n_audio, window)
    bid = bi.to("cuda")
    pos = O.make_positions(grid, n_audio)
    tab = h.rope_table(dev(pos))
    qp, kp, _, _ = h.qk_prep(q, k, tab, tab)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = h.attn_fwd(qp, kp, v, h.MODE_BLOCK_SPARSE, block_index=bid, status_word=status, logit_bound=bound)
    assert h.read_status(status) == 0
    rows = torch.cat([torch.arange(0, L, 4099), torch.tensor([L - 1, 1023, 1024, 1151, 1152])])
    qo, ko = O.qk_prep(q.cpu().double(), k.cpu().double(), *O.rope_table(pos))
    ref = O.attention(qo, ko, v.cpu().double(), csr=(bi.row_ptr.numpy(), bi.col_idx.numpy()), q_rows=rows)
    check(out[rows], ref.float(), mx=3e-2, mean=3e-3)
    o1 = h.attn_fwd(qp, kp, torch.ones_like(v), h.MODE_BLOCK_SPARSE, block_index=bid, logit_bound=bound)
    assert float((o1.float() - 1).abs().max()) <= 8e-3


# ------------------------------------------------------------------------------------------ errors
def test_errors_are_reported_not_swallowed(h):
    q, k, v = (dev(x) for x in bf16_inputs(256, 2, 60))
    with pytest.raises(ValueError):
        h.attn_fwd(q, k[:, :1], v)
    with pytest.raises(h.H3AError) as e:
        big = torch.zeros(256 * 260 + 512, dtype=torch.bfloat16, device="cuda")
        h.attn_fwd(big.as_strided((256, 2, 128), (260, 130, 1)), k, v)  # strides not multiples of 16 bytes
    assert e.value.status == h._lib.H3A_ERR_ALIGN
    with pytest.raises(ValueError):
        h.attn_fwd(q, k, v, h.MODE_BLOCK_SPARSE)
    with pytest.raises((TypeError, ValueError)):
        h.attn_fwd(q, k, v, h.MODE_FP8_QK)  # bf16 operands and no scales


# ------------------------------------------------------------------------------------------ host-buffer path
@pytest.mark.parametrize("mode_name,groups", [("dense", None), ("dense", [1, 2, 2]), ("fp8_qk", [5]), ("block_sparse", [2, 3])])
def test_host_buffer_path_pipelined_over_head_groups(h, mode_name, groups):
    grid, n_audio, H = (4, 8, 12), 100, 5
    pos = O.make_positions(grid, n_audio)
    L = pos.shape[0]
    q, k, v = bf16_inputs(L, H, 90)
    csr, bi, mode = None, None, h.MODE_DENSE_BF16
    if mode_name == "block_sparse":
        bih = h.build_block_index(grid, n_audio, (1, 2, 2))
        csr, bi, mode = (bih.row_ptr.numpy(), bih.col_idx.numpy()), bih.to("cuda"), h.MODE_BLOCK_SPARSE
    elif mode_name == "fp8_qk":
        mode = h.MODE_FP8_QK
    ref = O.joint_attention(q.float(), k.float(), v.float(), pos, mode_name, csr=csr)
    host = h.HostJointAttention(L, H, mode, bi, head_groups=groups)
    hq, hk, hv = (t.contiguous().pin_memory() for t in (q, k, v))
    ho = torch.full((L, H, 128), 9.0, dtype=torch.bfloat16).pin_memory()
    tab = h.rope_table(dev(pos))
    for _ in range(2):  # second call reuses the staging buffers and streams
        ho.fill_(9.0)
        host(hq, hk, hv, tab, ho)
        torch.cuda.current_stream().synchronize()
        if mode_name == "fp8_qk":
            assert O.error_stats(ho.float(), ref)["rel_l2"] <= FP8_REL
        else:
            check(ho, ref, mx=3e-2, mean=3e-3)
    with pytest.raises(ValueError):
        host(q, hk, hv, tab, ho)  # not pinned


# ------------------------------------------------------------------------------------------ fixed softmax reference
@pytest.mark.parametrize("L,Lk,H", [(300, 300, 2), (1000, 1500, 3), (129, 64, 1)])
def test_fixed_logit_bound_gives_the_same_softmax(h, L, Lk, H):
    q, k, v = bf16_inputs(L, H, 300 + L, Lk)
    ref, ref_lse = O.attention(q.float(), k.float(), v.float(), return_lse=True)
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) / 128 ** 0.5
    true_bound = float(s.abs().max())
    # tight; the largest bound that is its own reference; the sliding-reference range up to its end; too small (still exact)
    for bound in (true_bound * 1.05, 30.0, 45.0, 60.0, true_bound * 0.5):
        out, lse = h.attn_fwd(dev(q), dev(k), dev(v), return_lse=True, logit_bound=bound)
        check(out, ref, mx=3e-2 if Lk < 256 else BF16_MAX, mean=4e-3 if Lk < 256 else BF16_MEAN)
        assert float((lse.cpu().t() - ref_lse).abs().max()) < 2e-3
    out = h.attn_fwd(dev(q), dev(k), dev(v), logit_bound=1e6)  # unusable bound: falls back to the running maximum
    check(out, ref, mx=3e-2 if Lk < 256 else BF16_MAX, mean=4e-3 if Lk < 256 else BF16_MEAN)


@pytest.mark.parametrize("L,Lk,H", [(512, 1024, 2), (1000, 2304, 2)])
def test_large_logits_inside_the_sliding_reference_range(h, L, Lk, H):
    """Logits spread over +-50 (operands scaled up): a bound of 55 uses the sliding reference (60 - B = 5), on the
    single-CTA kernel (8 key tiles) and on CTA pairs (18); rows keep full accuracy although their maxima differ by
    tens of units, and the online kernels agree."""
    g = torch.Generator().manual_seed(17)
    q = (3.0 * torch.randn(L, H, 128, generator=g)).bfloat16()
    k = (3.0 * torch.randn(Lk, H, 128, generator=g)).bfloat16()
    v = torch.randn(Lk, H, 128, generator=g).bfloat16()
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float()) / 128 ** 0.5
    assert 30.0 < float(s.abs().max()) < 55.0
    ref = O.attention(q.double(), k.double(), v.double()).float()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for bound in (55.0, 0.0):
        ch = h.ops.kernel_choice(L, Lk, H, logit_bound=bound)
        assert ch["fixed_reference"] == (bound > 0) and ch["cta_pairs"] == (Lk >= 2048)
        out = h.attn_fwd(dev(q), dev(k), dev(v), logit_bound=bound, status_word=status)
        assert h.read_status(status) == 0
        check(out, ref, mx=4e-2, mean=3e-3, rel=1.5e-2)  # peaked rows: the output is close to single V rows, |v| up to 4


@pytest.mark.parametrize("Lk", [1024, 2304])
def test_a_logit_bound_that_does_not_hold_is_reported(h, Lk):
    """Operands far outside a stated bound of 12 (logits of several hundred): exponentials overflow, the row sums are
    infinite, and the launch says so through the status word (H3A_ERR_BOUND) instead of handing back garbage silently;
    the same data with no bound (online softmax) is fine."""
    from pika_h3_flex_b200 import _lib

    L, H = 512, 2
    g = torch.Generator().manual_seed(18)
    q = (8 * torch.randn(L, H, 128, generator=g)).bfloat16()
    k = (8 * torch.randn(Lk, H, 128, generator=g)).bfloat16()
    v = torch.randn(Lk, H, 128, generator=g).bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    h.attn_fwd(dev(q), dev(k), dev(v), logit_bound=12.0, status_word=status)
    assert h.read_status(status) & 0xFF == 11
    with pytest.raises(h.H3AError) as ei:
        h.check_status(status)
    assert ei.value.status == _lib.H3A_ERR_BOUND
    status.zero_()
    out = h.attn_fwd(dev(q), dev(k), dev(v), logit_bound=0.0, status_word=status)
    assert h.read_status(status) == 0
    check(out, O.attention(q.double(), k.double(), v.double()).float(), mx=5e-2, mean=4e-3, rel=2e-2)


@pytest.mark.parametrize("Lk", [1024, 2304])
def test_rows_below_the_range_of_a_large_bound_are_reported(h, Lk):
    """A bound of 104 that HOLDS (|logit| <= 104), but a block of query rows is strongly anti-aligned with every key
    (all their logits near -57, far below the line B - 138 = -34 the reference serves): their terms fall under fp32's range,
    which shows in the row sum and is reported (H3A_ERR_BOUND) instead of being returned as garbage; without those rows
    the same launch is clean and exact, and the online softmax serves all rows."""
    L, H = 512, 1
    g = torch.Generator().manual_seed(19)
    u = torch.zeros(128)
    u[0] = 1.0
    k = (0.5 * torch.randn(Lk, H, 128, generator=g) + 16.0 * u).bfloat16()
    q = (1.5 * torch.randn(L, H, 128, generator=g)).bfloat16()
    v = torch.randn(Lk, H, 128, generator=g).bfloat16()
    q_bad = q.clone()
    q_bad[128:256] = (-40.0 * u + 0.5 * torch.randn(128, H, 128, generator=g)).bfloat16()
    s = torch.einsum("qhd,khd->hqk", q_bad.float(), k.float()) / 128 ** 0.5
    assert float(s.abs().max()) < 104.0 and float(s[:, 128:256].max()) < -45.0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = h.attn_fwd(dev(q), dev(k), dev(v), logit_bound=104.0, status_word=status)
    assert h.read_status(status) == 0
    check(out, O.attention(q.double(), k.double(), v.double()).float(), mx=4e-2, mean=3e-3, rel=1.5e-2)
    h.attn_fwd(dev(q_bad), dev(k), dev(v), logit_bound=104.0, status_word=status)
    assert h.read_status(status) & 0xFF == 11
    status.zero_()
    out = h.attn_fwd(dev(q_bad), dev(k), dev(v), logit_bound=0.0, status_word=status)
    assert h.read_status(status) == 0
    check(out, O.attention(q_bad.double(), k.double(), v.double()).float(), mx=4e-2, mean=3e-3, rel=1.5e-2)


def test_online_softmax_in_two_launches(h):
    """No logit bound, 18 key tiles: the launch is the fixed-reference kernel with a per-row reference from the first key
    tile, followed by the running-maximum kernel over the CTA pairs that put themselves on the redo list.  Ordinary data
    redoes nothing; rows whose later logits outgrow the first tile's maximum by more than 2^60 (here by about 49 in
    natural units) are redone and come out exact; with a workspace too small for the list the launch is the
    running-maximum kernel alone, and both agree with the oracle."""
    L, Lk, H = 1024, 2304, 2
    g = torch.Generator().manual_seed(21)
    q = torch.randn(L, H, 128, generator=g).bfloat16()
    k = torch.randn(Lk, H, 128, generator=g).bfloat16()
    v = torch.randn(Lk, H, 128, generator=g).bfloat16()
    need = h.ops.split_workspace_bytes(L, Lk, H)
    assert need >= 4 * (4 + 2 * H)
    ch = h.ops.kernel_choice(L, Lk, H, workspace_bytes=need)
    assert ch["cta_pairs"] and not ch["fixed_reference"] and ch["online_two_launch"]
    assert not h.ops.kernel_choice(L, Lk, H, workspace_bytes=16)["online_two_launch"]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = O.attention(q.double(), k.double(), v.double()).float()
    ws = torch.full((need,), 0x77, dtype=torch.uint8, device="cuda")
    out, lse = h.attn_fwd(dev(q), dev(k), dev(v), workspace=ws, status_word=status, return_lse=True)
    assert h.read_status(status) == 0 and int(ws.view(torch.int32)[0]) == 0  # nothing to redo
    check(out, ref)
    lse_ref = O.attention(q.double(), k.double(), v.double(), return_lse=True)[1]
    assert float((lse.cpu().t().double() - lse_ref).abs().max()) < 2e-3
    single = h.attn_fwd(dev(q), dev(k), dev(v), workspace=torch.empty(16, dtype=torch.uint8, device="cuda"), status_word=status)
    check(single, ref)
    # rows 256..383 of both heads: tiny logits against the first key tile, then a handful of keys 49 above
    u = torch.zeros(128)
    u[5] = 1.0
    q2, k2 = q.clone(), k.clone()
    q2[256:384] = (24.0 * u + 0.3 * torch.randn(128, H, 128, generator=g)).bfloat16()
    k2[:128] = (0.3 * torch.randn(128, H, 128, generator=g)).bfloat16()
    k2[1000:1010] = (24.0 * u + 0.3 * torch.randn(10, H, 128, generator=g)).bfloat16()
    s = torch.einsum("qhd,khd->hqk", q2.float(), k2.float()) / 128 ** 0.5
    assert float((s[:, 256:384, 1000:1010].amax(-1) - s[:, 256:384, :128].amax(-1)).min()) > 45.0
    ref2 = O.attention(q2.double(), k2.double(), v.double()).float()
    ws.fill_(0x77)
    out2 = h.attn_fwd(dev(q2), dev(k2), dev(v), workspace=ws, status_word=status)
    assert h.read_status(status) == 0
    words = ws.view(torch.int32)
    assert int(words[0]) == H and sorted(words[4 : 4 + H].tolist()) == [0, 2]  # pair 0 (rows 0..511) of each head: pairs 0 and 2
    check(out2, ref2, mx=4e-2, mean=3e-3, rel=1.5e-2)
    single2 = h.attn_fwd(dev(q2), dev(k2), dev(v), workspace=torch.empty(16, dtype=torch.uint8, device="cuda"), status_word=status)
    check(single2, ref2, mx=4e-2, mean=3e-3, rel=1.5e-2)


def test_joint_path_bound_from_norm_weights(h):
    L, H = 700, 2
    q, k, v = bf16_inputs(L, H, 77)
    g = torch.Generator().manual_seed(6)
    qw, kw = 1 + 0.3 * torch.randn(128, generator=g), 1 + 0.3 * torch.randn(128, generator=g)
    pos = O.make_positions((4, 10, 15), 100)
    ref = O.joint_attention(q.float(), k.float(), v.float(), pos, "dense", q_weight=qw, k_weight=kw)
    tab = h.rope_table(dev(pos))
    from pika_h3_flex_b200.ops import normed_logit_bound
    b = normed_logit_bound(qw, kw)
    assert abs(b - 128 * float(qw.abs().max()) * float(kw.abs().max()) / 128 ** 0.5 * 1.02) < 1e-4
    for lb in (None, 0.0):  # derived bound / running maximum
        out = h.joint_attention(dev(q), dev(k), dev(v), tab, q_weight=dev(qw), k_weight=dev(kw), logit_bound=lb)
        check(out, ref)


# ------------------------------------------------------------------------------------------ config 4: cross-attention
def test_config4_cross_attention_shape(h):
    """49,384 joint tokens attend to 512 text tokens (config 4), 4 of the 40 heads, QK-RMSNorm without rotation."""
    Lq, Lk, H = 49384, 512, 4
    g = torch.Generator(device="cuda").manual_seed(1004)
    q = torch.randn(Lq, H, 128, device="cuda", generator=g).bfloat16()
    k = torch.randn(Lk, H, 128, device="cuda", generator=g).bfloat16()
    v = torch.randn(Lk, H, 128, device="cuda", generator=g).bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = h.joint_attention(q, k, v, None, status_word=status)
    assert h.read_status(status) == 0
    rows = torch.cat([torch.arange(0, Lq, 613), torch.tensor([Lq - 1, Lq - 104, Lq - 105])])
    qn, kn = O.rms_norm(q[rows].float().cpu()), O.rms_norm(k.float().cpu())
    check(out[rows], O.attention(qn, kn, v.float().cpu()))
    o1 = h.joint_attention(q, k, torch.ones_like(v), None)
    assert float((o1.float() - 1).abs().max()) <= 8e-3


# ------------------------------------------------------------------------------------------ persistent CTAs
_PERSIST_CASES = [  # (Lq, Lk, heads, fp8): more (head, query-tile group) items than SMs, the last pair of a head half empty
    (15360, 640, 6, False),   # 360 items of 5 key tiles: the 5-stage K/V ring wraps inside and across items
    (10000, 552, 5, False),   # 79 query tiles: every head ends on a pair with one tile; key tail of 40
    (8192, 1024, 8, True),    # FP8-QK below the CTA-pair threshold
    # at most 4 key tiles: K / V resident in a persistent CTA pair, which changes head a few times
    (20000, 512, 4, False),   # 160 groups of four query tiles on 74 pairs; the last group of a head is short
    (16000, 300, 5, False),   # 3 key tiles, the last with 44 keys
    (33000, 100, 3, False),   # one key tile with a tail
    (9000, 130, 9, False),    # 2 key tiles, the second nearly empty
]
_PERSIST_CHILD = r"""
import sys, torch
sys.path.insert(0, %(root)r)
import pika_h3_flex_b200 as h
outs = []
for i, (Lq, Lk, H, fp8) in enumerate(%(cases)r):
    g = torch.Generator().manual_seed(500 + i)
    q = torch.randn(Lq, H, 128, generator=g).bfloat16().cuda()
    k = torch.randn(Lk, H, 128, generator=g).bfloat16().cuda()
    v = torch.randn(Lk, H, 128, generator=g).bfloat16().cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = h.joint_attention(q, k, v, None, mode=h.MODE_FP8_QK if fp8 else h.MODE_DENSE_BF16, status_word=status)
    assert h.read_status(status) == 0
    outs.append(out.cpu())
torch.save(outs, %(path)r)
"""


def test_persistent_ctas_give_the_same_rows_as_one_cta_per_item(h, tmp_path):
    """Fixed softmax reference with few key tiles per item (cross-attention shapes): by default the CTAs are persistent -
    one CTA per SM walks the items of the single-CTA kernel, and with at most 4 key tiles a CTA pair keeps a head's K / V
    in shared memory.  H3A_PERSIST=0 H3A_RESIDENT=0 (read once per process, so a child process runs it) launches one
    single-CTA block per item.  The single-CTA kernel does the same arithmetic per row in the same order either way
    (bit-identical outputs); the pair kernel agrees to rounding; all match the oracle on sampled rows."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = tmp_path / "per_item.pt"
    code = _PERSIST_CHILD % {"root": root, "cases": _PERSIST_CASES, "path": str(path)}
    subprocess.run([sys.executable, "-c", code], check=True, env=dict(os.environ, H3A_PERSIST="0", H3A_RESIDENT="0"), timeout=300)
    per_item = torch.load(path)
    for i, (Lq, Lk, H, fp8) in enumerate(_PERSIST_CASES):
        g = torch.Generator().manual_seed(500 + i)
        q = torch.randn(Lq, H, 128, generator=g).bfloat16()
        k = torch.randn(Lk, H, 128, generator=g).bfloat16()
        v = torch.randn(Lk, H, 128, generator=g).bfloat16()
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = h.joint_attention(dev(q), dev(k), dev(v), None, mode=h.MODE_FP8_QK if fp8 else h.MODE_DENSE_BF16, status_word=status)
        assert h.read_status(status) == 0
        ch = h.ops.kernel_choice(Lq, Lk, H, h.MODE_FP8_QK if fp8 else h.MODE_DENSE_BF16, logit_bound=11.4)
        assert ch["persistent"] and ch["fixed_reference"] and ch["cta_pairs"] == (Lk <= 512 and not fp8), ch
        if Lk > 512:  # the same kernel, persistent or not: the same arithmetic in the same order
            assert torch.equal(out.cpu(), per_item[i]), (Lq, Lk, H, fp8)
        else:         # CTA pairs with resident K / V against the single-CTA kernel: another MMA shape, and a quarter of the
            # exponentials on the polynomial there against none here: an output may differ by one bf16 step (2^-8 of its size)
            want = per_item[i].float()
            d = (out.cpu().float() - want).abs()
            assert bool((d <= 2.0 ** -6 * want.abs().clamp_min(0.25)).all()) and float(d.mean()) <= 1e-4, (Lq, Lk, H, float(d.max()), float(d.mean()))  # a step either side of a power of two
        rows = torch.cat([torch.arange(0, Lq, 397), torch.tensor([Lq - 1, Lq - 129, 255, 256, 511, 512])])
        ref = O.attention(O.rms_norm(q[rows].float()), O.rms_norm(k.float()), v.float())
        if fp8:
            check(out[rows], ref, mx=FP8_MAX, mean=FP8_MEAN, rel=FP8_REL)
        else:
            check(out[rows], ref)
        o1 = h.joint_attention(dev(q), dev(k), torch.ones_like(dev(v)), None, mode=h.MODE_FP8_QK if fp8 else h.MODE_DENSE_BF16)
        assert float((o1.float() - 1).abs().max()) <= 8e-3


def test_persistent_ctas_on_block_sparse_lists(h, tmp_path):
    """Block-sparse launches keep one CTA per item by default; H3A_PERSIST=1 makes them persistent too (items of very
    different length, and items that list nothing).  Same rows, bit for bit."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = tmp_path / "persistent.pt"
    grid, n_audio, H, window = (24, 20, 30), 256, 3, (1, 2, 3)  # 58 pairs of query tiles x 3 heads, below 12 % density
    code = (
        "import sys, torch; sys.path.insert(0, %r)\n"
        "import pika_h3_flex_b200 as h\n"
        "bi = h.build_block_index(%r, %r, %r).to('cuda')\n"
        "L = %d\n"
        "g = torch.Generator().manual_seed(91)\n"
        "q, k, v = (torch.randn(L, %d, 128, generator=g).bfloat16().cuda() for _ in range(3))\n"
        "st = torch.zeros(1, dtype=torch.int32, device='cuda')\n"
        "out = h.attn_fwd(q, k, v, mode=h.MODE_BLOCK_SPARSE, block_index=bi, logit_bound=%r, status_word=st)\n"
        "assert h.read_status(st) == 0\n"
        "torch.save(out.cpu(), %r)\n" % (root, grid, n_audio, window, grid[0] * grid[1] * grid[2] + n_audio, H, PAIR_BOUND, str(path))
    )
    subprocess.run([sys.executable, "-c", code], check=True, env=dict(os.environ, H3A_PERSIST="1"), timeout=300)
    bih = h.build_block_index(grid, n_audio, window)
    nqb = bih.row_ptr.numel() - 1
    assert bih.col_idx.numel() < 0.12 * nqb * nqb  # the single-CTA kernel's range
    bi = bih.to("cuda")
    L = grid[0] * grid[1] * grid[2] + n_audio
    g = torch.Generator().manual_seed(91)
    q, k, v = (torch.randn(L, H, 128, generator=g).bfloat16().cuda() for _ in range(3))
    out = h.attn_fwd(q, k, v, mode=h.MODE_BLOCK_SPARSE, block_index=bi, logit_bound=PAIR_BOUND)
    assert torch.equal(out.cpu(), torch.load(path))


# ------------------------------------------------------------------------------------------ bounded waits
def test_wait_that_nothing_signals_runs_out_and_is_reported(h):
    """The bounded wait of the attention kernels, on a barrier nothing ever signals: it must give up after the
    limit, report through the status word (code 9) and leave the context usable - no trap, no hang."""
    import time

    lib = h._lib.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert lib.h3a_selftest_wait_timeout(status.data_ptr(), 20_000_000, stream) == 0  # 20 ms
    raw = h.read_status(status)
    dt = time.perf_counter() - t0
    assert (raw & 0xFF) == 9, hex(raw)
    assert 0.015 < dt < 5.0, dt
    assert lib.h3a_read_device_status(status.data_ptr(), stream, None) == h._lib.H3A_ERR_TIMEOUT
    assert lib.h3a_selftest_wait_timeout(status.data_ptr(), 0, stream) == h._lib.H3A_ERR_ARG
    # the context is still usable and a normal call reports no timeout
    q, k, v = (dev(x) for x in bf16_inputs(512, 2, 124))
    status.zero_()
    out = h.attn_fwd(q, k, v, status_word=status)
    assert h.read_status(status) == 0
    check(out, O.attention(q.float().cpu(), k.float().cpu(), v.float().cpu()))
    # a status word that is already non-zero makes a launch return at once without touching the output
    status.fill_(5)
    canary = torch.full_like(out, 3.0)
    h.attn_fwd(q, k, v, out=canary, status_word=status)
    torch.cuda.synchronize()
    assert float((canary.float() - 3).abs().max()) == 0.0


def test_sparse_heavy_first_schedule_does_not_change_results(h):
    q, k, v, csr, keep = sparse_case((6, 8, 16), 256, (1, 1, 2), 3, 52)
    bi = h.BlockIndex.from_csr(csr[0], csr[1], keep.shape[1]).to("cuda")
    assert bi.heavy_pairs in (0, 1)  # the two audio tiles form one dense leading pair
    outs = []
    for hint in (0, 1, 2, 3):
        bi.heavy_pairs = hint
        outs.append(h.attn_fwd(dev(q), dev(k), dev(v), h.MODE_BLOCK_SPARSE, block_index=bi))
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    check(outs[0], O.attention(q.float(), k.float(), v.float(), csr=csr))


def test_repeated_sparse_launches_with_uneven_streams_stay_finite(h, cfg0):
    """Regression: query-tile pairs whose two key lists differ in length let one warpgroup of a stream run ahead
    of its partner; the end-of-CTA exchange of row sums must wait for the stream's own last MMA (a one-in-ten
    race otherwise).  Forty launches on a poisoned output buffer, bit-identical every time."""
    q, k, v, pos, _ = cfg0
    bi = h.build_block_index(O.CONFIGS["cfg0"][0], 0, (1, 8, 8)).to("cuda")
    qp, kp, _, _ = h.qk_prep(dev(q), dev(k), h.rope_table(dev(pos)), h.rope_table(dev(pos)))
    vd = dev(v)
    from pika_h3_flex_b200.ops import normed_logit_bound
    first = None
    for _ in range(40):
        out = torch.full((q.shape[0], q.shape[1], 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        h.attn_fwd(qp, kp, vd, h.MODE_BLOCK_SPARSE, block_index=bi, out=out, logit_bound=normed_logit_bound())
        assert bool(torch.isfinite(out.float()).all())
        first = out if first is None else first
        assert torch.equal(out, first)


# ------------------------------------------------------------------------------------------ CTA-pair kernel
# Attention with a fixed softmax reference over at least 16 key tiles runs on pairs of CTAs (one MMA of 256 rows per
# pair).  The cases cover: one pair with its second CTA partly or wholly beyond the last query row, ragged key
# tails, several pairs per head, several heads, and the FP8 operands.
PAIR_BOUND = 14.0  # |q.k|/sqrt(128) of unit-normal rows stays far below this


@pytest.mark.parametrize("L,Lk,H", [(512, 2048, 1), (256, 2100, 1), (257, 1921, 2), (700, 2500, 3), (1536, 2048, 2), (4096, 4096, 4)])
def test_pair_kernel_dense_shapes(h, L, Lk, H):
    q, k, v = bf16_inputs(L, H, 900 + L + Lk, Lk)
    ref, ref_lse = O.attention(q.float(), k.float(), v.float(), return_lse=True)
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = h.attn_fwd(dev(q), dev(k), dev(v), return_lse=True, logit_bound=PAIR_BOUND, status_word=st)
    assert h.read_status(st) == 0
    check(out, ref, mx=3e-2 if Lk < 256 else BF16_MAX, mean=4e-3 if Lk < 256 else BF16_MEAN)
    assert float((lse.cpu().t() - ref_lse).abs().max()) < 2e-3


@pytest.mark.parametrize("L,H", [(512, 2), (1000, 2), (130, 1)])
def test_pair_kernel_fp8(h, L, H):
    q, k, v = bf16_inputs(L, H, 950 + L, 2304 - L % 7)
    qq, sq = O.quantize_e4m3_blocks(q.float())
    kq, sk = O.quantize_e4m3_blocks(k.float())
    ref = O.attention(O.dequantize_blocks(qq, sq), O.dequantize_blocks(kq, sk), v.float())
    to_dev = lambda x: dev(x.to(torch.float8_e4m3fn).view(torch.uint8).permute(1, 0, 2).contiguous()).permute(1, 0, 2)
    out = h.attn_fwd(to_dev(qq), to_dev(kq), dev(v), h.MODE_FP8_QK, dev(sq), dev(sk), logit_bound=PAIR_BOUND)
    check(out, ref, mx=3e-2 if L < 256 else BF16_MAX, mean=4e-3 if L < 256 else BF16_MEAN)


def test_pair_kernel_agrees_with_single_cta_kernel(h, tmp_path):
    """The same seeded case through the single-CTA kernel (H3A_PAIR=0 is read once per process, so a child
    process runs it): both kernels do the same arithmetic per row in the same order."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = tmp_path / "single.pt"
    code = (
        "import sys, torch; sys.path.insert(0, %r)\n"
        "import pika_h3_flex_b200 as h\n"
        "g = torch.Generator().manual_seed(77)\n"
        "q, k, v = (torch.randn(2200, 3, 128, generator=g).bfloat16().cuda() for _ in range(3))\n"
        "torch.save(h.attn_fwd(q, k, v, logit_bound=%r).cpu(), %r)\n" % (root, PAIR_BOUND, str(path))
    )
    env = dict(os.environ, H3A_PAIR="0")
    subprocess.run([sys.executable, "-c", code], check=True, env=env, timeout=300)
    g = torch.Generator().manual_seed(77)
    q, k, v = (torch.randn(2200, 3, 128, generator=g).bfloat16().cuda() for _ in range(3))
    out = h.attn_fwd(q, k, v, logit_bound=PAIR_BOUND).cpu()
    single = torch.load(path)
    assert float((out.float() - single.float()).abs().max()) <= 1e-3
    check(out, O.attention(q.float().cpu(), k.float().cpu(), v.float().cpu()))


def test_pair_kernel_skips_work_when_the_status_word_is_already_set(h):
    """A launch whose status word already holds an error does nothing: every pair reads rank 0's verdict,
    passes both cluster barriers and returns without touching TMEM or the output."""
    q, k, v = bf16_inputs(1024, 2, 970, 2048)
    st = torch.full((1,), 0x105, dtype=torch.int32, device="cuda")
    out = torch.full((1024, 2, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    h.attn_fwd(dev(q), dev(k), dev(v), out=out, logit_bound=PAIR_BOUND, status_word=st)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
    assert int(st.item()) == 0x105
    st.zero_()
    h.attn_fwd(dev(q), dev(k), dev(v), out=out, logit_bound=PAIR_BOUND, status_word=st)  # the context is still usable
    assert h.read_status(st) == 0
    check(out, O.attention(q.float(), k.float(), v.float()))


@pytest.mark.parametrize("Lq,Lk,H", [(20000, 512, 4), (15360, 640, 6)])
def test_persistent_kernels_skip_work_when_the_status_word_is_already_set(h, Lq, Lk, H):
    """The same for the persistent forms (CTA pairs with resident K / V; one single-CTA block per SM): every block leaves
    before it touches TMEM or the output, and the next launch on a cleared word is complete."""
    g = torch.Generator().manual_seed(971)
    q = torch.randn(Lq, H, 128, generator=g).bfloat16()
    k = torch.randn(Lk, H, 128, generator=g).bfloat16()
    v = torch.randn(Lk, H, 128, generator=g).bfloat16()
    st = torch.full((1,), 0x105, dtype=torch.int32, device="cuda")
    out = torch.full((Lq, H, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    h.attn_fwd(dev(q), dev(k), dev(v), out=out, logit_bound=PAIR_BOUND, status_word=st)
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
    assert int(st.item()) == 0x105
    st.zero_()
    h.attn_fwd(dev(q), dev(k), dev(v), out=out, logit_bound=PAIR_BOUND, status_word=st)
    assert h.read_status(st) == 0
    rows = torch.cat([torch.arange(0, Lq, 509), torch.tensor([Lq - 1])])
    check(out[rows], O.attention(q[rows].float(), k.float(), v.float()))
    out2, lse = h.attn_fwd(dev(q), dev(k), dev(v), logit_bound=PAIR_BOUND, return_lse=True)  # the log-sum-exp of the persistent forms
    assert torch.equal(out2, out)
    sc = (q[rows].float().transpose(0, 1) @ k.float().transpose(0, 1).transpose(1, 2)) / 128 ** 0.5  # [H, rows, Lk]
    assert float((lse[:, rows].cpu() - torch.logsumexp(sc, dim=-1)).abs().max()) <= 2e-3


def test_pair_kernel_repeated_launches_are_bit_identical(h):
    q, k, v = bf16_inputs(2304, 4, 980, 3000)
    qd, kd, vd = dev(q), dev(k), dev(v)
    first = None
    for _ in range(30):
        out = torch.full((2304, 4, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        h.attn_fwd(qd, kd, vd, out=out, logit_bound=PAIR_BOUND)
        assert bool(torch.isfinite(out.float()).all())
        first = out if first is None else first
        assert torch.equal(out, first)
    check(first, O.attention(q.float(), k.float(), v.float()))


def _ring_rows(n, width, empty, long_row=None):
    """n query tiles over n key tiles: tile i keeps `width` key tiles starting at 3 i (mod n); the tiles in `empty`
    keep none; `long_row` keeps every second key tile."""
    rows = [sorted({(3 * i + j) % n for j in range(width)}) for i in range(n)]
    for i in empty:
        rows[i] = []
    if long_row is not None:
        rows[long_row] = list(range(0, n, 2))
    return rows


@pytest.mark.parametrize("rows", [
    # query tiles with no key tile whose partner in the MMA (the adjacent tile) has some; uneven lists
    _ring_rows(16, 3, empty=(2, 5, 7), long_row=3),
    # four consecutive query tiles (one CTA pair) with no key tile at all, ragged last tile
    _ring_rows(18, 4, empty=(4, 5, 6, 7, 13), long_row=16),
])
def test_pair_kernel_block_sparse_structures(h, rows):
    """Block-sparse launches above 12 % density run on CTA pairs with one merged plan per four query tiles."""
    n = len(rows)
    nnz = sum(len(r) for r in rows)
    assert nnz / (n * n) >= 0.12
    L, H = n * 128 - 37, 2
    rp = np.cumsum([0] + [len(r) for r in rows]).astype(np.int32)
    ci = np.array([c for r in rows for c in r], dtype=np.int32)
    q, k, v = bf16_inputs(L, H, 990 + n)
    ref, ref_lse = O.attention(q.float(), k.float(), v.float(), csr=(rp, ci), return_lse=True)
    bi = h.BlockIndex.from_csr(rp, ci, n).to("cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    first = None
    for _ in range(10):
        out = torch.full((L, H, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        out, lse = h.attn_fwd(dev(q), dev(k), dev(v), h.MODE_BLOCK_SPARSE, block_index=bi, out=out, return_lse=True,
                              logit_bound=PAIR_BOUND, status_word=st)
        assert h.read_status(st) == 0
        first = out if first is None else first
        assert torch.equal(out, first)
    check(first, torch.nan_to_num(ref))
    empty = torch.tensor([len(r) == 0 for r in rows]).repeat_interleave(128)[:L]
    assert bool((first.float().cpu()[empty] == 0).all())
    assert bool(torch.isinf(lse.cpu()[:, empty]).all())
    assert float((lse.cpu().t()[~empty] - ref_lse[~empty]).abs().max()) < 2e-3


@pytest.mark.parametrize("L,Lk,H,fp8", [(1000, 2200, 3, False), (4096, 4096, 4, False), (2100, 8192, 5, False), (1536, 4096, 3, True)])
def test_pair_kernel_split_last_wave(h, L, Lk, H, fp8):
    """With the optional workspace the pairs of the last, partly filled wave each walk a share of the key tiles and a
    second kernel adds the shares; without it nothing is split.  Both must give the oracle's rows (and each other's,
    up to the order of the additions)."""
    from pika_h3_flex_b200 import _lib
    import ctypes as C

    q, k, v = bf16_inputs(L, H, 1200 + L, Lk)
    if fp8:
        qq, sq = O.quantize_e4m3_blocks(q.float())
        kq, sk = O.quantize_e4m3_blocks(k.float())
        ref, ref_lse = O.attention(O.dequantize_blocks(qq, sq), O.dequantize_blocks(kq, sk), v.float(), return_lse=True)
        to_dev = lambda x: dev(x.to(torch.float8_e4m3fn).view(torch.uint8).permute(1, 0, 2).contiguous()).permute(1, 0, 2)
        args = (to_dev(qq), to_dev(kq), dev(v), h.MODE_FP8_QK, dev(sq), dev(sk))
    else:
        ref, ref_lse = O.attention(q.float(), k.float(), v.float(), return_lse=True)
        args = (dev(q), dev(k), dev(v))
    # the size query says whether this shape splits on this device
    p = _lib.AttnParams()
    p.Lq, p.Lk, p.H, p.d, p.B, p.mode, p.logit_bound = L, Lk, H, 128, 1, int(h.MODE_FP8_QK if fp8 else h.MODE_DENSE_BF16), PAIR_BOUND
    need = C.c_size_t(0)
    assert _lib.load().h3a_attn_workspace_bytes(C.byref(p), C.byref(need)) == 0
    assert need.value > 0, "these shapes are chosen so that the last wave is split on a 148-SM device"
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    split, lse = h.attn_fwd(*args, logit_bound=PAIR_BOUND, return_lse=True, status_word=st)  # wrapper supplies the workspace
    assert h.read_status(st) == 0
    small = torch.empty(16, dtype=torch.uint8, device="cuda")  # too small: the launch must not split
    whole = h.attn_fwd(*args, logit_bound=PAIR_BOUND, workspace=small)
    check(split, ref)
    check(whole, ref)
    assert float((split.float() - whole.float()).abs().max()) <= 2e-3
    assert float((lse.cpu().t() - ref_lse).abs().max()) < 2e-3


def test_hot_path_replays_from_a_cuda_graph(h):
    """Preparation + attention (CTA pairs, split last wave, combine) captured once into a CUDA graph and replayed on
    new input values in the same buffers: the launches make no host synchronisation and take all their inputs
    from device memory or by value, so a sampler loop can replay them without per-step launch work."""
    from pika_h3_flex_b200.ops import normed_logit_bound

    grid, n_audio, H = (6, 16, 20), 128, 3
    pos = O.make_positions(grid, n_audio)
    L = pos.shape[0]
    q, k, v = (t.bfloat16() for t in O.seeded_qkv(L, H, seed=51))
    sq, sk, sv = dev(q).clone(), dev(k).clone(), dev(v).clone()
    tab = h.rope_table(dev(pos))
    bound = normed_logit_bound()
    out = torch.empty(L, H, 128, dtype=torch.bfloat16, device="cuda")

    def step():
        qp, kp, _, _ = h.qk_prep(sq, sk, tab, tab)
        h.attn_fwd(qp, kp, sv, out=out, logit_bound=bound)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture: one-time function attributes are set here
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for seed in (52, 53):
        q2, k2, v2 = (t.bfloat16() for t in O.seeded_qkv(L, H, seed=seed))
        sq.copy_(dev(q2)); sk.copy_(dev(k2)); sv.copy_(dev(v2))
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        check(out, O.joint_attention(q2.float(), k2.float(), v2.float(), pos, "dense"))
