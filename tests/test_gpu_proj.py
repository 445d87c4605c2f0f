"""GPU parity of the fused projection (h3a_proj_fwd): x W^T (+ LoRA) (+ bias), with the per-head RMSNorm + rotation
in its epilogue, against the fp32 oracle on the same bf16-rounded inputs.  Tolerance: rel-L2 <= 5e-3 and max-abs
<= 3e-2 on outputs of unit scale (bf16 output rounding is 2e-3 relative)."""
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def h(lib):
    import pika_h3_flex_b200 as pkg

    assert torch.cuda.is_available()
    return pkg


def _inputs(L, K, H, R, bias, seed):
    g = torch.Generator().manual_seed(seed)
    N = H * 128
    x = torch.randn(L, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, generator=g) if bias else None
    a = bmat = None
    if R:
        a = (torch.randn(R, K, generator=g) / K ** 0.5).bfloat16()
        bmat = (0.5 * torch.randn(N, R, generator=g) / R ** 0.5).bfloat16()
    return x, w, b, a, bmat


def _lora_t(x, a):
    # the thin product x A^T, rounded to bf16 as the caller hands it to the kernel
    return None if a is None else (x.float() @ a.float().t()).bfloat16()


@pytest.mark.parametrize("L,K,H,R,bias", [
    (256, 64, 2, 0, False),      # one tile, one step of the contraction
    (300, 520, 3, 0, True),      # ragged tokens, K not a multiple of 64, odd head count (half-empty column tile)
    (1000, 1024, 5, 128, True),  # LoRA rank 128
    (4100, 320, 20, 64, False),  # 170 tiles on 74 CTA pairs: every pair reuses both accumulator buffers
])
def test_projection_store(h, L, K, H, R, bias):
    x, w, b, a, bm = _inputs(L, K, H, R, bias, 40 + L)
    t = _lora_t(x, a)
    ref = O.lora_linear(x, w, b, None, None)
    if R:
        ref = ref + t.float() @ bm.float().t()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    dev = lambda z: None if z is None else z.cuda()
    out = h.proj_fwd(dev(x), dev(w), dev(b), dev(t), dev(bm), status_word=st)
    assert h.read_status(st) == 0
    assert out.shape == (L, H, 128) and out.dtype == torch.bfloat16
    s = O.error_stats(out.float().cpu(), ref.view(L, H, 128))
    assert s["rel_l2"] <= 5e-3 and s["max_abs"] <= 3e-2, s


@pytest.mark.parametrize("L,K,H,R,half,weighted", [(700, 512, 2, 0, False, False), (700, 512, 3, 64, True, True), (4100, 320, 20, 64, False, True)])
def test_projection_with_fused_norm_and_rotation(h, L, K, H, R, half, weighted):
    x, w, b, a, bm = _inputs(L, K, H, R, True, 60 + L)
    t = _lora_t(x, a)
    frames = max(1, (L - 40) // 16)
    pos = O.make_positions((frames, 4, 4), L - frames * 16)
    cos, sin = O.rope_table(pos)
    nw = 1 + 0.1 * torch.randn(128, generator=torch.Generator().manual_seed(5)) if weighted else None
    y = O.lora_linear(x, w, b, None, None)
    if R:
        y = y + t.float() @ bm.float().t()
    ref = O.apply_rope(O.rms_norm(y.view(L, H, 128), nw), cos, sin, not half)
    rope = torch.stack([cos, sin], dim=-1).float().contiguous().cuda()
    dev = lambda z: None if z is None else z.cuda()
    out = h.proj_fwd(dev(x), dev(w), dev(b), dev(t), dev(bm), prep=True, rope=rope, norm_weight=dev(nw), rope_half=half)
    s = O.error_stats(out.float().cpu(), ref)
    assert s["rel_l2"] <= 5e-3 and s["max_abs"] <= 3e-2, s
    # and it is what the two-step path (projection, then h3a_qk_prep) gives, up to the bf16 rounding in between
    two_step, _, _, _ = h.qk_prep(h.proj_fwd(dev(x), dev(w), dev(b), dev(t), dev(bm)), None, rope, None, dev(nw), None, 1e-6, False, half)
    assert float((two_step.float() - out.float()).abs().max()) <= 4e-2


def test_projection_rejects_bad_arguments(h):
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(130, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        h.proj_fwd(x, w)  # N not a multiple of 128
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        h.proj_fwd(x, w, lora_t=torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda"))  # LoRA halves go together
    with pytest.raises(ValueError):
        h.proj_fwd(x.float(), w)


def test_projection_token_major_output(h):
    """The output projection (to_out): same GEMM, rows written token-major [L, N]."""
    L, K, H = 900, 384, 3
    x, w, b, a, bm = _inputs(L, K, H, 64, True, 77)
    t = _lora_t(x, a)
    ref = O.lora_linear(x, w, b, None, None) + t.float() @ bm.float().t()
    out = h.proj_fwd(x.cuda(), w.cuda(), b.cuda(), t.cuda(), bm.cuda(), token_major=True)
    assert out.shape == (L, H * 128) and out.is_contiguous()
    s = O.error_stats(out.float().cpu(), ref)
    assert s["rel_l2"] <= 5e-3 and s["max_abs"] <= 3e-2, s


@pytest.mark.parametrize("L,K,H", [(700, 512, 3), (4100, 320, 20)])
def test_projection_with_fused_fp8_quantisation(h, L, K, H):
    """Epilogue H3A_PROJ_PREP_FP8: the prepared rows as e4m3 with per-(head, 128-token block) absmax scales, the
    layout h3a_qk_prep produces; dequantised they must match the oracle's preparation within e4m3 resolution, and
    the scales must be the block maxima / 448."""
    x, w, b, a, bm = _inputs(L, K, H, 64, True, 90 + L)
    t = _lora_t(x, a)
    frames = max(1, (L - 40) // 16)
    pos = O.make_positions((frames, 4, 4), L - frames * 16)
    cos, sin = O.rope_table(pos)
    y = O.lora_linear(x, w, b, None, None) + t.float() @ bm.float().t()
    ref = O.apply_rope(O.rms_norm(y.view(L, H, 128)), cos, sin, True)
    rope = torch.stack([cos, sin], dim=-1).float().contiguous().cuda()
    out, scale = h.proj_fwd(x.cuda(), w.cuda(), b.cuda(), t.cuda(), bm.cuda(), prep=True, rope=rope, fp8=True)
    assert out.dtype == torch.uint8 and out.shape == (L, H, 128) and scale.shape == (H, (L + 127) // 128)
    deq = O.dequantize_blocks(out.cpu().view(torch.float8_e4m3fn).float(), scale.cpu())
    s = O.error_stats(deq, ref)
    assert s["rel_l2"] <= 4e-2 and s["max_abs"] <= 0.3, s  # e4m3: 3 mantissa bits, values up to ~5
    nb = (L + 127) // 128
    pad = torch.zeros(nb * 128 - L, H, 128)
    blockmax = torch.cat([ref, pad]).abs().view(nb, 128, H, 128).amax(dim=(1, 3)).t()  # [H, nb]
    assert torch.allclose(scale.cpu(), blockmax / 448.0, rtol=2e-2, atol=1e-6)
