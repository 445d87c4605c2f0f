"""GPU parity of the adaptive layer norm (h3a_adaln_norm) against the fp32 oracle on the same bf16-rounded inputs.
Tolerance: bf16 output rounding (2^-9 relative) on values of a few units: max-abs <= 4e-2, rel-L2 <= 4e-3."""
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def h(lib):
    import pika_h3_flex_b200 as pkg

    assert torch.cuda.is_available()
    return pkg


@pytest.mark.parametrize("L,D,T,rms,affine", [(1, 8, 1, False, False), (300, 5120, 3, False, False), (257, 1024, 2, True, True),
                                              (64, 8192, 6, False, True), (1000, 520, 4, True, False)])
def test_adaln_matches_oracle(h, L, D, T, rms, affine):
    g = torch.Generator().manual_seed(L + D)
    x = (2.0 * torch.randn(L, D, generator=g) + 0.5).bfloat16()
    mod = (0.3 * torch.randn(T, 2 * D, generator=g)).bfloat16()  # one projection output, chunked like the reference does
    shift, scale = mod.chunk(2, dim=-1)
    idx = torch.randint(0, T, (L,), generator=g)
    w = 1 + 0.1 * torch.randn(D, generator=g) if affine else None
    b = 0.1 * torch.randn(D, generator=g) if affine else None
    ref = O.adaln_modulate(x, scale, shift, idx, 1e-6, rms, w, b)
    modd = mod.cuda()
    shd, scd = modd.chunk(2, dim=-1)  # strided views of the [T, 2 D] tensor: no copies
    out = h.adaln_norm(x.cuda(), scd, shd, idx.cuda(), 1e-6, rms, None if w is None else w.cuda(), None if b is None else b.cuda())
    assert out.shape == (L, D) and out.dtype == torch.bfloat16
    s = O.error_stats(out.float().cpu(), ref)
    assert s["max_abs"] <= 4e-2 and s["rel_l2"] <= 4e-3, s


def test_adaln_without_indices_and_argument_checks(h):
    x = torch.randn(16, 64).bfloat16().cuda()
    sc, sh = (0.1 * torch.randn(1, 64)).bfloat16().cuda(), (0.1 * torch.randn(1, 64)).bfloat16().cuda()
    out = h.adaln_norm(x, sc, sh)
    ref = O.adaln_modulate(x.cpu(), sc.cpu(), sh.cpu())
    assert float((out.float().cpu() - ref).abs().max()) <= 4e-2
    with pytest.raises(ValueError):
        h.adaln_norm(x, sc[:, :32], sh)
    with pytest.raises(ValueError):
        h.adaln_norm(x, sc, sh, torch.zeros(16, dtype=torch.int32, device="cuda"))
    from pika_h3_flex_b200 import _lib
    with pytest.raises(_lib.H3AError):
        h.adaln_norm(torch.zeros(4, 8200, dtype=torch.bfloat16, device="cuda"), torch.zeros(1, 8200, dtype=torch.bfloat16, device="cuda"),
                     torch.zeros(1, 8200, dtype=torch.bfloat16, device="cuda"))  # wider than one CTA holds
