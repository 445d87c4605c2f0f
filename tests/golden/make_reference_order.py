"""Regenerate ``reference_row_order.npz``:  python tests/golden/make_reference_order.py [reference checkout; default: ../reference beside this repository]

The one contract of the attention path that the reference project holds in importable code is the ORDER of the
video rows of the packed sequence: ``video_external_to_rows`` (``src/pika_h3/core/packing.py:65-69``) hands the
latent ``[B, F, C, H, W]`` to ``patchify_video_latents`` (``src/pika_h3/core/packing.py:49-54``, the stand-in the
reference uses when the diffusers port is absent), patch size ``(1, 2, 2)`` (``src/pika_h3/core/geometry.py``).
This script imports those functions from a checkout of the reference, pushes a latent through them whose value
at ``(f, c, y, x)`` encodes its own coordinates, and stores, for every resulting row, the (frame, patch row,
patch column) it came from, plus the channel / in-patch offsets of the 96 entries of a row.  The tests compare
the oracle's and the product's position grids with these arrays, so the row order is pinned to what the
reference itself computes; the fixture travels where the checkout does not.
"""
import importlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GRIDS = [(2, 3, 4), (3, 4, 6), (5, 16, 24), (4, 32, 32)]  # (frames, token rows, token columns)


def reference_rows(packing, geometry, grid):
    """Run the reference's own ``video_external_to_rows`` on a coordinate-carrying latent."""
    T, Hg, Wg = grid
    pt, ph, pw = geometry.PATCH_SIZE
    C = geometry.VIDEO_LATENT_CHANNELS
    F, Hl, Wl = T * pt, Hg * ph, Wg * pw
    f = torch.arange(F, dtype=torch.float64).view(F, 1, 1, 1)
    c = torch.arange(C, dtype=torch.float64).view(1, C, 1, 1)
    y = torch.arange(Hl, dtype=torch.float64).view(1, 1, Hl, 1)
    x = torch.arange(Wl, dtype=torch.float64).view(1, 1, 1, Wl)
    code = ((f * 64 + c) * 4096 + y) * 4096 + x  # exact in float64
    rows = packing.video_external_to_rows(code[None])  # [1, rows, C * ph * pw]
    back = packing.video_rows_to_external(rows, F, Hl, Wl)
    assert torch.equal(back, code[None]), "the reference's own inverse does not restore the latent"
    r = rows[0].to(torch.int64)
    xx, yy = r % 4096, (r // 4096) % 4096
    cc, ff = (r // (4096 * 4096)) % 64, r // (4096 * 4096 * 64)
    # every entry of a row belongs to one token: same frame / patch row / patch column
    tok = torch.stack([ff // pt, yy // ph, xx // pw], dim=-1)
    assert bool((tok == tok[:, :1]).all())
    within = torch.stack([cc, ff % pt, yy % ph, xx % pw], dim=-1)
    assert bool((within == within[:1]).all())
    return tok[:, 0].numpy().astype(np.int32), within[0].numpy().astype(np.int32)


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference"))
    sys.path.insert(0, os.path.join(ref, "src"))
    packing = importlib.import_module("pika_h3.core.packing")
    geometry = importlib.import_module("pika_h3.core.geometry")
    out = {"patch_size": np.asarray(geometry.PATCH_SIZE, dtype=np.int32),
           "have_diffusers_port": np.asarray(int(packing.HAVE_DIFFUSERS_H3))}
    for grid in GRIDS:
        tok, within = reference_rows(packing, geometry, grid)
        tag = "x".join(str(g) for g in grid)
        out[f"rows_{tag}"] = tok
        out[f"within_{tag}"] = within
    # audio rows: channel-major (src/pika_h3/core/packing.py:82-89): row r of 2 T rows = (channel, latent index)
    T = 7
    a = torch.arange(T, dtype=torch.float64).view(1, T, 1, 1) * 1000 + torch.arange(geometry.AUDIO_CHANNELS, dtype=torch.float64).view(1, 1, -1, 1) * 100 \
        + torch.arange(geometry.AUDIO_LATENT_CHANNELS, dtype=torch.float64).view(1, 1, 1, -1)
    rows = packing.audio_external_to_rows(a.reshape(1, T, geometry.AUDIO_EXTERNAL_DIM))[0].to(torch.int64)
    out["audio_rows_t7"] = torch.stack([(rows[:, 0] // 100) % 10, rows[:, 0] // 1000], dim=-1).numpy().astype(np.int32)  # (channel, index)
    np.savez_compressed(os.path.join(HERE, "reference_row_order.npz"), **out)
    print("wrote reference_row_order.npz:", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
