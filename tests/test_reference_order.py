"""CPU: the row order of the packed sequence, pinned to what the reference project's own code computes.

``tests/golden/reference_row_order.npz`` was produced by running the reference's ``video_external_to_rows`` /
``patchify_video_latents`` (``src/pika_h3/core/packing.py:65-69,49-54``) on a coordinate-carrying latent
(``tests/golden/make_reference_order.py``).  It is the only part of the attention path whose result the reference
computes in code that can be imported without its absent dependencies, so it is the one independent pin of the
oracle's and the product's position grids.  When a checkout of the reference is present the functions are also
run live and must reproduce the fixture.
"""
import importlib
import os
import sys

import numpy as np
import pytest
import torch

from oracle import oracle as O
from pika_h3_flex_b200 import layout

GRIDS = [(2, 3, 4), (3, 4, 6), (5, 16, 24), (4, 32, 32)]
# a checkout of the reference: named by the environment, else a directory `reference` beside this repository
REFERENCE = os.environ.get("H3_REFERENCE_CHECKOUT") or os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..", "reference"))


@pytest.fixture(scope="module")
def order(golden_dir):
    return dict(np.load(os.path.join(golden_dir, "reference_row_order.npz")))


def _tag(grid):
    return "x".join(str(g) for g in grid)


@pytest.mark.parametrize("grid", GRIDS)
@pytest.mark.parametrize("n_audio", [0, 5, 128])
def test_oracle_and_product_grids_follow_the_reference_row_order(order, grid, n_audio):
    rows = order[f"rows_{_tag(grid)}"]  # [rows, 3] = (frame, patch row, patch column) of every row, reference order
    assert rows.shape == (grid[0] * grid[1] * grid[2], 3)
    for make in (O.make_positions, layout.position_grid):
        pos = make(grid, n_audio)
        assert pos.shape == (n_audio + rows.shape[0], 3)
        np.testing.assert_array_equal(pos[n_audio:].to(torch.int64).numpy(), rows)
        # audio rows: one-dimensional positions ahead of the video rows
        np.testing.assert_array_equal(pos[:n_audio, 0].to(torch.int64).numpy(), np.arange(n_audio))
        assert n_audio == 0 or float(pos[:n_audio, 1:].abs().max()) == 0.0


def test_product_grid_equals_oracle_grid_at_the_benchmark_shapes():
    for grid, n_audio in (((31, 30, 52), 1024), ((31, 48, 84), 1024), ((4, 32, 32), 0)):
        a = O.make_positions(grid, n_audio)
        b = layout.position_grid(grid, n_audio, dtype=torch.float64)
        assert torch.equal(a, b)
        assert layout.position_grid(grid, n_audio).dtype == torch.float32


def test_row_entries_are_channel_major_patches(order):
    # a row holds channel c, then the (1, 2, 2) patch offsets: 24 x 1 x 2 x 2 = 96 entries
    within = order["within_3x4x6"]
    assert within.shape == (96, 4)
    c, pt, ph, pw = within.T
    np.testing.assert_array_equal(c, np.repeat(np.arange(24), 4))
    np.testing.assert_array_equal(pt, 0)
    np.testing.assert_array_equal(ph, np.tile([0, 0, 1, 1], 24))
    np.testing.assert_array_equal(pw, np.tile([0, 1, 0, 1], 24))
    np.testing.assert_array_equal(order["patch_size"], [1, 2, 2])


def test_audio_rows_are_channel_major(order):
    # all rows of the left channel, then all rows of the right one (src/pika_h3/core/packing.py:82-89)
    a = order["audio_rows_t7"]
    np.testing.assert_array_equal(a[:, 0], np.repeat([0, 1], 7))
    np.testing.assert_array_equal(a[:, 1], np.tile(np.arange(7), 2))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "src", "pika_h3")), reason="no checkout of the reference here")
def test_fixture_reproduces_from_the_reference_checkout(order, golden_dir):
    sys.path.insert(0, os.path.join(REFERENCE, "src"))
    sys.path.insert(0, golden_dir)
    try:
        packing = importlib.import_module("pika_h3.core.packing")
        geometry = importlib.import_module("pika_h3.core.geometry")
        gen = importlib.import_module("make_reference_order")
        for grid in GRIDS:
            tok, within = gen.reference_rows(packing, geometry, grid)
            np.testing.assert_array_equal(tok, order[f"rows_{_tag(grid)}"])
            np.testing.assert_array_equal(within, order[f"within_{_tag(grid)}"])
    finally:
        sys.path.remove(golden_dir)
        sys.path.remove(os.path.join(REFERENCE, "src"))
