"""Host-side layout helpers: the float position grid of the packed joint sequence.

Mirrors what the reference hands to its DiT as ``position_ids`` (``src/pika_h3/core/packing.py:126-133``):
a float ``[S, 3]`` grid built on the host.  Video rows are frame-major, then row, then column
(``src/pika_h3/core/packing.py:49-54``); audio rows are 1-D positions ``(a, 0, 0)`` and come first.
"""
from __future__ import annotations

from typing import Tuple

import torch


def position_grid(grid: Tuple[int, int, int], n_audio: int = 0, dtype=torch.float32) -> torch.Tensor:
    T, Hg, Wg = grid
    n = torch.arange(T * Hg * Wg, dtype=torch.int64)
    vid = torch.stack([n // (Hg * Wg), (n // Wg) % Hg, n % Wg], dim=1).to(dtype)
    aud = torch.zeros(n_audio, 3, dtype=dtype)
    aud[:, 0] = torch.arange(n_audio, dtype=dtype)
    return torch.cat([aud, vid], dim=0)
