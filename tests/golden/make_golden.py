"""Regenerate the golden fixtures in this directory:  python tests/golden/make_golden.py

The reference project ships no vectors for its attention path (its model file lives in an un-vendored
dependency), so these fixtures pin the float64 evaluation of the oracle's own definitions on small seeded
inputs.  They guard the fp32 oracle, and through it the CUDA path, against silent changes of convention
(pair order, axis split, norm/rotation order, scale rule, mask rule).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import oracle as O  # noqa: E402


def main():
    grid, n_audio, H = (3, 4, 6), 24, 2  # L = 96: one partial 128-tile
    L = n_audio + grid[0] * grid[1] * grid[2]
    q, k, v = O.seeded_qkv(L, H, seed=4242)
    q, k, v = (t.bfloat16().double() for t in (q, k, v))  # inputs exactly representable in bf16
    pos = O.make_positions(grid, n_audio)
    cos, sin = O.rope_table(pos)
    out = {"pos": pos.numpy(), "cos": cos.numpy().astype(np.float32), "sin": sin.numpy().astype(np.float32)}
    out["q"], out["k"], out["v"] = (t.float().numpy() for t in (q, k, v))
    for inter in (True, False):
        qp, kp = O.qk_prep(q, k, cos, sin, interleaved=inter)
        tag = "inter" if inter else "half"
        out[f"qp_{tag}"] = qp.float().numpy()
        out[f"kp_{tag}"] = kp.float().numpy()
        out[f"dense_{tag}"] = O.attention(qp, kp, v).float().numpy()
    qp, kp = O.qk_prep(q, k, cos, sin)
    qq, sq = O.quantize_e4m3_blocks(qp.float())
    out["q_e4m3"] = qq.numpy()
    out["q_scale"] = sq.numpy()
    out["fp8"] = O.attention_fp8_qk(qp.float(), kp.float(), v.float()).numpy()
    np.savez_compressed(os.path.join(HERE, "small_joint.npz"), **out)

    # block-sparse case: 2x6x10 grid + 128 audio, window (1,1,2), tiles of 128
    grid, n_audio, H = (5, 8, 16), 128, 1
    L = n_audio + grid[0] * grid[1] * grid[2]
    keep = O.neighbourhood_block_mask(grid, n_audio, (1, 1, 2))
    rp, ci = O.mask_to_csr(keep)
    q, k, v = O.seeded_qkv(L, H, seed=4243)
    q, k, v = (t.bfloat16().double() for t in (q, k, v))
    rows = torch.arange(0, L, 7)
    o = O.attention(q, k, v, csr=(rp, ci), q_rows=rows)
    np.savez_compressed(
        os.path.join(HERE, "small_sparse.npz"), keep=keep, row_ptr=rp, col_idx=ci, rows=rows.numpy(),
        out_rows=o.float().numpy(), grid=np.array(grid), n_audio=np.array(n_audio),
    )
    print("written", os.listdir(HERE))


if __name__ == "__main__":
    main()
