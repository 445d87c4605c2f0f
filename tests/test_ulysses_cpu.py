"""CPU ranks (gloo): the Ulysses reshard logic — head padding, seq->head and head->seq exchanges, FP8
scale resharding — against the single-process oracle.  The CUDA prep/attention calls are replaced by
oracle stand-ins here; the GPU tests cover the real kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from pika_h3_flex_b200 import _lib
from pika_h3_flex_b200.ulysses import UlyssesAttention, head_to_seq, padded_heads, seq_to_head


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cpu_prep(q, k, q_rope, k_rope, fp8):
    """Host stand-in for the CUDA preparation; either of q, k may be None (one tensor at a time)."""
    outs = []
    for x, rope in ((q, q_rope), (k, k_rope)):
        if x is None:
            outs.append((None, None))
            continue
        if rope is not None:
            cos, sin = rope[..., 0].double(), rope[..., 1].double()
            xp = O.qk_prep(x, x, cos, sin)[0]
        else:
            xp = O.rms_norm(x)
        outs.append(O.quantize_e4m3_blocks(xp) if fp8 else (xp, None))
    return outs[0][0], outs[1][0], outs[0][1], outs[1][1]


def _cpu_attn(q, k, v, mode, q_scale, k_scale, block_index):
    if mode == _lib.MODE_FP8_QK:
        q, k = O.dequantize_blocks(q, q_scale), O.dequantize_blocks(k, k_scale)
    csr = None
    if mode == _lib.MODE_BLOCK_SPARSE:
        csr = (block_index.row_ptr.numpy(), block_index.col_idx.numpy())
    return O.attention(q, k, v, csr=csr)


def _worker(rank, world, port, H, L, mode, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        q, k, v = O.seeded_qkv(L, H, seed=77)
        pos = O.make_positions((L // 16, 4, 4), L - (L // 16) * 16)
        cos, sin = O.rope_table(pos)
        rope = torch.stack([cos, sin], dim=-1).float()
        Ls = L // world
        sl = slice(rank * Ls, (rank + 1) * Ls)
        bi = None
        if mode == _lib.MODE_BLOCK_SPARSE:
            from pika_h3_flex_b200.ops import BlockIndex

            keep = O.neighbourhood_block_mask((L // 16, 4, 4), L - (L // 16) * 16, (1, 1, 1))
            bi = BlockIndex.from_csr(*O.mask_to_csr(keep), n_k_tiles=keep.shape[1])
        ua = UlyssesAttention(None, mode, bi, prep_fn=_cpu_prep, attn_fn=_cpu_attn)
        out = ua(q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), rope[sl].contiguous())
        # raw exchange round trip
        x = torch.arange(padded_heads(H, world) * Ls * 4, dtype=torch.float32).view(-1, Ls, 4) + 1000 * rank
        y, _ = seq_to_head(x)
        z, _ = head_to_seq(y)
        torch.save({"out": out.clone(), "roundtrip": bool(torch.equal(x, z)), "y": y}, os.path.join(result_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _run(world, H, L, mode, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), H, L, mode, str(tmp_path)), nprocs=world, join=True)
    res = [torch.load(os.path.join(tmp_path, f"r{r}.pt")) for r in range(world)]
    q, k, v = O.seeded_qkv(L, H, seed=77)
    pos = O.make_positions((L // 16, 4, 4), L - (L // 16) * 16)
    csr = None
    if mode == _lib.MODE_BLOCK_SPARSE:
        csr = O.mask_to_csr(O.neighbourhood_block_mask((L // 16, 4, 4), L - (L // 16) * 16, (1, 1, 1)))
    ref = O.joint_attention(q, k, v, pos, {0: "dense", 1: "fp8_qk", 2: "block_sparse"}[mode], csr=csr)
    out = torch.cat([r["out"] for r in res], dim=0)
    assert out.shape == ref.shape
    assert all(r["roundtrip"] for r in res)
    return out, ref, res


@pytest.mark.parametrize("world,H", [(2, 4), (2, 3), (4, 6)])
def test_ulysses_dense_matches_single_rank(world, H, tmp_path):
    out, ref, res = _run(world, H, 256, _lib.MODE_DENSE_BF16, tmp_path)
    assert float((out - ref).abs().max()) < 1e-5
    # after seq->head rank r holds heads [r*hp, (r+1)*hp) of every source rank's tokens, in rank order
    hp = padded_heads(H, world) // world
    Ls = 256 // world
    y1 = res[1]["y"]
    assert y1.shape == (hp, world * Ls, 4)
    for src in range(world):
        assert float(y1[0, src * Ls, 0]) == 1000 * src + (1 * hp) * Ls * 4


def test_ulysses_fp8_scales_follow_their_blocks(tmp_path):
    out, ref, _ = _run(2, 4, 512, _lib.MODE_FP8_QK, tmp_path)
    assert float((out - ref).abs().max()) < 1e-5


def test_ulysses_block_sparse(tmp_path):
    out, ref, _ = _run(2, 2, 512, _lib.MODE_BLOCK_SPARSE, tmp_path)
    assert float((out - ref).abs().max()) < 1e-5


def test_ulysses_rejects_bad_shapes():
    assert padded_heads(40, 8) == 40 and padded_heads(6, 4) == 8 and padded_heads(1, 8) == 8


def _mismatch_worker(rank, world, port, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pika_h3_flex_b200.ops import BlockIndex

        H = 2
        Ls = 64 if rank == 0 else 80  # rank 1 brings a longer shard
        q, k, v = O.seeded_qkv(Ls, H, seed=5 + rank)
        ua = UlyssesAttention(None, _lib.MODE_DENSE_BF16, None, prep_fn=_cpu_prep, attn_fn=_cpu_attn)
        try:
            ua(q, k, v, None)
            verdict = "no error"
        except ValueError as e:
            verdict = "ValueError: " + str(e)
        # a block index that does not describe the whole sequence is refused before any exchange
        keep = O.neighbourhood_block_mask((4, 4, 4), 0, (1, 1, 1))
        bi = BlockIndex.from_csr(*O.mask_to_csr(keep), n_k_tiles=keep.shape[1])  # 64 tokens = 1 tile
        ub = UlyssesAttention(None, _lib.MODE_BLOCK_SPARSE, bi, prep_fn=_cpu_prep, attn_fn=_cpu_attn)
        q, k, v = O.seeded_qkv(128, H, seed=9)  # 2 x 128 tokens = 2 tiles
        try:
            ub(q, k, v, None)
            verdict2 = "no error"
        except ValueError as e:
            verdict2 = "ValueError: " + str(e)
        torch.save({"shape": verdict, "index": verdict2}, os.path.join(result_dir, f"m{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_ulysses_shape_mismatch_between_ranks_raises_on_every_rank(tmp_path):
    """Ranks that bring shards of different length would block in an exchange whose sizes disagree; the one-time
    host-side check must turn that into a ValueError on every rank instead."""
    mp.spawn(_mismatch_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(os.path.join(tmp_path, f"m{r}.pt"))
        assert res["shape"].startswith("ValueError") and "disagree" in res["shape"], res
        assert res["index"].startswith("ValueError") and "block index" in res["index"], res


def test_round_robin_head_assignment_of_the_host_path_simulated():
    """The index arithmetic of the host-buffer Ulysses pipeline (heads dealt round-robin, blocks packed per peer,
    placed per source rank, unpacked per owner) with all ranks simulated in one process: after the inbound
    exchange rank p must hold heads j*P + p over ALL tokens, and the outbound exchange must restore every rank's
    token shard of every head.  5 heads on 2 ranks and 6 on 4 pad."""
    for P, H in ((2, 6), (2, 5), (4, 6), (3, 7)):
        Ls, Cc = 4, 2
        hp = (H + P - 1) // P
        full = torch.arange(P * Ls * H * Cc, dtype=torch.float32).view(P * Ls, H, Cc)  # [token, head, c]
        shards = [full[r * Ls : (r + 1) * Ls] for r in range(P)]
        for j0, n in ((0, 1), (1, hp - 1)) if hp > 1 else ((0, 1),):
            h0, h1 = j0 * P, min((j0 + n) * P, H)

            def pack(x_hm):  # HostUlyssesAttention._pack
                if x_hm.shape[0] < n * P:
                    x_hm = torch.cat([x_hm, x_hm.new_zeros(n * P - x_hm.shape[0], Ls, Cc)], dim=0)
                return x_hm.view(n, P, Ls, Cc).permute(1, 0, 2, 3).contiguous()

            sends = [pack(shards[r][:, h0:h1].permute(1, 0, 2).contiguous()) for r in range(P)]
            # all_to_all: rank p receives sends[src][p] from every src
            recvs = [torch.stack([sends[src][p] for src in range(P)]) for p in range(P)]
            outs_send = []
            for p in range(P):
                got = recvs[p].permute(1, 0, 2, 3).reshape(n, P * Ls, Cc)  # [slot, all tokens, c]
                for j in range(n):
                    h = (j0 + j) * P + p
                    want = full[:, h] if h < H else torch.zeros(P * Ls, Cc)
                    assert torch.equal(got[j], want), (P, H, p, j)
                outs_send.append(got.view(n, P, Ls, Cc).permute(1, 0, 2, 3).contiguous())  # [dest rank, slot, its tokens, c]
            for r in range(P):
                back = torch.stack([outs_send[p][r] for p in range(P)])  # [owner p, slot j, my tokens, c]
                heads = back.permute(1, 0, 2, 3).reshape(n * P, Ls, Cc)[: h1 - h0]
                assert torch.equal(heads.permute(1, 0, 2), shards[r][:, h0:h1]), (P, H, r)
