"""GPU: the CUDA code path of the Ulysses wrapper (prep -> exchange -> attention -> exchange) on a one-rank NCCL
group; the multi-rank reshard logic itself is covered on CPU ranks (tests/test_ulysses_cpu.py) and the 2/4/8-GPU
runs by bench.py --gpus N."""
import os
import socket

import pytest
import torch
import torch.distributed as dist

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nccl_group(lib):
    assert torch.cuda.is_available()
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    yield None
    dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["nccl", "peer"])
@pytest.mark.parametrize("mode_name", ["dense", "fp8_qk", "block_sparse"])
def test_ulysses_wrapper_cuda_path(nccl_group, mode_name, transport):
    import pika_h3_flex_b200 as h
    from pika_h3_flex_b200.ulysses import UlyssesAttention

    grid, n_audio, H = (4, 8, 12), 128, 3
    pos = O.make_positions(grid, n_audio)
    L = pos.shape[0]
    q, k, v = (t.bfloat16() for t in O.seeded_qkv(L, H, seed=31))
    csr, bi, mode = None, None, h.MODE_DENSE_BF16
    if mode_name == "block_sparse":
        bih = h.build_block_index(grid, n_audio, (1, 2, 2))
        csr, bi, mode = (bih.row_ptr.numpy(), bih.col_idx.numpy()), bih.to("cuda"), h.MODE_BLOCK_SPARSE
    elif mode_name == "fp8_qk":
        mode = h.MODE_FP8_QK
    ref = O.joint_attention(q.float(), k.float(), v.float(), pos, mode_name, csr=csr)
    ua = UlyssesAttention(None, mode, bi, transport=transport)
    for _ in range(2):  # the peer transport reuses its buffers: the second call must not see the first one's leftovers
        out = ua(q.cuda(), k.cuda(), v.cuda(), h.rope_table(pos.cuda()))
        assert ua.transport == transport and out.shape == (L, H, 128)
        st = O.error_stats(out.float().cpu(), ref)
        if mode_name == "fp8_qk":
            assert st["rel_l2"] <= 6e-2, st
        else:
            assert st["max_abs"] <= 3e-2 and st["mean_abs"] <= 3e-3, st
    ua.check_status()
    ua.close()


_CHILD = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
import pika_h3_flex_b200 as h
from pika_h3_flex_b200.ulysses import UlyssesAttention
from oracle import oracle as O
grid, n_audio, H = (4, 8, 12), 128, {heads}
pos = O.make_positions(grid, n_audio)
L = pos.shape[0]
q, k, v = (t.bfloat16() for t in O.seeded_qkv(L, H, seed=33))
Ls = L // world
sl = slice(rank * Ls, (rank + 1) * Ls)
ok = True
for mode_name in ("dense", "fp8_qk", "block_sparse"):
    csr, bi, mode = None, None, h.MODE_DENSE_BF16
    if mode_name == "block_sparse":
        bih = h.build_block_index(grid, n_audio, (1, 2, 2))
        csr, bi, mode = (bih.row_ptr.numpy(), bih.col_idx.numpy()), bih.to("cuda"), h.MODE_BLOCK_SPARSE
    elif mode_name == "fp8_qk":
        mode = h.MODE_FP8_QK
    ref = O.joint_attention(q.float(), k.float(), v.float(), pos, mode_name, csr=csr)[sl]
    hp = (H + world - 1) // world
    # direct stores into the owners' memory (twice: buffers are reused); then the staged all_to_all with one launch,
    # the automatic choice of head groups, and one exchange + launch per head slot
    for transport, groups in (("peer", 1), ("peer", 1), ("nccl", 1), ("nccl", 2), ("nccl", [1] * hp)):
        ua = UlyssesAttention(None, mode, bi, head_groups=groups, transport=transport)
        out = ua(q[sl].cuda(), k[sl].cuda(), v[sl].cuda(), h.rope_table(pos[sl].cuda()))
        st = O.error_stats(out.float().cpu(), ref)
        good = st["rel_l2"] <= (6e-2 if mode_name == "fp8_qk" else 1e-2)
        print(rank, mode_name, transport, groups, st, flush=True)
        ok = ok and good and tuple(out.shape) == (Ls, H, 128) and ua.transport == transport
        ua.check_status()
        ua.close()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if int(flag.item()) == 1 else 1)
"""


@pytest.mark.parametrize("world,heads", [(2, 4), (2, 3), (4, 6)])
def test_ulysses_multi_gpu_exchange_matches_oracle(world, heads, tmp_path):
    """Ranks as child processes, one per GPU: both transports (rows stored straight into the owning rank's memory over
    NVLink; blocks staged per peer and exchanged with NCCL's all_to_all) must give every rank the oracle's rows of its
    sequence shard, in all three modes; heads = 3 on 2 ranks and 6 on 4 also pads."""
    import subprocess
    import sys

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(_CHILD.format(root=root, heads=heads))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o.decode(errors="replace"))
    assert all(p.returncode == 0 for p in procs), "\n".join(x[-2000:] for x in outs)


_HOST_CHILD = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
import pika_h3_flex_b200 as h
from pika_h3_flex_b200.host_path import HostUlyssesAttention
from oracle import oracle as O
grid, n_audio, H = (4, 8, 12), 128, {heads}
pos = O.make_positions(grid, n_audio)
L = pos.shape[0]
Ls = L // world
sl = slice(rank * Ls, (rank + 1) * Ls)
rope = h.rope_table(pos[sl].cuda())
ok = True
for mode_name, transport in (("dense", "peer"), ("fp8_qk", "peer"), ("block_sparse", "peer"), ("dense", "nccl"), ("block_sparse", "nccl")):
    csr, bi, mode = None, None, h.MODE_DENSE_BF16
    if mode_name == "block_sparse":
        bih = h.build_block_index(grid, n_audio, (1, 2, 2))
        csr, bi, mode = (bih.row_ptr.numpy(), bih.col_idx.numpy()), bih.to("cuda"), h.MODE_BLOCK_SPARSE
    elif mode_name == "fp8_qk":
        mode = h.MODE_FP8_QK
    ha = HostUlyssesAttention(Ls, H, mode, bi, slot_groups={groups!r}, transport=transport)
    for seed in (35, 36):  # twice through the same staging buffers, different values
        q, k, v = (t.bfloat16() for t in O.seeded_qkv(L, H, seed=seed))
        ref = O.joint_attention(q.float(), k.float(), v.float(), pos, mode_name, csr=csr)[sl]
        hq, hk, hv = (t[sl].contiguous().pin_memory() for t in (q, k, v))
        ho = torch.full((Ls, H, 128), float("nan"), dtype=torch.bfloat16).pin_memory()
        ha(hq, hk, hv, rope, ho)
        torch.cuda.synchronize()
        st = O.error_stats(ho.float(), ref)
        print(rank, mode_name, transport, seed, st, ha.stage_ms(), flush=True)
        ok = ok and bool(torch.isfinite(ho.float()).all()) and st["rel_l2"] <= (6e-2 if mode_name == "fp8_qk" else 1e-2)
    ha.check_status()
    ha.close()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if int(flag.item()) == 1 else 1)
"""


@pytest.mark.parametrize("world,heads,groups", [(2, 6, [1, 2]), (2, 5, [1, 1, 1]), (4, 6, None)])
def test_host_buffer_path_under_ulysses(world, heads, groups, tmp_path):
    """Ranks as child processes: pinned host shards in, pinned host shard out, pipelined over head-slot groups with
    round-robin head assignment (5 heads on 2 ranks and 6 on 4 pad), on both transports; every rank must get the
    oracle's rows."""
    import subprocess
    import sys

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(_HOST_CHILD.format(root=root, heads=heads, groups=groups))
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    outs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        outs.append(o.decode(errors="replace"))
    assert all(p.returncode == 0 for p in procs), "\n".join(x[-2000:] for x in outs)
