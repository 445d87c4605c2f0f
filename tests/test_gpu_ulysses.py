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


@pytest.mark.parametrize("mode_name", ["dense", "fp8_qk", "block_sparse"])
def test_ulysses_wrapper_cuda_path(nccl_group, mode_name):
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
    ua = UlyssesAttention(None, mode, bi)
    out = ua(q.cuda(), k.cuda(), v.cuda(), h.rope_table(pos.cuda()))
    assert out.shape == (L, H, 128)
    st = O.error_stats(out.float().cpu(), ref)
    if mode_name == "fp8_qk":
        assert st["rel_l2"] <= 6e-2, st
    else:
        assert st["max_abs"] <= 3e-2 and st["mean_abs"] <= 3e-3, st
