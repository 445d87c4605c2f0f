"""GPU: the pieces of the sequence-parallel path that store rows where they are needed (h3a_qk_prep_scatter, the
per-rank output bases of h3a_attn_fwd, the peer arena), with several ranks EMULATED on one GPU: every "rank" is a
separate local buffer, so the index arithmetic of all ranks runs in one process.  The real multi-process runs over
NVLink are the child-process tests of tests/test_gpu_ulysses.py (they need 2 or 4 GPUs) and bench.py --gpus N."""
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def h(lib):
    import pika_h3_flex_b200 as pkg

    assert torch.cuda.is_available()
    return pkg


@pytest.mark.parametrize("P,H,round_robin,half", [(1, 3, False, False), (2, 4, False, True), (4, 6, False, False), (3, 7, True, False), (4, 6, True, True), (8, 40, True, False)])
def test_prepared_rows_land_at_their_heads_owner(h, P, H, round_robin, half):
    """Every emulated rank prepares its token shard of all heads and scatters the rows; afterwards owner p must hold,
    for each of its head slots, exactly what the plain preparation gives for that head over the FULL sequence
    (bit-identical: the arithmetic per row is the same kernel code).  7 heads on 3 ranks and 6 on 4 pad."""
    from pika_h3_flex_b200 import ops

    Ls = 200 if P < 8 else 130
    L = P * Ls
    hp = (H + P - 1) // P
    g = torch.Generator().manual_seed(90 + P)
    x = torch.randn(L, H, 128, generator=g).bfloat16().cuda()
    w = (1 + 0.1 * torch.randn(128, generator=g)).cuda()
    pos = O.make_positions((L // 16, 4, 4), L - (L // 16) * 16)
    tab = h.rope_table(pos.cuda())
    want, _, _, _ = h.qk_prep(x, None, tab, None, q_weight=w, rope_half=half)  # logical [L, H, 128]
    want_v, _, _, _ = h.qk_prep(x, None, None, None, no_norm=True)
    assert torch.equal(want_v, x)  # the re-layout is an exact copy
    bufs = [torch.full((hp, L, 128), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    bufs_v = [torch.full((hp, L, 128), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    for r in range(P):
        sl = slice(r * Ls, (r + 1) * Ls)
        # in two head ranges, as the host-buffer pipeline does (head0 names the first head of the piece)
        cut = max(1, H // 2)
        for h0, h1 in ((0, cut), (cut, H)):
            if h1 <= h0:
                continue
            to = ops.HeadOwners([b.data_ptr() for b in bufs], hp, round_robin, r * Ls, L, head0=h0, start_head=r + 1)  # any order of the heads
            ops.prep_scatter(x[sl, h0:h1], to, tab[sl].contiguous(), w, rope_half=half)
            tov = ops.HeadOwners([b.data_ptr() for b in bufs_v], hp, round_robin, r * Ls, L, head0=h0)
            ops.prep_scatter(x[sl, h0:h1], tov, no_norm=True)
    for head in range(H):
        owner, slot = (head % P, head // P) if round_robin else (head // hp, head % hp)
        assert torch.equal(bufs[owner][slot], want[:, head]), (head, owner, slot)
        assert torch.equal(bufs_v[owner][slot], x[:, head])
    # padded slots were never touched
    for p in range(P):
        for slot in range(hp):
            head = slot * P + p if round_robin else p * hp + slot
            if head >= H:
                assert bool((bufs[p][slot] == 9.0).all())


@pytest.mark.parametrize("P,H,round_robin", [(2, 4, False), (4, 6, False), (3, 6, True), (2, 6, False), (8, 40, False)])  # the last two: an odd
# number of heads per rank, so a 256-column tile (two heads) belongs to two owners
def test_projection_epilogue_stores_rows_at_their_heads_owner(h, P, H, round_robin):
    """The fused projection with `out_to`: every emulated rank projects its token shard (LoRA, RMSNorm and rotation in
    the epilogue) and the epilogue stores the rows at the heads' owners; each owner must end up with exactly what the
    projection of the FULL sequence writes for its heads (same kernel arithmetic per row: bit-identical)."""
    from pika_h3_flex_b200 import ops

    Ls, K, R = 300, 320, 64
    L = P * Ls
    hp = (H + P - 1) // P
    g = torch.Generator().manual_seed(95)
    x = torch.randn(L, K, generator=g).bfloat16().cuda()
    w = (torch.randn(H * 128, K, generator=g) / K ** 0.5).bfloat16().cuda()
    la = (torch.randn(R, K, generator=g) / K ** 0.5).bfloat16().cuda()
    lb = (0.5 * torch.randn(H * 128, R, generator=g) / R ** 0.5).bfloat16().cuda()
    nw = (1 + 0.1 * torch.randn(128, generator=g)).cuda()
    pos = O.make_positions((L // 16, 4, 4), L - (L // 16) * 16)
    tab = h.rope_table(pos.cuda())
    t = torch.nn.functional.linear(x, la)
    want = h.proj_fwd(x, w, None, t, lb, prep=True, rope=tab, norm_weight=nw)  # logical [L, H, 128]
    bufs = [torch.full((hp, L, 128), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for r in range(P):
        sl = slice(r * Ls, (r + 1) * Ls)
        to = ops.HeadOwners([b.data_ptr() for b in bufs], hp, round_robin, r * Ls, L, start_head=2 * r)
        assert h.proj_fwd(x[sl], w, None, t[sl].contiguous(), lb, prep=True, rope=tab[sl].contiguous(), norm_weight=nw, out_to=to,
                          status_word=status) is None
    assert h.read_status(status) == 0
    for head in range(H):
        owner, slot = (head % P, head // P) if round_robin else (head // hp, head % hp)
        assert torch.equal(bufs[owner][slot], want[:, head]), (head, owner, slot)


def test_scatter_argument_checks(h):
    from pika_h3_flex_b200 import _lib, ops

    x = torch.zeros(64, 2, 128, dtype=torch.bfloat16, device="cuda")
    buf = torch.zeros(1, 128, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(h.H3AError):  # rows beyond the full sequence
        ops.prep_scatter(x, ops.HeadOwners([buf.data_ptr(), buf.data_ptr()], 1, False, 100, 128))
    with pytest.raises(h.H3AError):  # more heads than the ranks have slots for
        ops.prep_scatter(x, ops.HeadOwners([buf.data_ptr()], 1, False, 0, 128))
    with pytest.raises(h.H3AError):  # a missing base
        ops.prep_scatter(x, ops.HeadOwners([buf.data_ptr(), 0], 1, False, 0, 128))


@pytest.mark.parametrize("L,Lk,H,P,bound,sparse", [(600, 600, 3, 3, 0.0, False), (1000, 2200, 3, 4, 12.0, False), (4096, 4096, 4, 8, 12.0, False),
                                                    (2304, 2304, 2, 2, 12.0, True), (1024, 1024, 2, 4, 0.0, True),
                                                    # short key ranges on persistent blocks: CTA pairs with resident K / V (whose
                                                    # rows otherwise leave as TMA tile stores) and one single-CTA block per SM
                                                    (9600, 512, 4, 3, 12.0, False), (40000, 640, 2, 2, 12.0, False)])
def test_output_rows_land_at_their_tokens_owner(h, L, Lk, H, P, bound, sparse):
    """The attention launch stores query row g at the emulated rank g // rows: single-CTA kernels (running maximum and
    fixed reference), CTA pairs with the split last wave (whose combining kernel stores too) and block-sparse.  The rows
    must equal the ordinary launch bit for bit, in a token-major buffer with more heads than the launch computes."""
    from pika_h3_flex_b200 import ops

    g = torch.Generator().manual_seed(91)
    q = torch.randn(L, H, 128, generator=g).bfloat16().cuda()
    k = torch.randn(Lk, H, 128, generator=g).bfloat16().cuda()
    v = torch.randn(Lk, H, 128, generator=g).bfloat16().cuda()
    mode, bi = h.MODE_DENSE_BF16, None
    if sparse:
        keep = O.neighbourhood_block_mask((L // 64, 8, 8), 0, (2, 8, 8))
        bi = h.BlockIndex.from_csr(*O.mask_to_csr(keep), n_k_tiles=keep.shape[1]).to("cuda")
        mode = h.MODE_BLOCK_SPARSE
    want = h.attn_fwd(q, k, v, mode, block_index=bi, logit_bound=bound)
    rows = (L + P - 1) // P
    Hall, head0, step = 2 * H + 1, 1, 2  # the launch's head j is head 1 + 2 j of a [rows, 2 H + 1, 128] token-major buffer
    bufs = [torch.full((rows, Hall, 128), 5.0, dtype=torch.bfloat16, device="cuda") for _ in range(P)]
    to = ops.RankOutputs([b.data_ptr() + head0 * 128 * 2 for b in bufs], rows, Hall * 128, step * 128)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert h.attn_fwd(q, k, v, mode, block_index=bi, logit_bound=bound, out_ranks=to, status_word=status) is None
    assert h.read_status(status) == 0
    got = torch.cat(bufs, dim=0)[:L]
    assert torch.equal(got[:, head0::step][:, :H], want)
    untouched = torch.ones(Hall, dtype=torch.bool)
    untouched[head0::step][:H] = False
    assert bool((got[:, untouched] == 5.0).all())


def test_peer_arena_on_one_rank(h):
    """Allocation through the library, torch views of the local arena, address arithmetic and release; with one rank no
    handle is exchanged."""
    from pika_h3_flex_b200.peer import Carver, PeerArena

    c = Carver()
    a_off, b_off = c.take(1000), c.take(4096)
    assert a_off == 0 and b_off == 1024 and c.size == 5120
    before = torch.cuda.memory_allocated()
    ar = PeerArena(c.size)
    assert torch.cuda.memory_allocated() - before < 4096  # not from torch's allocator (other processes must be able to map it); only the barrier's flag is
    t = ar.tensor(b_off, (16, 128), torch.bfloat16)
    t.fill_(3.0)
    u = ar.tensor(b_off, (16 * 128,), torch.bfloat16)
    assert t.data_ptr() == ar.addr(0, b_off) and float(u.float().sum()) == 3.0 * 16 * 128
    with pytest.raises(ValueError):
        ar.tensor(b_off, (4096,), torch.bfloat16)
    ar.barrier()
    del t, u
    ar.close()
