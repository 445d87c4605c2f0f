"""GPU: the processor call shape on a stand-in attention module (LoRA-wrapped projections named as the
reference's DEFAULT_LORA_TARGETS, src/pika_h3/core/loader.py:9) against the oracle."""
import pytest
import torch
import torch.nn as nn

from oracle import oracle as O

pytestmark = pytest.mark.gpu


class LoraLinear(nn.Module):
    """base Linear + (alpha/r) B A, the structure PEFT gives to_q/to_k/to_v/to_out.0 (rank = alpha = 128 in
    the reference, src/pika_h3/pipeline.py:34; smaller here)."""

    def __init__(self, din, dout, r=8):
        super().__init__()
        self.base = nn.Linear(din, dout, bias=True)
        self.A = nn.Linear(din, r, bias=False)
        self.B = nn.Linear(r, dout, bias=False)

    def forward(self, x):
        return self.base(x) + self.B(self.A(x))


class RMSNorm(nn.Module):
    def __init__(self, d, eps=1e-6):
        super().__init__()
        self.weight = nn.Parameter(1 + 0.1 * torch.randn(d))
        self.eps = eps


class StubAttention(nn.Module):
    def __init__(self, dim, heads, ctx_dim=None):
        super().__init__()
        self.heads = heads
        inner = heads * 128
        self.to_q = LoraLinear(dim, inner)
        self.to_k = LoraLinear(ctx_dim or dim, inner)
        self.to_v = LoraLinear(ctx_dim or dim, inner)
        self.to_out = nn.ModuleList([LoraLinear(inner, dim), nn.Dropout(0.0)])
        self.norm_q = RMSNorm(128)
        self.norm_k = RMSNorm(128)


def oracle_forward(attn, x, ctx, pos, mode="dense", csr=None):
    H = attn.heads
    src = x if ctx is None else ctx
    q = attn.to_q(x).view(-1, H, 128).float().cpu()
    k = attn.to_k(src).view(-1, H, 128).float().cpu()
    v = attn.to_v(src).view(-1, H, 128).float().cpu()
    qw, kw = attn.norm_q.weight.float().cpu(), attn.norm_k.weight.float().cpu()
    if ctx is None:
        o = O.joint_attention(q, k, v, pos, mode, csr=csr, q_weight=qw, k_weight=kw)
    else:
        o = O.attention(O.rms_norm(q, qw), O.rms_norm(k, kw), v)
    o = o.reshape(1, x.shape[1], -1).to(x)
    return attn.to_out[0](o)


@pytest.fixture(scope="module")
def setup(lib):
    assert torch.cuda.is_available()
    torch.manual_seed(3)
    torch.backends.cuda.matmul.allow_tf32 = False
    attn = StubAttention(256, 2).cuda().bfloat16()
    grid, n_audio = (4, 8, 8), 64
    pos = O.make_positions(grid, n_audio)
    x = torch.randn(1, pos.shape[0], 256, device="cuda").bfloat16()
    return attn, x, pos, grid, n_audio


@torch.no_grad()
def test_self_attention_with_position_ids(setup):
    from pika_h3_flex_b200.processor import B200AttnProcessor

    attn, x, pos, _, _ = setup
    proc = B200AttnProcessor()
    y = proc(attn, x, position_ids=pos.cuda(), token_tags=None, timestep_indices=None)  # extra kwargs pass through
    ref = oracle_forward(attn, x, None, pos)
    assert y.shape == x.shape and y.dtype == x.dtype
    assert float((y.float() - ref.float()).abs().max()) < 3e-2
    # the table is cached per position GRID: the reference makes a new device copy of its layout every forward
    # (src/pika_h3/core/wrapper.py:164-166), so an equal-valued but distinct tensor must hit
    c = proc._rope_cache
    assert len(c) == 1 and c.misses == 1
    p2 = pos.cuda()
    proc(attn, x, position_ids=p2)
    assert len(c) == 1 and c.misses == 1 and c.content_hits == 1
    proc(attn, x, position_ids=p2)  # the same tensor object again (the next block of the same forward): identity hit
    assert c.hits == 1 and c.content_hits == 1
    del p2
    other = pos.cuda() + 1.0
    proc(attn, x, position_ids=other)
    assert len(c) == 2 and c.misses == 2
    proc(attn, x, position_ids=(pos.cuda() + 2.0))
    assert len(c) == 2  # two grids are kept


@torch.no_grad()
def test_self_attention_with_cos_sin_tuple_and_modes(setup):
    from pika_h3_flex_b200 import build_block_index
    from pika_h3_flex_b200.processor import B200AttnProcessor

    attn, x, pos, grid, n_audio = setup
    cos, sin = O.rope_table(pos)
    full = (cos.float().repeat_interleave(2, dim=1).cuda(), sin.float().repeat_interleave(2, dim=1).cuda())
    ref = oracle_forward(attn, x, None, pos)
    y = B200AttnProcessor()(attn, x, image_rotary_emb=full)
    assert float((y.float() - ref.float()).abs().max()) < 3e-2
    y8 = B200AttnProcessor("fp8_qk")(attn, x, image_rotary_emb=(cos.float().cuda(), sin.float().cuda()))
    assert float(((y8.float() - ref.float()).norm() / ref.float().norm())) < 8e-2
    bi = build_block_index(grid, n_audio, (1, 2, 2))
    ys = B200AttnProcessor("block_sparse", bi.to("cuda"))(attn, x, position_ids=pos.cuda())
    refs = oracle_forward(attn, x, None, pos, "block_sparse", (bi.row_ptr.numpy(), bi.col_idx.numpy()))
    assert float((ys.float() - refs.float()).abs().max()) < 3e-2


@torch.no_grad()
def test_cross_attention_to_text_tokens(setup):
    from pika_h3_flex_b200.processor import B200AttnProcessor

    _, x, _, _, _ = setup
    torch.manual_seed(4)
    attn = StubAttention(256, 2, ctx_dim=512).cuda().bfloat16()
    text = torch.randn(1, 77, 512, device="cuda").bfloat16()
    y = B200AttnProcessor()(attn, x, encoder_hidden_states=text)
    ref = oracle_forward(attn, x, text, None)
    assert float((y.float() - ref.float()).abs().max()) < 3e-2


def test_processor_rejects_what_it_cannot_do(setup):
    from pika_h3_flex_b200.processor import B200AttnProcessor

    attn, x, pos, _, _ = setup
    proc = B200AttnProcessor()
    with pytest.raises(NotImplementedError):
        proc(attn, x, attention_mask=torch.ones(1, 1, device="cuda"))
    with pytest.raises(ValueError):
        proc(attn, torch.cat([x, x]), position_ids=pos.cuda())
    with pytest.raises(RuntimeError):
        proc(attn, x.cpu(), position_ids=pos)
    with pytest.raises(ValueError):
        B200AttnProcessor("block_sparse")


@torch.no_grad()
def test_processor_refuses_norms_it_does_not_implement(setup):
    """The library's preparation is a per-head RMSNorm with one [128] weight.  A norm across heads ([heads * 128]
    weight), a LayerNorm, a norm with a bias, or a module without norm_q / norm_k (unless qk_norm=True asks for the
    unit-weight norm) must raise instead of silently computing something else."""
    import copy

    from pika_h3_flex_b200.processor import B200AttnProcessor

    attn, x, pos, _, _ = setup
    proc = B200AttnProcessor()
    wide = copy.deepcopy(attn)
    wide.norm_q.weight = nn.Parameter(torch.ones(attn.heads * 128, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(NotImplementedError, match="across heads"):
        proc(wide, x, position_ids=pos.cuda())
    ln = copy.deepcopy(attn)
    ln.norm_k = nn.LayerNorm(128).cuda().bfloat16()
    with pytest.raises(NotImplementedError, match="LayerNorm"):
        proc(ln, x, position_ids=pos.cuda())
    biased = copy.deepcopy(attn)
    biased.norm_q.bias = nn.Parameter(torch.zeros(128, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(NotImplementedError, match="bias"):
        proc(biased, x, position_ids=pos.cuda())
    bare = copy.deepcopy(attn)
    bare.norm_q = bare.norm_k = None
    with pytest.raises(NotImplementedError, match="qk_norm=True"):
        proc(bare, x, position_ids=pos.cuda())
    y = B200AttnProcessor(qk_norm=True)(bare, x, position_ids=pos.cuda())  # on purpose: unit-weight per-head RMSNorm
    H = attn.heads
    q, k, v = (m(x).view(-1, H, 128).float().cpu() for m in (bare.to_q, bare.to_k, bare.to_v))
    ref = bare.to_out[0](O.joint_attention(q, k, v, pos, "dense").reshape(1, x.shape[1], -1).to(x))
    assert float((y.float() - ref.float()).abs().max()) < 3e-2


@torch.no_grad()
@pytest.mark.parametrize("factor,fixed", [(1.5, True), (2.3, True), (4.0, False)])
def test_learned_norm_weights_of_growing_size(factor, fixed):
    """norm_q / norm_k weights (1 + 0.1 N(0,1), largest about 1.27) scaled by 1.5, 2.3 and 4: the bound from the weights
    (128 max|w_q| max|w_k| / sqrt(128)) is about 40, 100 and 290.  Up to 110 the launch keeps the fixed softmax reference
    (beyond 64 with the row-sum check as its safety net); above, it is the online softmax, on CTA pairs at this length
    (18 key tiles).  All must match the oracle: up to sixteen times the usual logit scale gives peaked rows and outputs
    of order one."""
    from pika_h3_flex_b200 import ops
    from pika_h3_flex_b200.processor import B200AttnProcessor

    torch.manual_seed(5)
    attn = StubAttention(256, 2).cuda().bfloat16()
    attn.norm_q.weight.mul_(factor)
    attn.norm_k.weight.mul_(factor)
    grid, n_audio = (8, 16, 16), 256  # 2,304 tokens
    pos = O.make_positions(grid, n_audio)
    x = torch.randn(1, pos.shape[0], 256, device="cuda").bfloat16()
    proc = B200AttnProcessor()
    y = proc(attn, x, position_ids=pos.cuda())
    proc.check_status()
    bound = ops.normed_logit_bound(attn.norm_q.weight, attn.norm_k.weight)
    ch = ops.kernel_choice(pos.shape[0], pos.shape[0], 2, logit_bound=bound)
    assert ch["cta_pairs"] and ch["fixed_reference"] == fixed and (bound <= 110.0) == fixed, (bound, ch)
    ref = oracle_forward(attn, x, None, pos).float()
    # logits of up to +-100: the bf16 rounding of the prepared Q and K alone moves a logit by several hundredths, i.e. the
    # weights of near-tied keys by several per cent; the bounds below are what that allows at outputs of order one
    assert float((y.float() - ref).abs().max()) < 0.15
    assert float((y.float() - ref).norm() / ref.norm()) < 2e-2


@torch.no_grad()
def test_processor_surfaces_a_wait_that_gave_up(setup):
    """Every launch of a processor carries the processor's own status word.  A bounded wait that runs out (made to
    run out here with the library's self-test, on that very word) is raised by check_status() as H3A_ERR_TIMEOUT,
    launches made while the word is set do nothing, and after a reset the processor works again."""
    import pika_h3_flex_b200 as h3
    from pika_h3_flex_b200.processor import B200AttnProcessor

    attn, x, pos, _, _ = setup
    proc = B200AttnProcessor()
    y0 = proc(attn, x, position_ids=pos.cuda())
    proc.check_status()  # clean
    word = proc.status.tensor()
    lib = h3._lib.load()
    assert lib.h3a_selftest_wait_timeout(word.data_ptr(), 5_000_000, torch.cuda.current_stream().cuda_stream) == 0
    with pytest.raises(h3.H3AError) as ei:
        proc.check_status()
    assert ei.value.status == h3._lib.H3A_ERR_TIMEOUT
    with pytest.raises(h3.H3AError):
        B200AttnProcessor(status=proc.status, check_every_call=True)(attn, x, position_ids=pos.cuda())
    proc.status.reset()
    y1 = proc(attn, x, position_ids=pos.cuda())
    proc.check_status()
    assert torch.equal(y0, y1)


class PeftLikeLinear(nn.Module):
    """The attribute layout of PEFT's lora.Linear: base_layer, lora_A / lora_B ModuleDicts keyed by adapter name,
    a scaling dict, lora_dropout, merged / disable_adapters flags."""

    def __init__(self, din, dout, r=16, alpha=8.0):
        super().__init__()
        self.base_layer = nn.Linear(din, dout, bias=True)
        self.lora_A = nn.ModuleDict({"default": nn.Linear(din, r, bias=False)})
        self.lora_B = nn.ModuleDict({"default": nn.Linear(r, dout, bias=False)})
        self.lora_dropout = nn.ModuleDict({"default": nn.Identity()})
        self.scaling = {"default": alpha / r}
        self.active_adapters = ["default"]
        self.merged = False
        self.disable_adapters = False

    def forward(self, x):
        return self.base_layer(x) + self.scaling["default"] * self.lora_B["default"](self.lora_A["default"](x))


@torch.no_grad()
@pytest.mark.parametrize("wrapper", ["stub", "peft_like", "plain"])
def test_fused_projection_matches_module_calls(setup, wrapper):
    """fused_projection=True: to_q / to_k / to_v run through the library's GEMM with norm + rotation in its epilogue;
    the result must match the processor that calls the modules (and the oracle)."""
    from pika_h3_flex_b200 import build_block_index
    from pika_h3_flex_b200.processor import B200AttnProcessor, _linear_parts

    attn0, x, pos, grid, n_audio = setup
    torch.manual_seed(11)
    attn = StubAttention(256, 2).cuda().bfloat16()
    if wrapper != "stub":
        mk = (lambda i, o: PeftLikeLinear(i, o)) if wrapper == "peft_like" else (lambda i, o: nn.Linear(i, o))
        attn.to_q, attn.to_k, attn.to_v = (mk(256, 256).cuda().bfloat16() for _ in range(3))
    assert all(_linear_parts(m) is not None for m in (attn.to_q, attn.to_k, attn.to_v))
    ref = oracle_forward(attn, x, None, pos)
    y_mod = B200AttnProcessor()(attn, x, position_ids=pos.cuda())
    y_fused = B200AttnProcessor(fused_projection=True)(attn, x, position_ids=pos.cuda())
    assert float((y_fused.float() - ref.float()).abs().max()) < 3e-2
    assert float((y_fused.float() - y_mod.float()).abs().max()) < 3e-2
    bi = build_block_index(grid, n_audio, (1, 2, 2))
    ys = B200AttnProcessor("block_sparse", bi.to("cuda"), fused_projection=True, rope_half=True)(attn, x, position_ids=pos.cuda())
    ym = B200AttnProcessor("block_sparse", bi.to("cuda"), rope_half=True)(attn, x, position_ids=pos.cuda())
    assert float((ys.float() - ym.float()).abs().max()) < 3e-2
    # FP8-QK: the quantisation runs in the GEMM epilogue too
    y8 = B200AttnProcessor("fp8_qk", fused_projection=True)(attn, x, position_ids=pos.cuda())
    assert float(((y8.float() - ref.float()).norm() / ref.float().norm())) < 8e-2


@torch.no_grad()
def test_merged_lora_projection_is_one_launch_and_agrees(setup):
    """merge_lora=True: the LoRA update is folded into a bf16 copy of the base weight once per module; the projection
    then needs no thin matmul in front.  Results agree with the un-merged form to the rounding of the merged weight."""
    from pika_h3_flex_b200.processor import B200AttnProcessor

    _, x, pos, _, _ = setup
    torch.manual_seed(12)
    attn = StubAttention(256, 2).cuda().bfloat16()
    attn.to_q, attn.to_k, attn.to_v = (PeftLikeLinear(256, 256).cuda().bfloat16() for _ in range(3))
    ref = oracle_forward(attn, x, None, pos)
    apart = B200AttnProcessor(fused_projection=True)
    merged = B200AttnProcessor(fused_projection=True, merge_lora=True)
    y_a = apart(attn, x, position_ids=pos.cuda())
    y_m = merged(attn, x, position_ids=pos.cuda())
    assert len(merged._merged_w) == 4 and len(merged._scaled_b) == 0 and len(apart._merged_w) == 0  # to_q, to_k, to_v, to_out.0
    assert float((y_m.float() - ref.float()).abs().max()) < 3e-2
    assert float((y_m.float() - y_a.float()).abs().max()) < 3e-2
    w0 = merged._merged_w[next(iter(merged._merged_w))]
    y_m2 = merged(attn, x, position_ids=pos.cuda())  # the merged weights are reused
    assert len(merged._merged_w) == 4 and merged._merged_w[next(iter(merged._merged_w))] is w0 and torch.equal(y_m, y_m2)
    merged.forget_merged()
    assert len(merged._merged_w) == 0
    merged.check_status()


@torch.no_grad()
def test_fused_projection_cross_attention(setup):
    from pika_h3_flex_b200.processor import B200AttnProcessor

    _, x, _, _, _ = setup
    torch.manual_seed(4)
    attn = StubAttention(256, 2, ctx_dim=512).cuda().bfloat16()
    text = torch.randn(1, 77, 512, device="cuda").bfloat16()
    y = B200AttnProcessor(fused_projection=True)(attn, x, encoder_hidden_states=text)
    ref = oracle_forward(attn, x, text, None)
    assert float((y.float() - ref.float()).abs().max()) < 3e-2


def test_unrecognised_projection_modules_fall_back_to_the_module_call(setup):
    from pika_h3_flex_b200.processor import _linear_parts

    assert _linear_parts(nn.Sequential(nn.Linear(8, 8))) is None
    two = PeftLikeLinear(8, 8)
    two.lora_A["other"] = nn.Linear(8, 16, bias=False)
    two.lora_B["other"] = nn.Linear(16, 8, bias=False)
    two.active_adapters = ["default", "other"]
    assert _linear_parts(two) is None  # two active adapters: not taken apart
    merged = PeftLikeLinear(8, 8)
    merged.merged = True
    assert _linear_parts(merged)[2] is None  # merged: the base weight already holds the update


_SP_CHILD = r"""
import os, sys, importlib.util, torch, torch.distributed as dist
sys.path.insert(0, {root!r})
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
spec = importlib.util.spec_from_file_location("stubs", {this!r})
stubs = importlib.util.module_from_spec(spec)
spec.loader.exec_module(stubs)
from oracle import oracle as O
from pika_h3_flex_b200 import build_block_index
from pika_h3_flex_b200.processor import B200AttnProcessor
torch.manual_seed(3)
torch.backends.cuda.matmul.allow_tf32 = False
attn = stubs.StubAttention(256, 3).cuda().bfloat16()      # 3 heads on 2 ranks: padded to 4
grid, n_audio = (4, 8, 8), 256
pos = O.make_positions(grid, n_audio)
S = pos.shape[0]
x = torch.randn(1, S, 256, device="cuda").bfloat16()
Ss = S // world
sl = slice(rank * Ss, (rank + 1) * Ss)
bi = build_block_index(grid, n_audio, (1, 2, 2)).to("cuda")
ok = True
with torch.no_grad():
    for mode, idx in (("dense_bf16", None), ("fp8_qk", None), ("block_sparse", bi)):
        whole = B200AttnProcessor(mode, idx)(attn, x, position_ids=pos.cuda())
        shard = B200AttnProcessor(mode, idx, sequence_parallel=True)(attn, x[:, sl].contiguous(), position_ids=pos[sl].cuda())
        err = float((shard.float() - whole[:, sl].float()).abs().max())
        print(rank, mode, err, flush=True)
        ok = ok and tuple(shard.shape) == (1, Ss, 256) and err < (6e-2 if mode == "fp8_qk" else 2e-2)
        # projections through the library's GEMM, prepared operands on the wire
        fused = B200AttnProcessor(mode, idx, sequence_parallel=True, fused_projection=True)(attn, x[:, sl].contiguous(), position_ids=pos[sl].cuda())
        errf = float((fused.float() - whole[:, sl].float()).abs().max())
        print(rank, mode, "fused", errf, flush=True)
        ok = ok and errf < (8e-2 if mode == "fp8_qk" else 3e-2)
    text = torch.randn(1, 77, 256, device="cuda").bfloat16()
    c_whole = B200AttnProcessor()(attn, x, encoder_hidden_states=text)
    c_shard = B200AttnProcessor(sequence_parallel=True)(attn, x[:, sl].contiguous(), encoder_hidden_states=text)
    ok = ok and float((c_shard.float() - c_whole[:, sl].float()).abs().max()) < 2e-2
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.destroy_process_group()
sys.exit(0 if int(flag.item()) == 1 else 1)
"""


def test_sequence_parallel_processor_matches_single_gpu(tmp_path):
    """Two ranks as child processes (NCCL): the processor with ``sequence_parallel=True`` on each rank's shard of
    the packed sequence returns that shard of what the single-GPU processor returns (all three modes, padded
    heads, cross-attention without an exchange)."""
    import os
    import socket
    import subprocess
    import sys

    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "child.py"
    script.write_text(_SP_CHILD.format(root=root, this=os.path.abspath(__file__)))
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
