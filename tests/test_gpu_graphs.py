"""GPU: one generator evaluation captured as a CUDA graph and the reference's re-noising loop around it
(src/pika_h3/core/sampling.py:87-109,160-169), on a stand-in stack of transformer blocks whose attention runs
through B200AttnProcessor: adaptive layer norm (library kernel) -> attention (fused projections, library kernels) ->
residual.  The replayed loop must reproduce the eager loop bit for bit (same kernels, same inputs, same noise)."""
import importlib.util
import os

import pytest
import torch
import torch.nn as nn

from oracle import oracle as O

pytestmark = pytest.mark.gpu

_spec = importlib.util.spec_from_file_location("proc_stubs", os.path.join(os.path.dirname(os.path.abspath(__file__)), "test_gpu_processor.py"))
stubs = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(stubs)


class Block(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.attn = stubs.StubAttention(dim, heads)
        self.mod = nn.Linear(1, 2 * dim)  # timestep -> (shift, scale), the shape of the reference's modulation tables


class Stack(nn.Module):
    def __init__(self, dim, heads, n_blocks, proc):
        super().__init__()
        self.blocks = nn.ModuleList([Block(dim, heads) for _ in range(n_blocks)])
        self.proc = proc

    def forward(self, x, sigma, pos):
        import pika_h3_flex_b200 as h3

        h = x
        for b in self.blocks:
            shift, scale = (0.1 * b.mod(sigma.to(h.dtype).view(1, 1))).chunk(2, dim=-1)  # [1, D] each: one timestep row
            y = h3.adaln_norm(h[0], scale.contiguous(), shift.contiguous(), None)
            h = h + self.proc(b.attn, y[None], position_ids=pos)
        return h


@torch.no_grad()
@pytest.mark.parametrize("mode,fused", [("dense_bf16", True), ("fp8_qk", False)])
def test_captured_step_replays_the_sampler_loop(lib, mode, fused):
    from pika_h3_flex_b200.graphs import StepGraph, renoise_sample
    from pika_h3_flex_b200.processor import B200AttnProcessor

    assert torch.cuda.is_available()
    torch.manual_seed(11)
    dim, heads = 256, 2
    grid, n_audio = (8, 16, 16), 256  # 2,304 tokens: the CTA-pair kernels
    pos = O.make_positions(grid, n_audio).cuda()
    S = pos.shape[0]
    proc = B200AttnProcessor(mode, fused_projection=fused)
    model = Stack(dim, heads, 3, proc).cuda().bfloat16()
    x_noise = torch.randn(1, S, dim, device="cuda").bfloat16()
    sigmas = [1.0, 0.75, 0.5, 0.25, 0.1, 0.04, 0.0]  # the reference's six evaluations (knots 1000 ... 40, 0)

    eager = renoise_sample(lambda x, sigma, pos: model(x, sigma, pos), x_noise, sigmas, torch.Generator(device="cuda").manual_seed(5), pos=pos)
    proc.check_status()
    step = StepGraph(model, {"x": x_noise, "sigma": torch.ones(1, device="cuda"), "pos": pos}, constants=("pos",))
    replayed = renoise_sample(step, x_noise, sigmas, torch.Generator(device="cuda").manual_seed(5), pos=pos)
    proc.check_status()
    assert step.replays == 6
    assert torch.isfinite(replayed.float()).all()
    assert torch.equal(replayed, eager)
    # a second trajectory through the same graph, other noise: still equal to eager
    x2 = torch.randn(1, S, dim, device="cuda").bfloat16()
    assert torch.equal(renoise_sample(step, x2, sigmas, torch.Generator(device="cuda").manual_seed(6), pos=pos),
                       renoise_sample(lambda x, sigma, pos: model(x, sigma, pos), x2, sigmas, torch.Generator(device="cuda").manual_seed(6), pos=pos))
    with pytest.raises(ValueError):
        step(x=x_noise[:, :100], sigma=torch.ones(1, device="cuda"), pos=pos)
    with pytest.raises(ValueError):
        step(x=x_noise, sigma=torch.ones(1, device="cuda"), pos=pos.clone())

    # launch gaps: eager against replay, one evaluation
    def timed(fn, n=10):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    s1 = torch.ones(1, device="cuda")
    t_eager = timed(lambda: model(x_noise, s1, pos))
    t_graph = timed(lambda: step(x=x_noise, sigma=s1, pos=pos))
    print(f"one evaluation of 3 blocks ({mode}, fused={fused}): eager {t_eager:.3f} ms, graph replay {t_graph:.3f} ms")
    assert t_graph <= t_eager * 1.05
