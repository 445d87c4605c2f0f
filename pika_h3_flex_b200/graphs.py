"""The sampler loop around the attention path, with each generator evaluation replayed from a CUDA graph.

The reference samples with six generator evaluations and fresh noise in between
(``few_step_trajectory`` / ``few_step_sample``, reference ``src/pika_h3/core/sampling.py:87-109,160-169``): every
evaluation is one forward of the DiT on the same geometry - the same sequence of kernels on buffers of the same
shapes - launched eagerly, kernel by kernel, from Python.  With the attention at a few milliseconds per block the gaps
between launches start to show, most of all under sequence parallelism.  :class:`StepGraph` captures ONE evaluation
(any callable built from this library's launches and capturable torch operations, e.g. a stack of transformer blocks
whose attention modules carry a ``B200AttnProcessor``) into a CUDA graph and replays it; :func:`renoise_sample` is the
reference's loop around such a step.  What varies between evaluations (the noisy latents, the timestep) lives in static
device buffers that are overwritten before each replay, so the graph never bakes a value in.

Capture rules the step must obey (the processor does, once warmed up): no host synchronisation, no new device
allocation outside torch's caching allocator, every launch on the current stream.  The warm-up runs before the capture
take care of everything that happens once - per-device kernel attributes, the rotary table of the position grid, the
logit bound read from the norm weights, scaled LoRA factors, the status word.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Sequence

import torch


class StepGraph:
    """``StepGraph(fn, example)``: ``fn(**inputs) -> Tensor | tuple[Tensor]`` with ``example`` a dict of device tensors
    of the shapes every call will have.  The inputs are copied into static buffers, ``fn`` runs ``warmup`` times on a
    side stream, then once more under capture.  ``graph(**inputs)`` copies the new values in, replays and returns the
    static output tensor(s), which the next replay overwrites.  Tensors of ``example`` listed in ``constants`` are
    captured by reference instead (weights of a geometry: position grids, block indices), not copied per call."""

    def __init__(self, fn: Callable, example: Dict[str, torch.Tensor], warmup: int = 2, constants: Sequence[str] = ()):
        if not example:
            raise ValueError("a step needs at least one tensor input")
        dev = next(iter(example.values())).device
        if dev.type != "cuda":
            raise RuntimeError("StepGraph captures CUDA work (there is no CPU path)")
        self.fn = fn
        self.constants = set(constants)
        self.static_in = {k: (v if k in self.constants else v.clone()) for k, v in example.items()}
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):
                fn(**self.static_in)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = fn(**self.static_in)
        self.replays = 0

    def __call__(self, **inputs: torch.Tensor):
        for k, v in inputs.items():
            if k in self.constants:
                if v is not self.static_in[k]:
                    raise ValueError(f"{k} was captured by reference: pass the same tensor")
                continue
            dst = self.static_in[k]
            if v.shape != dst.shape or v.dtype != dst.dtype:
                raise ValueError(f"{k}: the graph was captured for {tuple(dst.shape)} {dst.dtype}")
            dst.copy_(v, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_out


def add_noise(x0: torch.Tensor, eps: torch.Tensor, sigma) -> torch.Tensor:
    """``x_t = (1 - sigma) x0 + sigma eps`` in fp32, returned in ``x0``'s dtype (reference
    ``src/pika_h3/core/sampling.py:14-21``)."""
    s = torch.as_tensor(sigma, dtype=torch.float32, device=x0.device)
    return ((1 - s) * x0.float() + s * eps.float()).to(x0.dtype)


@torch.no_grad()
def renoise_sample(step: Callable, x_noise: torch.Tensor, sigmas: Sequence[float], noise_generator: Optional[torch.Generator] = None,
                   **fixed) -> torch.Tensor:
    """The reference's K-evaluation re-noising sampler around ``step(x=..., sigma=..., **fixed) -> x0``: a ladder of
    K + 1 knots ending in 0; for i < K - 1 the prediction is re-noised to the next knot with fresh fp32 noise, the last
    evaluation returns the clean prediction and the terminal 0 is never fed to the model
    (``src/pika_h3/core/sampling.py:87-109,160-169``).  ``step`` is typically a :class:`StepGraph`; ``sigma`` reaches
    it as a one-element fp32 device tensor."""
    sig = [float(s) for s in sigmas]
    if len(sig) < 2 or sig[-1] != 0.0:
        raise ValueError("the ladder must hold K + 1 knots ending in 0")
    K = len(sig) - 1
    x_t = x_noise
    for i in range(K):
        s = torch.full((1,), sig[i], dtype=torch.float32, device=x_noise.device)
        x0 = step(x=x_t, sigma=s, **fixed)
        if i == K - 1:
            return x0.clone()
        eps = torch.randn(x0.shape, device=x0.device, dtype=torch.float32, generator=noise_generator)
        x_t = add_noise(x0, eps, sig[i + 1])
    raise AssertionError("unreachable")
