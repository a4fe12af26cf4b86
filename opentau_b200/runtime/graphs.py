"""CUDA-graph replay of fixed-shape inference functions.

The reference removes the launch overhead of the 10 x 18-layer denoise loop with
``torch.compile(mode="reduce-overhead")`` (OpenTau ``src/opentau/scripts/benchmark_inference.py:249-259``).
Here the whole sampler (prefix pass + Euler loop) is a sequence of hand-written kernels with static
shapes, so it is captured once per input signature and replayed: one graph launch per action chunk.
"""

from __future__ import annotations

from typing import Any, Callable, Sequence

import torch
from torch import Tensor


def _signature(args: Sequence[Any]) -> tuple:
    sig = []
    for a in args:
        if isinstance(a, Tensor):
            sig.append((tuple(a.shape), a.dtype, str(a.device)))
        elif isinstance(a, (list, tuple)):
            sig.append(_signature(a))
        else:
            sig.append(a)
    return tuple(sig)


def _clone_static(a: Any) -> Any:
    if isinstance(a, Tensor):
        return a.clone()
    if isinstance(a, (list, tuple)):
        return type(a)(_clone_static(x) for x in a)
    return a


def _copy_into(dst: Any, src: Any) -> None:
    if isinstance(dst, Tensor):
        dst.copy_(src, non_blocking=True)
    elif isinstance(dst, (list, tuple)):
        for d, s in zip(dst, src):
            _copy_into(d, s)


class CudaGraphRunner:
    """Wraps ``fn(*tensors) -> Tensor | tuple``; each new input signature is warmed up eagerly, captured,
    then replayed.  Outputs are returned as views of the graph's static output buffers: copy them if they
    must survive the next call."""

    def __init__(self, fn: Callable, warmup: int = 2):
        self.fn, self.warmup = fn, warmup
        self._graphs: dict[tuple, tuple] = {}

    def __call__(self, *args):
        key = _signature(args)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(args)
            self._graphs[key] = entry
        graph, static_in, static_out, n_kernels = entry
        _copy_into(static_in, args)
        graph.replay()
        from ..ops import cuda_ops
        cuda_ops.launch_count += n_kernels     # the replay runs every kernel node recorded at capture
        return static_out

    def _capture(self, args):
        static_in = _clone_static(args)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self.warmup):       # lazy one-time set-up (attributes, status word) happens here
                self.fn(*static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        from ..ops import cuda_ops
        graph = torch.cuda.CUDAGraph()
        before = cuda_ops.launch_count
        with torch.cuda.graph(graph):
            static_out = self.fn(*static_in)
        n_kernels = cuda_ops.launch_count - before
        cuda_ops.launch_count = before         # capture records, it does not run
        return graph, static_in, static_out, n_kernels

    @property
    def num_graphs(self) -> int:
        return len(self._graphs)
