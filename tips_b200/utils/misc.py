"""Small helpers, the counterpart of tips/tensorflow/utils.py:5-38.

The reference's helpers exist because TensorFlow has two execution modes: ``executing_eagerly`` tells them apart,
``make_subgraph`` turns a Python function into a traced ``tf.function``, ``cache`` memoises on the arguments plus
the eager flag, ``vars_to_refs`` / ``refs_to_vars`` make variables hashable.  Here the two modes are eager
launches and CUDA-graph capture: ``make_subgraph`` captures a function once into a CUDA graph and replays it,
which removes the launch overhead of a step made of many small kernels (the CTR trainer does the same by hand,
models/ctr.py).
"""
from __future__ import annotations

import functools

import torch


def executing_eagerly() -> bool:
    """False while the current CUDA stream is being captured into a graph."""
    return not (torch.cuda.is_available() and torch.cuda.is_current_stream_capturing())


def cache(fn):
    """Memoise `fn` on its (hashable) arguments and on whether a graph capture is under way."""
    memo = {}

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        key = (args, tuple(sorted(kwargs.items())), executing_eagerly())
        if key not in memo:
            memo[key] = fn(*args, **kwargs)
        return memo[key]

    wrapper.cache = memo
    return wrapper


def vars_to_refs(params):
    """Hashable references of parameters (ids), and back."""
    return tuple(id(p) for p in params)


def refs_to_vars(refs, params):
    by_id = {id(p): p for p in params}
    return [by_id[r] for r in refs]


class _Subgraph:
    """A function captured into a CUDA graph: inputs are copied into static buffers, the graph is replayed, the
    static outputs are returned (valid until the next call)."""

    def __init__(self, fn, example_inputs, warmup):
        self.fn = fn
        self.static_in = [t.clone() if isinstance(t, torch.Tensor) else t for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # warm up off the capturing stream: lazy initialisation must not be captured
            for _ in range(max(1, warmup)):
                fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = fn(*self.static_in)
        self.replays = 0

    def __call__(self, *inputs):
        if len(inputs) != len(self.static_in):
            raise TypeError(f"expected {len(self.static_in)} arguments, got {len(inputs)}")
        for dst, src in zip(self.static_in, inputs):
            if isinstance(dst, torch.Tensor):
                if dst.shape != src.shape or dst.dtype != src.dtype:
                    raise ValueError("a captured subgraph takes the shapes and dtypes it was captured with")
                if dst.data_ptr() != src.data_ptr():
                    dst.copy_(src, non_blocking=True)
            elif dst != src:
                raise ValueError("non-tensor arguments of a captured subgraph are constants")
        self.graph.replay()
        self.replays += 1
        return self.static_out


def make_subgraph(fn, *example_inputs, warmup: int = 3):
    """Return a callable that runs `fn(*inputs)` as one CUDA-graph replay.

    `example_inputs` fix the shapes and dtypes.  `fn` must be capture-safe: no host synchronisation, no allocation
    whose address later calls depend on, every kernel on the current stream.  Without CUDA (or without tensor
    arguments on a GPU) `fn` itself is returned, so callers need no second code path."""
    tensors = [t for t in example_inputs if isinstance(t, torch.Tensor)]
    if not torch.cuda.is_available() or not tensors or not all(t.is_cuda for t in tensors):
        return fn
    return _Subgraph(fn, example_inputs, warmup)
