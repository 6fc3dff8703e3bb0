"""A layer call of fixed shape replayed from a captured CUDA graph.

No counterpart in the reference (whose call synchronises with the host some twenty times and cannot be captured).  A
call of ``AdaptiveSparseAttention`` is a chain of a few dozen launches; at moderate sizes their host cost exceeds their
device time (measured at 4 x 16384 tokens: 1.3 ms per eager call of which 0.9 ms is kernel time).  When the call never
waits for the host - shortlist mode that cannot turn dense (alpha >= 0.95), no keep threshold, candidate pieces within
L - it can be captured once and replayed: the prototype EMA and the other state updates are kernels on the layer's
own buffers and replay with it; the telemetry record is re-armed after every replay and decoded on first access."""
from __future__ import annotations

import torch

from .aspa import AdaptiveSparseAttention


class CapturedLayerCall:
    """``CapturedLayerCall(layer, example)(x)`` == ``layer(x)`` for every ``x`` of the example's shape and dtype.

    The graph is captured on a stream of priority -2, so inside it the routing chain outranks the projection GEMM the
    layer forks onto its second stream.  ``__call__`` copies ``x`` (device or pinned host memory) into the static
    input, replays on the current stream and returns the static output tensor, which the next call overwrites."""

    def __init__(self, layer: AdaptiveSparseAttention, example: torch.Tensor, *, priority: int = -2) -> None:
        if not example.is_cuda:
            raise RuntimeError("the example input must live on the CUDA device the layer is on")
        self.layer = layer
        self.static_in = example.detach().clone()
        stream = torch.cuda.Stream(device=example.device, priority=priority)
        stream.wait_stream(torch.cuda.current_stream())
        state = {n: b.detach().clone() for n, b in layer.named_buffers()}   # EMAs, memory bank: a call moves them
        with torch.no_grad(), torch.cuda.stream(stream):   # eager warm-up on a side stream, as graph capture requires
            for _ in range(2):
                layer(self.static_in)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(example.device)
        pending = layer.__dict__.get("_pending")
        if not (isinstance(pending, dict) and pending.get("lazy")):
            self._restore(state)
            raise RuntimeError("this layer call waits for row counts on the host (alpha < 0.95, a keep threshold, or "
                               "candidate pieces that may exceed L) and cannot be captured into a CUDA graph")
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph, stream=stream):
            self.static_out = layer(self.static_in)
        self._pending = layer.__dict__.get("_pending")
        torch.cuda.synchronize(example.device)
        self._restore(state)   # the warm-up and capture calls moved the state; put it back, in place

    def _restore(self, state) -> None:
        with torch.no_grad():
            for n, b in self.layer.named_buffers():
                b.copy_(state[n])

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape != self.static_in.shape or x.dtype != self.static_in.dtype:
            raise ValueError(f"captured for {tuple(self.static_in.shape)} {self.static_in.dtype}, got {tuple(x.shape)} {x.dtype}")
        self.layer.check_previous_call()   # an expired router wait of the previous replay surfaces here
        if x.data_ptr() != self.static_in.data_ptr():
            self.static_in.copy_(x, non_blocking=True)
        self.graph.replay()
        if self._pending is not None:  # the replay refreshed the pinned record: decode it again on the next telemetry access
            self.layer.__dict__["_pending"] = dict(self._pending)
            self.layer.__dict__["_head_stats_value"] = None
            self.layer.__dict__["_sparse_state_value"] = None
        return self.static_out


class CapturedModelCall:
    """The same for any module that contains ASPA layers (a transformer block, a whole decoder): ``CapturedModelCall(
    model, example)(x)`` == ``model(x)`` for inputs of the example's shape and dtype, replayed from one CUDA graph.

    Every ``AdaptiveSparseAttention`` inside must make a call that never waits for the host at this shape (see
    ``CapturedLayerCall``); otherwise a ``RuntimeError`` is raised before anything is captured and the model is left as
    it was.  Buffers the calls move (prototype EMAs, memory banks) are restored after warm-up and capture; from then on
    every replay moves them as an eager call would.  The static output is overwritten by the next call."""

    def __init__(self, model: torch.nn.Module, example: torch.Tensor, *, priority: int = -2) -> None:
        if not example.is_cuda:
            raise RuntimeError("the example input must live on the CUDA device the model is on")
        self.model = model
        self.layers = [m for m in model.modules() if isinstance(m, AdaptiveSparseAttention)]
        self.static_in = example.detach().clone()
        stream = torch.cuda.Stream(device=example.device, priority=priority)
        stream.wait_stream(torch.cuda.current_stream())
        state = {n: b.detach().clone() for n, b in model.named_buffers()}
        with torch.no_grad(), torch.cuda.stream(stream):
            for _ in range(2):
                model(self.static_in)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize(example.device)
        for layer in self.layers:
            pending = layer.__dict__.get("_pending")
            if not (isinstance(pending, dict) and pending.get("lazy")):
                self._restore(state)
                raise RuntimeError("a layer of this model waits for row counts on the host at this shape (dense modes, "
                                   "alpha < 0.95, a keep threshold, or candidate pieces that may exceed L): the model "
                                   "cannot be captured into a CUDA graph")
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph, stream=stream):
            self.static_out = model(self.static_in)
        self._pending = [layer.__dict__.get("_pending") for layer in self.layers]
        torch.cuda.synchronize(example.device)
        self._restore(state)

    def _restore(self, state) -> None:
        with torch.no_grad():
            for n, b in self.model.named_buffers():
                b.copy_(state[n])

    def __call__(self, x: torch.Tensor):
        if x.shape != self.static_in.shape or x.dtype != self.static_in.dtype:
            raise ValueError(f"captured for {tuple(self.static_in.shape)} {self.static_in.dtype}, got {tuple(x.shape)} {x.dtype}")
        for layer in self.layers:
            layer.check_previous_call()
        if x.data_ptr() != self.static_in.data_ptr():
            self.static_in.copy_(x, non_blocking=True)
        self.graph.replay()
        for layer, pending in zip(self.layers, self._pending):
            if pending is not None:
                layer.__dict__["_pending"] = dict(pending)
                layer.__dict__["_head_stats_value"] = None
                layer.__dict__["_sparse_state_value"] = None
        return self.static_out
