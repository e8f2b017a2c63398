"""CUDA-graph capture of a serving forward.

A recommender request at serving batch sizes is bound by kernel launches (tens of small kernels for a few hundred microseconds of
device work), so the whole forward -- lengths-to-offsets scan, quantized lookup, interaction, towers -- is captured once into a
CUDA graph over static input buffers and replayed per request: one launch instead of dozens.

Jagged inputs keep a static *capacity*: ``values`` is a buffer of ``values_capacity`` ids of which a request fills a prefix; the
offsets are computed from the request's lengths inside the graph, so the unused tail is never read.  Requests with more ids than
the capacity, another batch size or other keys fall back to the eager module.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class CudaGraphDenseSparseModule(nn.Module):
    """Wraps ``module(dense [B, n], KJT) -> Tensor`` (e.g. a DLRM in eval mode).

    Args:
        module: the model; called under ``torch.no_grad()``.
        sample_dense / sample_kjt: a representative request (fixes batch size, keys and dtypes).
        values_capacity: ids the static buffer holds (default: 1.5x the sample's count, at least the sample's).
        warmup: eager runs on the capture stream before capturing (lets lazy initialisers and caches settle).
    """

    def __init__(self, module: nn.Module, sample_dense: torch.Tensor, sample_kjt: KeyedJaggedTensor, values_capacity: Optional[int] = None, warmup: int = 3) -> None:
        super().__init__()
        assert sample_dense.is_cuda, "CUDA graphs need CUDA inputs"
        self.module = module
        self._keys = list(sample_kjt.keys())
        self._B = sample_kjt.stride()
        n = sample_kjt.values().numel()
        self._capacity = max(int(values_capacity) if values_capacity is not None else int(n * 1.5) + 1, n)
        self._dense = sample_dense.clone()
        self._values = torch.zeros(self._capacity, dtype=sample_kjt.values().dtype, device=sample_dense.device)
        self._values[:n].copy_(sample_kjt.values())
        self._lengths = sample_kjt.lengths().clone()
        self._weighted = sample_kjt.weights_or_none() is not None
        self._weights = torch.zeros(self._capacity, dtype=torch.float32, device=sample_dense.device) if self._weighted else None
        if self._weighted:
            self._weights[:n].copy_(sample_kjt.weights())
        self._graph: Optional[torch.cuda.CUDAGraph] = torch.cuda.CUDAGraph()
        self.capture_error: Optional[str] = None
        side = torch.cuda.Stream(device=sample_dense.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                self._run_static()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        try:
            with torch.no_grad(), torch.cuda.graph(self._graph):
                self._out = self._run_static()
        except Exception as e:  # a module that synchronises with the host cannot be captured: serve it eagerly
            self._graph = None
            self.capture_error = f"{type(e).__name__}: {e}"
            torch.cuda.synchronize()
        self.replays = 0
        self.fallbacks = 0

    @property
    def captured(self) -> bool:
        return self._graph is not None

    def _run_static(self) -> torch.Tensor:
        kjt = KeyedJaggedTensor(keys=self._keys, values=self._values, lengths=self._lengths, weights=self._weights, stride=self._B)
        return self.module(self._dense, kjt)

    def _fits(self, dense: torch.Tensor, kjt: KeyedJaggedTensor) -> bool:
        return (kjt.keys() == self._keys and kjt.stride() == self._B and dense.shape == self._dense.shape and kjt.values().numel() <= self._capacity
                and (kjt.weights_or_none() is not None) == self._weighted and not kjt.variable_stride_per_key())

    @torch.no_grad()
    def forward(self, dense: torch.Tensor, kjt: KeyedJaggedTensor) -> torch.Tensor:
        """Returns the static output buffer: it is overwritten by the next call, copy it if it must live longer."""
        if self._graph is None or not self._fits(dense, kjt):
            self.fallbacks += 1
            dev = self._dense.device
            return self.module(dense.to(dev, non_blocking=True), kjt.to(dev, non_blocking=True))
        n = kjt.values().numel()
        self._dense.copy_(dense, non_blocking=True)
        self._values[:n].copy_(kjt.values(), non_blocking=True)
        self._lengths.copy_(kjt.lengths(), non_blocking=True)
        if self._weighted:
            self._weights[:n].copy_(kjt.weights(), non_blocking=True)
        self._graph.replay()
        self.replays += 1
        return self._out
