"""Executors of the dynamic-batching serving runtime: one thread per device pulls merged batches from the native batching queue,
asks the resource manager for an in-flight slot, runs the predict module and routes the per-request slices of the result back.
Counterpart of the reference's legacy runtime (``torchrec/inference/inference_legacy/src/GPUExecutor.cpp:134-153``): batches are
rejected when no slot frees up in time or the executor is shutting down, instead of queueing without bound."""
from __future__ import annotations

import threading
from typing import Callable, List, Optional

import torch
from torch import nn

from torchrec_b200.ops import _ext
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class BatchingExecutor:
    """``module(dense [B, n], KJT) -> [B, k]`` served through ``torch.classes.trb_inference.BatchingQueue``.

    Args:
        module: model in eval mode on ``devices[i]`` (one replica per device is built with ``replicate``).
        feature_names: keys of the sparse features, in the order requests carry them.
        devices: serving devices (``cpu`` works for tests).
        max_batch_size / batching_timeout_ms: a batch is formed when this many samples wait or the oldest has waited this long.
        max_outstanding_batches: in-flight batches allowed per device.
    """

    def __init__(self, module: nn.Module, feature_names: List[str], devices: List[torch.device], max_batch_size: int = 2048, batching_timeout_ms: int = 5,
                 max_outstanding_batches: int = 2, replicate: Optional[Callable[[nn.Module, torch.device], nn.Module]] = None) -> None:
        assert _ext.has_cpu_ext(), f"native host library unavailable: {_ext.cpu_error()}"
        self._feature_names = list(feature_names)
        self._devices = list(devices)
        self._queue = torch.classes.trb_inference.BatchingQueue(max_batch_size, batching_timeout_ms, len(devices), len(feature_names),
                                                                any(d.type == "cuda" for d in devices))
        self._resources = torch.classes.trb_inference.ResourceManager(len(devices), max_outstanding_batches)
        replicate = replicate or (lambda m, d: m.to(d))
        self._modules = [module if i == 0 and next(module.parameters(), torch.empty(0)).device == d else replicate(module, d) for i, d in enumerate(devices)]
        self._stop = threading.Event()
        self.rejected_batches = 0
        self._threads = [threading.Thread(target=self._run, args=(i,), name=f"trb-executor-{i}", daemon=True) for i in range(len(devices))]
        for t in self._threads:
            t.start()

    # ---- client side ---------------------------------------------------------------------------------------------
    def predict(self, dense: torch.Tensor, kjt: KeyedJaggedTensor, timeout_ms: int = 10000) -> torch.Tensor:
        """Blocking call from a client thread: enqueue one request, wait for its slice of the batched result."""
        assert kjt.keys() == self._feature_names
        rid = self._queue.add_request(dense.cpu().float(), kjt.lengths().cpu().long().view(-1), kjt.values().cpu().long())
        out = self._queue.wait_result(rid, timeout_ms)
        if out.numel() == 0 and dense.shape[0] > 0:
            raise TimeoutError(f"request {rid} was rejected or timed out")
        return out

    # ---- executor threads ---------------------------------------------------------------------------------------------
    @torch.no_grad()
    def _run(self, idx: int) -> None:
        dev, module = self._devices[idx], self._modules[idx]
        if dev.type == "cuda":
            torch.cuda.set_device(dev)
        while not self._stop.is_set():
            dense, lengths, values, rids, sizes = self._queue.get_batch(idx, 50)
            if rids.numel() == 0:
                continue
            if self._stop.is_set() or not self._resources.occupy(idx, 100):
                self.rejected_batches += 1
                self._queue.set_results(rids, sizes, torch.empty(0, 1))  # clients see an empty result: rejected
                continue
            try:
                B = int(sizes.sum())
                kjt = KeyedJaggedTensor(keys=self._feature_names, values=values.to(dev, non_blocking=True), lengths=lengths.to(dev, non_blocking=True), stride=B)
                out = module(dense.to(dev, non_blocking=True), kjt)
                out = out.float().reshape(B, -1).cpu()
                self._queue.set_results(rids, sizes, out)
            except Exception:
                self._queue.set_results(rids, sizes, torch.empty(0, 1))
            finally:
                self._resources.release(idx)

    @property
    def batches_formed(self) -> int:
        return int(self._queue.batches_formed())

    @property
    def peak_outstanding(self) -> List[int]:
        return [int(self._resources.peak(i)) for i in range(len(self._devices))]

    def shutdown(self) -> None:
        self._stop.set()
        for t in self._threads:
            t.join(timeout=2)
        self._queue.stop()
