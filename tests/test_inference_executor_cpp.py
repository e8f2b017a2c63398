"""C++ serving runtime: validation, batching functions, result split and the executor threads that run a TorchScript module
on batches from the batching queue (CPU here; the same classes drive a GPU by device index)."""
import os
import tempfile
import threading
import time

import pytest
import torch

from torchrec_b200.ops import _ext

pytestmark = pytest.mark.skipif(not _ext.has_cpu_ext(), reason="native CPU library not built")

F, D = 2, 4


class _Model(torch.nn.Module):
    def forward(self, dense: torch.Tensor, lengths: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
        n = lengths.numel()
        bag = torch.repeat_interleave(torch.arange(n), lengths.to(torch.long))
        sums = torch.zeros(n).index_add_(0, bag, values.to(torch.float32))
        return (dense.sum(1) + sums.view(2, -1).sum(0)).unsqueeze(1)


def _request(seed, b):
    g = torch.Generator().manual_seed(seed)
    dense = torch.randn(b, D, generator=g)
    lengths = torch.randint(0, 4, (F * b,), generator=g)
    values = torch.randint(0, 100, (int(lengths.sum()),), generator=g)
    return dense, lengths, values


def _scripted(tmp):
    path = os.path.join(tmp, "m.pt")
    torch.jit.script(_Model()).save(path)
    return path


def test_executor_serves_concurrent_requests():
    ops = torch.classes.trb_inference
    with tempfile.TemporaryDirectory() as tmp:
        q = ops.BatchingQueue(64, 5, 1, F, False)
        ex = ops.GPUExecutor(q, _scripted(tmp), -1, 0, 2, 0, "")
        results = {}

        def client(i):
            dense, lengths, values = _request(i, 1 + i % 5)
            rid = q.add_request(dense, lengths, values)
            results[i] = (q.wait_result(rid, 5000), _Model()(dense, lengths, values))

        threads = [threading.Thread(target=client, args=(i,)) for i in range(40)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        for i, (got, want) in results.items():
            torch.testing.assert_close(got, want)
        st = ex.stats()
        assert st["requests"] == 40 and st["batches"] >= 1 and st["rejected_batches"] == 0 and st["failed_batches"] == 0
        assert st["batches"] < 40, "requests were not batched"
        ex.stop()
        q.stop()


def test_executor_rejects_batches_that_waited_too_long():
    ops = torch.classes.trb_inference
    with tempfile.TemporaryDirectory() as tmp:
        q = ops.BatchingQueue(8, 1, 1, F, False)
        rid = q.add_request(*_request(0, 2))
        time.sleep(0.2)  # the batch is formed and then sits in the executor queue
        ex = ops.GPUExecutor(q, _scripted(tmp), -1, 0, 1, 20, "")
        with pytest.raises(RuntimeError, match="rejected"):
            q.wait_result(rid, 5000)
        assert ex.stats()["rejected_batches"] == 1
        ex.stop()
        q.stop()


def test_validation_batching_and_result_split():
    ops = torch.ops.trb_inference
    dense, lengths, values = _request(3, 4)
    assert ops.validate_sparse(values, lengths, None) == ""
    assert "differs" in ops.validate_sparse(values[:-1], lengths, None) or lengths.sum() == 0
    assert "non-negative" in ops.validate_sparse(values, -lengths - 1, None)
    assert ops.validate_dense(dense, 4, D) == "" and "expected" in ops.validate_dense(dense, 5, D)
    # sparse batching: feature-major merge equals what the model sees request by request
    reqs = [_request(10 + i, 1 + i) for i in range(3)]
    merged_len, merged_ids = ops.batch_requests("sparse", [[l, v] for _, l, v in reqs], F)
    merged_dense = ops.batch_requests("dense", [[d] for d, _, _ in reqs], F)[0]
    want = torch.cat([_Model()(*r) for r in reqs])
    torch.testing.assert_close(_Model()(merged_dense, merged_len, merged_ids), want)
    sizes = torch.tensor([1, 2, 3])
    parts = ops.split_dict_of_tensor({"score": want, "aux": want * 2}, sizes)
    assert [p["score"].shape[0] for p in parts] == [1, 2, 3]
    torch.testing.assert_close(torch.cat([p["aux"] for p in parts]), want * 2)
    lists = ops.split_dict_of_tensors({"heads": [want, want + 1]}, sizes)
    assert len(lists) == 3 and len(lists[1]["heads"]) == 2 and lists[1]["heads"][1].shape[0] == 2
    mask = torch.tensor([1, 0, 1, 1, 0, 0])
    masked = ops.split_dict_with_mask_tensor({"score": want}, {"score": mask}, sizes)
    assert [m["score"].shape[0] for m in masked] == [1, 1, 1]
    torch.testing.assert_close(masked[2]["score"], want[3:4])
