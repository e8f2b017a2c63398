"""C++ dynamic batching queue: requests from several client threads are merged feature-major, executed by a consumer
thread and answered per request (cf. the reference's ``torchrec/inference`` batching tests)."""
import threading

import pytest
import torch

from torchrec_b200.ops import _ext


@pytest.fixture(scope="module", autouse=True)
def _lib():
    if not _ext.has_cpu_ext():
        pytest.skip("native CPU library not built")


def _request(b, F, seed):
    g = torch.Generator().manual_seed(seed)
    dense = torch.randn(b, 3, generator=g)
    lengths = torch.randint(0, 4, (F, b), generator=g)
    values = torch.randint(0, 100, (int(lengths.sum()),), generator=g)
    return dense, lengths.reshape(-1), values


def test_batches_are_feature_major_and_results_routed():
    F = 2
    q = torch.classes.trb_inference.BatchingQueue(8, 200, 1, F, False)
    reqs = [_request(b, F, 10 + i) for i, b in enumerate([3, 2, 3])]  # 8 samples: one full batch
    ids = [q.add_request(*r) for r in reqs]
    dense, lengths, values, rids, sizes = q.get_batch(0, 2000)
    assert rids.tolist() == ids and sizes.tolist() == [3, 2, 3]
    torch.testing.assert_close(dense, torch.cat([r[0] for r in reqs]))
    # expected sparse layout: feature 0 of every request, then feature 1 of every request
    exp_len, exp_val = [], []
    for f in range(F):
        for d, l, v in reqs:
            l2 = l.view(F, -1)
            per_f = l2.sum(1).tolist()
            parts = v.split(per_f)
            exp_len.append(l2[f]); exp_val.append(parts[f])
    assert torch.equal(lengths, torch.cat(exp_len)) and torch.equal(values, torch.cat(exp_val))
    q.set_results(rids, sizes, dense.sum(1, keepdim=True))
    for rid, (d, _, _) in zip(ids, reqs):
        torch.testing.assert_close(q.wait_result(rid, 1000), d.sum(1, keepdim=True))
    q.stop()


def test_timeout_flushes_partial_batch_and_threads():
    F = 1
    q = torch.classes.trb_inference.BatchingQueue(64, 30, 2, F, False)
    stop = threading.Event()

    def executor(idx):
        while not stop.is_set():
            dense, lengths, values, rids, sizes = q.get_batch(idx, 50)
            if rids.numel():
                q.set_results(rids, sizes, dense * 2)

    workers = [threading.Thread(target=executor, args=(i,)) for i in range(2)]
    for w in workers:
        w.start()
    results = {}

    def client(i):
        d, l, v = _request(2, F, 100 + i)
        rid = q.add_request(d, l, v)
        results[i] = (d, q.wait_result(rid, 5000))

    clients = [threading.Thread(target=client, args=(i,)) for i in range(6)]
    for c in clients:
        c.start()
    for c in clients:
        c.join()
    stop.set()
    for w in workers:
        w.join()
    assert len(results) == 6
    for d, out in results.values():
        torch.testing.assert_close(out, d * 2)
    assert q.batches_formed() >= 1
    q.stop()
    with pytest.raises(RuntimeError):
        q.wait_result(12345, 10)


def test_resource_manager_bounds_in_flight_batches():
    rm = torch.classes.trb_inference.ResourceManager(2, 2)
    assert rm.occupy(0, 10) and rm.occupy(0, 10)
    assert not rm.occupy(0, 20)  # third batch on device 0 is refused after the wait
    assert rm.occupy(1, 10)
    assert rm.outstanding(0) == 2 and rm.peak(0) == 2 and rm.rejected() == 1
    t = threading.Timer(0.05, lambda: rm.release(0))
    t.start()
    assert rm.occupy(0, 2000)  # a slot frees up while waiting
    t.join()
    rm.release(0); rm.release(0); rm.release(1)
    with pytest.raises(RuntimeError):
        rm.release(1)


def test_batching_executor_merges_concurrent_clients():
    from torchrec_b200.inference.executor import BatchingExecutor
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    torch.manual_seed(0)

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ebc = EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="t", embedding_dim=4, num_embeddings=50, feature_names=["a", "b"])])
            self.lin = torch.nn.Linear(3 + 8, 2)

        def forward(self, dense, kjt):
            return self.lin(torch.cat([dense, self.ebc(kjt).values()], dim=1))

    m = M().eval()
    ex = BatchingExecutor(m, ["a", "b"], [torch.device("cpu")], max_batch_size=16, batching_timeout_ms=20)
    results = {}

    def client(i):
        g = torch.Generator().manual_seed(i)
        b = 1 + i % 3
        lengths = torch.randint(0, 3, (2 * b,), generator=g)
        kjt = KeyedJaggedTensor(keys=["a", "b"], values=torch.randint(0, 50, (int(lengths.sum()),), generator=g), lengths=lengths)
        dense = torch.randn(b, 3, generator=g)
        got = ex.predict(dense, kjt)
        with torch.no_grad():
            results[i] = (got, m(dense, kjt))

    threads = [threading.Thread(target=client, args=(i,)) for i in range(12)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    ex.shutdown()
    assert len(results) == 12
    for got, want in results.values():
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
    assert ex.batches_formed < 12  # requests were merged
    assert ex.peak_outstanding[0] >= 1 and ex.rejected_batches == 0
