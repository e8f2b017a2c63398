"""Quantized DLRM-DCNv2 inference latency: 26 tables of dim 128 with int8 row-wise quantized weights (fp16 scale and bias per
row; ``--int4-big`` stores the four 40M-row tables in int4), dense towers in 16-bit, requests of 2048 samples with the training
configuration's pooling factors and Zipf(1.05) ids.  Every request is copied from pinned host memory, run, and its predictions
are read back; p50 / p99 latency are over device-timed requests, QPS is requests per second with requests issued back to back.

    python -m torchrec_b200.distributed.benchmark.benchmark_quant_inference --requests 300 --warmup 20
"""
from __future__ import annotations

import argparse
import json
import time
from typing import List

import torch

ROWS = [40000000, 39060, 17295, 7424, 20265, 3, 7122, 1543, 63, 40000000, 3067956, 405282, 10, 2209, 11938, 155, 4, 976, 14, 40000000, 40000000, 40000000,
        590152, 12973, 108, 36]
POOLING = [3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1]


def _fill_quantized(weight: torch.Tensor, gen: torch.Generator) -> None:
    """Random payload, scale 1/128 and bias -1 in the trailing fp16 pair of every row."""
    rows = weight.shape[0]
    step = 4_000_000
    tail = torch.tensor([1.0 / 128, -1.0], dtype=torch.float16).view(torch.uint8).to(weight.device)
    for lo in range(0, rows, step):
        hi = min(rows, lo + step)
        weight[lo:hi].random_(0, 256, generator=gen)
        weight[lo:hi, -4:] = tail


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--requests", type=int, default=300)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--request-size", type=int, default=2048)
    p.add_argument("--int4-big", action="store_true", help="int4 for the four 40M-row tables")
    p.add_argument("--row-cap", type=int, default=0, help="cap table rows (smoke runs)")
    p.add_argument("--gpus", type=int, default=1, help="place the tables table-wise over this many GPUs of one process; requests arrive at GPU 0, "
                   "every GPU's lookup kernel stores its pooled rows straight into GPU 0's buffer")
    p.add_argument("--cuda-graph", action="store_true", help="replay the forward as one CUDA graph (static buffers) instead of launching it eagerly")
    a = p.parse_args()

    from torchrec_b200.datasets.random import RandomRecDataset
    from torchrec_b200.models.dlrm import DLRM_DCN
    from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig
    from torchrec_b200.ops import _ext, dense_ops
    from torchrec_b200.quant.embedding_modules import EmbeddingBagCollection as QuantEmbeddingBagCollection

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    _ext.require_cuda_ext("benchmark_quant_inference")
    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    rows = [min(r, a.row_cap) if a.row_cap else r for r in ROWS]
    keys = [f"cat_{i}" for i in range(len(rows))]
    tables = [EmbeddingBagConfig(name=f"t_{k}", embedding_dim=128, num_embeddings=r, feature_names=[k],
                                 data_type=DataType.INT4 if (a.int4_big and r >= 40_000_000) else DataType.INT8) for k, r in zip(keys, rows)]
    sharded_serving = a.gpus > 1
    # several GPUs: the unsharded module only describes the tables (meta device); every shard is created and filled on its own GPU
    qebc = QuantEmbeddingBagCollection(tables=tables, is_weighted=False, device=torch.device("meta") if sharded_serving else device, output_dtype=torch.bfloat16)
    if not sharded_serving:
        gen = torch.Generator(device=device).manual_seed(7)
        for m in qebc.embedding_bags.values():
            _fill_quantized(m.weight, gen)
    torch.manual_seed(0)
    model = DLRM_DCN(qebc, dense_in_features=13, dense_arch_layer_sizes=[512, 256, 128], over_arch_layer_sizes=[1024, 1024, 512, 256, 1], dcn_num_layers=3,
                     dcn_low_rank_dim=512, dense_device=device).eval()
    table_bytes = sum(t.num_embeddings * (t.embedding_dim * (4 if t.data_type == DataType.INT4 else 8) // 8 + 4) for t in tables)
    if sharded_serving:
        from torchrec_b200.distributed.quant_embeddingbag import ShardedQuantEmbeddingBagCollection
        from torchrec_b200.distributed.types import ParameterSharding, ShardingEnv

        assert not a.cuda_graph, "the multi-GPU path is launched eagerly"
        # largest tables first, each onto the GPU that holds the fewest bytes so far
        load = [0] * a.gpus
        plan = {}
        for t in sorted(tables, key=lambda t: -t.num_embeddings):
            r = min(range(a.gpus), key=lambda i: load[i])
            load[r] += t.num_embeddings * 132
            plan[t.name] = ParameterSharding(sharding_type="table_wise", compute_kernel="quant", ranks=[r])
        sharded = ShardedQuantEmbeddingBagCollection(qebc, plan, ShardingEnv.from_local(world_size=a.gpus, rank=0), device=device)
        for r, shard in enumerate(sharded._shards):
            if hasattr(shard, "embedding_bags"):
                gen_r = torch.Generator(device=torch.device("cuda", r)).manual_seed(7 + r)
                for m in shard.embedding_bags.values():
                    _fill_quantized(m.weight, gen_r)
        model.sparse_arch.embedding_bag_collection = sharded
        qebc = sharded
        for r in range(a.gpus):
            torch.cuda.synchronize(r)

    ds = RandomRecDataset(keys=keys, batch_size=a.request_size, hash_sizes=rows, ids_per_features=POOLING, min_ids_per_features=POOLING, num_dense=13, manual_seed=99,
                          num_generated_batches=16, zipf_s=1.05, idx_dtype=torch.int32, label_positive_rate=0.25, dense_log_transform=True)
    host = [b.pin_memory() for b in ds.batch_generator._generated_batches]
    out_host = torch.empty(a.request_size, dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (host[0].dense_features, host[0].sparse_features.values(), host[0].sparse_features.lengths()))

    class _Scores(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, dense, kjt):
            return torch.sigmoid(self.m(dense, kjt).float()).view(-1)

    scorer = _Scores(model)
    if a.cuda_graph:
        from torchrec_b200.inference.cuda_graph import CudaGraphDenseSparseModule

        b0 = host[0]
        scorer = CudaGraphDenseSparseModule(scorer, b0.dense_features.to(device), b0.sparse_features.to(device))

    @torch.no_grad()
    def serve(i: int) -> None:
        b = host[i % len(host)]
        if a.cuda_graph:
            # the wrapper copies straight from the pinned request into its static buffers
            pred = scorer(b.dense_features, b.sparse_features)
        else:
            pred = scorer(b.dense_features.to(device, non_blocking=True), b.sparse_features.to(device, non_blocking=True))
        out_host.copy_(pred, non_blocking=True)

    for i in range(a.warmup):
        serve(i)
    torch.cuda.synchronize()
    lat: List[float] = []
    for i in range(a.requests):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        serve(i)
        e1.record()
        e1.synchronize()
        lat.append(e0.elapsed_time(e1))
    lat.sort()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.requests):
        serve(i)
    e1.record()
    torch.cuda.synchronize()
    back_to_back_ms = e0.elapsed_time(e1)
    wall = time.perf_counter() - t0
    for part in (qebc._shards if sharded_serving else [qebc]):
        for emb in getattr(part, "_emb_modules", []):
            emb.check_error()
    print(json.dumps({
        "metric": "quantized DLRM-DCNv2 inference latency", "n_gpus": a.gpus, "request_size": a.request_size, "requests": a.requests, "warmup": a.warmup,
        "p50_ms": lat[len(lat) // 2], "p99_ms": lat[min(len(lat) - 1, int(len(lat) * 0.99))], "mean_ms": sum(lat) / len(lat),
        "qps_requests": a.requests / (back_to_back_ms / 1e3), "samples_per_s": a.requests * a.request_size / (back_to_back_ms / 1e3), "host_wall_s": wall,
        "h2d_bytes_per_request": h2d, "d2h_bytes_per_request": a.request_size * 4, "table_bytes": table_bytes,
        "config": {"tables": "26 x dim 128, int8 row-wise" + (" (int4 on the four 40M-row tables)" if a.int4_big else ""), "dense": "bf16 towers on the tcgen05 GEMMs", "launch": "one CUDA graph replay per request" if a.cuda_graph else "eager",
                   "rows": "full" if not a.row_cap else f"capped at {a.row_cap}", "data": "synthetic Zipf(1.05) ids, random quantized weights"}}))


if __name__ == "__main__":
    main()
