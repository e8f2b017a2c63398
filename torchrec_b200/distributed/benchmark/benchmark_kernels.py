"""Micro-benchmarks of the hand-written kernels at DLRM-DCNv2 shapes: the tcgen05 GEMMs (plain and fused
epilogues) against ``torch.matmul``/``F.linear`` and the table-batched embedding forward / sort / backward.

    python -m torchrec_b200.distributed.benchmark.benchmark_kernels --op all
    python -m torchrec_b200.distributed.benchmark.benchmark_kernels --op tbe_bwd --small   # profiler-sized case

Times are medians of CUDA-event timings with an L2 flush (a 256 MiB write) before every timed call.
Counterpart of the raw table-batched-embedding benchmark of the reference
(``torchrec/distributed/benchmark/benchmark_split_table_batched_embeddings.py``).
"""
from __future__ import annotations

import argparse
from typing import Callable, List

import torch

DLRM_ROWS = [40000000, 39060, 17295, 7424, 20265, 3, 7122, 1543, 63, 40000000, 3067956, 405282, 10, 2209, 11938, 155, 4, 976,
             14, 40000000, 40000000, 40000000, 590152, 12973, 108, 36]
DLRM_POOLING = [3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1]


def timeit(fn: Callable[[], object], n: int = 10, warm: int = 3) -> float:
    """Median milliseconds of ``fn`` over ``n`` runs after ``warm`` warm-ups, L2 flushed before each run."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda")
    for s, e in evs:
        flush.zero_()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) for s, e in evs)
    return ts[len(ts) // 2]


def bench_gemm_nt(M: int, shapes: List[tuple], n: int, warm: int) -> None:
    ops = torch.ops.trb200
    for (N, K) in shapes:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn(N, K, device="cuda").bfloat16()
        bias = torch.randn(N, device="cuda")
        t0 = timeit(lambda: ops.gemm_nt_bf16(a, b, None, 0, False), n, warm)
        t1 = timeit(lambda: ops.gemm_nt_bf16(a, b, bias, 1, False), n, warm)
        t2 = timeit(lambda: torch.relu(torch.nn.functional.linear(a, b, bias.bfloat16())), n, warm)
        t3 = timeit(lambda: torch.matmul(a, b.t()), n, warm)
        fl = 2 * M * N * K
        print(f"NT  M={M} N={N} K={K}: tcgen05 plain {t0:.3f} ms ({fl / t0 / 1e9:.0f} TF) | tcgen05+bias+relu {t1:.3f} ms ({fl / t1 / 1e9:.0f} TF) | torch linear+relu {t2:.3f} ms | "
              f"matmul only {t3:.3f} ms ({fl / t3 / 1e9:.0f} TF)", flush=True)


def bench_gemm_cross(M: int, D: int, R: int, n: int, warm: int) -> None:
    """The low-rank cross layer's second GEMM with its fused epilogue ``y = x0 * (v W^T + b) + xl``."""
    ops = torch.ops.trb200
    v = torch.randn(M, R, device="cuda").bfloat16()
    w = torch.randn(D, R, device="cuda").bfloat16()
    bias = torch.randn(D, device="cuda")
    x0 = torch.randn(M, D, device="cuda").bfloat16()
    xl = torch.randn(M, D, device="cuda").bfloat16()
    t1 = timeit(lambda: ops.gemm_nt_bf16_cross(v, w, bias, x0, xl), n, warm)
    t2 = timeit(lambda: x0 * torch.nn.functional.linear(v, w, bias.bfloat16()) + xl, n, warm)
    fl = 2 * M * D * R
    byt = 4 * M * D * 2
    print(f"CROSS M={M} N={D} K={R}: tcgen05 fused {t1:.3f} ms ({fl / t1 / 1e9:.0f} TF, {byt / t1 / 1e6:.0f} GB/s epilogue traffic) | "
          f"torch unfused {t2:.3f} ms", flush=True)


def bench_gemm_tn(M: int, shapes: List[tuple], n: int, warm: int) -> None:
    ops = torch.ops.trb200
    for (N, K) in shapes:
        a = torch.randn(M, N, device="cuda").bfloat16()
        b = torch.randn(M, K, device="cuda").bfloat16()
        t1 = timeit(lambda: ops.gemm_tn_bf16(a, b), n, warm)
        t3 = timeit(lambda: torch.matmul(a.t(), b), n, warm)
        fl = 2 * M * N * K
        print(f"TN  Mc={M} N={N} K={K}: tcgen05 {t1:.3f} ms ({fl / t1 / 1e9:.0f} TF) | torch {t3:.3f} ms ({fl / t3 / 1e9:.0f} TF)", flush=True)


def bench_tbe(B: int, row_cap: int, which: str, n: int, warm: int) -> None:
    from torchrec_b200.modules.embedding_configs import PoolingMode
    from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags

    rows = [min(r, row_cap) for r in DLRM_ROWS]
    m = TableBatchedEmbeddingBags(
        [(r, 128) for r in rows], pooling_mode=PoolingMode.SUM, output_dtype=torch.bfloat16,
        optimizer_args=OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.005), device="cuda",
    )
    m.init_embedding_weights_uniform(-0.01, 0.01)
    g = torch.Generator(device="cuda").manual_seed(0)
    idx, lens = [], []
    for r, p in zip(rows, DLRM_POOLING):
        u = torch.rand(B * p, device="cuda", generator=g)
        ids = ((r ** u) - 1).long().clamp(0, r - 1)  # heavy-headed (Zipf-like) ids
        idx.append((ids * 2654435761) % r)
        lens.append(torch.full((B,), p, device="cuda", dtype=torch.int64))
    idx = torch.cat(idx).to(torch.int32)
    off = torch.cat([torch.zeros(1, device="cuda", dtype=torch.int64), torch.cat(lens).cumsum(0)]).to(torch.int32)
    N = idx.numel()
    print(f"TBE B={B} ids={N} rows<= {row_cap} weights {m.weights.numel() * 4 / 2**30:.1f} GiB", flush=True)
    if which in ("tbe_fwd", "tbe", "all"):
        with torch.no_grad():
            t = timeit(lambda: m(idx, off), n, warm)
        print(f"tbe fwd {t:.3f} ms  {N * 512 / t / 1e6:.0f} GB/s gathered", flush=True)
    if which in ("tbe_sort", "tbe", "all"):
        t = timeit(lambda: m.build_plan(idx, off, None, B), n, warm)
        print(f"tbe plan (linearize + radix sort) {t:.3f} ms", flush=True)
    if which in ("tbe_bwd", "tbe", "all"):
        grad = torch.randn(B, 26 * 128, device="cuda").bfloat16()
        plan = m.build_plan(idx, off, None, B)
        uniq = int(torch.unique(plan.keys).numel())
        t = timeit(lambda: m._backward_impl(grad, idx, off, None, B, plan), n, warm)
        byt = uniq * 128 * 4 * 2 + grad.numel() * 2
        print(f"tbe bwd apply {t:.3f} ms  unique rows {uniq}  minimum traffic {byt / 1e9:.2f} GB -> {byt / t / 1e6:.0f} GB/s", flush=True)
    m.check_error()


def bench_tbe_uniform(B: int, n: int, warm: int) -> None:
    """Pooled lookup with UNIFORM ids over tables far larger than L2 (4 tables x 2M rows x 512 B = 4 GiB): every id is a DRAM
    row fetch, so gathered bytes / time is a DRAM figure (the Zipf case above is partly served from L2)."""
    from torchrec_b200.modules.embedding_configs import PoolingMode
    from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags

    rows, pf = 2_000_000, 8
    m = TableBatchedEmbeddingBags([(rows, 128)] * 4, pooling_mode=PoolingMode.SUM, output_dtype=torch.bfloat16,
                                  optimizer_args=OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.005), device="cuda")
    m.init_embedding_weights_uniform(-0.01, 0.01)
    g = torch.Generator(device="cuda").manual_seed(0)
    idx = torch.randint(0, rows, (4 * B * pf,), device="cuda", generator=g, dtype=torch.int32)
    off = (torch.arange(4 * B + 1, device="cuda", dtype=torch.int64) * pf).to(torch.int32)
    N = idx.numel()
    with torch.no_grad():
        t = timeit(lambda: m(idx, off), n, warm)
    print(f"tbe fwd uniform ids: {N} ids, {t:.3f} ms, {N * 512 / t / 1e6:.0f} GB/s of rows from DRAM (+ {B * 4 * 256 / t / 1e6:.0f} GB/s output)", flush=True)
    grad = torch.randn(B, 4 * 128, device="cuda").bfloat16()
    plan = m.build_plan(idx, off, None, B)
    uniq = int(torch.unique(plan.keys).numel())
    t = timeit(lambda: m._backward_impl(grad, idx, off, None, B, plan), n, warm)
    byt = uniq * 128 * 4 * 2 + N * 256  # row read + write per unique row, one bf16 gradient row slice per id
    print(f"tbe bwd uniform ids: unique rows {uniq}, {t:.3f} ms, algorithmic traffic {byt / 1e9:.2f} GB -> {byt / t / 1e6:.0f} GB/s", flush=True)


def bench_qtbe(B: int, n: int, warm: int) -> None:
    """int8 / int4 row-wise quantized pooled lookup (inference)."""
    from torchrec_b200.modules.embedding_configs import PoolingMode
    from torchrec_b200.ops.qtbe import QuantTableBatchedEmbeddingBags

    rows, pf = 4_000_000, 8
    for bits in (8, 4):
        m = QuantTableBatchedEmbeddingBags([(rows, 128, bits)] * 4, pooling_mode=PoolingMode.SUM, output_dtype=torch.float16, device=torch.device("cuda"))
        m.weights.random_(0, 255)  # arbitrary row bytes: the kernel's traffic does not depend on the values
        idx = torch.randint(0, rows, (4 * B * pf,), device="cuda", dtype=torch.int32)
        off = (torch.arange(4 * B + 1, device="cuda", dtype=torch.int64) * pf).to(torch.int32)
        t = timeit(lambda: m(idx, off), n, warm)
        row_bytes = 128 * bits // 8 + 4
        print(f"qtbe fwd int{bits}: {idx.numel()} ids, {t:.3f} ms, {idx.numel() * row_bytes / t / 1e6:.0f} GB/s of quantized rows", flush=True)


def bench_dense_small(M: int, n: int, warm: int) -> None:
    """Dot interaction forward / backward, the fused cross-layer backward pass and the one-launch dense optimizer."""
    ops = torch.ops.trb200
    dense = torch.randn(M, 128, device="cuda").bfloat16()
    sparse = torch.randn(M, 26, 128, device="cuda").bfloat16()
    t = timeit(lambda: ops.dot_interaction_fwd(dense, sparse), n, warm)
    out = ops.dot_interaction_fwd(dense, sparse)
    byt = (dense.numel() + sparse.numel() + out.numel()) * 2
    print(f"dot fwd M={M}: {t:.3f} ms, {byt / t / 1e6:.0f} GB/s", flush=True)
    dout = torch.randn_like(out)
    t = timeit(lambda: ops.dot_interaction_bwd(dout, dense, sparse), n, warm)
    print(f"dot bwd M={M}: {t:.3f} ms, {(2 * (dense.numel() + sparse.numel()) + out.numel()) * 2 / t / 1e6:.0f} GB/s", flush=True)
    D = 3456
    dy, x0, u = (torch.randn(M, D, device="cuda").bfloat16() for _ in range(3))
    acc = torch.randn(M, D, device="cuda").bfloat16()
    t = timeit(lambda: ops.cross_bwd_fused(dy, x0, u, acc, False), n, warm)
    print(f"cross bwd fused M={M} D={D}: {t:.3f} ms, {6 * M * D * 2 / t / 1e6:.0f} GB/s (4 reads + 2 writes)", flush=True)
    from torchrec_b200.optim.fused_dense import FusedDenseOptimizer

    params = [torch.nn.Parameter(torch.randn(r, c, device="cuda")) for r, c in ((1024, 3456), (3456, 512), (512, 3456), (1024, 1024), (512, 1024))]
    opt = FusedDenseOptimizer(params, "adagrad", lr=0.01)
    opt.buffer.grad.normal_()
    t = timeit(lambda: opt.step(), n, warm)
    nel = sum(p.numel() for p in params)
    print(f"dense optimizer (Adagrad + bf16 copies) {nel} elements: {t:.3f} ms, {nel * (4 * 5 + 2 * 2) / t / 1e6:.0f} GB/s", flush=True)


def bench_sparse_kernels(B: int, n: int, warm: int) -> None:
    """Row-wise bucketization and the 2-D jagged permute of the library-collective input distribution."""
    from torchrec_b200.ops import sparse_ops as sops

    F, pf, rows, W = 26, 8, 4_000_000, 8
    lengths = torch.full((F * B,), pf, dtype=torch.int64, device="cuda")
    idx = torch.randint(0, rows, (F * B * pf,), device="cuda", dtype=torch.int64)
    block = torch.full((F,), (rows + W - 1) // W, dtype=torch.int64, device="cuda")
    t = timeit(lambda: sops.block_bucketize_sparse_features(lengths, idx, bucketize_pos=False, sequence=False, block_sizes=block, my_size=W), n, warm)
    print(f"block bucketize {idx.numel()} ids into {W} buckets: {t:.3f} ms, {idx.numel() * 16 / t / 1e6:.0f} GB/s (read + write ids)", flush=True)
    perm = torch.randperm(F, device="cuda").to(torch.int32)
    t = timeit(lambda: sops.permute_2D_sparse_data(perm, lengths.view(F, B), idx, None, idx.numel()), n, warm)
    print(f"permute 2-D jagged {idx.numel()} ids: {t:.3f} ms, {idx.numel() * 16 / t / 1e6:.0f} GB/s", flush=True)
    # the small jagged helpers
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), lengths.cumsum(0)])
    t = timeit(lambda: sops.offsets_range(offsets[:-1], idx.numel()), n, warm)
    print(f"offsets_range over {idx.numel()} positions: {t:.3f} ms, {idx.numel() * 8 / t / 1e6:.0f} GB/s written", flush=True)
    csr = torch.arange(0, F * pf + 1, pf, dtype=torch.int64, device="cuda")
    vals = torch.rand(idx.numel(), device="cuda")
    t = timeit(lambda: sops.segment_sum_csr(B, csr, vals), n, warm)
    print(f"segment_sum_csr of {idx.numel()} floats into {F} segments: {t:.3f} ms, {idx.numel() * 4 / t / 1e6:.0f} GB/s", flush=True)
    base = torch.arange(F, dtype=torch.int64, device="cuda") * rows
    bound = torch.tensor([F * rows], device="cuda")
    t = timeit(lambda: sops.unique_ids_per_feature(base, offsets, idx, bound), n, warm)
    t_lib = timeit(lambda: torch.unique(idx + base.repeat_interleave(B * pf), sorted=True, return_inverse=True), n, warm)
    print(f"per-feature unique of {idx.numel()} ids (sort + flags + scan + scatter): {t:.3f} ms (torch.unique on pre-linearized keys: {t_lib:.3f} ms)", flush=True)
    D = 256
    values = torch.randn(idx.numel() // 4, D, device="cuda").bfloat16()
    seq_len = torch.randint(20, 201, (values.shape[0] // 110,), device="cuda")
    seq_len[-1] += values.shape[0] - int(seq_len.sum()) if int(seq_len.sum()) < values.shape[0] else 0
    seq_off = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), seq_len.cumsum(0)]).clamp(max=values.shape[0])
    t = timeit(lambda: sops.jagged_to_padded_dense(values, seq_off, 200, 0.0), n, warm)
    print(f"jagged_to_padded_dense {values.shape[0]} x {D} bf16 rows -> [{seq_len.numel()}, 200, {D}]: {t:.3f} ms, "
          f"{(values.numel() + seq_len.numel() * 200 * D) * 2 / t / 1e6:.0f} GB/s", flush=True)
    from torchrec_b200.ops.quant_ops import quantize_rowwise_nbit

    w = torch.randn(4_000_000, 128, device="cuda")
    for bits in (8, 4):
        t = timeit(lambda: quantize_rowwise_nbit(w, bits), n, warm)
        print(f"row-wise int{bits} quantization of [{w.shape[0]}, 128] fp32: {t:.3f} ms, {(w.numel() * 4 + w.shape[0] * (128 * bits // 8 + 4)) / t / 1e6:.0f} GB/s", flush=True)


def bench_engine(B: int, n: int, warm: int) -> None:
    """The fused sparse engine's own kernels with two virtual ranks on this GPU (every phase runs for both ranks before the next
    one, so nothing waits): id scatter, finalize, gradient publish.  Local memory stands in for the peer's, so these are the
    kernels' HBM-side figures, not NVLink ones."""
    import sys

    sys.path.insert(0, "tests")
    from test_fused_sparse_engine_gpu import _build, _kjt  # the virtual-rank harness of the tests

    kinds = ["rw", "tw", "tw", "cw"]
    tables, engines, _, _ = _build(2, kinds, [128, 128, 128, 128], [1_000_000, 500_000, 200_000, 100_000], ["sum"] * 4, stage_dtype=torch.float16, grad_dtype=torch.bfloat16)
    kjts = [_kjt(tables, B, 16, r, idx_dtype=torch.int32) for r in range(2)]
    for e, k in zip(engines, kjts):
        e.prepare(k)
    for e in engines:
        e.prepare_finish()
    grads = [torch.randn(B, 512, device="cuda").bfloat16() for _ in range(2)]

    def step():
        hs = [e.new_handle(k) for e, k in zip(engines, kjts)]
        for ph in (0, 1):
            for e, h in zip(engines, hs):
                e.phase_send(h, ph)
        for e, h in zip(engines, hs):
            e.phase_push(h, build_plans=True)
        for e, h in zip(engines, hs):
            e.phase_finalize(h)
        for e, h, g in zip(engines, hs, grads):
            e.phase_publish(h, g, 1.0)
        for e, h in zip(engines, hs):
            e.phase_pull(h)

    t = timeit(step, n, warm)
    ids = sum(int(k.values().numel()) for k in kjts)
    print(f"engine step, 2 virtual ranks, B={B}/rank, {ids} ids: {t:.3f} ms for both ranks", flush=True)
    for e in engines:
        e.peer.check_error()


def bench_transformer(B: int, n: int, warm: int) -> None:
    """Packed attention (forward, backward), the fused layer-norm / GELU kernels and the sampled-softmax cross entropy on BERT4Rec
    shapes: ``B`` sequences with lengths uniform in [20, 200], 4 heads of 64, hidden 256, feed-forward 1024, 8192 negatives."""
    from torchrec_b200.ops import transformer_ops as tops

    ops = torch.ops.trb200
    sink = torch.zeros(1, device="cuda")
    for chains, per_sm in ((1, 1), (4, 2), (8, 4), (8, 8)):
        flops = ops.mma_sync_probe(sink, 4096, chains, per_sm)
        t = timeit(lambda: ops.mma_sync_probe(sink, 4096, chains, per_sm), n, warm)
        print(f"mma.sync m16n8k16 bf16 issue rate, {chains} independent chains x {8 * per_sm} warps per SM: {flops / t / 1e9:.0f} TFLOP/s", flush=True)
    gen = torch.Generator().manual_seed(0)
    lengths = torch.randint(20, 201, (B,), generator=gen)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)]).cuda()
    T, H, D = int(lengths.sum()), 4, 256
    pair_flops = 2.0 * float((lengths.double() ** 2).sum()) * 64 * H  # one [len, 64] x [64, len] product per head
    qkv = torch.randn(T, 3 * D, device="cuda").bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for p in (0.0, 0.1):
        t = timeit(lambda: ops.varlen_attn_fwd(qkv, offsets, H, 200, p, 7, err), n, warm)
        print(f"packed attention fwd p={p} T={T}: {t:.3f} ms, {2 * pair_flops / t / 1e9:.0f} TFLOP/s (2 products), {(qkv.numel() + T * D) * 2 / t / 1e6:.0f} GB/s", flush=True)
        out, lse = ops.varlen_attn_fwd(qkv, offsets, H, 200, p, 7, err)
        dout = torch.randn_like(out)
        t = timeit(lambda: ops.varlen_attn_bwd(dout, qkv, out, lse, offsets, H, 200, p, 7, err), n, warm)
        print(f"packed attention bwd p={p} T={T}: {t:.3f} ms, {7 * pair_flops / t / 1e9:.0f} TFLOP/s (7 products), {(2 * qkv.numel() + 2 * T * D) * 2 / t / 1e6:.0f} GB/s", flush=True)
    a, r = (torch.randn(T, D, device="cuda").bfloat16() for _ in range(2))
    w, b = torch.ones(D, device="cuda"), torch.zeros(D, device="cuda")
    t = timeit(lambda: ops.ln_residual_fwd(a, r, w, b, 0.1, 7, 1e-5), n, warm)
    print(f"dropout + residual + layer norm fwd [{T}, {D}]: {t:.3f} ms, {4 * T * D * 2 / t / 1e6:.0f} GB/s", flush=True)
    z = torch.randn(T, 4 * D, device="cuda").bfloat16()
    t = timeit(lambda: ops.gelu_dropout_fwd(z, 0.1, 7), n, warm)
    print(f"gelu + dropout fwd [{T}, {4 * D}]: {t:.3f} ms, {2 * z.numel() * 2 / t / 1e6:.0f} GB/s", flush=True)
    dh = torch.randn_like(z)
    t = timeit(lambda: ops.gelu_dropout_bwd(dh, z, 0.1, 7), n, warm)
    print(f"gelu + dropout bwd [{T}, {4 * D}]: {t:.3f} ms, {3 * z.numel() * 2 / t / 1e6:.0f} GB/s", flush=True)
    P, N = max(8, int(0.15 * T) // 8 * 8), 8192
    scores = torch.randn(P, N, device="cuda").bfloat16()
    pos = torch.randn(P, device="cuda")
    t = timeit(lambda: ops.sampled_ce_fwd_bwd(pos, scores, 1.0 / P), n, warm)
    print(f"sampled-softmax cross entropy + gradient [{P}, {N}]: {t:.3f} ms, {2 * scores.numel() * 2 / t / 1e6:.0f} GB/s", flush=True)
    assert tops.attention_error(qkv.device) == 0 and int(err.item()) == 0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "gemm_nt", "gemm_tn", "gemm_cross", "tbe", "tbe_fwd", "tbe_sort", "tbe_bwd",
                                                       "tbe_uniform", "qtbe", "dense_small", "sparse", "engine", "transformer"])
    ap.add_argument("--shape", type=str, default="", help="N,K: run the GEMM benchmarks on this one shape only (profiler captures)")
    ap.add_argument("--small", action="store_true", help="profiler-sized case: few launches, a few GB on the device")
    ap.add_argument("--quick", action="store_true", help="full-size operands (larger than L2) but one warm-up and two timed launches per kernel: what a profiler capture runs")
    ap.add_argument("--batch", type=int, default=65536)
    ap.add_argument("--row-cap", type=int, default=4000000)
    args = ap.parse_args()
    from torchrec_b200.ops import _ext

    _ext.require_cuda_ext("benchmark_kernels")
    M = 16384 if args.small else args.batch
    n, warm = (2, 1) if (args.small or args.quick) else (10, 3)
    row_cap = min(args.row_cap, 200000) if args.small else args.row_cap
    one = [tuple(int(x) for x in args.shape.split(","))] if args.shape else None
    if args.op in ("all", "gemm_nt"):
        bench_gemm_nt(M, one or [(512, 3456), (3456, 512), (1024, 3456), (1024, 1024), (512, 1024), (256, 512), (128, 256)], n, warm)
    if args.op in ("all", "gemm_cross"):
        bench_gemm_cross(M, 3456, 512, n, warm)
    if args.op in ("all", "gemm_tn"):
        bench_gemm_tn(M, one or [(512, 3456), (3456, 512), (1024, 3456), (1024, 1024), (512, 1024), (256, 512)], n, warm)
    if args.op in ("all", "tbe", "tbe_fwd", "tbe_sort", "tbe_bwd"):
        bench_tbe(M, row_cap, args.op, n, warm)
    if args.op in ("all", "tbe_uniform"):
        bench_tbe_uniform(M, n, warm)
    if args.op in ("all", "qtbe"):
        bench_qtbe(M, n, warm)
    if args.op in ("all", "dense_small"):
        bench_dense_small(M, n, warm)
    if args.op in ("all", "sparse"):
        bench_sparse_kernels(M, n, warm)
    if args.op in ("all", "engine"):
        bench_engine(M // 4, n, warm)
    if args.op in ("all", "transformer"):
        bench_transformer(512 if args.small else 4096, n, warm)
    print("gemm status", int(torch.ops.trb200.gemm_error_status()), flush=True)


if __name__ == "__main__":
    main()
