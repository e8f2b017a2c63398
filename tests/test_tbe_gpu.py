"""CUDA TBE kernels against the CPU (plain torch, fp32) implementation of the same module."""
import copy

import pytest
import torch

from torchrec_b200.modules.embedding_configs import PoolingMode
from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags

pytestmark = pytest.mark.gpu


def _make_inputs(specs, ftm, B, max_len, weighted, seed, zipf=False, idx_dtype=torch.int64):
    g = torch.Generator().manual_seed(seed)
    F = len(ftm)
    lengths = torch.randint(0, max_len + 1, (F * B,), generator=g)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)])
    idx = []
    for f in range(F):
        n = int(lengths[f * B:(f + 1) * B].sum())
        rows = specs[ftm[f]][0]
        if zipf:
            r = torch.rand(n, generator=g)
            ids = (rows ** r - 1).long().clamp(0, rows - 1)  # heavy head -> long duplicate runs
        else:
            ids = torch.randint(0, rows, (n,), generator=g)
        idx.append(ids)
    idx = torch.cat(idx)
    psw = torch.rand(idx.numel(), generator=g) if weighted else None
    return idx.to(idx_dtype), offsets.to(idx_dtype), psw


def _pair(specs, ftm, pooling, opt, wdtype=torch.float32, fused=True, out_dtype=torch.float32):
    torch.manual_seed(1)
    cpu = TableBatchedEmbeddingBags(specs, ftm, pooling, wdtype, out_dtype, copy.deepcopy(opt), fused=fused)
    cpu.init_embedding_weights_uniform(-0.5, 0.5)
    gpu = TableBatchedEmbeddingBags(specs, ftm, pooling, wdtype, out_dtype, copy.deepcopy(opt), fused=fused, device="cuda")
    with torch.no_grad():
        gpu.weights.copy_(cpu.weights)
    return cpu, gpu


@pytest.mark.parametrize("pooling", [PoolingMode.SUM, PoolingMode.MEAN])
@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_forward_pooled(pooling, weighted, idx_dtype):
    specs = [(1000, 128), (50, 64), (300, 256), (7, 8)]
    ftm = [0, 1, 2, 2, 3]
    cpu, gpu = _pair(specs, ftm, pooling, OptimizerArgs())
    idx, off, psw = _make_inputs(specs, ftm, 37, 9, weighted, 3, idx_dtype=idx_dtype)
    with torch.no_grad():
        ref = cpu(idx, off, psw)
        out = gpu(idx.cuda(), off.cuda(), None if psw is None else psw.cuda())
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-5)
    gpu.check_error()


@pytest.mark.parametrize("wdtype,out_dtype", [(torch.float16, torch.float16), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)])
def test_forward_low_precision(wdtype, out_dtype):
    specs = [(500, 128), (200, 512)]
    ftm = [0, 1]
    cpu, gpu = _pair(specs, ftm, PoolingMode.SUM, OptimizerArgs(), wdtype, out_dtype=out_dtype)
    idx, off, _ = _make_inputs(specs, ftm, 64, 20, False, 5)
    with torch.no_grad():
        ref = cpu(idx, off)
        out = gpu(idx.cuda(), off.cuda())
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_forward_sequence():
    specs = [(400, 64), (90, 64)]
    ftm = [0, 1, 0]
    cpu, gpu = _pair(specs, ftm, PoolingMode.NONE, OptimizerArgs())
    idx, off, _ = _make_inputs(specs, ftm, 19, 40, False, 9)
    with torch.no_grad():
        ref = cpu(idx, off)
        out = gpu(idx.cuda(), off.cuda())
    torch.testing.assert_close(out.cpu(), ref)


OPTS = [
    OptimizerArgs(EmbOptimType.EXACT_SGD, 0.1),
    OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.05, eps=1e-8),
    OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.05, eps=1e-8, weight_decay=0.01),
    OptimizerArgs(EmbOptimType.EXACT_ADAGRAD, 0.05, eps=1e-8),
    OptimizerArgs(EmbOptimType.ADAM, 0.01, eps=1e-8),
    OptimizerArgs(EmbOptimType.PARTIAL_ROWWISE_ADAM, 0.01, eps=1e-8),
    OptimizerArgs(EmbOptimType.LAMB, 0.01, eps=1e-6, weight_decay=0.01),
    OptimizerArgs(EmbOptimType.PARTIAL_ROWWISE_LAMB, 0.01, eps=1e-6),
    OptimizerArgs(EmbOptimType.LARS_SGD, 0.1, eta=0.01),
]


@pytest.mark.parametrize("opt", OPTS, ids=lambda o: f"{o.optimizer.value}-wd{o.weight_decay}")
@pytest.mark.parametrize("zipf", [False, True])
def test_backward_fused_optimizers(opt, zipf):
    """Two steps, hot rows included (zipf) so that rows spanning several 64-entry blocks are hit."""
    specs = [(2000, 128), (64, 64), (900, 256)]
    ftm = [0, 1, 2, 0]
    cpu, gpu = _pair(specs, ftm, PoolingMode.SUM, opt)
    for step in range(2):
        idx, off, psw = _make_inputs(specs, ftm, 257, 30, step == 1, 11 + step, zipf=zipf)
        ref = cpu(idx, off, psw)
        out = gpu(idx.cuda(), off.cuda(), None if psw is None else psw.cuda())
        g = torch.randn(ref.shape, generator=torch.Generator().manual_seed(step))
        ref.backward(g)
        out.backward(g.cuda())
        torch.testing.assert_close(out.detach().cpu(), ref.detach(), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(gpu.weights.detach().cpu(), cpu.weights.detach(), rtol=1e-3, atol=5e-5)
        if cpu.momentum1.numel():
            torch.testing.assert_close(gpu.momentum1.cpu(), cpu.momentum1, rtol=2e-3, atol=1e-6)
        if cpu.momentum2.numel():
            torch.testing.assert_close(gpu.momentum2.cpu(), cpu.momentum2, rtol=2e-3, atol=1e-7)
    gpu.check_error()


def test_backward_mean_and_bf16_grad():
    specs = [(3000, 128)]
    ftm = [0, 0]
    opt = OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.05)
    cpu, gpu = _pair(specs, ftm, PoolingMode.MEAN, opt, out_dtype=torch.float32)
    idx, off, _ = _make_inputs(specs, ftm, 300, 12, False, 21, zipf=True)
    ref = cpu(idx, off)
    out = gpu(idx.cuda(), off.cuda())
    g = torch.randn(ref.shape).bfloat16()
    ref.backward(g.float())
    out.backward(g.cuda().float())
    torch.testing.assert_close(gpu.weights.detach().cpu(), cpu.weights.detach(), rtol=2e-4, atol=2e-5)


def test_backward_sequence_adam():
    specs = [(500, 64), (100, 64)]
    ftm = [0, 1]
    opt = OptimizerArgs(EmbOptimType.ADAM, 0.01)
    cpu, gpu = _pair(specs, ftm, PoolingMode.NONE, opt)
    idx, off, _ = _make_inputs(specs, ftm, 33, 50, False, 31, zipf=True)
    ref = cpu(idx, off)
    out = gpu(idx.cuda(), off.cuda())
    g = torch.randn(ref.shape)
    ref.backward(g)
    out.backward(g.cuda())
    torch.testing.assert_close(gpu.weights.detach().cpu(), cpu.weights.detach(), rtol=2e-4, atol=2e-5)


def test_backward_dense_grad():
    specs = [(300, 128), (40, 32)]
    ftm = [0, 1]
    cpu, gpu = _pair(specs, ftm, PoolingMode.SUM, OptimizerArgs(), fused=False)
    idx, off, _ = _make_inputs(specs, ftm, 50, 10, False, 41, zipf=True)
    ref = cpu(idx, off)
    out = gpu(idx.cuda(), off.cuda())
    g = torch.randn(ref.shape)
    ref.backward(g)
    out.backward(g.cuda())
    torch.testing.assert_close(gpu.weights.grad.cpu(), cpu.weights.grad, rtol=1e-4, atol=1e-5)


def test_fp16_weights_backward():
    specs = [(800, 256)]
    opt = OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.05)
    cpu, gpu = _pair(specs, [0], PoolingMode.SUM, opt, torch.float16, out_dtype=torch.float32)
    idx, off, _ = _make_inputs(specs, [0], 128, 20, False, 51)
    ref = cpu(idx, off)
    out = gpu(idx.cuda(), off.cuda())
    g = torch.randn(ref.shape)
    ref.backward(g)
    out.backward(g.cuda())
    torch.testing.assert_close(gpu.weights.detach().cpu().float(), cpu.weights.detach().float(), rtol=2e-3, atol=2e-3)


def test_out_of_range_id_is_reported():
    specs = [(10, 8)]
    _, gpu = _pair(specs, [0], PoolingMode.SUM, OptimizerArgs())
    idx = torch.tensor([1, 99], device="cuda")
    off = torch.tensor([0, 2], device="cuda")
    with torch.no_grad():
        gpu(idx, off)
    with pytest.raises(IndexError):
        gpu.check_error()


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_backward_reads_a_column_slice_without_copy(gdtype):
    """The gradient of a concat arrives as a column slice of a wider tensor (row stride > width)."""
    specs = [(2000, 128), (500, 128)]
    ftm = [0, 1, 0]
    opt = OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.05)
    cpu, gpu = _pair(specs, ftm, PoolingMode.SUM, opt, out_dtype=gdtype)
    idx, off, _ = _make_inputs(specs, ftm, 300, 12, False, 31, zipf=True)
    ref = cpu(idx, off)
    out = gpu(idx.cuda(), off.cuda())
    wide = torch.randn(300, 64 + 384, generator=torch.Generator().manual_seed(3)).to(gdtype)
    g = wide[:, 64:]
    assert not g.is_contiguous()
    ref.backward(g.contiguous())
    out.backward(wide.cuda()[:, 64:])
    torch.testing.assert_close(gpu.weights.detach().cpu(), cpu.weights.detach(), rtol=2e-3 if gdtype == torch.bfloat16 else 2e-4, atol=2e-5)
    gpu.check_error()


@pytest.mark.parametrize("pooling", [PoolingMode.SUM, PoolingMode.MEAN])
def test_per_sample_weight_gradient(pooling):
    specs = [(400, 64), (300, 32)]
    ftm = [0, 1, 1]
    opt = OptimizerArgs(EmbOptimType.EXACT_SGD, 0.1)
    cpu, gpu = _pair(specs, ftm, pooling, opt)
    idx, off, psw = _make_inputs(specs, ftm, 50, 6, True, 41)
    w0 = [t.clone() for t in cpu.split_embedding_weights()]
    pc = psw.clone().requires_grad_(True)
    pg = psw.cuda().requires_grad_(True)
    ref = cpu(idx, off, pc)
    out = gpu(idx.cuda(), off.cuda(), pg)
    g = torch.randn(ref.shape, generator=torch.Generator().manual_seed(5))
    ref.backward(g)
    out.backward(g.cuda())
    torch.testing.assert_close(pg.grad.cpu(), pc.grad, rtol=1e-4, atol=1e-5)
    # oracle: autograd through plain embedding bags on the weights as they were before the update
    po = psw.clone().requires_grad_(True)
    cols, outs = 0, []
    B = 50
    for f, t in enumerate(ftm):
        o = off[f * B:(f + 1) * B + 1]
        s, e = int(o[0]), int(o[-1])
        r = torch.nn.functional.embedding_bag(idx[s:e], w0[t], o[:-1] - s, mode="sum", per_sample_weights=po[s:e])
        if pooling == PoolingMode.MEAN:
            r = r / (o[1:] - o[:-1]).clamp(min=1).unsqueeze(1).float()
        outs.append(r)
    torch.cat(outs, 1).backward(g)
    torch.testing.assert_close(pc.grad, po.grad, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("idx_dtype", [torch.int64, torch.int32])
def test_forward_sequence_one_huge_bag_and_empty_feature(idx_dtype):
    """Unpooled lookups are spread over ids, not bags: one bag with most of the batch and a feature without ids."""
    specs = [(400, 64), (90, 64), (50, 64)]
    ftm = [0, 1, 2, 0]
    B = 7
    g = torch.Generator().manual_seed(3)
    lengths = torch.zeros(len(ftm) * B, dtype=torch.int64)
    lengths[0] = 5000           # feature 0, sample 0
    lengths[B + 3] = 13         # feature 1
    lengths[3 * B:] = torch.randint(0, 5, (B,), generator=g)  # feature 3; feature 2 stays empty
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)])
    idx = torch.cat([torch.randint(0, 400, (5000,), generator=g), torch.randint(0, 90, (13,), generator=g), torch.randint(0, 400, (int(lengths[3 * B:].sum()),), generator=g)])
    cpu, gpu = _pair(specs, ftm, PoolingMode.NONE, OptimizerArgs())
    with torch.no_grad():
        ref = cpu(idx.to(idx_dtype), offsets.to(idx_dtype))
        out = gpu(idx.to(idx_dtype).cuda(), offsets.to(idx_dtype).cuda())
    torch.testing.assert_close(out.cpu(), ref)
    gpu.check_error()


def test_out_of_range_id_leaves_row_zero_alone():
    """An id outside its table contributes nothing to the forward; the backward must not update row 0 for it either."""
    specs = [(10, 8)]
    _, gpu = _pair(specs, [0], PoolingMode.SUM, OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.1))
    before = gpu.weights.detach().clone()
    idx = torch.tensor([3, 99, -5], device="cuda")
    off = torch.tensor([0, 3], device="cuda")
    out = gpu(idx, off)
    out.backward(torch.ones_like(out))
    after = gpu.weights.detach().view(10, 8)
    b = before.view(10, 8)
    assert not torch.equal(after[3], b[3]), "the valid id must be updated"
    torch.testing.assert_close(after[0], b[0], rtol=0, atol=0)
    assert float(gpu.momentum1[0]) == 0.0
    with pytest.raises(IndexError):
        gpu.check_error()


def test_stochastic_rounding_is_unbiased_where_nearest_rounding_stalls():
    """bf16 table, updates of a small fraction of one unit in the last place: rounding to nearest never moves the weights,
    stochastic rounding moves them by the right amount on average."""
    rows, D, steps, lr = 4096, 128, 50, 1.0
    specs = [(rows, D)]
    idx = torch.arange(rows, device="cuda")
    off = torch.arange(rows + 1, device="cuda")
    results = {}
    for sr in (False, True):
        opt = OptimizerArgs(EmbOptimType.EXACT_SGD, lr, stochastic_rounding=sr)
        tbe = TableBatchedEmbeddingBags(specs, [0], PoolingMode.SUM, torch.bfloat16, torch.float32, opt, device="cuda")
        with torch.no_grad():
            tbe.weights.fill_(1.0)  # one unit in the last place of bf16 at 1.0 is 2**-7
        g = torch.full((rows, D), 2.0 ** -7 / 16, device="cuda")  # each step moves a weight by 1/16 of that unit
        for _ in range(steps):
            out = tbe(idx, off)
            out.backward(g)
        results[sr] = float((1.0 - tbe.weights.detach().float()).mean())
    expected = steps * 2.0 ** -7 / 16
    assert results[False] == 0.0
    assert abs(results[True] - expected) < 0.1 * expected, (results, expected)


@pytest.mark.parametrize("D", [512, 1024])
@pytest.mark.parametrize("zipf", [False, True])
def test_wide_rows_against_embedding_bag_and_python_rowwise_adagrad(D, zipf):
    """Wide rows at a four-digit batch, checked directly against ``torch.nn.functional.embedding_bag`` and a row-wise Adagrad written out
    in plain torch (state += mean(g^2) per row; w -= lr * g / (sqrt(state) + eps)), two steps so that the state matters."""
    import torch.nn.functional as F

    lr, eps = 0.05, 1e-8
    specs, ftm, B = [(3000, D), (500, D)], [0, 1, 0], 2048
    torch.manual_seed(2)
    tbe = TableBatchedEmbeddingBags(specs, ftm, PoolingMode.SUM, torch.float32, torch.float32, OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, lr, eps=eps),
                                    fused=True, device="cuda")
    tbe.init_embedding_weights_uniform(-0.1, 0.1)
    tables = [w.detach().clone() for w in tbe.split_embedding_weights()]
    state = [torch.zeros(r, device="cuda") for r, _ in specs]
    for step in range(2):
        idx, off, _ = _make_inputs(specs, ftm, B, 12, False, 21 + step, zipf=zipf)
        idx, off = idx.cuda(), off.cuda()
        out = tbe(idx, off)
        params = [t.clone().requires_grad_(True) for t in tables]
        cols = []
        for f, t in enumerate(ftm):
            lo, hi = int(off[f * B]), int(off[(f + 1) * B])
            cols.append(F.embedding_bag(idx[lo:hi], params[t], off[f * B:(f + 1) * B] - lo, mode="sum"))
        want = torch.cat(cols, dim=1)
        torch.testing.assert_close(out.detach(), want.detach(), rtol=1e-5, atol=1e-5)
        g = torch.randn(want.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(step))
        out.backward(g)
        want.backward(g)
        for t in range(len(specs)):
            grad = params[t].grad
            state[t] += grad.pow(2).mean(1)
            tables[t] = tables[t] - lr * grad / (state[t].sqrt().unsqueeze(1) + eps)  # rows without gradient stay as they are
        for got, ref in zip(tbe.split_embedding_weights(), tables):
            torch.testing.assert_close(got.detach(), ref, rtol=1e-4, atol=2e-6)
    tbe.check_error()
