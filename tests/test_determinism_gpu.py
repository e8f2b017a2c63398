"""Run-twice determinism of the sparse path: the fused embedding backward + optimizer combines the contributions to a row in a
fixed order (sorted ids, fixed block order), so two runs from the same state over the same batch give bit-identical tables and
optimizer states even when hot ids span many blocks.  (The dense side accumulates split-K partial sums with fp32 atomics and is
not bitwise repeatable; it is not covered here.)"""
import pytest
import torch

from torchrec_b200.modules.embedding_configs import PoolingMode
from torchrec_b200.ops.tbe import EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags

pytestmark = pytest.mark.gpu


def _run(opt, wdtype, pooling, steps=3):
    specs = [(5000, 128), (40, 64 if pooling != PoolingMode.NONE else 128), (100000, 128)]  # unpooled groups share one width
    ftm, B = [0, 1, 2, 2], 512
    torch.manual_seed(1)
    tbe = TableBatchedEmbeddingBags(specs, ftm, pooling, wdtype, torch.float32, opt, fused=True, device="cuda")
    tbe.init_embedding_weights_uniform(-0.1, 0.1)
    g = torch.Generator().manual_seed(5)
    for _ in range(steps):
        lengths = torch.randint(0, 30, (len(ftm) * B,), generator=g)
        offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)])
        ids = []
        for f, t in enumerate(ftm):
            n = int(lengths[f * B:(f + 1) * B].sum())
            rows = specs[t][0]
            ids.append((rows ** torch.rand(n, generator=g) - 1).long().clamp(0, rows - 1))  # heavy head: one id thousands of times
        idx = torch.cat(ids).cuda()
        if pooling == PoolingMode.NONE:
            out = tbe(idx, offsets.cuda())
        else:
            out = tbe(idx, offsets.cuda(), torch.rand(idx.numel(), generator=g).cuda())
        grad = torch.randn(out.shape, generator=g).cuda()
        out.backward(grad)
    tbe.check_error()
    states = [v.clone() for st in tbe.split_optimizer_states() for v in st.values()]
    return tbe.weights.detach().clone(), states


@pytest.mark.parametrize("opt", [OptimizerArgs(EmbOptimType.EXACT_ROWWISE_ADAGRAD, 0.05, eps=1e-8), OptimizerArgs(EmbOptimType.ADAM, 0.01, eps=1e-8),
                                 OptimizerArgs(EmbOptimType.EXACT_SGD, 0.1)])
@pytest.mark.parametrize("wdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pooling", [PoolingMode.SUM, PoolingMode.NONE])
def test_two_runs_are_bit_identical(opt, wdtype, pooling):
    import copy

    w1, s1 = _run(copy.deepcopy(opt), wdtype, pooling)
    w2, s2 = _run(copy.deepcopy(opt), wdtype, pooling)
    assert torch.equal(w1, w2)
    assert len(s1) == len(s2) and all(torch.equal(a, b) for a, b in zip(s1, s2))
