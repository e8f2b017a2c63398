"""The allocation-free C entry point ``trb_tbe_backward_apply_noalloc`` against the regular operator
``trb200::tbe_backward_apply`` on the same sorted plan: two calls in a row must give the same weights
and optimizer state.  Called through ctypes on the exported symbol, like a C host would.

Collected last (file name) so that it also runs after every other GPU test has used the library.
"""
import ctypes

import pytest
import torch

from torchrec_b200.modules.embedding_configs import PoolingMode
from torchrec_b200.ops import _ext
from torchrec_b200.ops.tbe import _OPT_CODE, EmbOptimType, OptimizerArgs, TableBatchedEmbeddingBags

pytestmark = pytest.mark.gpu

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class _Args(ctypes.Structure):
    _fields_ = [
        ("weights", ctypes.c_void_p), ("weights_dtype", ctypes.c_int32), ("grad_dtype", ctypes.c_int32),
        ("mom1", ctypes.c_void_p), ("mom2", ctypes.c_void_p), ("dense_grad", ctypes.c_void_p),
        ("meta", ctypes.c_void_p), ("sorted_keys", ctypes.c_void_p), ("sorted_src", ctypes.c_void_p),
        ("sorted_w", ctypes.c_void_p), ("src_feature", ctypes.c_void_p), ("bag_scale", ctypes.c_void_p),
        ("grad", ctypes.c_void_p), ("grad_stride", ctypes.c_int64), ("N", ctypes.c_int64),
        ("B", ctypes.c_int32), ("F", ctypes.c_int32), ("max_D", ctypes.c_int32), ("pooled", ctypes.c_int32),
        ("opt_type", ctypes.c_int32), ("step", ctypes.c_int32),
        ("lr", ctypes.c_float), ("eps", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
        ("weight_decay", ctypes.c_float), ("max_grad", ctypes.c_float),
    ]


def _lib():
    assert _ext.has_cuda_ext(), "the CUDA extension must be built in-tree"
    lib = ctypes.CDLL(_ext.CUDA_LIB_PATH)
    fn = lib.trb_tbe_backward_apply_noalloc
    fn.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    fn.restype = ctypes.c_int
    return fn


def _ptr(t):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _call_noalloc(fn, tbe, plan, grad, B, step):
    o = tbe.optimizer_args
    w = tbe.weights.detach()
    meta = tbe._meta_tensor(w.device)
    a = _Args(
        weights=w.data_ptr(), weights_dtype=_DT[w.dtype], grad_dtype=_DT[grad.dtype],
        mom1=_ptr(tbe.momentum1), mom2=_ptr(tbe.momentum2), dense_grad=None, meta=meta.data_ptr(),
        sorted_keys=plan.keys.data_ptr(), sorted_src=plan.src.data_ptr(), sorted_w=_ptr(plan.w),
        src_feature=_ptr(plan.src_feature), bag_scale=_ptr(plan.bag_scale), grad=grad.data_ptr(),
        grad_stride=grad.stride(0), N=plan.keys.numel(), B=B, F=meta.size(1), max_D=tbe.max_D,
        pooled=int(tbe.pooling_mode != PoolingMode.NONE), opt_type=_OPT_CODE[o.optimizer], step=step,
        lr=o.learning_rate, eps=o.eta if o.optimizer == EmbOptimType.LARS_SGD else o.eps, beta1=o.beta1, beta2=o.beta2,
        weight_decay=o.weight_decay, max_grad=o.max_gradient,
    )
    err = ctypes.create_string_buffer(512)
    rc = fn(ctypes.byref(a), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, len(err))
    return rc, err.value.decode()


def _call_regular(tbe, plan, grad, B, step):
    o = tbe.optimizer_args
    w = tbe.weights.detach()
    torch.ops.trb200.tbe_backward_apply(
        w, tbe.momentum1 if tbe.momentum1.numel() else None, tbe.momentum2 if tbe.momentum2.numel() else None, None,
        tbe._meta_tensor(w.device), plan.keys, plan.src, plan.w, plan.src_feature, plan.bag_scale, grad, grad.stride(0), B,
        tbe.max_D, tbe.pooling_mode != PoolingMode.NONE, _OPT_CODE[o.optimizer], o.learning_rate,
        o.eta if o.optimizer == EmbOptimType.LARS_SGD else o.eps, o.beta1, o.beta2, o.weight_decay, step, o.max_gradient, None,
    )


def _inputs(specs, ftm, B, max_len, seed):
    g = torch.Generator().manual_seed(seed)
    F = len(ftm)
    lengths = torch.randint(0, max_len + 1, (F * B,), generator=g)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)])
    idx = []
    for f in range(F):
        n = int(lengths[f * B:(f + 1) * B].sum())
        rows = specs[ftm[f]][0]
        r = torch.rand(n, generator=g)
        idx.append((rows ** r - 1).long().clamp(0, rows - 1))  # heavy head: rows that span many blocks
    return torch.cat(idx).cuda(), offsets.cuda()


@pytest.mark.parametrize(
    "opt",
    [
        OptimizerArgs(optimizer=EmbOptimType.EXACT_ROWWISE_ADAGRAD, learning_rate=0.05, eps=1e-8),
        OptimizerArgs(optimizer=EmbOptimType.ADAM, learning_rate=0.01, eps=1e-8, beta1=0.9, beta2=0.999),
    ],
    ids=["rowwise_adagrad", "adam"],
)
def test_noalloc_matches_operator_two_calls(opt):
    specs = [(4000, 128), (300, 64), (20, 128)]
    ftm = [0, 1, 2, 0]
    B = 512
    fn = _lib()
    torch.manual_seed(7)
    a = TableBatchedEmbeddingBags(specs, ftm, PoolingMode.SUM, torch.float32, torch.float32, opt, device="cuda")
    a.init_embedding_weights_uniform(-0.5, 0.5)
    b = TableBatchedEmbeddingBags(specs, ftm, PoolingMode.SUM, torch.float32, torch.float32, opt, device="cuda")
    with torch.no_grad():
        b.weights.copy_(a.weights)
    for step in (1, 2):  # two calls in a row: the second one sees the scratch the first one left behind
        idx, off = _inputs(specs, ftm, B, 12, seed=10 + step)
        plan = a.build_plan(idx, off, None, B)
        assert plan.keys.numel() <= 262144
        grad = torch.randn(B, a.total_D, device="cuda")
        _call_regular(a, plan, grad, B, step)
        rc, msg = _call_noalloc(fn, b, plan, grad, B, step)
        assert rc == 0, msg
        torch.cuda.synchronize()
        torch.testing.assert_close(b.weights, a.weights, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(b.momentum1, a.momentum1, rtol=1e-5, atol=1e-6)
        if a.momentum2.numel():
            torch.testing.assert_close(b.momentum2, a.momentum2, rtol=1e-5, atol=1e-6)
    a.check_error()


def test_noalloc_rejects_oversize():
    fn = _lib()
    a = _Args(N=262145, B=1, F=1, max_D=128, pooled=1)
    # pointers only have to be non-null to reach the size check; nothing is launched for a rejected call
    dummy = torch.zeros(8, device="cuda")
    for name in ("weights", "meta", "sorted_keys", "sorted_src", "grad"):
        setattr(a, name, dummy.data_ptr())
    err = ctypes.create_string_buffer(512)
    rc = fn(ctypes.byref(a), None, err, len(err))
    assert rc == 2
    assert "beyond the fixed scratch" in err.value.decode()


def _mem_counters():
    st = torch.cuda.memory_stats()
    return st["allocation.all.allocated"], st["segment.all.allocated"], torch.cuda.mem_get_info()[0]


def test_noalloc_allocates_nothing_and_covers_wide_rows_half_types_and_long_chains():
    """bf16 tables with dim 256 and fp16 gradients (the second scratch limit, blocks x dim, is the binding one here), one id
    repeated far more than 17 x 64 times (a chain that the third pass folds), and allocator counters unchanged across the call."""
    specs = [(2000, 256)]
    B = 1024
    opt = OptimizerArgs(optimizer=EmbOptimType.EXACT_ROWWISE_ADAGRAD, learning_rate=0.05, eps=1e-8, stochastic_rounding=False)
    fn = _lib()
    torch.manual_seed(3)
    a = TableBatchedEmbeddingBags(specs, [0], PoolingMode.SUM, torch.bfloat16, torch.float32, opt, device="cuda")
    a.init_embedding_weights_uniform(-0.5, 0.5)
    b = TableBatchedEmbeddingBags(specs, [0], PoolingMode.SUM, torch.bfloat16, torch.float32, opt, device="cuda")
    with torch.no_grad():
        b.weights.copy_(a.weights)
    lengths = torch.full((B,), 8, dtype=torch.int64)
    idx = torch.randint(0, 2000, (B * 8,))
    idx[: 3000] = 7  # one hot row: 3000 consecutive sorted entries span about 47 blocks
    off = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)]).cuda()
    plan = a.build_plan(idx.cuda(), off, None, B)
    grad = torch.randn(B, 256, device="cuda").half()
    _call_regular(a, plan, grad, B, 1)
    b._meta_tensor(b.weights.device)  # the module's metadata and error word exist before the measured window
    torch.cuda.synchronize()
    before = _mem_counters()
    rc, msg = _call_noalloc(fn, b, plan, grad, B, 1)
    torch.cuda.synchronize()
    after = _mem_counters()
    assert rc == 0, msg
    assert before[0] == after[0] and before[1] == after[1], "the tensor library's allocator was used"
    assert after[2] >= before[2] - (1 << 20), "device memory was allocated behind the allocator's back"
    torch.testing.assert_close(b.weights.float(), a.weights.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(b.momentum1, a.momentum1, rtol=1e-4, atol=1e-6)


def test_noalloc_unpooled_matches_operator():
    specs = [(500, 64)]
    opt = OptimizerArgs(optimizer=EmbOptimType.EXACT_SGD, learning_rate=0.1)
    fn = _lib()
    a = TableBatchedEmbeddingBags(specs, [0], PoolingMode.NONE, torch.float32, torch.float32, opt, device="cuda")
    a.init_embedding_weights_uniform(-0.5, 0.5)
    b = TableBatchedEmbeddingBags(specs, [0], PoolingMode.NONE, torch.float32, torch.float32, opt, device="cuda")
    with torch.no_grad():
        b.weights.copy_(a.weights)
    B = 64
    idx, off = _inputs(specs, [0], B, 9, seed=4)
    plan = a.build_plan(idx, off, None, B)
    grad = torch.randn(idx.numel(), 64, device="cuda")
    _call_regular(a, plan, grad, B, 1)
    rc, msg = _call_noalloc(fn, b, plan, grad, B, 1)
    assert rc == 0, msg
    torch.cuda.synchronize()
    torch.testing.assert_close(b.weights, a.weights, rtol=1e-5, atol=1e-6)


def test_noalloc_rejects_second_limit_and_bad_arguments():
    fn = _lib()
    dummy = torch.zeros(8, device="cuda")
    err = ctypes.create_string_buffer(512)
    # N is below the entry limit, but ceil(N / 64) * max_D exceeds the block x dim limit
    a = _Args(N=200000, B=1, F=1, max_D=1024, pooled=1)
    for name in ("weights", "meta", "sorted_keys", "sorted_src", "grad"):
        setattr(a, name, dummy.data_ptr())
    assert fn(ctypes.byref(a), None, err, len(err)) == 2
    # a missing mandatory pointer and an unknown dtype code are argument errors, nothing is launched
    a = _Args(N=64, B=1, F=1, max_D=128, pooled=1)
    for name in ("meta", "sorted_keys", "sorted_src", "grad"):
        setattr(a, name, dummy.data_ptr())
    assert fn(ctypes.byref(a), None, err, len(err)) == 1
    a.weights = dummy.data_ptr()
    a.weights_dtype = 9
    assert fn(ctypes.byref(a), None, err, len(err)) == 1
