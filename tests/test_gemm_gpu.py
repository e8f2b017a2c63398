"""tcgen05 GEMM kernels against fp32 torch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from torchrec_b200.ops import _ext
    return _ext.cuda_ops()


def _check_status():
    assert _ops().gemm_error_status() == 0, "a GEMM kernel gave up waiting on a barrier"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (1000, 512, 104), (4096, 3456, 512), (333, 136, 3456), (2048, 1024, 1024), (128, 8, 64)])
def test_gemm_nt_plain(M, N, K):
    torch.manual_seed(0)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    out = _ops().gemm_nt_bf16(a, b, None, 0, True)
    ref = a.float() @ b.float().t()
    _check_status()
    torch.testing.assert_close(out, ref, rtol=1e-3, atol=1e-2 * (K ** 0.5) / 8)


@pytest.mark.parametrize("act", [0, 1, 2])
def test_gemm_nt_bias_act_bf16(act):
    torch.manual_seed(1)
    M, N, K = 1536, 1024, 512
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") / K ** 0.5).bfloat16()
    bias = torch.randn(N, device="cuda")
    out = _ops().gemm_nt_bf16(a, b, bias, act, False)
    ref = a.float() @ b.float().t() + bias
    if act == 1:
        ref = torch.relu(ref)
    elif act == 2:
        ref = torch.sigmoid(ref)
    _check_status()
    torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)


def test_gemm_nt_cross_and_add():
    torch.manual_seed(2)
    M, N, K = 2048, 3456, 512
    v = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") / K ** 0.5).bfloat16()
    bias = torch.randn(N, device="cuda") * 0.1
    x0 = torch.randn(M, N, device="cuda").bfloat16()
    xl = torch.randn(M, N, device="cuda").bfloat16()
    u, y = _ops().gemm_nt_bf16_cross(v, w, bias, x0, xl)
    u_ref = v.float() @ w.float().t() + bias
    _check_status()
    torch.testing.assert_close(u.float(), u_ref, rtol=2e-2, atol=2e-2)
    y_ref = x0.float() * u.float() + xl.float()
    torch.testing.assert_close(y.float(), y_ref, rtol=2e-2, atol=2e-2)
    out = _ops().gemm_nt_bf16_add(v, w, xl)
    torch.testing.assert_close(out.float(), v.float() @ w.float().t() + xl.float(), rtol=2e-2, atol=2e-2)
    _check_status()


@pytest.mark.parametrize("Mc,N,K", [(512, 128, 128), (4096, 512, 3456), (8192, 1024, 1024), (1000, 136, 264), (65536, 256, 512)])
def test_gemm_tn(Mc, N, K):
    torch.manual_seed(3)
    a = (torch.randn(Mc, N, device="cuda") * 0.25).bfloat16()
    b = (torch.randn(Mc, K, device="cuda") * 0.25).bfloat16()
    out = _ops().gemm_tn_bf16(a, b)
    ref = a.float().t() @ b.float()
    _check_status()
    torch.testing.assert_close(out, ref, rtol=2e-3, atol=2e-3 * (Mc ** 0.5))


def test_fused_linear_autograd_matches_fp32():
    """linear_act / lowrank_cross_layer (bf16 tensor-core path) against fp32 autograd of the same math."""
    from torchrec_b200.ops import dense_ops
    torch.manual_seed(4)
    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    try:
        B, N, r = 1024, 512, 128
        x = torch.randn(B, N, device="cuda")
        W1 = torch.nn.Parameter(torch.randn(256, N, device="cuda") / N ** 0.5)
        b1 = torch.nn.Parameter(torch.randn(256, device="cuda") * 0.1)
        xr = x.clone().requires_grad_(True)
        y = dense_ops.linear_act(xr, W1, b1, dense_ops.ACT_RELU)
        g = torch.randn_like(y.float())
        y.float().backward(g)
        # fp32 reference that uses the same ReLU mask as the fused path (a bf16 output that rounds to
        # the other side of zero would otherwise flip single mask bits and hide GEMM errors)
        x16, W16 = x.bfloat16().float(), W1.detach().bfloat16().float()
        yr = torch.relu(x16 @ W16.t() + b1.detach())
        torch.testing.assert_close(y.float(), yr, rtol=3e-2, atol=3e-2)
        dz = (g * (y > 0)).bfloat16().float()
        torch.testing.assert_close(xr.grad, dz @ W16, rtol=3e-2, atol=3e-2)
        torch.testing.assert_close(W1.grad, dz.t() @ x16, rtol=3e-2, atol=5e-2)
        torch.testing.assert_close(b1.grad, dz.sum(0), rtol=3e-2, atol=5e-2)
        # cross layer
        V = torch.nn.Parameter(torch.randn(r, N, device="cuda") / N ** 0.5)
        W = torch.nn.Parameter(torch.randn(N, r, device="cuda") / r ** 0.5)
        bb = torch.nn.Parameter(torch.randn(N, device="cuda") * 0.1)
        x0 = torch.randn(B, N, device="cuda").bfloat16().requires_grad_(True)
        y = dense_ops.lowrank_cross_layer(x0, x0, V, W, bb)
        g = torch.randn(B, N, device="cuda")
        y.float().backward(g)
        Vr, Wr, br = (t.detach().clone().requires_grad_(True) for t in (V, W, bb))
        x0r = x0.detach().float().requires_grad_(True)
        yr = x0r * (torch.nn.functional.linear(torch.nn.functional.linear(x0r, Vr), Wr) + br) + x0r
        yr.backward(g)
        def rel(a, b):
            return ((a.float() - b.float()).norm() / b.float().norm()).item()

        assert rel(y, yr) < 2e-2
        assert rel(x0.grad, x0r.grad) < 3e-2
        assert rel(V.grad, Vr.grad) < 3e-2
        assert rel(W.grad, Wr.grad) < 3e-2
        assert rel(bb.grad, br.grad) < 3e-2
        assert _ops().gemm_error_status() == 0
    finally:
        dense_ops.set_dense_compute_dtype(torch.float32)


def test_lowrank_cross_stack_autograd_matches_fp32():
    """Three-layer low-rank cross network as one autograd node (running dx0, fused bias gradient) against fp32
    autograd of the same math."""
    from torchrec_b200.ops import dense_ops
    torch.manual_seed(5)
    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    try:
        B, N, r, L = 777, 384, 64, 3   # B not a multiple of the tile sizes
        Vs = [torch.nn.Parameter(torch.randn(r, N, device="cuda") / N ** 0.5) for _ in range(L)]
        Ws = [torch.nn.Parameter(torch.randn(N, r, device="cuda") / r ** 0.5) for _ in range(L)]
        bs = [torch.nn.Parameter(torch.randn(N, device="cuda") * 0.1) for _ in range(L)]
        x0 = torch.randn(B, N, device="cuda").bfloat16().requires_grad_(True)
        y = dense_ops.lowrank_cross_stack(x0, Vs, Ws, bs)
        g = torch.randn(B, N, device="cuda")
        y.float().backward(g)
        Vr = [t.detach().clone().requires_grad_(True) for t in Vs]
        Wr = [t.detach().clone().requires_grad_(True) for t in Ws]
        br = [t.detach().clone().requires_grad_(True) for t in bs]
        x0r = x0.detach().float().requires_grad_(True)
        xl = x0r
        for l in range(L):
            xl = x0r * (torch.nn.functional.linear(torch.nn.functional.linear(xl, Vr[l]), Wr[l]) + br[l]) + xl
        xl.backward(g)

        def rel(a, b):
            return ((a.float() - b.float()).norm() / b.float().norm()).item()

        assert rel(y, xl) < 2e-2
        assert rel(x0.grad, x0r.grad) < 3e-2
        for l in range(L):
            assert rel(Vs[l].grad, Vr[l].grad) < 4e-2, l
            assert rel(Ws[l].grad, Wr[l].grad) < 4e-2, l
            assert rel(bs[l].grad, br[l].grad) < 4e-2, l
        assert _ops().gemm_error_status() == 0
    finally:
        dense_ops.set_dense_compute_dtype(torch.float32)


@pytest.mark.parametrize("Mc,N,K", [(4096, 512, 256), (300, 1024, 3456), (8192, 128, 512)])
def test_gemm_tn_accumulates_into_a_given_tensor(Mc, N, K):
    torch.manual_seed(0)
    a = torch.randn(Mc, N, device="cuda").bfloat16()
    b = torch.randn(Mc, K, device="cuda").bfloat16()
    base = torch.randn(N, K, device="cuda")
    acc = base.clone()
    torch.ops.trb200.gemm_tn_bf16_acc(a, b, acc)
    want = base + a.float().t() @ b.float()
    torch.testing.assert_close(acc, want, rtol=2e-3, atol=2e-2 * (Mc ** 0.5) / 16)


def test_colsum_accumulates_into_a_given_tensor():
    x = torch.randn(5000, 256, device="cuda").bfloat16()
    base = torch.randn(256, device="cuda")
    acc = base.clone()
    torch.ops.trb200.colsum_bf16_acc(x, acc)
    torch.testing.assert_close(acc, base + x.float().sum(0), rtol=1e-3, atol=1e-2)


def test_linear_backward_writes_into_flat_gradients():
    """With parameters in a flat buffer whose gradient was zeroed, the weight and bias gradients are reduced straight into it
    (no autograd accumulation) and equal the fp32 reference."""
    from torchrec_b200.ops import dense_ops
    from torchrec_b200.optim.fused_dense import FusedDenseOptimizer

    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    try:
        torch.manual_seed(1)
        lin = torch.nn.Linear(256, 512).cuda()
        ref_w, ref_b = lin.weight.detach().clone().requires_grad_(), lin.bias.detach().clone().requires_grad_()
        opt = FusedDenseOptimizer(lin.parameters(), "sgd", lr=0.0)
        x = torch.randn(1024, 256, device="cuda")
        for _ in range(2):  # the second pass accumulates on top of the first
            y = dense_ops.linear_act(x, lin.weight, lin.bias, dense_ops.ACT_RELU)
            y.float().sum().backward()
            torch.relu(torch.nn.functional.linear(x.bfloat16().float(), ref_w.bfloat16().float(), ref_b)).sum().backward()
            if _ == 0:
                opt.zero_grad()  # arms direct accumulation; drop the first pass on both sides
                ref_w.grad = None
                ref_b.grad = None
        torch.testing.assert_close(lin.weight.grad, ref_w.grad, rtol=2e-2, atol=2e-1)
        torch.testing.assert_close(lin.bias.grad, ref_b.grad, rtol=2e-2, atol=2e-1)
        assert lin.weight.grad.data_ptr() == opt.buffer.grad.data_ptr()
    finally:
        dense_ops.set_dense_compute_dtype(torch.float32)
        dense_ops.bf16_cache.clear()
