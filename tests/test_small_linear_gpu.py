"""Linear layers on the CUDA cores (``small_linear_kernels.cu``): a layer with 13 input features and the one-logit layer, against
fp32 torch on the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K,N,act", [(13, 512, 1), (5, 64, 0), (27, 128, 2)])
def test_small_k_layer_matches_torch(K, N, act):
    from torchrec_b200.ops import dense_ops

    torch.manual_seed(K)
    M = 3001
    x = torch.randn(M, K, device="cuda")
    w = (torch.randn(N, K, device="cuda") * 0.3).requires_grad_(True)
    b = torch.randn(N, device="cuda").requires_grad_(True)
    prev = dense_ops.get_dense_compute_dtype()
    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    try:
        assert dense_ops._small_k_ok(x, w)
        y = dense_ops.linear_act(x, w, b, act)
        go = torch.randn(M, N, device="cuda").bfloat16()
        (y.float() * go.float()).sum().backward()
    finally:
        dense_ops.set_dense_compute_dtype(prev)
    w32, b32 = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    z = x.bfloat16().float() @ w32.t() + b32
    want = torch.relu(z) if act == 1 else torch.sigmoid(z) if act == 2 else z
    assert y.dtype == torch.bfloat16
    torch.testing.assert_close(y.float(), want.detach(), rtol=1e-2, atol=1e-2)
    # the kernel differentiates through the bf16-rounded output, the oracle through fp32: compare with a tolerance for that
    (want * go.float()).sum().backward()
    torch.testing.assert_close(w.grad, w32.grad, rtol=3e-2, atol=0.5)
    torch.testing.assert_close(b.grad, b32.grad, rtol=3e-2, atol=0.5)


@pytest.mark.parametrize("K", [256, 64, 1024])
def test_logit_layer_matches_torch(K):
    from torchrec_b200.ops import dense_ops

    torch.manual_seed(K)
    M = 4099
    x = torch.randn(M, K, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(1, K, device="cuda") * 0.1).requires_grad_(True)
    b = torch.randn(1, device="cuda").requires_grad_(True)
    y = dense_ops.linear_small_out(x, w, b)
    assert y.dtype == torch.float32 and y.shape == (M, 1)
    x32, w32, b32 = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    want = x32 @ w32.t() + b32
    torch.testing.assert_close(y, want.detach(), rtol=1e-4, atol=1e-4)
    go = torch.randn(M, 1, device="cuda")
    (y * go).sum().backward()
    (want * go).sum().backward()
    torch.testing.assert_close(x.grad.float(), x32.grad, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(w.grad, w32.grad, rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(b.grad, b32.grad, rtol=1e-3, atol=1e-3)


def test_logit_layer_accumulates_into_a_flat_gradient():
    """With the parameters living in a flat buffer whose gradient was zeroed for the step, the kernels add straight into it."""
    from torchrec_b200.ops import dense_ops
    from torchrec_b200.optim.fused_dense import FlatParamBuffer

    torch.manual_seed(0)
    lin = torch.nn.Linear(256, 1).cuda()
    flat = FlatParamBuffer(list(lin.parameters()))
    flat.zero_grad()
    x = torch.randn(1000, 256, device="cuda").bfloat16()
    y = dense_ops.linear_small_out(x, lin.weight, lin.bias)
    y.sum().backward()
    want = x.float().sum(0, keepdim=True)
    torch.testing.assert_close(lin.weight.grad, want, rtol=1e-3, atol=1e-2)
    torch.testing.assert_close(lin.bias.grad, torch.full((1,), 1000.0, device="cuda"))
