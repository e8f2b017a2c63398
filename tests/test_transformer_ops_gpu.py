"""Fused transformer pieces against plain fp32 torch: ``residual + dropout + layer norm`` and ``gelu + dropout`` (forward and
backward), and the packed encoder against the padded ``nn.TransformerEncoder`` it shares its parameters with."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D", [256, 512, 1024])
@pytest.mark.parametrize("with_a", [False, True])
def test_residual_layer_norm_matches_torch_without_dropout(D, with_a):
    from torchrec_b200.ops.transformer_ops import residual_layer_norm

    torch.manual_seed(D)
    T = 1237  # not a multiple of the rows a block handles
    r = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True)
    a = torch.randn(T, D, device="cuda").bfloat16().requires_grad_(True) if with_a else None
    w = (torch.rand(D, device="cuda") + 0.5).requires_grad_(True)
    b = torch.randn(D, device="cuda").requires_grad_(True)
    s, y = residual_layer_norm(a, r, w, b, 0.0, True)
    # oracle in fp32 on the same bf16 inputs; the stream is rounded to bf16 before it is normalised
    r32, a32 = r.detach().float().requires_grad_(True), (a.detach().float().requires_grad_(True) if with_a else None)
    w32, b32 = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    s32 = (r32 + a32) if with_a else r32
    s_ref = s32.detach().bfloat16().float() + (s32 - s32.detach())  # value rounded, gradient straight through
    y_ref = torch.nn.functional.layer_norm(s_ref, (D,), w32, b32, 1e-5)
    torch.testing.assert_close(s.float(), s_ref.detach(), rtol=0, atol=0)
    torch.testing.assert_close(y.float(), y_ref.detach(), rtol=2e-2, atol=2e-2)
    gy = torch.randn(T, D, device="cuda").bfloat16()
    gs = torch.randn(T, D, device="cuda").bfloat16()
    (y.float() * gy.float()).sum().backward(retain_graph=True) if not with_a else ((y.float() * gy.float()).sum() + (s.float() * gs.float()).sum()).backward()
    (y_ref * gy.float()).sum().backward(retain_graph=True) if not with_a else ((y_ref * gy.float()).sum() + (s_ref * gs.float()).sum()).backward()
    torch.testing.assert_close(r.grad.float(), r32.grad, rtol=3e-2, atol=3e-2)
    if with_a:
        torch.testing.assert_close(a.grad.float(), a32.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(w.grad, w32.grad, rtol=2e-2, atol=0.5)
    torch.testing.assert_close(b.grad, b32.grad, rtol=2e-2, atol=0.5)


def test_dropout_mask_is_shared_by_forward_and_backward():
    from torchrec_b200.ops.transformer_ops import gelu_dropout, residual_layer_norm

    torch.manual_seed(1)
    T, D, p = 4096, 256, 0.25
    r = torch.zeros(T, D, device="cuda").bfloat16().requires_grad_(True)
    a = torch.ones(T, D, device="cuda").bfloat16().requires_grad_(True)
    w, b = torch.ones(D, device="cuda").requires_grad_(True), torch.zeros(D, device="cuda").requires_grad_(True)
    s, _ = residual_layer_norm(a, r, w, b, p, True)
    kept = s.detach().float() != 0
    assert abs(float(kept.float().mean()) - (1 - p)) < 0.01
    torch.testing.assert_close(s.detach().float()[kept], torch.full_like(s.detach().float()[kept], 1 / (1 - p)), rtol=1e-2, atol=1e-2)
    s.float().sum().backward()
    torch.testing.assert_close(a.grad.float(), kept.float() / (1 - p), rtol=1e-2, atol=1e-2)  # the same elements, the same scale
    # two calls draw different masks
    s2, _ = residual_layer_norm(a.detach(), r.detach(), w.detach(), b.detach(), p, True)
    assert float(((s2.float() != 0) != kept).float().mean()) > 0.1
    # evaluation mode drops nothing
    s3, _ = residual_layer_norm(a.detach(), r.detach(), w.detach(), b.detach(), p, False)
    assert bool((s3.float() == 1).all())
    z = torch.randn(T, 1024, device="cuda").bfloat16().requires_grad_(True)
    h = gelu_dropout(z, p, True)
    kept = h.detach().float() != 0
    ref = torch.nn.functional.gelu(z.detach().float()) / (1 - p)
    torch.testing.assert_close(h.detach().float()[kept], ref[kept], rtol=2e-2, atol=2e-2)
    h.float().sum().backward()
    zz = z.detach().float().requires_grad_(True)
    torch.nn.functional.gelu(zz).sum().backward()
    sure = ref.abs() > 1e-2  # where gelu(z) itself rounds to zero, h == 0 says nothing about the mask
    torch.testing.assert_close(z.grad.float()[sure], (zz.grad * kept.float() / (1 - p))[sure], rtol=3e-2, atol=3e-2)


def test_packed_encoder_matches_padded_encoder():
    from torchrec_b200.models.bert4rec import BERT4RecSampled
    from torchrec_b200.ops import dense_ops

    torch.manual_seed(0)
    dev = torch.device("cuda")
    model = BERT4RecSampled(2000, 40, 256, nhead=4, num_layers=2, dim_feedforward=512, dropout=0.1, device=dev).eval()
    B = 33
    g = torch.Generator().manual_seed(3)
    lengths = torch.randint(1, 41, (B,), generator=g)
    items = torch.randint(1, 1999, (int(lengths.sum()),), generator=g)
    off = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)])
    row = torch.repeat_interleave(torch.arange(B), lengths)
    col = torch.arange(items.numel()) - off[:-1][row]
    sel = torch.randperm(items.numel(), generator=g)[:50]
    positions = (row * 40 + col)[sel].to(dev)
    kjt = BERT4RecSampled.make_input(items, lengths, items[sel], torch.randint(1, 1999, (64,), generator=g)).to(dev)
    model.packed = False
    with torch.no_grad():
        want = model(kjt, positions)  # fp32 library path on padded tensors
    model.packed = True
    prev = dense_ops.get_dense_compute_dtype()
    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    try:
        with torch.no_grad():
            got = model(kjt, positions)  # packed tokens, bf16 tensor-core GEMMs, fused kernels
        torch.testing.assert_close(got.float(), want, rtol=5e-2, atol=5e-2 * float(want.abs().max()))
        # one training step runs end to end and produces finite gradients everywhere
        model.train()
        out = model(kjt, positions)
        loss = torch.nn.functional.cross_entropy(out.float(), torch.zeros(out.shape[0], dtype=torch.long, device=dev))
        loss.backward()
        for name, p in model.encoder.named_parameters():
            assert p.grad is not None and bool(torch.isfinite(p.grad).all()), name
    finally:
        dense_ops.set_dense_compute_dtype(prev)
