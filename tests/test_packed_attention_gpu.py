"""Attention over packed sequences (``varlen_attention.cu``) against one fp32 attention per sequence in plain torch: values and
the gradients of q, k and v, with and without dropout (the dropped probabilities are read back through one-hot values)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _oracle(qkv32: torch.Tensor, bounds, heads: int, keep=None) -> torch.Tensor:
    """Per sequence and head, fp32.  ``keep`` (optional): [T, heads, max_n] factors multiplied onto the probabilities."""
    T, three_d = qkv32.shape
    D = three_d // 3
    dh = D // heads
    out = torch.zeros(T, D, device=qkv32.device, dtype=torch.float32)
    pieces = []
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        if hi == lo:
            continue
        n = hi - lo
        q, k, v = (qkv32[lo:hi, i * D:(i + 1) * D].reshape(n, heads, dh).transpose(0, 1) for i in range(3))
        p = torch.softmax(q @ k.transpose(1, 2) / math.sqrt(dh), dim=-1)  # [H, n, n]
        if keep is not None:
            p = p * keep[lo:hi, :, :n].transpose(0, 1)
        pieces.append((lo, hi, (p @ v).transpose(0, 1).reshape(n, D)))
    return torch.cat([o for _, _, o in pieces]) if pieces else out


@pytest.mark.parametrize("heads", [1, 4])
def test_packed_attention_matches_per_sequence_attention(heads):
    from torchrec_b200.ops.transformer_ops import attention_error, packed_attention, packed_attention_supported

    torch.manual_seed(heads)
    lengths = [1, 7, 16, 17, 31, 32, 33, 64, 100, 129, 200, 0, 5]  # tile edges, an empty sequence, one token
    bounds = [0]
    for n in lengths:
        bounds.append(bounds[-1] + n)
    T, D = bounds[-1], heads * 64
    qkv = (torch.randn(T, 3 * D, device="cuda") * 1.5).bfloat16().requires_grad_(True)
    offsets = torch.tensor(bounds, device="cuda")
    assert packed_attention_supported(qkv, heads, 200)
    out = packed_attention(qkv, offsets, heads, 200, 0.0)
    q32 = qkv.detach().float().requires_grad_(True)
    want = _oracle(q32, bounds, heads)
    torch.testing.assert_close(out.float(), want.detach(), rtol=2e-2, atol=2e-2)
    go = torch.randn(T, D, device="cuda").bfloat16()
    (out.float() * go.float()).sum().backward()
    (want * go.float()).sum().backward()
    err = (qkv.grad.float() - q32.grad).abs().max().item()
    assert err <= 3e-2 * max(1.0, q32.grad.abs().max().item()), err
    torch.testing.assert_close(qkv.grad.float(), q32.grad, rtol=5e-2, atol=5e-2)
    assert attention_error(qkv.device) == 0


def test_packed_attention_dropout_is_consistent_between_forward_and_backward():
    """With one-hot values the output IS the dropped probability matrix: read the mask from it, then check the values, the
    keep rate and the gradients against an oracle that uses that mask."""
    from torchrec_b200.ops.transformer_ops import packed_attention

    torch.manual_seed(3)
    heads, p = 2, 0.25
    lengths = [64, 40, 9, 64]
    bounds = [0]
    for n in lengths:
        bounds.append(bounds[-1] + n)
    T, D = bounds[-1], heads * 64
    qkv = torch.randn(T, 3 * D, device="cuda") * 0.5
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        for h in range(heads):
            qkv[lo:hi, 2 * D + h * 64:2 * D + (h + 1) * 64] = torch.eye(64, device="cuda")[: hi - lo]  # v_j = e_j
    qkv = qkv.bfloat16().requires_grad_(True)
    offsets = torch.tensor(bounds, device="cuda")
    torch.manual_seed(11)
    out = packed_attention(qkv, offsets, heads, 64, p)
    probs = out.detach().float().reshape(T, heads, 64)  # [token, head, key]
    kept = probs != 0
    valid = torch.zeros_like(kept)
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        valid[lo:hi, :, : hi - lo] = True
    assert not (kept & ~valid).any()
    rate = kept[valid].float().mean().item()
    assert abs(rate - (1 - p)) < 0.02, rate
    keep = kept.float() / (1 - p)
    q32 = qkv.detach().float().requires_grad_(True)
    want = _oracle(q32, bounds, heads, keep)
    torch.testing.assert_close(out.float(), want.detach(), rtol=2e-2, atol=1e-2)
    go = torch.randn(T, D, device="cuda").bfloat16()
    (out.float() * go.float()).sum().backward()
    (want * go.float()).sum().backward()
    torch.testing.assert_close(qkv.grad.float(), q32.grad, rtol=5e-2, atol=3e-2)
    # another call draws another mask
    out2 = packed_attention(qkv.detach(), offsets, heads, 64, p)
    assert ((out2 != 0) != (out.detach() != 0)).any()


def test_sequence_longer_than_the_launch_cap_is_reported_and_zero_filled():
    from torchrec_b200.ops.transformer_ops import _attn_err, attention_error, packed_attention

    qkv = torch.randn(50, 3 * 64, device="cuda").bfloat16()
    offsets = torch.tensor([0, 50], device="cuda")
    out = packed_attention(qkv, offsets, 1, 32, 0.0)
    assert attention_error(qkv.device) == 1
    assert (out[32:] == 0).all() and torch.isfinite(out.float()).all()
    _attn_err[qkv.device].zero_()


def test_packed_encoder_uses_the_packed_attention_kernel_and_matches_the_padded_mode():
    from torch import nn

    from torchrec_b200.modules import jagged_transformer as jt
    from torchrec_b200.ops import dense_ops

    torch.manual_seed(0)
    layer = nn.TransformerEncoderLayer(d_model=256, nhead=4, dim_feedforward=1024, dropout=0.0, activation="gelu", batch_first=True, norm_first=True)
    enc = nn.TransformerEncoder(layer, num_layers=2, norm=nn.LayerNorm(256)).cuda()
    lengths = torch.tensor([20, 200, 77, 131, 64, 1])
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)]).cuda()
    x = torch.randn(int(lengths.sum()), 256, device="cuda")
    prev = dense_ops.get_dense_compute_dtype()
    dense_ops.set_dense_compute_dtype(torch.bfloat16)
    try:
        outs = {}
        for mode in ("kernel", "padded"):
            jt.ATTENTION_MODE = mode
            outs[mode] = jt.jagged_encoder_forward(enc, x, offsets, 200, training=False).float()
    finally:
        jt.ATTENTION_MODE = "kernel"
        dense_ops.set_dense_compute_dtype(prev)
    torch.testing.assert_close(outs["kernel"], outs["padded"], rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("P,N", [(1000, 8192), (37, 64), (5, 16392)])
def test_sampled_softmax_loss_matches_cross_entropy(P, N):
    from torchrec_b200.ops.transformer_ops import sampled_softmax_loss

    torch.manual_seed(P)
    D = 256
    h = (torch.randn(P, D, device="cuda") * 0.3).bfloat16().requires_grad_(True)
    pos = (torch.randn(P, D, device="cuda") * 0.3).bfloat16().requires_grad_(True)
    neg = (torch.randn(N, D, device="cuda") * 0.3).bfloat16().requires_grad_(True)
    loss = sampled_softmax_loss(h, pos, neg)
    (loss * 3.0).backward()
    h32, p32, n32 = (t.detach().float().requires_grad_(True) for t in (h, pos, neg))
    scores = torch.cat([(h32 * p32).sum(-1, keepdim=True), h32 @ n32.t()], dim=1)
    want = torch.nn.functional.cross_entropy(scores, torch.zeros(P, dtype=torch.long, device="cuda"))
    (want * 3.0).backward()
    torch.testing.assert_close(loss, want, rtol=2e-2, atol=2e-2)
    for got, ref in ((h.grad, h32.grad), (pos.grad, p32.grad), (neg.grad, n32.grad)):
        scale = ref.abs().max().item()
        assert (got.float() - ref).abs().max().item() <= 0.05 * scale + 1e-6, ((got.float() - ref).abs().max().item(), scale)
