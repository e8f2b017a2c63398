"""Numerics of the smaller sm_100a kernels (quantization, fused BCE, multi-probe hash, pruning remap, keyed-tensor regroup)
against plain torch / the host implementation."""
import os

import pytest
import torch

from torchrec_b200.ops import dense_ops, quant_ops
from torchrec_b200.ops import sparse_ops as sops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits", [8, 4, 2])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_rowwise_quantize_matches_host(bits, dtype):
    torch.manual_seed(0)
    w = (torch.randn(513, 96) * 0.3).to(dtype)
    w[7] = 0.25  # constant row: scale 0 is stored as 1
    ref = quant_ops.quantize_rowwise_nbit(w.float(), bits)
    got = quant_ops.quantize_rowwise_nbit(w.cuda(), bits).cpu()
    assert got.shape == ref.shape and got.dtype == torch.uint8
    nb = 96 * bits // 8
    assert torch.equal(got[:, nb:], ref[:, nb:])  # scale and bias bit-exact
    deq_g = quant_ops.dequantize_rowwise_nbit(got, 96, bits)
    deq_r = quant_ops.dequantize_rowwise_nbit(ref, 96, bits)
    # payload may differ by one step only where a value sits on a rounding boundary
    scale = ref[:, nb:nb + 2].contiguous().view(torch.float16).float()
    assert ((deq_g - deq_r).abs() <= scale + 1e-6).all()
    assert (got[:, :nb] != ref[:, :nb]).float().mean() < 1e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("weighted", [False, True])
def test_fused_bce_matches_torch(dtype, weighted):
    torch.manual_seed(1)
    n = 70001
    x = (torch.randn(n, device="cuda") * 4).to(dtype).requires_grad_(True)
    y = (torch.rand(n, device="cuda") < 0.3).float()
    w = torch.rand(n, device="cuda") if weighted else None
    loss = dense_ops.bce_with_logits_mean(x, y, w)
    (loss * 3.0).backward()
    xr = x.detach().float().requires_grad_(True)
    ref = torch.nn.functional.binary_cross_entropy_with_logits(xr, y, weight=w)
    (ref * 3.0).backward()
    torch.testing.assert_close(loss, ref, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2 if dtype == torch.bfloat16 else 1e-4, atol=1e-7)


def test_zch_probe_device_invariants_and_host_agreement():
    S, nb = 1 << 14, 8
    seg = torch.arange(nb + 1) * (S // nb)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 10**15, (6000,), generator=g)
    ids = torch.cat([ids, ids[:1500]])
    ident_d = torch.full((S,), -1, dtype=torch.int64, device="cuda")
    slots, ev = sops.zch_probe(ids.cuda(), ident_d, None, seg, max_probe=128)
    slots = slots.cpu()
    assert (ev == -1).all() and (slots >= 0).all()
    seen = {}
    for i, s in zip(ids.tolist(), slots.tolist()):
        assert seen.setdefault(i, s) == s
        assert s // (S // nb) == i % nb
    assert len(set(seen.values())) == len(seen)
    assert torch.equal(ident_d.cpu()[slots], ids)
    # read-only lookups on the device and on the host agree on the table the device built
    probe = torch.cat([ids[:500], torch.randint(0, 10**15, (500,), generator=g)])
    d, _ = sops.zch_probe(probe.cuda(), ident_d, None, seg, max_probe=128, readonly=True)
    h, _ = sops.zch_probe(probe, ident_d.cpu(), None, seg, max_probe=128, readonly=True)
    assert torch.equal(d.cpu(), h)
    d2, _ = sops.zch_probe(probe.cuda(), ident_d, None, seg, max_probe=128, readonly=True, disable_fallback=True)
    assert (d2[:500] >= 0).all()


def test_zch_probe_device_ttl_eviction():
    S = 64
    seg = torch.tensor([0, S])
    ident = torch.full((S,), -1, dtype=torch.int64, device="cuda")
    meta = torch.full((S,), sops.ZCH_EMPTY_SCORE, dtype=torch.int32, device="cuda")
    first = torch.arange(1000, 1000 + S, device="cuda")
    s0, _ = sops.zch_probe(first, ident, meta, seg, max_probe=S, input_metadata=torch.full((S,), 10, dtype=torch.int32, device="cuda"), eviction_threshold=5, eviction_policy=sops.ZCH_TTL)
    assert sorted(ident.tolist()) == first.tolist() and (meta == 10).all()
    batch = torch.cat([first[:8], torch.arange(5000, 5016, device="cuda")])
    s1, e1 = sops.zch_probe(batch, ident, meta, seg, max_probe=S, input_metadata=torch.full((24,), 30, dtype=torch.int32, device="cuda"), eviction_threshold=20, eviction_policy=sops.ZCH_TTL)
    assert torch.equal(s1[:8], s0[:8]) and (e1[:8] == -1).all()
    assert (e1[8:] >= 0).all() and torch.equal(e1[8:], s1[8:])
    assert len(set(s1.tolist())) == 24
    assert torch.equal(ident[s1], batch) and (meta[s1] == 30).all()


def test_itep_remap_device_matches_host():
    g = torch.Generator().manual_seed(4)
    sizes = [1000, 50, 700]
    buffer_offsets = torch.tensor([0, 1000, 1050, 1750])
    al = torch.randint(-300, 300, (1750,), generator=g)
    lengths = [4000, 100, 3000, 2500]
    feature_buffer = torch.tensor([0, -1, 2, 1], dtype=torch.int32)
    vals = torch.cat([torch.randint(0, 1000, (4000,), generator=g), torch.randint(0, 10**6, (100,), generator=g),
                      torch.randint(0, 700, (3000,), generator=g), torch.randint(0, 50, (2500,), generator=g)])
    fo = torch.tensor([0, 4000, 4100, 7100, 9600])
    util_h, util_d = torch.zeros(1750), torch.zeros(1750, device="cuda")
    h = sops.itep_remap(vals, fo, feature_buffer, al, util_h, buffer_offsets, True)
    d = sops.itep_remap(vals.cuda(), fo, feature_buffer, al.cuda(), util_d, buffer_offsets, True)
    assert torch.equal(h, d.cpu()) and torch.equal(util_h, util_d.cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kt_regroup_forward_backward(dtype):
    torch.manual_seed(5)
    B = 1000
    in_keys = [["a", "b", "c"], ["d", "e"]]
    in_lengths = [[16, 8, 4], [32, 12]]
    groups = [["e", "a"], ["c"], ["a", "d", "b"]]  # "a" twice, nothing dropped
    vals = [torch.randn(B, sum(l), device="cuda").to(dtype).requires_grad_(True) for l in in_lengths]
    outs = sops.permute_multi_embedding(vals, in_lengths, in_keys, groups)
    os.environ["TRB200_COMPOSITE"] = ""
    refs_in = [v.detach().clone().requires_grad_(True) for v in vals]
    sops._COMPOSITE_ONLY.add("kt_regroup")
    try:
        refs = sops.permute_multi_embedding(refs_in, in_lengths, in_keys, groups)
    finally:
        sops._COMPOSITE_ONLY.discard("kt_regroup")
    for o, r in zip(outs, refs):
        assert torch.equal(o, r)
    ws = [torch.randn_like(o) for o in outs]
    sum((o.float() * w.float()).sum() for o, w in zip(outs, ws)).backward()
    sum((r.float() * w.float()).sum() for r, w in zip(refs, ws)).backward()
    for v, r in zip(vals, refs_in):
        torch.testing.assert_close(v.grad.float(), r.grad.float(), rtol=1e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-2 if dtype == torch.bfloat16 else 1e-6)
    # a key that no group reads gets a zero gradient
    vals2 = [v.detach().clone().requires_grad_(True) for v in vals]
    (o2,) = sops.permute_multi_embedding(vals2, in_lengths, in_keys, [["b"]])
    o2.sum().backward()
    assert vals2[1].grad.abs().sum() == 0 and vals2[0].grad[:, 16:24].eq(1).all() and vals2[0].grad[:, :16].eq(0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,F,D", [(torch.bfloat16, 26, 128), (torch.bfloat16, 31, 64), (torch.bfloat16, 3, 16), (torch.bfloat16, 40, 32), (torch.float32, 26, 128)])
def test_dot_interaction_matches_torch(dtype, F, D):
    """bf16 with at most 32 vectors per sample runs on the tensor cores, everything else on the scalar kernel; both against the
    triu(X X^T) definition in fp32 on the same inputs, forward and backward."""
    import os

    from torchrec_b200.ops.dense_ops import dot_interaction

    torch.manual_seed(F * D)
    B = 77  # not a multiple of the samples a block handles
    dense = (torch.randn(B, D, device="cuda") * 0.5).to(dtype).requires_grad_(True)
    sparse = (torch.randn(B, F, D, device="cuda") * 0.5).to(dtype).requires_grad_(True)
    out = dot_interaction(dense, sparse)
    d32, s32 = dense.detach().float().requires_grad_(True), sparse.detach().float().requires_grad_(True)
    x = torch.cat((d32.unsqueeze(1), s32), dim=1)
    z = torch.bmm(x, x.transpose(1, 2))
    iu = torch.triu_indices(F + 1, F + 1, offset=1, device="cuda")
    want = torch.cat((d32, z[:, iu[0], iu[1]]), dim=1)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert out.shape == want.shape
    torch.testing.assert_close(out.float(), want.detach(), rtol=tol, atol=tol * float(want.abs().max()))
    g = torch.randn_like(want).to(dtype)
    out.backward(g)
    want.backward(g.float())
    torch.testing.assert_close(dense.grad.float(), d32.grad, rtol=tol, atol=tol * float(d32.grad.abs().max()))
    torch.testing.assert_close(sparse.grad.float(), s32.grad, rtol=tol, atol=tol * float(s32.grad.abs().max()))


def test_zch_reserved_slots_and_admission_on_the_device():
    """Opt-in admission on CUDA: claimed slots lie in front of the reserved block of their bucket, ids that were not admitted share a
    reserved row, and the read-only pass reproduces the mapping."""
    from torchrec_b200.ops import sparse_ops as sops

    torch.manual_seed(0)
    S, buckets, reserved = 8192, 8, 64
    ident = torch.full((S,), -1, dtype=torch.int64, device="cuda")
    seg = torch.arange(0, S + 1, S // buckets, device="cuda")
    ids = (torch.arange(1, 3001, device="cuda") * 104729)
    admit = torch.rand(3000, device="cuda") < 0.5
    slots, _ = sops.zch_probe(ids, ident, None, seg, max_probe=64, reserved_slots=reserved, admit=admit)
    claimed = ident[slots] == ids
    pos = slots % (S // buckets)
    assert (pos[claimed] < S // buckets - reserved).all() and (pos[~claimed] >= S // buckets - reserved).all()
    assert torch.equal(claimed, admit)  # the table has room for every admitted id
    assert (ident.view(buckets, -1)[:, -reserved:] == -1).all()
    again, _ = sops.zch_probe(ids, ident, None, seg, max_probe=64, readonly=True, reserved_slots=reserved)
    assert torch.equal(again, slots)
    # the host implementation takes the same decisions
    ident_cpu = torch.full((S,), -1, dtype=torch.int64)
    slots_cpu, _ = sops.zch_probe(ids.cpu(), ident_cpu, None, seg.cpu(), max_probe=64, reserved_slots=reserved, admit=admit.cpu())
    assert torch.equal((ident_cpu[slots_cpu] == ids.cpu()), claimed.cpu())
    assert torch.equal(slots_cpu[~claimed.cpu()], slots.cpu()[~claimed.cpu()])  # shared rows are a pure function of the id
