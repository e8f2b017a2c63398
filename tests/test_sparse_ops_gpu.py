"""CUDA sparse kernels against the composite torch implementation run on CPU."""
import pytest
import torch

from torchrec_b200.ops import sparse_ops as sops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_complete_cumsum(dtype):
    x = torch.randint(0, 50, (100003,), dtype=dtype)
    torch.testing.assert_close(sops.asynchronous_complete_cumsum(x.cuda()).cpu(), sops.asynchronous_complete_cumsum(x))


@pytest.mark.parametrize("weighted", [False, True])
def test_permute_2d(weighted):
    T, B = 7, 33
    lengths = torch.randint(0, 6, (T, B), dtype=torch.int32)
    N = int(lengths.sum())
    values = torch.randint(0, 1000, (N,), dtype=torch.int64)
    w = torch.rand(N) if weighted else None
    for perm in ([3, 0, 6, 1, 2, 5, 4], [1, 1, 4], [2, 5]):
        p = torch.tensor(perm, dtype=torch.int32)
        rl, rv, rw = sops.permute_2D_sparse_data(p, lengths, values, w)
        gl, gv, gw = sops.permute_2D_sparse_data(p.cuda(), lengths.cuda(), values.cuda(), None if w is None else w.cuda())
        assert torch.equal(gl.cpu(), rl) and torch.equal(gv.cpu(), rv)
        if weighted:
            assert torch.equal(gw.cpu(), rw)


@pytest.mark.parametrize("my_size", [2, 8])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_block_bucketize(my_size, dtype):
    F, B = 3, 41
    rows = [1000, 77, 5000]
    lengths = torch.randint(0, 50, (F * B,), dtype=dtype)
    idx = torch.cat([torch.randint(0, rows[f], (int(lengths[f * B:(f + 1) * B].sum()),)) for f in range(F)]).to(dtype)
    w = torch.rand(idx.numel())
    blk = torch.tensor([(r + my_size - 1) // my_size for r in rows], dtype=dtype)
    ref = sops.block_bucketize_sparse_features(lengths, idx, True, True, blk, my_size, w)
    got = sops.block_bucketize_sparse_features(lengths.cuda(), idx.cuda(), True, True, blk.cuda(), my_size, w.cuda())
    for r, g in zip(ref, got):
        assert torch.equal(g.cpu(), r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_jagged_padded_roundtrip(dtype):
    B, L, D = 29, 12, 64
    lengths = torch.randint(0, 20, (B,))
    off = torch.cat([torch.zeros(1, dtype=torch.int64), lengths.cumsum(0)])
    v = torch.randn(int(off[-1]), D).to(dtype)
    ref = sops.jagged_to_padded_dense(v, off, L, 0.5)
    got = sops.jagged_to_padded_dense(v.cuda(), off.cuda(), L, 0.5)
    assert torch.equal(got.cpu(), ref)
    lens_c = lengths.clamp(max=L)
    off_c = torch.cat([torch.zeros(1, dtype=torch.int64), lens_c.cumsum(0)])
    back = sops.padded_dense_to_jagged(got, off_c.cuda(), int(off_c[-1]))
    assert torch.equal(back.cpu(), sops.padded_dense_to_jagged(ref, off_c))


def test_jagged_padded_kernels_are_differentiable():
    import os

    from torchrec_b200.ops import sparse_ops as sops

    torch.manual_seed(0)
    lengths = torch.tensor([3, 0, 7, 2, 5])
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)]).cuda()
    v = torch.randn(int(lengths.sum()), 16, device="cuda", requires_grad=True)
    w = torch.randn(5, 4, 16, device="cuda")
    out = sops.jagged_to_padded_dense(v, offsets, 4, 0.0)  # bag 2 and 4 are truncated
    (out * w).sum().backward()
    vr = v.detach().clone().requires_grad_(True)
    sops._COMPOSITE_ONLY.add("jagged_to_padded_dense")
    try:
        ref = sops.jagged_to_padded_dense(vr, offsets, 4, 0.0)
    finally:
        sops._COMPOSITE_ONLY.discard("jagged_to_padded_dense")
    (ref * w).sum().backward()
    torch.testing.assert_close(out, ref)
    torch.testing.assert_close(v.grad, vr.grad)
    d = torch.randn(5, 8, 16, device="cuda", requires_grad=True)
    j = sops.padded_dense_to_jagged(d, offsets, int(lengths.sum()))
    wj = torch.randn_like(j)
    (j * wj).sum().backward()
    dr = d.detach().clone().requires_grad_(True)
    mask = torch.arange(8, device="cuda").unsqueeze(0) < lengths.cuda().unsqueeze(1)
    (dr[mask] * wj).sum().backward()
    torch.testing.assert_close(d.grad, dr.grad)


def test_offsets_range_and_segment_sum_match_composite():
    from torchrec_b200.ops import sparse_ops as sops

    g = torch.Generator().manual_seed(0)
    lens = torch.randint(0, 9, (500,), generator=g)
    starts = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)[:-1]])
    total = int(lens.sum())
    for dt in (torch.int32, torch.int64):
        got = sops.offsets_range(starts.to(dt).cuda(), total)
        want = sops.offsets_range(starts.to(dt), total)
        assert got.dtype == dt and torch.equal(got.cpu(), want)
    csr = torch.cat([torch.zeros(1, dtype=torch.long), torch.randint(0, 5, (300,), generator=g).cumsum(0)])
    batch = 7
    n = int(csr[-1]) * batch
    for values in (torch.randint(0, 100, (n,), generator=g), torch.rand(n, generator=g)):
        got = sops.segment_sum_csr(batch, csr.int().cuda(), values.cuda())
        # oracle: every segment summed on its own in float64 (a prefix-sum difference in fp32 loses digits on long inputs)
        bounds = (csr * batch).tolist()
        want = torch.stack([values[lo:hi].double().sum() for lo, hi in zip(bounds[:-1], bounds[1:])]).to(values.dtype)
        torch.testing.assert_close(got.cpu(), want, rtol=1e-6, atol=1e-6)
        torch.testing.assert_close(sops.segment_sum_csr(batch, csr, values), want, rtol=1e-4, atol=2e-4)


def test_vbe_expand_matches_index_select_and_routes_gradients():
    from torchrec_b200.ops import sparse_ops as sops

    torch.manual_seed(1)
    rows, dims, B = [5, 1, 9], [16, 8, 40], 33
    flat = torch.randn(sum(r * d for r, d in zip(rows, dims)), device="cuda", requires_grad=True)
    inverse = torch.stack([torch.randint(0, r, (B,)) for r in rows]).cuda()
    got = sops.vbe_expand(flat, inverse, rows, dims)
    ref_in = flat.detach().cpu().requires_grad_(True)
    want = sops.vbe_expand(ref_in, inverse.cpu(), rows, dims)
    torch.testing.assert_close(got.detach().cpu(), want.detach(), rtol=0, atol=0)
    g = torch.randn(B, sum(dims))
    got.backward(g.cuda())
    want.backward(g)
    torch.testing.assert_close(flat.grad.cpu(), ref_in.grad, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_jagged_unique_indices_matches_the_composite(dtype):
    from torchrec_b200.ops import sparse_ops as sops

    g = torch.Generator().manual_seed(0)
    F, B = 5, 64
    table_rows = torch.tensor([1000, 50, 7000])
    cumsum = torch.cat([torch.zeros(1, dtype=torch.long), table_rows.cumsum(0)])
    feature_table = torch.tensor([0, 1, 1, 2, 2, 3])  # features 1,2 share table 1; 3,4 share table 2
    lengths = torch.randint(0, 9, (F * B,), generator=g)
    lengths[B:B + 5] = 0  # empty bags at a feature's start
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)])
    rows_of_feature = table_rows[feature_table[:-1]]
    ids = torch.cat([torch.randint(0, int(rows_of_feature[f]), (int(lengths[f * B:(f + 1) * B].sum()),), generator=g) for f in range(F)]).to(dtype)
    want = sops.jagged_unique_indices(cumsum, feature_table, offsets, ids)
    got = sops.jagged_unique_indices(cumsum.cuda(), feature_table.cuda(), offsets.cuda(), ids.cuda())
    for a, b in zip(got, want):
        assert a.dtype == b.dtype and torch.equal(a.cpu(), b), (a, b)
    uniq, rev = got[2], got[3]
    assert torch.equal(uniq[rev.long()].cpu() , ids)
