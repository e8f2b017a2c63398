"""Host C++ operators (``torch.ops.trb200_cpu``) against the composite torch implementations, and the semantics of the
multi-probe hash and the pruning remap."""
import os

import pytest
import torch

from torchrec_b200.ops import _ext
from torchrec_b200.ops import sparse_ops as sops

pytestmark = pytest.mark.skipif(not _ext.has_cpu_ext(), reason="host library not built")


def _composite(fn, *a, **k):
    old = os.environ.get("TRB200_CPU_NATIVE")
    os.environ["TRB200_CPU_NATIVE"] = "0"
    try:
        return fn(*a, **k)
    finally:
        if old is None:
            del os.environ["TRB200_CPU_NATIVE"]
        else:
            os.environ["TRB200_CPU_NATIVE"] = old


def _eq(a, b):
    assert (a is None) == (b is None)
    if a is not None:
        assert a.dtype == b.dtype and a.shape == b.shape
        assert torch.equal(a, b)


@pytest.mark.parametrize("ldtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("weighted", [False, True])
def test_permute_2d_native_matches_composite(ldtype, weighted):
    g = torch.Generator().manual_seed(0)
    T, B = 5, 7
    lengths = torch.randint(0, 4, (T, B), generator=g).to(ldtype)
    n = int(lengths.sum())
    values = torch.randint(0, 1000, (n,), generator=g)
    weights = torch.rand(n, generator=g) if weighted else None
    permute = torch.tensor([3, 0, 0, 4, 2], dtype=torch.int32)
    got = sops.permute_2D_sparse_data(permute, lengths, values, weights)
    ref = _composite(sops.permute_2D_sparse_data, permute, lengths, values, weights)
    for a, b in zip(got, ref):
        _eq(a, b)


@pytest.mark.parametrize("pos,seq,keep", [(False, False, False), (True, True, False), (False, True, True)])
def test_block_bucketize_native_matches_composite(pos, seq, keep):
    g = torch.Generator().manual_seed(1)
    F, B, W = 3, 6, 4
    lengths = torch.randint(0, 5, (F * B,), generator=g)
    n = int(lengths.sum())
    block_sizes = torch.tensor([25, 10, 7])
    indices = torch.randint(0, 120, (n,), generator=g)  # some ids lie past block*W and wrap
    weights = torch.rand(n, generator=g)
    got = sops.block_bucketize_sparse_features(lengths, indices, pos, seq, block_sizes, W, weights, keep_orig_idx=keep)
    ref = _composite(sops.block_bucketize_sparse_features, lengths, indices, pos, seq, block_sizes, W, weights, keep_orig_idx=keep)
    for a, b in zip(got, ref):
        _eq(a, b)


def test_cumsum_and_padded_dense_native():
    ops = _ext.cpu_ops()
    x = torch.tensor([3, 0, 2, 5])
    assert ops.complete_cumsum(x).tolist() == [0, 3, 3, 5, 10]
    values = torch.arange(20, dtype=torch.float32).view(10, 2)
    offsets = torch.tensor([0, 3, 3, 10])
    got = ops.jagged_to_padded_dense(values, offsets, 4, -1.0)
    ref = _composite(sops.jagged_to_padded_dense, values, offsets, 4, -1.0)
    assert torch.equal(got, ref)


def _segments(size, buckets):
    return torch.arange(buckets + 1) * (size // buckets)


def test_zch_probe_inserts_without_collisions_and_is_stable():
    S = 256
    identities = torch.full((S,), -1, dtype=torch.int64)
    seg = _segments(S, 4)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 10**12, (150,), generator=g)
    ids = torch.cat([ids, ids[:20]])  # duplicates inside the batch
    slots, ev = sops.zch_probe(ids, identities, None, seg, max_probe=64)
    assert (ev == -1).all()
    assert (slots >= 0).all() and (slots < S).all()
    # same id -> same slot, different ids -> different slots, and the bucket rule holds
    uniq = {}
    for i, s in zip(ids.tolist(), slots.tolist()):
        assert uniq.setdefault(i, s) == s
        assert s // (S // 4) == i % 4
    assert len(set(uniq.values())) == len(uniq)
    assert torch.equal(identities[slots], ids)
    # a read-only pass returns the same slots and does not touch the table
    before = identities.clone()
    again, _ = sops.zch_probe(ids, identities, None, seg, max_probe=64, readonly=True)
    assert torch.equal(again, slots) and torch.equal(before, identities)
    # unknown ids in read-only mode: fallback row, or -1 when the fallback is off
    unknown = torch.tensor([10**13 + 1, 10**13 + 2])
    fb, _ = sops.zch_probe(unknown, identities, None, seg, max_probe=64, readonly=True)
    assert (fb >= 0).all()
    no_fb, _ = sops.zch_probe(unknown, identities, None, seg, max_probe=64, readonly=True, disable_fallback=True)
    assert (no_fb == -1).all()


def test_zch_probe_ttl_eviction_spares_ids_of_the_batch():
    S = 8
    identities = torch.full((S,), -1, dtype=torch.int64)
    metadata = torch.full((S,), sops.ZCH_EMPTY_SCORE, dtype=torch.int32)
    seg = _segments(S, 1)
    first = torch.arange(100, 108)
    sops.zch_probe(first, identities, metadata, seg, max_probe=8, input_metadata=torch.full((8,), 10, dtype=torch.int32), eviction_threshold=5, eviction_policy=sops.ZCH_TTL)
    assert sorted(identities.tolist()) == first.tolist() and (metadata == 10).all()
    # hour 20: everything stored has expired (score 10 < 20); id 100 comes again together with two new ids
    batch = torch.tensor([100, 200, 201])
    slots, ev = sops.zch_probe(batch, identities, metadata, seg, max_probe=8, input_metadata=torch.full((3,), 30, dtype=torch.int32), eviction_threshold=20, eviction_policy=sops.ZCH_TTL)
    assert ev[0] == -1 and ev[1] >= 0 and ev[2] >= 0 and ev[1] != ev[2]
    assert identities[slots[0]] == 100 and identities[slots[1]] == 200 and identities[slots[2]] == 201
    assert len(set(slots.tolist())) == 3
    assert (metadata[slots] == 30).all()
    # without expired slots a full table falls back to a shared row and evicts nothing
    s2, e2 = sops.zch_probe(torch.tensor([999]), identities, metadata, seg, max_probe=8, input_metadata=torch.tensor([31], dtype=torch.int32), eviction_threshold=5, eviction_policy=sops.ZCH_TTL)
    assert e2[0] == -1 and identities[s2[0]] != 999


def test_zch_probe_lru_evicts_the_oldest_probed_slot():
    S = 4
    identities = torch.full((S,), -1, dtype=torch.int64)
    metadata = torch.full((S,), sops.ZCH_EMPTY_SCORE, dtype=torch.int32)
    seg = _segments(S, 1)
    for t, i in enumerate([11, 12, 13, 14]):
        sops.zch_probe(torch.tensor([i]), identities, metadata, seg, max_probe=4, input_metadata=torch.tensor([t + 1], dtype=torch.int32), eviction_policy=sops.ZCH_LRU)
    sops.zch_probe(torch.tensor([11]), identities, metadata, seg, max_probe=4, input_metadata=torch.tensor([9], dtype=torch.int32), eviction_policy=sops.ZCH_LRU)  # touch 11
    slots, ev = sops.zch_probe(torch.tensor([15]), identities, metadata, seg, max_probe=4, input_metadata=torch.tensor([10], dtype=torch.int32), eviction_policy=sops.ZCH_LRU)
    assert ev[0] == slots[0] and 12 not in identities.tolist() and 11 in identities.tolist() and 15 in identities.tolist()


def test_itep_remap():
    # two buffers: table A (6 unpruned ids -> 3 rows), table B (4 -> 2); feature 1 is not pruned
    address_lookup = torch.tensor([0, 1, 2, -1, -2, -3, 0, 1, -1, -2])
    row_util = torch.zeros(10)
    buffer_offsets = torch.tensor([0, 6, 10])
    values = torch.tensor([0, 4, 5, 77, 78, 3, 1])
    feature_offsets = torch.tensor([0, 3, 5, 7])
    feature_buffer = torch.tensor([0, -1, 1], dtype=torch.int32)
    out = sops.itep_remap(values, feature_offsets, feature_buffer, address_lookup, row_util, buffer_offsets, True)
    assert out.tolist() == [0, 1, 2, 77, 78, 1, 1]
    assert row_util.tolist() == [1, 0, 0, 0, 1, 1, 0, 1, 0, 1]
    out2 = sops.itep_remap(values, feature_offsets, feature_buffer, address_lookup, row_util, buffer_offsets, False)
    assert out2.tolist() == out.tolist() and row_util.sum() == 5


def test_jagged_unique_indices_semantics():
    """Distinct ids per feature (features that share a table are deduplicated together and counted under the last of them), sorted
    inside a feature, with a reverse index that reproduces the input."""
    import torch

    from torchrec_b200.ops import sparse_ops as sops

    cumsum = torch.tensor([0, 10, 30])          # two tables: 10 and 20 rows
    feature_table = torch.tensor([0, 1, 1, 2])   # feature 0 -> table 0, features 1 and 2 -> table 1
    # B = 2 bags per feature
    lengths = torch.tensor([2, 1, 0, 3, 2, 0])
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)])
    ids = torch.tensor([3, 3, 9, 5, 7, 5, 7, 19])
    out_len, out_off, uniq, rev = sops.jagged_unique_indices(cumsum, feature_table, offsets, ids)
    assert out_len.tolist() == [2, 0, 3] and out_off.tolist() == [0, 2, 2, 5]
    assert uniq.tolist() == [3, 9, 5, 7, 19]
    assert torch.equal(uniq[rev], ids)
