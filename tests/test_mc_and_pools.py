"""Managed collision (admission, eviction, remap stability), object pools, feature processors (cf. the reference's
``torchrec/modules/tests/test_mc_modules.py``, ``test_tensor_pool.py``, ``test_kjt_pool_lookup.py``)."""
import pytest
import torch

from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.mc_embedding_modules import ManagedCollisionEmbeddingBagCollection
from torchrec_b200.modules.mc_modules import DistanceLFU_EvictionPolicy, LFU_EvictionPolicy, LRU_EvictionPolicy, ManagedCollisionCollection, MCHManagedCollisionModule
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


def _jt(ids):
    ids = torch.tensor(ids, dtype=torch.int64)
    return {"f": JaggedTensor(values=ids, lengths=torch.ones(ids.numel(), dtype=torch.int64))}


def test_mch_lfu_admits_frequent_ids_and_keeps_slots():
    mc = MCHManagedCollisionModule(zch_size=3, device=torch.device("cpu"), eviction_policy=LFU_EvictionPolicy(), eviction_interval=2)
    mc.train()
    mc(_jt([1000, 1000, 1000, 2000, 2000, 3000]))
    out = mc(_jt([4000, 1000]))["f"].values()  # second batch triggers the rebuild after profiling
    # 4 candidates for 3 slots: 1000 (4x), 2000 (2x) and one of the singletons are admitted
    members = set(mc._mch_sorted_raw_ids[mc._mch_sorted_raw_ids != torch.iinfo(torch.int64).max].tolist())
    assert {1000, 2000} <= members and len(members) == 3
    a = mc.remap(_jt([1000, 2000]))["f"].values().tolist()
    assert len(set(a)) == 2 and all(0 <= x < 3 for x in a)
    # stable: the same ids keep their slots over later rebuilds as long as they stay popular
    for _ in range(4):
        mc(_jt([1000, 2000, 1000]))
    assert mc.remap(_jt([1000, 2000]))["f"].values().tolist() == a
    assert int(mc.open_slots()) == 0


def test_mch_lru_evicts_stale_ids_and_reports_rows():
    mc = MCHManagedCollisionModule(zch_size=2, device=torch.device("cpu"), eviction_policy=LRU_EvictionPolicy(), eviction_interval=1)
    mc.train()
    mc(_jt([10, 20]))
    slots = dict(zip([10, 20], mc.remap(_jt([10, 20]))["f"].values().tolist()))
    assert mc.evict() is None
    mc(_jt([20]))          # refresh 20
    mc(_jt([30]))          # 30 enters, 10 is the stalest member
    ev = mc.evict()
    assert ev is not None and ev.tolist() == [slots[10]]
    assert mc.remap(_jt([30]))["f"].values().tolist() == [slots[10]]
    assert mc.remap(_jt([20]))["f"].values().tolist() == [slots[20]]
    # eval mode does not profile
    mc.eval()
    mc(_jt([40, 40, 40]))
    assert 40 not in mc._mch_sorted_raw_ids.tolist()


def test_distance_lfu_score_prefers_recent_over_old_frequent():
    p = DistanceLFU_EvictionPolicy(decay_exponent=2.0)
    s = p.score(torch.tensor([10, 3]), torch.tensor([0, 9]), 10)
    assert s[1] > s[0]


def test_mc_ebc_resets_rows_of_evicted_ids():
    cfg = EmbeddingBagConfig(name="t", num_embeddings=2, embedding_dim=4, feature_names=["f"])
    ebc = EmbeddingBagCollection([cfg])
    mcc = ManagedCollisionCollection({"t": MCHManagedCollisionModule(zch_size=2, device=torch.device("cpu"), eviction_policy=LRU_EvictionPolicy(), eviction_interval=1)}, [cfg])
    m = ManagedCollisionEmbeddingBagCollection(ebc, mcc, return_remapped_features=True)
    m.train()
    kjt = lambda ids: KeyedJaggedTensor.from_lengths_sync(keys=["f"], values=torch.tensor(ids), lengths=torch.ones(len(ids), dtype=torch.int64))
    m(kjt([111, 222]))
    with torch.no_grad():
        ebc.embedding_bags["t"].weight.fill_(7.0)
    m(kjt([222]))
    out, remapped = m(kjt([333]))   # 333 takes 111's slot: that row is re-initialised, 222's row is untouched
    w = ebc.embedding_bags["t"].weight.detach()
    slot_333 = int(remapped.values()[0])
    assert (w[slot_333].abs() < 7.0).all() and (w[1 - slot_333] == 7.0).all()
    torch.testing.assert_close(out.values()[0], w[slot_333])


def test_hash_zch_module_train_eval_evict_and_rebuild():
    from torchrec_b200.modules.hash_mc_evictions import HashZchEvictionConfig, HashZchEvictionPolicyName
    from torchrec_b200.modules.hash_mc_modules import HashZchManagedCollisionModule
    from torchrec_b200.sparse.jagged_tensor import JaggedTensor

    m = HashZchManagedCollisionModule(zch_size=64, device=torch.device("cpu"), total_num_buckets=4, max_probe=16, name="t", tb_logging_frequency=1,
                                      eviction_policy_name=HashZchEvictionPolicyName.SINGLE_TTL_EVICTION, eviction_config=HashZchEvictionConfig(features=["f"], single_ttl=24))
    ids = torch.tensor([10**10 + 3, 7, 7, 123456789, 42])
    jt = JaggedTensor(values=ids, lengths=torch.tensor([2, 0, 3]))
    out = m({"f": jt})["f"]
    v = out.values()
    assert v[1] == v[2] and len(set(v.tolist())) == 4 and (v < 64).all() and (v >= 0).all()
    assert torch.equal(out.lengths(), jt.lengths())
    assert int(m.open_slots()) == 60
    m.validate_state()
    assert m._scalar_logger.last_report["t/train/insert_rate"] == 1.0
    assert m.evict() is None
    sd = m.state_dict()
    assert "_hash_zch_identities" in sd and "_hash_zch_metadata" in sd
    # eval: read-only, known ids keep their rows
    m.eval()
    again = m({"f": JaggedTensor(values=torch.tensor([42, 7, 999]), lengths=torch.tensor([3]))})["f"].values()
    assert again[0] == v[4] and again[1] == v[1] and int(m.open_slots()) == 60
    # a shard of buckets [2, 4) keeps global row numbers
    shard = m.rebuild_with_output_id_range((32, 64))
    shard.train()
    o = shard({"f": JaggedTensor(values=torch.tensor([2, 6, 10, 3]), lengths=torch.tensor([4]))})["f"].values()
    assert ((o >= 32) & (o < 64)).all() and (o[:3] < 48).all() and o[3] >= 48
    with pytest.raises(RuntimeError):
        m.rebuild_with_output_id_range((5, 64))
    # disable_fallback drops unknown ids from their bags in eval
    m2 = HashZchManagedCollisionModule(zch_size=8, device=torch.device("cpu"), total_num_buckets=1, max_probe=8, disable_fallback=True)
    m2({"f": JaggedTensor(values=torch.tensor([1, 2]), lengths=torch.tensor([2]))})
    m2.eval()
    r = m2({"f": JaggedTensor(values=torch.tensor([1, 55, 2, 66]), lengths=torch.tensor([2, 2]))})["f"]
    assert r.lengths().tolist() == [1, 1] and r.values().numel() == 2


def test_itep_unsharded_prunes_and_remaps():
    from torchrec_b200.modules.itep_embedding_modules import ITEPEmbeddingBagCollection
    from torchrec_b200.modules.itep_modules import GenericITEPModule
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    torch.manual_seed(0)
    ebc = EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="t0", embedding_dim=4, num_embeddings=4, feature_names=["f0"]),
                                         EmbeddingBagConfig(name="t1", embedding_dim=4, num_embeddings=10, feature_names=["f1"])])
    itep = GenericITEPModule({"t0": 12}, lookups=[ebc], pruning_interval=1001)
    m = ITEPEmbeddingBagCollection(ebc, itep)
    assert itep.address_lookup.tolist() == [0, 1, 2, 3, -1, -2, -3, -4, -1, -2, -3, -4]
    sd = m.state_dict()
    assert "_itep_module.t0_itp_address_lookup" in sd and "_itep_module.t0_itp_row_util" in sd and "_iter" in sd

    def batch(ids0):
        return KeyedJaggedTensor(keys=["f0", "f1"], values=torch.tensor(ids0 + [9, 3]), lengths=torch.tensor([len(ids0), 0, 1, 1]))

    w0 = ebc.embedding_bags["t0"].weight.detach().clone()
    # iterations 0 and 1: id 9 (a sharer of row 1) is hot, owners 1..3 are never seen
    out = m(batch([9, 9, 9, 0]))
    torch.testing.assert_close(out["f0"][0], 3 * w0[1] + w0[0])
    m(batch([9, 9, 0, 0]))
    # iteration 2 prunes before its lookup: id 9 takes the row of the least used owner (id 1 -> row 1, first among the unused)
    m(batch([9, 0]))
    assert itep.last_pruned_iter == 2
    al = itep.address_lookup.tolist()
    assert al[9] >= 0 and al[0] == 0 and sum(1 for v in al if v >= 0) == 4
    lost = [i for i in (1, 2, 3) if al[i] < 0]
    assert len(lost) == 1
    # the handed-over row was re-initialised, the others were not
    w1 = ebc.embedding_bags["t0"].weight.detach()
    assert not torch.equal(w1[al[9]], w0[al[9]]) and torch.equal(w1[0], w0[0])
    assert int(m._iter) == 3
    # state round trip keeps the views live
    m2 = ITEPEmbeddingBagCollection(EmbeddingBagCollection(tables=ebc.embedding_bag_configs()), GenericITEPModule({"t0": 12}, lookups=[ebc]))
    m2.load_state_dict(m.state_dict())
    assert m2._itep_module.address_lookup.tolist() == al
    m.eval()
    before = itep.row_util.clone()
    m(batch([9, 5]))
    assert torch.equal(before, itep.row_util)


def test_mpzch_opt_in_admission_and_reserved_rows():
    """With opt-in admission no id claims a reserved slot, an id that was not admitted shares a reserved row of its bucket, an
    admitted id keeps its own slot afterwards, and about ``opt_in_prob`` percent of new ids are admitted per occurrence."""
    import torch

    from torchrec_b200.modules.hash_mc_modules import HashZchManagedCollisionModule
    from torchrec_b200.sparse.jagged_tensor import JaggedTensor

    torch.manual_seed(0)
    mc = HashZchManagedCollisionModule(zch_size=4000, device=torch.device("cpu"), total_num_buckets=4, max_probe=64, opt_in_prob=30, percent_reserved_slots=10)
    assert mc.get_reserved_slots_per_bucket() == 100
    mc.train()
    ids = torch.arange(1, 1001) * 7919
    out = mc.remap({"f": JaggedTensor(values=ids, lengths=torch.ones(1000, dtype=torch.long))})["f"].values()
    ident = mc._hash_zch_identities.data.view(-1)
    in_bucket = out % 1000
    claimed = ident[out] == ids
    assert (in_bucket[claimed] < 900).all() and (in_bucket[~claimed] >= 900).all()
    assert (ident.view(4, 1000)[:, 900:] == -1).all()  # nobody owns a reserved slot
    assert 0.2 < claimed.float().mean().item() < 0.4
    # evaluation: admitted ids find their slot, the others land on the same reserved row as before
    mc.eval()
    again = mc.remap({"f": JaggedTensor(values=ids, lengths=torch.ones(1000, dtype=torch.long))})["f"].values()
    assert torch.equal(again, out)
    # every further training pass admits more of the remaining ids
    mc.train()
    for _ in range(10):
        out = mc.remap({"f": JaggedTensor(values=ids, lengths=torch.ones(1000, dtype=torch.long))})["f"].values()
    assert (ident[out] == ids).float().mean().item() > 0.9
    # sampling off: everything is admitted and nothing is reserved
    plain = HashZchManagedCollisionModule(zch_size=4000, device=torch.device("cpu"), total_num_buckets=4, max_probe=64)
    plain.train()
    o2 = plain.remap({"f": JaggedTensor(values=ids, lengths=torch.ones(1000, dtype=torch.long))})["f"].values()
    assert (plain._hash_zch_identities.data.view(-1)[o2] == ids).all() and plain.get_reserved_slots_per_bucket() == -1


def test_inference_tensor_pool_over_virtual_devices():
    """One process, four row blocks (all on the host here): lookups return the trained pool's rows in the caller's order."""
    import torch

    from torchrec_b200.distributed.tensor_pool import ShardedInferenceTensorPool
    from torchrec_b200.distributed.types import ObjectPoolShardingPlan, ObjectPoolShardingType, ShardingEnv
    from torchrec_b200.modules.tensor_pool import TensorPool

    pool = TensorPool(pool_size=37, dim=6, dtype=torch.float32, device=torch.device("cpu"))
    pool.update(torch.arange(37), torch.arange(37 * 6, dtype=torch.float32).view(37, 6))
    sharded = ShardedInferenceTensorPool(ShardingEnv.from_local(world_size=4, rank=0), 37, 6, torch.float32,
                                         ObjectPoolShardingPlan(sharding_type=ObjectPoolShardingType.ROW_WISE), pool, torch.device("cpu"))
    assert [p._shard.shape[0] for p in sharded._local_shard_pools] == [10, 10, 10, 7]
    ids = torch.tensor([36, 0, 9, 10, 29, 30, 5, 36])
    torch.testing.assert_close(sharded(ids), pool.lookup(ids))


def test_inference_kjt_pool_over_virtual_devices():
    import torch

    from torchrec_b200.distributed.keyed_jagged_tensor_pool import ShardedInferenceKeyedJaggedTensorPool
    from torchrec_b200.distributed.types import ObjectPoolShardingPlan, ObjectPoolShardingType, ShardingEnv
    from torchrec_b200.modules.keyed_jagged_tensor_pool import KeyedJaggedTensorPool
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    caps = {"a": 3, "b": 2}
    pool = KeyedJaggedTensorPool(pool_size=11, feature_max_lengths=caps, device=torch.device("cpu"))
    g = torch.Generator().manual_seed(0)
    la, lb = torch.randint(0, 4, (11,), generator=g), torch.randint(0, 3, (11,), generator=g)
    vals = torch.randint(0, 100, (int(la.sum() + lb.sum()),), generator=g)
    pool.update(torch.arange(11), KeyedJaggedTensor.from_lengths_sync(keys=["a", "b"], values=vals, lengths=torch.cat([la, lb])))
    sharded = ShardedInferenceKeyedJaggedTensorPool(ShardingEnv.from_local(world_size=3, rank=0), 11, caps, torch.int64, False,
                                                    ObjectPoolShardingPlan(sharding_type=ObjectPoolShardingType.ROW_WISE), pool, torch.device("cpu"))
    ids = torch.tensor([10, 0, 4, 3, 8, 10])
    got, want = sharded(ids), pool.lookup(ids)
    assert got.keys() == want.keys() and torch.equal(got.lengths(), want.lengths()) and torch.equal(got.values(), want.values())


def test_small_helpers_of_sparse_and_feature_modules():
    """``jt_is_equal`` / ``regroup_kts`` / position-weight helpers / ``TrainInputMapper`` / ``apply_mc_method_to_jt_dict``."""
    from torchrec_b200.modules.feature_processor import PositionWeightedModule
    from torchrec_b200.modules.feature_processor_ import get_stride_per_key_per_rank, get_weights_list
    from torchrec_b200.modules.hash_mc_modules import TrainInputMapper
    from torchrec_b200.modules.mc_modules import apply_mc_method_to_jt_dict
    from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor, KeyedTensor, jt_is_equal, regroup_kts

    a = JaggedTensor(values=torch.tensor([1.0, 2.0, 3.0]), lengths=torch.tensor([2, 0, 1]))
    b = JaggedTensor(values=torch.tensor([1.0, 2.0, 3.0]), offsets=torch.tensor([0, 2, 2, 3]))
    assert jt_is_equal(a, b) and not jt_is_equal(a, JaggedTensor(values=torch.tensor([1.0, 2.0, 3.0]), lengths=torch.tensor([1, 1, 1])))
    assert not jt_is_equal(a, "a") and not jt_is_equal(a, JaggedTensor(values=a.values(), lengths=a.lengths(), weights=torch.ones(3)))

    kt1 = KeyedTensor(keys=["x", "y"], length_per_key=[2, 3], values=torch.arange(10.0).view(2, 5))
    kt2 = KeyedTensor(keys=["z"], length_per_key=[1], values=torch.tensor([[100.0], [200.0]]))
    got = regroup_kts([kt1, kt2], [["z", "x"], ["y", "x"]])
    want = KeyedTensor.regroup([kt1, kt2], [["z", "x"], ["y", "x"]])
    assert all(torch.equal(g, w) for g, w in zip(got, want)) and got[0].tolist() == [[100.0, 0.0, 1.0], [200.0, 5.0, 6.0]]

    kjt = KeyedJaggedTensor(keys=["f0", "f1"], values=torch.arange(6), lengths=torch.tensor([2, 1, 3, 0]))
    seq = torch.tensor([0, 1, 0, 0, 1, 2])
    w = get_weights_list(seq, kjt, {"f1": torch.nn.Parameter(torch.tensor([0.5, 0.25, 0.125]))})
    assert w.tolist() == [1.0, 1.0, 1.0, 0.5, 0.25, 0.125]
    assert get_stride_per_key_per_rank(kjt) is None
    vb = KeyedJaggedTensor(keys=["f0", "f1"], values=torch.arange(3), lengths=torch.tensor([1, 1, 1]), stride_per_key_per_rank=[[2], [1]])
    assert get_stride_per_key_per_rank(vb) == [[2], [1]]

    pw = PositionWeightedModule({"f1": 4})
    out = pw({"f0": a, "f1": JaggedTensor(values=torch.tensor([7, 8, 9]), lengths=torch.tensor([3]))})
    assert set(out) == {"f0", "f1"} and out["f0"].weights_or_none() is None and out["f1"].weights().tolist() == [1.0, 1.0, 1.0]

    # ids dealt to 4 chunks of unequal size, modulo rule and block rule
    sizes, starts = torch.tensor([10, 20, 30, 40]), torch.tensor([0, 10, 30, 60])
    ids = torch.tensor([0, 5, 6, 7, 103])
    seen, local, off = TrainInputMapper(0, 4, sizes, starts, inference_dispatch_div_train_world_size=True)(ids)
    assert seen.tolist() == [0, 1, 1, 1, 25] and local.tolist() == [10, 20, 30, 40, 40] and off.tolist() == [0, 10, 30, 60, 60]
    seen, local, off = TrainInputMapper(100, 4, sizes, starts)(torch.tensor([0, 24, 25, 99]), output_offset=torch.tensor(10))
    assert seen.tolist() == [0, 24, 25, 99] and local.tolist() == [10, 10, 20, 40] and off.tolist() == [-10, -10, 0, 50]

    class _Mc(torch.nn.Module):
        def remap(self, features):
            return {k: JaggedTensor(values=v.values() + 1, lengths=v.lengths()) for k, v in features.items()}

    assert apply_mc_method_to_jt_dict(_Mc(), "remap", {"f": a})["f"].values().tolist() == [2.0, 3.0, 4.0]
