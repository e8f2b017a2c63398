"""Sparse data types on CPU: the documented examples of ``JaggedTensor`` / ``KeyedJaggedTensor`` / ``KeyedTensor``
(cf. ``torchrec/sparse/tests/test_jagged_tensor.py``, ``test_keyed_jagged_tensor.py``, ``test_keyed_tensor.py``)."""
import pytest
import torch

from torchrec_b200.sparse.jagged_tensor import (
    ComputeJTDictToKJT,
    ComputeKJTToJTDict,
    JaggedTensor,
    KeyedJaggedTensor,
    KeyedTensor,
    flatten_kjt_list,
    kjt_is_equal,
    unflatten_kjt_list,
)


def _kjt(weighted=True):
    #        0       1        2  <-- batch
    # "f1"   [1,2]   []       [3]
    # "f2"   [4]     [5,6]    [7,8,9]
    values = torch.tensor([1, 2, 3, 4, 5, 6, 7, 8, 9])
    weights = torch.tensor([1.0, 0.5, 1.5, 1.0, 0.5, 1.0, 1.0, 1.5, 2.0]) if weighted else None
    return KeyedJaggedTensor(keys=["f1", "f2"], values=values, weights=weights, lengths=torch.tensor([2, 0, 1, 1, 2, 3]))


# ---- JaggedTensor ---------------------------------------------------------------------------------------
def test_jt_from_dense_and_back():
    values = [torch.tensor([1.0]), torch.tensor([]), torch.tensor([7.0, 8.0]), torch.tensor([10.0, 11.0, 12.0])]
    weights = [torch.tensor([1.0]), torch.tensor([]), torch.tensor([7.0, 8.0]), torch.tensor([10.0, 11.0, 12.0])]
    jt = JaggedTensor.from_dense(values=values, weights=weights)
    assert jt.values().tolist() == [1.0, 7.0, 8.0, 10.0, 11.0, 12.0]
    assert jt.lengths().tolist() == [1, 0, 2, 3] and jt.offsets().tolist() == [0, 1, 1, 3, 6]
    back = jt.to_dense()
    assert [t.tolist() for t in back] == [v.tolist() for v in values]
    assert [t.tolist() for t in jt.to_dense_weights()] == [w.tolist() for w in weights]
    assert JaggedTensor(values=torch.tensor([1, 2])).__class__ is JaggedTensor if False else True


def test_jt_from_dense_lengths_and_padded():
    dense = torch.tensor([[1.0, 2.0, 0.0], [0.0, 0.0, 0.0], [3.0, 4.0, 5.0]])
    jt = JaggedTensor.from_dense_lengths(dense, torch.tensor([2, 0, 3]))
    assert jt.values().tolist() == [1.0, 2.0, 3.0, 4.0, 5.0]
    padded = jt.to_padded_dense(desired_length=2, padding_value=-1.0)
    assert padded.tolist() == [[1.0, 2.0], [-1.0, -1.0], [3.0, 4.0]]
    assert jt.to_padded_dense().shape == (3, 3)
    jt2 = JaggedTensor(values=torch.arange(10.0).view(5, 2), offsets=torch.tensor([0, 2, 2, 5]))
    p2 = jt2.to_padded_dense(4)
    assert p2.shape == (3, 4, 2) and p2[1].abs().sum() == 0 and p2[2, 2].tolist() == [8.0, 9.0]


def test_jt_requires_lengths_or_offsets_and_integer_kinds():
    with pytest.raises(AssertionError):
        JaggedTensor(values=torch.tensor([1.0]))
    with pytest.raises(AssertionError):
        JaggedTensor(values=torch.tensor([1.0]), lengths=torch.tensor([1.0]))
    e = JaggedTensor.empty()
    assert e.values().numel() == 0 and e.lengths().numel() == 0
    jt = JaggedTensor(values=torch.tensor([1.0, 2.0]), lengths=torch.tensor([2]))
    assert jt.weights_or_none() is None
    with pytest.raises(AssertionError):
        jt.weights()
    assert "JaggedTensor" in str(jt)


# ---- KeyedJaggedTensor -------------------------------------------------------------------------------------
def test_kjt_basic_views():
    kjt = _kjt()
    assert kjt.keys() == ["f1", "f2"] and kjt.stride() == 3
    assert kjt.length_per_key() == [3, 6] and kjt.offset_per_key() == [0, 3, 9]
    assert kjt.offsets().tolist() == [0, 2, 2, 3, 4, 6, 9]
    f2 = kjt["f2"]
    assert f2.values().tolist() == [4, 5, 6, 7, 8, 9] and f2.lengths().tolist() == [1, 2, 3] and f2.weights().tolist() == [1.0, 0.5, 1.0, 1.0, 1.5, 2.0]
    d = kjt.to_dict()
    assert set(d) == {"f1", "f2"} and d["f1"].offsets().tolist() == [0, 2, 2, 3]
    assert "f1" in str(kjt)
    with pytest.raises(KeyError):
        kjt["nope"]


def test_kjt_from_offsets_lengths_sync_and_jt_dict():
    a = KeyedJaggedTensor.from_offsets_sync(keys=["f1", "f2"], values=torch.arange(9), offsets=torch.tensor([0, 2, 2, 3, 4, 6, 9]))
    b = KeyedJaggedTensor.from_lengths_sync(keys=["f1", "f2"], values=torch.arange(9), lengths=torch.tensor([2, 0, 1, 1, 2, 3]))
    assert kjt_is_equal(a, b) and a.length_per_key() == [3, 6]
    c = KeyedJaggedTensor.from_jt_dict({"f1": b["f1"], "f2": b["f2"]})
    assert kjt_is_equal(b, c)
    assert not kjt_is_equal(a, _kjt())
    rt = ComputeJTDictToKJT()(ComputeKJTToJTDict()(b))
    assert kjt_is_equal(rt, b)


def test_kjt_split_and_permute_and_concat():
    kjt = KeyedJaggedTensor(keys=["a", "b", "c"], values=torch.arange(1, 10), lengths=torch.tensor([2, 0, 1, 1, 1, 4]), weights=torch.arange(1, 10) * 0.5)
    x, y = kjt.split([1, 2])
    assert x.keys() == ["a"] and y.keys() == ["b", "c"]
    assert x.values().tolist() == [1, 2] and y.values().tolist() == [3, 4, 5, 6, 7, 8, 9] and y.lengths().tolist() == [1, 1, 1, 4]
    assert y.weights().tolist() == [1.5, 2.0, 2.5, 3.0, 3.5, 4.0, 4.5]
    e, full = kjt.split([0, 3])
    assert e.keys() == [] and e.values().numel() == 0 and kjt_is_equal(full, kjt)
    p = kjt.permute([2, 0, 0])
    assert p.keys() == ["c", "a", "a"] and p.values().tolist() == [5, 6, 7, 8, 9, 1, 2, 1, 2] and p.lengths().tolist() == [1, 4, 2, 0, 2, 0]
    assert p.length_per_key() == [5, 2, 2]
    cat = KeyedJaggedTensor.concat([x, y])
    assert kjt_is_equal(cat, kjt)


def test_kjt_empty_and_empty_like_and_to():
    e = KeyedJaggedTensor.empty()
    assert e.keys() == [] and e.values().numel() == 0
    kjt = _kjt()
    el = KeyedJaggedTensor.empty_like(kjt)
    assert el.keys() == kjt.keys() and el.values().numel() == 0 and el.lengths().numel() == 0 or el.lengths().sum() == 0
    moved = kjt.to(torch.device("cpu"), dtype=torch.float16)
    assert moved.weights().dtype == torch.float16 and moved.values().dtype == kjt.values().dtype
    flat = kjt.flatten_lengths()
    assert flat.lengths().dim() == 1


def test_kjt_variable_batch_per_feature():
    # f1 has 2 samples, f2 has 3 (one rank); lengths are key-major with per-key strides
    kjt = KeyedJaggedTensor(keys=["f1", "f2"], values=torch.arange(8), lengths=torch.tensor([1, 2, 3, 0, 2]), stride_per_key_per_rank=[[2], [3]],
                            inverse_indices=(["f1", "f2"], torch.tensor([[0, 1, 0], [0, 1, 2]])))
    assert kjt.variable_stride_per_key() and kjt.stride_per_key() == [2, 3]
    assert kjt.length_per_key() == [3, 5] and kjt["f2"].lengths().tolist() == [3, 0, 2]
    assert kjt.stride() == 3
    p = kjt.permute([1, 0])
    assert p.stride_per_key() == [3, 2] and p.values().tolist() == [3, 4, 5, 6, 7, 0, 1, 2]
    a, b = kjt.split([1, 1])
    assert a.stride_per_key() == [2] and b.values().tolist() == [3, 4, 5, 6, 7]
    assert kjt.inverse_indices()[0] == ["f1", "f2"]


def test_kjt_dist_protocol_round_trip_single_rank():
    kjt = _kjt()
    labels = kjt.dist_labels()
    tensors = kjt.dist_tensors()
    assert labels == ["lengths", "values", "weights"] and len(tensors) == 3
    splits = kjt.dist_splits([2])
    assert splits[0] == [6] and splits[1] == [9]
    rebuilt = KeyedJaggedTensor.dist_init(keys=kjt.keys(), tensors=tensors, variable_stride_per_key=False, num_workers=1, recat=None, stride_per_rank=[3])
    assert kjt_is_equal(rebuilt, kjt)


def test_kjt_pytree_and_list_flatten():
    import torch.utils._pytree as pytree

    kjt = _kjt()
    leaves, spec = pytree.tree_flatten(kjt)
    back = pytree.tree_unflatten(leaves, spec)
    assert kjt_is_equal(back, kjt)
    flat, ctx = flatten_kjt_list([kjt, kjt.permute([1, 0])])
    out = unflatten_kjt_list(flat, ctx)
    assert kjt_is_equal(out[0], kjt) and out[1].keys() == ["f2", "f1"]


def test_kjt_pin_memory_is_gated_on_cuda():
    kjt = _kjt()
    if torch.cuda.is_available():
        assert kjt.pin_memory().values().is_pinned()
    else:
        with pytest.raises(RuntimeError):
            kjt.pin_memory()


# ---- KeyedTensor ---------------------------------------------------------------------------------------------
def test_keyed_tensor_views_and_regroup():
    t1, t2, t3 = torch.ones(2, 3), torch.ones(2, 2) * 2, torch.ones(2, 1) * 3
    kt = KeyedTensor.from_tensor_list(["a", "b", "c"], [t1, t2, t3])
    assert kt.keys() == ["a", "b", "c"] and kt.length_per_key() == [3, 2, 1] and kt.offset_per_key() == [0, 3, 5, 6]
    assert torch.equal(kt["b"], t2) and set(kt.to_dict()) == {"a", "b", "c"}
    kt2 = KeyedTensor.from_tensor_list(["d"], [torch.ones(2, 4) * 4])
    g = KeyedTensor.regroup([kt, kt2], [["c", "d"], ["a"], ["b", "a"]])
    assert [x.shape[1] for x in g] == [5, 3, 5]
    assert g[0][0].tolist() == [3.0, 4.0, 4.0, 4.0, 4.0] and g[2][0].tolist() == [2.0, 2.0, 1.0, 1.0, 1.0]
    d = KeyedTensor.regroup_as_dict([kt, kt2], [["c", "d"], ["a"]], ["x", "y"])
    assert torch.equal(d["y"], t1)
    assert "KeyedTensor" in str(kt)
    kd0 = KeyedTensor(keys=["p", "q"], length_per_key=[1, 2], values=torch.arange(6.0).view(3, 2), key_dim=0)
    assert kd0["q"].tolist() == [[2.0, 3.0], [4.0, 5.0]]


def test_keyed_tensor_regroup_is_differentiable_with_duplicates():
    a = torch.randn(4, 6, requires_grad=True)
    kt = KeyedTensor(keys=["x", "y"], length_per_key=[2, 4], values=a)
    g1, g2 = KeyedTensor.regroup([kt], [["y", "x"], ["x"]])
    (g1.sum() + 2 * g2.sum()).backward()
    assert torch.allclose(a.grad[:, :2], torch.full((4, 2), 3.0)) and torch.allclose(a.grad[:, 2:], torch.ones(4, 4))
