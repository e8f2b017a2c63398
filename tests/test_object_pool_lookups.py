"""Pool storage back ends."""
import torch

from torchrec_b200.modules.object_pool_lookups import TensorJaggedIndexSelectLookup, TensorLookup, UVMCachingFloatLookup
from torchrec_b200.sparse.jagged_tensor import JaggedTensor


def test_tensor_lookup_roundtrip_and_state():
    lk = TensorLookup(pool_size=6, dim=3, dtype=torch.float32, device=torch.device("cpu"))
    lk.update(torch.tensor([4, 1]), torch.tensor([[1.0, 2, 3], [4, 5, 6]]))
    torch.testing.assert_close(lk(torch.tensor([1, 0, 4])), torch.tensor([[4.0, 5, 6], [0, 0, 0], [1, 2, 3]]))
    (name, state), = list(lk.states_to_register())
    assert name == "_pool" and state.shape == (6, 3)
    lk.set_state(torch.ones(6, 3))
    assert float(lk(torch.tensor([2])).sum()) == 3.0
    assert UVMCachingFloatLookup is TensorLookup


def test_jagged_lookup_roundtrip_truncation_and_weights():
    lk = TensorJaggedIndexSelectLookup(pool_size=5, values_dtype=torch.int64, feature_max_lengths={"a": 2, "b": 3}, is_weighted=True, device=torch.device("cpu"))
    # ids [3, 0]; feature a: [10, 11, 12] (truncated to 2), [13]; feature b: [], [20, 21]
    vals = torch.tensor([10, 11, 12, 13, 20, 21])
    jt = JaggedTensor(values=vals, weights=vals.float() / 10, lengths=torch.tensor([3, 1, 0, 2]))
    lk.update(torch.tensor([3, 0]), jt)
    out = lk(torch.tensor([0, 3, 1]))
    assert out.lengths().tolist() == [1, 2, 0, 2, 0, 0]
    assert out.values().tolist() == [13, 10, 11, 20, 21]
    torch.testing.assert_close(out.weights(), torch.tensor([1.3, 1.0, 1.1, 2.0, 2.1]))
    assert [n for n, _ in lk.states_to_register()] == ["values", "key_lengths", "weights"]
