"""Test-helper packages shipped for users' own tests."""
import numpy as np
import torch


def test_keyed_jagged_tensor_equals():
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor
    from torchrec_b200.sparse.test_utils import keyed_jagged_tensor_equals

    a = KeyedJaggedTensor.from_lengths_sync(keys=["x", "y"], values=torch.tensor([3, 1, 2, 9]), lengths=torch.tensor([2, 1, 1, 0]))
    b = KeyedJaggedTensor.from_lengths_sync(keys=["x", "y"], values=torch.tensor([1, 3, 2, 9]), lengths=torch.tensor([2, 1, 1, 0]))
    assert keyed_jagged_tensor_equals(a, a) and not keyed_jagged_tensor_equals(a, b)
    assert keyed_jagged_tensor_equals(a, b, is_pooled_features=True)
    c = KeyedJaggedTensor.from_lengths_sync(keys=["x", "y"], values=torch.tensor([1, 2, 3, 9]), lengths=torch.tensor([2, 1, 1, 0]))
    assert not keyed_jagged_tensor_equals(a, c, is_pooled_features=True)  # 2 moved to another bag
    assert keyed_jagged_tensor_equals(None, None) and not keyed_jagged_tensor_equals(a, None)


def test_dummy_keyed_optimizer():
    from torchrec_b200.optim.test_utils import DummyKeyedOptimizer

    p = torch.nn.Parameter(torch.ones(2))
    opt = DummyKeyedOptimizer({"p": p}, {p: {"momentum": torch.zeros(2)}}, [{"params": [p], "lr": 0.1}])
    opt.step()
    assert "p" in opt.state_dict()["state"] and torch.equal(p.detach(), torch.ones(2))


def test_criteo_fixtures_feed_the_datapipes():
    from torchrec_b200.datasets.criteo import criteo_kaggle
    from torchrec_b200.datasets.test_utils.criteo_test_utils import CriteoTest, create_dataset_npys, create_dataset_tsv, validate_sample

    with create_dataset_tsv(num_rows=7, seed=1) as path:
        rows = list(criteo_kaggle(path))
        assert len(rows) == 7
        for r in rows:
            validate_sample(r)
    with create_dataset_npys(num_rows=5, seed=2) as (dense, sparse, labels):
        assert np.load(dense).shape == (5, 13) and np.load(sparse).shape == (5, 26) and np.load(labels).shape == (5, 1)
    with CriteoTest._create_dataset_tsv(num_rows=2, train=False) as path:
        assert len(open(path).read().strip().splitlines()) == 2
