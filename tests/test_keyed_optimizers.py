"""Keyed optimizers: FQN-keyed state dicts, in-place loads, combination, in-backward registration and the row-wise Adagrad
reference implementation (cf. ``torchrec/optim/tests``)."""
import copy

import pytest
import torch
from torch import nn

from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizer, KeyedOptimizerWrapper, OptimizerWrapper
from torchrec_b200.optim.optimizers import in_backward_optimizer_filter
from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(4, 3), nn.Linear(3, 1))


def _step(m, opt):
    opt.zero_grad()
    m(torch.ones(2, 4)).sum().backward()
    opt.step()


def test_wrapper_state_dict_is_keyed_by_fqn_and_loads_in_place():
    m = _model()
    opt = KeyedOptimizerWrapper(dict(m.named_parameters()), lambda ps: torch.optim.Adagrad(ps, lr=0.1))
    _step(m, opt)
    sd = opt.state_dict()
    assert set(sd["state"].keys()) == {"0.weight", "0.bias", "1.weight", "1.bias"}
    assert "param_groups" not in sd
    opt.save_param_groups(True)
    assert sorted(opt.state_dict()["param_groups"][0]["params"]) == ["0.bias", "0.weight", "1.bias", "1.weight"]
    # load into a fresh optimizer whose state was initialised: tensors are overwritten in place
    m2 = _model()
    opt2 = KeyedOptimizerWrapper(dict(m2.named_parameters()), lambda ps: torch.optim.Adagrad(ps, lr=0.1))
    opt2.init_state()
    before = opt2.state[m2[0].weight]["sum"]
    ptr = before.data_ptr()
    opt2.load_state_dict(copy.deepcopy(sd))
    after = opt2.state[m2[0].weight]["sum"]
    assert after.data_ptr() == ptr
    torch.testing.assert_close(after, opt.state[m[0].weight]["sum"])
    # strictness: a missing key or a changed shape is an error
    bad = copy.deepcopy(sd)
    bad["state"].pop("0.bias")
    with pytest.raises(ValueError):
        opt2.load_state_dict(bad)
    bad = copy.deepcopy(sd)
    bad["state"]["0.weight"]["sum"] = torch.zeros(9)
    with pytest.raises((ValueError, RuntimeError)):
        opt2.load_state_dict(bad)


def test_combined_optimizer_prefixes_and_steps_all():
    m = _model()
    a = KeyedOptimizerWrapper({"0.weight": m[0].weight, "0.bias": m[0].bias}, lambda ps: torch.optim.SGD(ps, lr=0.5, momentum=0.9))
    b = KeyedOptimizerWrapper({"1.weight": m[1].weight, "1.bias": m[1].bias}, lambda ps: torch.optim.Adagrad(ps, lr=0.1))
    combo = CombinedOptimizer([("first", a), b])
    assert set(combo.params.keys()) == {"first.0.weight", "first.0.bias", "1.weight", "1.bias"}
    w0, w1 = m[0].weight.detach().clone(), m[1].weight.detach().clone()
    _step(m, combo)
    assert not torch.equal(m[0].weight, w0) and not torch.equal(m[1].weight, w1)
    sd = combo.state_dict()
    assert "1.weight" in sd["state"] and "first.0.weight" in sd["state"]
    assert len(combo.param_groups) == 2 and [n for n, _ in combo.optimizers] == ["first", ""]
    combo.load_state_dict(copy.deepcopy(sd))
    with pytest.raises(ValueError):
        CombinedOptimizer([a, KeyedOptimizerWrapper({"0.weight": m[0].weight}, lambda ps: torch.optim.SGD(ps, lr=0.5))])
    assert isinstance(OptimizerWrapper(combo).state_dict(), dict)


def test_apply_optimizer_in_backward_marks_parameters_and_filter_skips_them():
    m = _model()
    apply_optimizer_in_backward(torch.optim.SGD, m[0].parameters(), {"lr": 0.25})
    assert m[0].weight._optimizer_classes == [torch.optim.SGD] and m[0].weight._optimizer_kwargs == [{"lr": 0.25}]
    w0, w1 = m[0].weight.detach().clone(), m[1].weight.detach().clone()
    m(torch.ones(2, 4)).sum().backward()
    assert not torch.equal(m[0].weight, w0), "updated inside backward"
    assert torch.equal(m[1].weight, w1)
    rest = dict(in_backward_optimizer_filter(m.named_parameters()))
    assert set(rest) == {"1.weight", "1.bias"}
    only = dict(in_backward_optimizer_filter(m.named_parameters(), include=True))
    assert set(only) == {"0.weight", "0.bias"}


def test_rowwise_adagrad_reference_math():
    torch.manual_seed(0)
    w = nn.Parameter(torch.randn(5, 4))
    opt = RowWiseAdagrad([w], lr=0.1, eps=1e-8)
    w0 = w.detach().clone()
    g = torch.randn(5, 4)
    g[2] = 0
    w.grad = g.clone()
    opt.step()
    state_sum = opt.state[w]["sum"]
    expect_sum = g.pow(2).mean(dim=1)
    torch.testing.assert_close(state_sum.view(-1), expect_sum)
    expect = w0 - 0.1 * g / (expect_sum.sqrt().unsqueeze(1) + 1e-8)
    torch.testing.assert_close(w.detach(), expect)
    # second step accumulates
    w.grad = g.clone()
    opt.step()
    torch.testing.assert_close(opt.state[w]["sum"].view(-1), 2 * expect_sum)
    assert torch.equal(w.detach()[2], w0[2])
