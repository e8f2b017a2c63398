"""Clipping / warm-up / semi-sync wrappers (cf. ``torchrec/optim/tests/test_clipping.py``, ``test_warmup.py``)."""
import math

import torch

from torchrec_b200.optim.clipping import GradientClipping, GradientClippingOptimizer
from torchrec_b200.optim.keyed import KeyedOptimizerWrapper
from torchrec_b200.optim.semi_sync import SemisyncOptimizer
from torchrec_b200.optim.warmup import WarmupOptimizer, WarmupPolicy, WarmupStage


def _keyed(params, lr=1.0):
    return KeyedOptimizerWrapper({f"p{i}": p for i, p in enumerate(params)}, lambda ps: torch.optim.SGD(ps, lr=lr))


def test_clip_norm_and_value():
    p = torch.nn.Parameter(torch.tensor([1.0, 1.0]))
    opt = GradientClippingOptimizer(_keyed([p]), clipping=GradientClipping.NORM, max_gradient=1.0, norm_type=2.0)
    p.grad = torch.tensor([3.0, 4.0])
    opt.step()
    torch.testing.assert_close(p.detach(), torch.tensor([1 - 0.6, 1 - 0.8]), rtol=1e-4, atol=1e-5)
    q = torch.nn.Parameter(torch.tensor([0.0, 0.0]))
    opt = GradientClippingOptimizer(_keyed([q]), clipping=GradientClipping.VALUE, max_gradient=0.5)
    q.grad = torch.tensor([3.0, -0.2])
    opt.step()
    torch.testing.assert_close(q.detach(), torch.tensor([-0.5, 0.2]))


def test_global_norm_with_sharded_param():
    a = torch.nn.Parameter(torch.zeros(2)); b = torch.nn.Parameter(torch.zeros(2))
    b._is_sharded = True
    opt = GradientClippingOptimizer(_keyed([a, b]), clipping=GradientClipping.NORM, max_gradient=1.0, enable_global_grad_clip=True)
    a.grad = torch.tensor([3.0, 0.0]); b.grad = torch.tensor([0.0, 4.0])
    opt.step()
    assert math.isclose(float(opt._last_total_norm), 5.0, rel_tol=1e-5)
    torch.testing.assert_close(torch.cat([a.detach(), b.detach()]), -torch.tensor([0.6, 0.0, 0.0, 0.8]), rtol=1e-4, atol=1e-5)


def test_warmup_schedule_and_state_dict():
    p = torch.nn.Parameter(torch.zeros(1))
    stages = [WarmupStage(WarmupPolicy.LINEAR, max_iters=4, value=0.0), WarmupStage(WarmupPolicy.CONSTANT, max_iters=6, value=0.5)]
    opt = WarmupOptimizer(_keyed([p]), stages, lr=2.0)
    lrs = []
    for _ in range(8):
        lrs.append(opt.param_groups[0]["lr"])
        p.grad = torch.ones(1)
        opt.step()
    assert lrs == [0.0, 0.5, 1.0, 1.5, 1.0, 1.0, 2.0, 2.0]
    sd = opt.state_dict()
    opt2 = WarmupOptimizer(_keyed([torch.nn.Parameter(torch.zeros(1))]), stages, lr=2.0)
    opt2.load_state_dict(sd)
    assert opt2.param_groups[0]["lr"] == 2.0


def test_semisync_single_rank_matches_outer_sgd():
    p = torch.nn.Parameter(torch.tensor([1.0]))
    local = _keyed([p], lr=0.1)
    outer = _keyed([p], lr=1.0)  # outer SGD with lr 1 on the drift = plain local training
    opt = SemisyncOptimizer([p], outer, local, num_local_steps=2)
    for _ in range(4):
        p.grad = torch.ones(1)
        opt.step()
    torch.testing.assert_close(p.detach(), torch.tensor([0.6]))
    assert int(opt._global_step_counter) == 2
