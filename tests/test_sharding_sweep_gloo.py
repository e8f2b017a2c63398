"""Seeded sweep over (sharding type x compute kernel x quantised comms x optimizer x pooling x weighted input): every drawn
combination trains a sharded model for two steps on two gloo ranks and must track the unsharded model (predictions each step,
tables at the end).  The combinations are a fixed-seed sample of the full product, so the file covers pairings that no
hand-written case names (cf. ``torchrec/distributed/test_utils/test_model_parallel.py:306-1079``, which draws the same axes
with hypothesis)."""
import copy
import itertools
import random

import pytest
import torch
import torch.distributed as dist

import test_sharding_gloo as T
from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process

AXES = {
    "sharding": ["tw", "rw", "cw", "twrw", "grid", "mixed"],
    "kernel": ["fused", "dense"],
    "qcomm": ["none", "fp16"],
    "optimizer": ["sgd", "adagrad", "rowwise_adagrad", "adam"],
    "pooling": ["SUM", "MEAN"],
    "weighted": [False, True],
}


def _valid(c) -> bool:
    if c["weighted"] and c["pooling"] == "MEAN":
        return False  # a weighted mean has no unsharded counterpart in the module under test
    if c["optimizer"] == "rowwise_adagrad" and c["sharding"] in ("cw", "grid", "mixed"):
        return False  # a column shard keeps its own row-wise state: not the unsharded update
    if c["kernel"] == "dense" and c["optimizer"] != "sgd":
        return False  # dense kernels hand their gradient to an ordinary optimizer; one of them is enough
    return True


def _draw(n: int, seed: int):
    product = [dict(zip(AXES, values)) for values in itertools.product(*AXES.values())]
    valid = [c for c in product if _valid(c)]
    return random.Random(seed).sample(valid, n)


CASES = _draw(10, seed=2024)


def _case_id(c) -> str:
    return "-".join(str(c[k]) for k in AXES)


def _run(rank, world_size, case):
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.fbgemm_qcomm_codec import CommType, QCommsConfig, get_qcomm_codecs_registry
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.modules.embedding_configs import PoolingType
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    optimizers = {"sgd": (torch.optim.SGD, {"lr": 0.1}), "adagrad": (torch.optim.Adagrad, {"lr": 0.1, "eps": 1e-8}),
                  "rowwise_adagrad": (RowWiseAdagrad, {"lr": 0.1, "eps": 1e-8}), "adam": (torch.optim.Adam, {"lr": 0.05, "eps": 1e-8})}
    opt_cls, kw = optimizers[case["optimizer"]]
    weighted, B = case["weighted"], 6
    loose = case["qcomm"] != "none"
    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        global_model = T._Model(T._make_ebc(PoolingType[case["pooling"]], weighted))
        local_model = copy.deepcopy(global_model)
        fused = case["kernel"] == "fused"
        if fused:
            apply_optimizer_in_backward(opt_cls, local_model.ebc.parameters(), kw)
        registry = None
        if case["qcomm"] == "fp16":
            registry = get_qcomm_codecs_registry(QCommsConfig(forward_precision=CommType.FP16, backward_precision=CommType.FP16))
        sharder = EmbeddingBagCollectionSharder(qcomm_codecs_registry=registry)
        module_plan = T._plan_for(local_model.ebc, case["sharding"], world_size)
        if not fused:
            for ps in module_plan.values():
                ps.compute_kernel = "dense"
        dmp = DistributedModelParallel(local_model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"),
                                       plan=ShardingPlan({"ebc": module_plan}), sharders=[sharder])
        dmp.load_state_dict(copy.deepcopy(global_model.state_dict()))
        if fused:
            local_opt = torch.optim.SGD([p for n, p in dmp.named_parameters() if "ebc" not in n], lr=0.1)
        else:  # dense kernels: the tables are ordinary parameters of the local optimizer (their gradient is already complete)
            local_opt = torch.optim.SGD([p for _, p in dmp.named_parameters()], lr=0.1)
        g_emb_opt = opt_cls(global_model.ebc.parameters(), **kw) if fused else torch.optim.SGD(global_model.ebc.parameters(), lr=0.1)
        g_dense_opt = torch.optim.SGD(global_model.over.parameters(), lr=0.1)
        kjts = [T._make_kjt(B, 100 + r, weighted) for r in range(world_size)]
        keys = kjts[0].keys()
        vals, lens, ws = [], [], []
        for k in keys:
            for kj in kjts:
                jt = kj[k]
                vals.append(jt.values())
                lens.append(jt.lengths())
                if weighted:
                    ws.append(jt.weights())
        global_kjt = KeyedJaggedTensor.from_lengths_sync(keys=keys, values=torch.cat(vals), lengths=torch.cat(lens), weights=torch.cat(ws) if weighted else None)
        rtol, atol = (2e-2, 2e-3) if loose else (1e-4, 1e-5)
        for _ in range(2):
            g_emb_opt.zero_grad()
            g_dense_opt.zero_grad()
            g_pred, _ = global_model(global_kjt)
            g_pred.mean().backward()
            g_emb_opt.step()
            g_dense_opt.step()
            local_opt.zero_grad()
            l_pred, _ = dmp(kjts[rank])
            l_pred.mean().backward()
            local_opt.step()
            torch.testing.assert_close(l_pred.detach(), g_pred.detach()[rank * B:(rank + 1) * B], rtol=rtol, atol=atol)
        sd = dmp.state_dict()
        for name, want in global_model.state_dict().items():
            got = sd[name]
            if hasattr(got, "local_shards"):
                mine = torch.zeros_like(want)
                for s in got.local_shards():
                    (r0, c0), (nr, nc) = s.metadata.shard_offsets, s.metadata.shard_sizes
                    mine[r0:r0 + nr, c0:c0 + nc] = s.tensor
                dist.all_reduce(mine)
                got = mine
            torch.testing.assert_close(got, want, rtol=rtol, atol=atol * 10 if loose else atol)


@pytest.mark.parametrize("case", CASES, ids=[_case_id(c) for c in CASES])
def test_drawn_combination_tracks_the_unsharded_model(case):
    run_multi_process(_run, world_size=2, case=case)


def test_the_draw_is_stable_and_spans_the_axes():
    assert CASES == _draw(10, seed=2024)
    for axis, values in AXES.items():
        seen = {c[axis] for c in CASES}
        assert len(seen) >= min(2, len(values)), f"axis {axis} is not exercised: {seen}"
