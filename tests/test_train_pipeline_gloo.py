"""Pipelined training must produce the same losses and parameters as the plain loop
(cf. ``torchrec/distributed/train_pipeline/tests/test_train_pipelines.py``)."""
import copy

import pytest
import torch

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def _build(rank, world_size, ctx, seed=0):
    from torchrec_b200.datasets.utils import Batch
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.models.dlrm import DLRM, DLRMTrain
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    torch.manual_seed(seed)
    cfgs = [EmbeddingBagConfig(name=f"t{i}", num_embeddings=1000, embedding_dim=16, feature_names=[f"f{i}"]) for i in range(4)]
    ebc = EmbeddingBagCollection(cfgs)
    model = DLRMTrain(DLRM(ebc, dense_in_features=8, dense_arch_layer_sizes=[16, 16], over_arch_layer_sizes=[16, 1]))
    apply_optimizer_in_backward(RowWiseAdagrad, model.model.sparse_arch.parameters(), {"lr": 0.01})
    gens = {f"t{i}": (sp.table_wise(rank=i % world_size) if i != 1 else sp.row_wise()) for i in range(4)}
    plan = ShardingPlan({"model.sparse_arch.embedding_bag_collection": sp.construct_module_sharding_plan(
        ebc, gens, sharder=EmbeddingBagCollectionSharder(), world_size=world_size, local_size=world_size, device_type="cpu")})
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan)
    return dmp


def _batches(rank, n, B=32):
    from torchrec_b200.datasets.utils import Batch
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    g = torch.Generator().manual_seed(1234 + rank)
    out = []
    for _ in range(n):
        lengths = torch.randint(0, 6, (4 * B,), generator=g)
        values = torch.randint(0, 1000, (int(lengths.sum()),), generator=g)
        kjt = KeyedJaggedTensor.from_lengths_sync(keys=[f"f{i}" for i in range(4)], values=values, lengths=lengths)
        out.append(Batch(dense_features=torch.randn(B, 8, generator=g), sparse_features=kjt, labels=torch.randint(0, 2, (B,), generator=g).float()))
    return out


def _run(rank, world_size, pipeline_name):
    from torchrec_b200.distributed.train_pipeline import (
        TrainPipelineBase, TrainPipelineFusedSparseDist, TrainPipelineSemiSync, TrainPipelineSparseDist, PrefetchTrainPipelineSparseDist,
    )
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        n = 6
        batches = _batches(rank, n)

        def make():
            dmp = _build(rank, world_size, ctx)
            dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda p: torch.optim.SGD(p, lr=0.05))
            return dmp, CombinedOptimizer([dmp.fused_optimizer, dense])

        ref, ref_opt = make()
        ref_losses = []
        for b in batches:
            ref_opt.zero_grad()
            loss, _ = ref(b)
            loss.backward()
            ref_opt.step()
            ref_losses.append(loss.detach().clone())

        dmp, opt = make()
        cls = {"base": TrainPipelineBase, "sparse": TrainPipelineSparseDist, "fused": TrainPipelineFusedSparseDist,
               "semisync": TrainPipelineSemiSync, "prefetch": PrefetchTrainPipelineSparseDist}[pipeline_name]
        kwargs = {"start_batch": 10 ** 9} if pipeline_name == "semisync" else {}
        pipe = cls(dmp, opt, torch.device("cpu"), **kwargs)
        it = iter(batches)
        losses = []
        for _ in range(n):
            out = pipe.progress(it)
            losses.append(out[0])
        with pytest.raises(StopIteration):
            pipe.progress(it)
        for a, b in zip(losses, ref_losses):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
        for (n1, p1), (n2, p2) in zip(sorted(dmp.state_dict().items()), sorted(ref.state_dict().items())):
            if hasattr(p1, "local_shards"):
                for s1, s2 in zip(p1.local_shards(), p2.local_shards()):
                    torch.testing.assert_close(s1.tensor, s2.tensor, rtol=1e-5, atol=1e-6)
            else:
                torch.testing.assert_close(p1, p2, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("pipeline_name", ["base", "sparse", "fused", "semisync", "prefetch"])
def test_pipeline_matches_plain_loop(pipeline_name):
    run_multi_process(_run, world_size=2, pipeline_name=pipeline_name)


def _run_eval_and_staged(rank, world_size):
    from torchrec_b200.distributed.train_pipeline import EvalPipelineSparseDist, StagedTrainPipeline, TrainPipelinePT2
    from torchrec_b200.distributed.train_pipeline.pipeline_stage import PipelineStage, SparseDataDistUtil
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        batches = _batches(rank, 5)
        dmp = _build(rank, world_size, ctx)
        dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda p: torch.optim.SGD(p, lr=0.05))
        opt = CombinedOptimizer([dmp.fused_optimizer, dense])
        before = {k: (v.local_shards()[0].tensor.clone() if hasattr(v, "local_shards") and v.local_shards() else None) for k, v in dmp.state_dict().items()}
        # evaluation pipeline: same outputs as plain eval forwards, nothing is updated
        dmp.eval()
        with torch.no_grad():
            want = [dmp(b)[0].clone() for b in batches]
        pipe = EvalPipelineSparseDist(dmp, opt, torch.device("cpu"))
        it = iter(batches)
        got = [pipe.progress(it)[0] for _ in range(5)]
        with pytest.raises(StopIteration):
            pipe.progress(it)
        for a, b in zip(got, want):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
        for k, v in dmp.state_dict().items():
            if before[k] is not None:
                assert torch.equal(v.local_shards()[0].tensor, before[k])
        # staged pipeline: a transform stage and the sparse data dist stage run ahead of the model
        dmp.train()
        seen = []

        def tag(batch):
            seen.append(float(batch.dense_features.sum()))
            return batch

        util = SparseDataDistUtil(model=dmp, data_dist_stream=None)
        staged = StagedTrainPipeline(pipeline_stages=[
            PipelineStage(name="tag", runnable=tag, stream=None),
            PipelineStage(name="start_sparse_data_dist", runnable=util.start_sparse_data_dist, stream=None),
        ])
        it = iter(batches)
        losses = []
        while True:
            batch = staged.progress(it)
            if batch is None:
                break
            batch = util.wait_sparse_data_dist(batch)
            opt.zero_grad()
            loss, _ = dmp(batch)
            loss.backward()
            opt.step()
            losses.append(float(loss))
        assert len(losses) == 5 and len(seen) == 5
        assert all(l == l for l in losses)
        # the PT2 pipeline runs the uncompiled path when no compile config is given
        util.detach()
        pt2 = TrainPipelinePT2(dmp, opt, torch.device("cpu"))
        it = iter(batches[:2])
        assert pt2.progress(it) is not None and pt2.progress(it) is not None
        with pytest.raises(StopIteration):
            pt2.progress(it)


def test_eval_staged_and_pt2_pipelines():
    run_multi_process(_run_eval_and_staged, world_size=2)
