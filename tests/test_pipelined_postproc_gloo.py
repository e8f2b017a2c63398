"""A parameter-free module between the batch and the sharded embedding module is pipelined with the input dist: it runs once per
batch, ahead of the forward, and training matches the plain loop (``torchrec/distributed/train_pipeline/tests/test_train_pipelines.py``,
postproc cases)."""
import torch
from torch import nn

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


class _Remap(nn.Module):
    """ids -> (ids * 7 + 3) % 1000; counts its calls."""

    def __init__(self):
        super().__init__()
        self.calls = 0

    def forward(self, kjt):
        from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

        self.calls += 1
        return KeyedJaggedTensor(keys=kjt.keys(), values=(kjt.values() * 7 + 3) % 1000, lengths=kjt.lengths())


class _Net(nn.Module):
    def __init__(self, inner):
        super().__init__()
        self.remap = _Remap()
        self.inner = inner

    def forward(self, batch):
        from torchrec_b200.datasets.utils import Batch

        return self.inner(Batch(dense_features=batch.dense_features, sparse_features=self.remap(batch.sparse_features), labels=batch.labels))


def _run(rank, world_size):
    from tests.test_train_pipeline_gloo import _batches
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.train_pipeline import TrainPipelineSparseDist
    from torchrec_b200.distributed.train_pipeline.postproc import PipelinedPostproc
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.models.dlrm import DLRM, DLRMTrain
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        def make():
            torch.manual_seed(0)
            cfgs = [EmbeddingBagConfig(name=f"t{i}", num_embeddings=1000, embedding_dim=16, feature_names=[f"f{i}"]) for i in range(4)]
            ebc = EmbeddingBagCollection(cfgs)
            net = _Net(DLRMTrain(DLRM(ebc, dense_in_features=8, dense_arch_layer_sizes=[16, 16], over_arch_layer_sizes=[16, 1])))
            apply_optimizer_in_backward(RowWiseAdagrad, ebc.parameters(), {"lr": 0.01})
            gens = {f"t{i}": (sp.table_wise(rank=i % world_size) if i != 1 else sp.row_wise()) for i in range(4)}
            plan = ShardingPlan({"inner.model.sparse_arch.embedding_bag_collection": sp.construct_module_sharding_plan(
                ebc, gens, sharder=EmbeddingBagCollectionSharder(), world_size=world_size, local_size=world_size, device_type="cpu")})
            dmp = DistributedModelParallel(net, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan)
            dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda p: torch.optim.SGD(p, lr=0.05))
            return dmp, CombinedOptimizer([dmp.fused_optimizer, dense])

        n = 6
        batches = _batches(rank, n)
        ref, ref_opt = make()
        ref_losses = []
        for b in batches:
            ref_opt.zero_grad()
            loss, _ = ref(b)
            loss.backward()
            ref_opt.step()
            ref_losses.append(loss.detach().clone())

        dmp, opt = make()
        pipe = TrainPipelineSparseDist(dmp, opt, torch.device("cpu"), pipeline_postproc=True)
        it = iter(batches)
        losses = []
        for _ in range(n):
            out = pipe.progress(it)
            losses.append((out[0] if isinstance(out, tuple) else out).detach().clone())
        for a, b in zip(losses, ref_losses):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
        wrapped = [m for m in dmp.modules() if isinstance(m, PipelinedPostproc)]
        assert len(wrapped) == 1 and wrapped[0].fqn.endswith("remap")
        # the embedding module is pipelined (its input comes from the batch through the remap module) and the remap ran once per batch
        assert len(pipe._pipelined_modules) == 1
        assert wrapped[0].postproc_module.calls == n
        # detaching gives the original module back
        pipe.detach()
        assert not any(isinstance(m, PipelinedPostproc) for m in dmp.modules())

        # without the flag the embedding module's input is computed inside the model: nothing is pipelined, results are equal
        dmp2, opt2 = make()
        pipe2 = TrainPipelineSparseDist(dmp2, opt2, torch.device("cpu"), pipeline_postproc=False)
        it2 = iter(batches)
        for i in range(n):
            out = pipe2.progress(it2)
            torch.testing.assert_close((out[0] if isinstance(out, tuple) else out).detach(), ref_losses[i], rtol=1e-5, atol=1e-6)
        assert len(pipe2._pipelined_modules) == 0


def test_pipelined_postproc():
    run_multi_process(_run, world_size=2)
