"""The plumbing configuration: tiny DLRM, 4 tables x 1000 rows x dim 16 (sum pooling, U(+-1/sqrt(rows)) init), 8 dense features,
bottom MLP 8-16-16, dot interaction, top MLP 16-1, BCE, batch 32 per rank, row-wise Adagrad lr 0.01 on the tables and SGD on the
dense part; table-wise sharded over two gloo ranks and trained through ``TrainPipelineSparseDist``.  The loss must fall and every
rank must end with identical dense weights."""
import torch
import torch.distributed as dist

from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def _run(rank, world_size):
    from torchrec_b200.datasets.utils import Batch
    from torchrec_b200.distributed import sharding_plan as sp
    from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder
    from torchrec_b200.distributed.model_parallel import DistributedModelParallel
    from torchrec_b200.distributed.train_pipeline import TrainPipelineSparseDist
    from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan
    from torchrec_b200.models.dlrm import DLRM, DLRMTrain
    from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig
    from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
    from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward
    from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper
    from torchrec_b200.optim.optimizers import in_backward_optimizer_filter
    from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad
    from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

    with MultiProcessContext(rank, world_size, "gloo") as ctx:
        torch.manual_seed(0)
        tables = [EmbeddingBagConfig(name=f"t{i}", embedding_dim=16, num_embeddings=1000, feature_names=[f"f{i}"]) for i in range(4)]
        ebc = EmbeddingBagCollection(tables=tables, device=torch.device("meta"))
        model = DLRMTrain(DLRM(ebc, dense_in_features=8, dense_arch_layer_sizes=[16, 16], over_arch_layer_sizes=[16, 1]))
        apply_optimizer_in_backward(RowWiseAdagrad, model.model.sparse_arch.parameters(), {"lr": 0.01})
        plan = ShardingPlan({"model.sparse_arch.embedding_bag_collection": sp.construct_module_sharding_plan(
            ebc, {f"t{i}": sp.table_wise(rank=i % world_size) for i in range(4)}, sharder=EmbeddingBagCollectionSharder(), world_size=world_size,
            local_size=world_size, device_type="cpu")})
        dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(ctx.pg), device=torch.device("cpu"), plan=plan)
        w = dict(dmp.state_dict())["model.sparse_arch.embedding_bag_collection.embedding_bags.t0.weight"]
        local = w.local_shards()
        if local:
            assert local[0].tensor.abs().max() <= 1000 ** -0.5 + 1e-6  # U(-1/sqrt(rows), 1/sqrt(rows))
        dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda ps: torch.optim.SGD(ps, lr=0.1))
        opt = CombinedOptimizer([dmp.fused_optimizer, dense])
        pipe = TrainPipelineSparseDist(dmp, opt, torch.device("cpu"))
        g = torch.Generator().manual_seed(100 + rank)
        true_w = torch.randn(8, generator=torch.Generator().manual_seed(5))

        def batches(n):
            for _ in range(n):
                lengths = torch.randint(0, 6, (4 * 32,), generator=g)
                values = torch.randint(0, 1000, (int(lengths.sum()),), generator=g)
                x = torch.randn(32, 8, generator=g)
                labels = (torch.rand(32, generator=g) < torch.sigmoid(x @ true_w)).float()  # learnable from the dense features
                yield Batch(dense_features=x, sparse_features=KeyedJaggedTensor(keys=[f"f{i}" for i in range(4)], values=values, lengths=lengths), labels=labels)

        it = iter(batches(120))
        losses = []
        while True:
            try:
                out = pipe.progress(it)  # the model's auxiliary output: (loss, logits, labels)
                losses.append(float(out[0]))
            except StopIteration:
                break
        assert len(losses) == 120
        first, last = sum(losses[:20]) / 20, sum(losses[-20:]) / 20
        assert last < first - 0.015, (first, last)
        for name, p in dmp.named_parameters():
            if "embedding_bags" in name:
                continue
            ref = p.detach().clone()
            dist.broadcast(ref, src=0)
            torch.testing.assert_close(p.detach(), ref, msg=lambda m: f"{name}: {m}")


def test_tiny_dlrm_table_wise_two_ranks():
    run_multi_process(_run, world_size=2)
