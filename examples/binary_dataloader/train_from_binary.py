"""Train DLRM from pre-processed binary Criteo files (``*_dense.npy`` / ``*_sparse.npy`` / ``*_labels.npy``): every rank maps its
row range of every file, batches come out of host memory as KJTs, and the sparse-dist pipeline overlaps the host-to-device copy
and the input distribution of the next batch with the current step.  Without ``--data_dir`` the script first writes small
synthetic files of the right format.

    python examples/binary_dataloader/train_from_binary.py --num_rows 4096 --batch_size 256
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/binary_dataloader/train_from_binary.py --data_dir /data/criteo_npy

This is the role ``examples/nvt_dataloader`` plays in the reference (a binary loader feeding the trainer); the files here are the
ones ``torchrec_b200/datasets/scripts/npy_preproc_criteo.py`` produces."""
from __future__ import annotations

import argparse
import contextlib
import glob
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from torchrec_b200.datasets.criteo import CAT_FEATURE_COUNT, DEFAULT_CAT_NAMES, INT_FEATURE_COUNT, InMemoryBinaryCriteoIterDataPipe  # noqa: E402
from torchrec_b200.datasets.test_utils.criteo_test_utils import create_dataset_npys  # noqa: E402
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder  # noqa: E402
from torchrec_b200.distributed.model_parallel import DistributedModelParallel  # noqa: E402
from torchrec_b200.distributed.planner import EmbeddingShardingPlanner, Topology  # noqa: E402
from torchrec_b200.distributed.train_pipeline import TrainPipelineSparseDist  # noqa: E402
from torchrec_b200.distributed.types import ShardingEnv  # noqa: E402
from torchrec_b200.models.dlrm import DLRM, DLRMTrain  # noqa: E402
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig  # noqa: E402
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward  # noqa: E402
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper  # noqa: E402
from torchrec_b200.optim.optimizers import in_backward_optimizer_filter  # noqa: E402
from torchrec_b200.optim.rowwise_adagrad import RowWiseAdagrad  # noqa: E402


def main(argv=None) -> float:
    p = argparse.ArgumentParser()
    p.add_argument("--data_dir", default="", help="folder with *_dense.npy, *_sparse.npy, *_labels.npy")
    p.add_argument("--num_rows", type=int, default=4096, help="rows of the synthetic files when no --data_dir is given")
    p.add_argument("--batch_size", type=int, default=256)
    p.add_argument("--hash_size", type=int, default=1000)
    p.add_argument("--embedding_dim", type=int, default=32)
    p.add_argument("--epochs", type=int, default=1)
    a = p.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        torch.cuda.set_device(device)
    else:
        device = torch.device("cpu")
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29547")
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", rank=rank, world_size=world)
    with contextlib.ExitStack() as stack:
        if a.data_dir:
            dense, sparse, labels = (sorted(glob.glob(os.path.join(a.data_dir, f"*_{kind}.npy"))) for kind in ("dense", "sparse", "labels"))
        else:
            d, s, l = stack.enter_context(create_dataset_npys(num_rows=a.num_rows, seed=0))
            dense, sparse, labels = [d], [s], [l]
        data = InMemoryBinaryCriteoIterDataPipe("train", dense, sparse, labels, batch_size=a.batch_size, rank=rank, world_size=world, drop_last=True,
                                                shuffle_batches=True, hashes=[a.hash_size] * CAT_FEATURE_COUNT, mmap_mode=True)
        tables = [EmbeddingBagConfig(name=f"t_{k}", embedding_dim=a.embedding_dim, num_embeddings=a.hash_size, feature_names=[k]) for k in DEFAULT_CAT_NAMES]
        model = DLRMTrain(DLRM(EmbeddingBagCollection(tables=tables, device=torch.device("meta")), dense_in_features=INT_FEATURE_COUNT,
                               dense_arch_layer_sizes=[64, a.embedding_dim], over_arch_layer_sizes=[128, 64, 1], dense_device=device))
        apply_optimizer_in_backward(RowWiseAdagrad, model.model.sparse_arch.parameters(), {"lr": 0.05})
        sharders = [EmbeddingBagCollectionSharder()]
        plan = EmbeddingShardingPlanner(topology=Topology(world_size=world, local_world_size=world, compute_device=device.type),
                                        batch_size=a.batch_size).collective_plan(model, sharders, dist.group.WORLD)
        dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=plan, sharders=sharders)
        dense_opt = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda params: torch.optim.Adagrad(params, lr=0.05))
        pipe = TrainPipelineSparseDist(dmp, CombinedOptimizer([dmp.fused_optimizer, dense_opt]), device)
        first = last = None
        for epoch in range(a.epochs):
            it, n, total = iter(data), 0, 0.0
            while True:
                try:
                    out = pipe.progress(it)
                except StopIteration:
                    break
                loss = float((out[0] if isinstance(out, tuple) else out).detach())
                first = loss if first is None else first
                total, n, last = total + loss, n + 1, loss
            if rank == 0:
                print(f"epoch {epoch}: {n} batches of {a.batch_size}, mean loss {total / max(n, 1):.4f}")
        return float(last if last is not None else float("nan"))


if __name__ == "__main__":
    main()
