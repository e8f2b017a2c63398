"""Start a sharded model from a pretrained embedding table: the table is written to a shared tensor file, every rank maps it and
copies only the rows / columns of its own shards into the sharded module (cf. ``examples/transfer_learning/
train_from_pretrained_embedding.py`` of the reference).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/transfer_learning/train_from_pretrained_embedding.py
"""
from __future__ import annotations

import os
import sys
import tempfile

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from torchrec_b200.distributed import sharding_plan as sp  # noqa: E402
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder  # noqa: E402
from torchrec_b200.distributed.model_parallel import DistributedModelParallel  # noqa: E402
from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan  # noqa: E402
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig  # noqa: E402
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402


def main() -> None:
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if torch.cuda.is_available() else torch.device("cpu")
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29553")
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", rank=rank, world_size=world)
    rows, dim = 1000, 32
    path = os.path.join(tempfile.gettempdir(), "trb200_pretrained_embedding.pt")
    if rank == 0:
        torch.manual_seed(0)
        torch.save(torch.arange(rows, dtype=torch.float32).unsqueeze(1).repeat(1, dim) / rows, path)  # row r holds r/rows: easy to check
    dist.barrier()
    pretrained = torch.load(path, mmap=True)
    model = torch.nn.Module()
    model.ebc = EmbeddingBagCollection(tables=[EmbeddingBagConfig(name="t", embedding_dim=dim, num_embeddings=rows, feature_names=["f"])], device=torch.device("meta"))
    sharder = EmbeddingBagCollectionSharder()
    plan = ShardingPlan({"ebc": sp.construct_module_sharding_plan(model.ebc, {"t": sp.row_wise()}, sharder=sharder, world_size=world, local_size=world, device_type=device.type)})
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=plan, sharders=[sharder])
    with torch.no_grad():
        for shard in dmp.state_dict()["ebc.embedding_bags.t.weight"].local_shards():
            (r0, c0), (nr, nc) = shard.metadata.shard_offsets, shard.metadata.shard_sizes
            shard.tensor.copy_(pretrained[r0:r0 + nr, c0:c0 + nc])
    ids = torch.tensor([3, 500, 999], device=device)
    out = dmp.module.ebc(KeyedJaggedTensor(keys=["f"], values=ids, lengths=torch.ones(3, dtype=torch.int64, device=device))).wait()
    assert torch.allclose(out["f"][:, 0].cpu(), ids.cpu().float() / rows), out["f"][:, 0]
    if rank == 0:
        print("sharded lookups return the pretrained rows:", out["f"][:, 0].tolist())
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
