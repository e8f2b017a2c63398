"""The same two tables under every sharding type: prints which rank holds which block of each table and checks that the sharded
lookup equals the unsharded one (cf. the sharding tutorials under ``examples/sharding`` of the reference).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 examples/sharding/sharding_types.py
"""
from __future__ import annotations

import copy
import os
import sys

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
        os.environ.setdefault("MASTER_PORT", "29554")
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    tables = [EmbeddingBagConfig(name="large", embedding_dim=64, num_embeddings=4096, feature_names=["f_large"]),
              EmbeddingBagConfig(name="small", embedding_dim=64, num_embeddings=64, feature_names=["f_small"])]
    reference = EmbeddingBagCollection(tables=tables)
    lengths = torch.randint(0, 4, (2 * 8,), generator=torch.Generator().manual_seed(rank))
    kjt = KeyedJaggedTensor(keys=["f_large", "f_small"], values=torch.randint(0, 64, (int(lengths.sum()),), generator=torch.Generator().manual_seed(10 + rank)), lengths=lengths)
    want = reference(kjt).values()
    generators = {"table_wise": lambda i: sp.table_wise(rank=i % world), "row_wise": lambda i: sp.row_wise(), "data_parallel": lambda i: sp.data_parallel(),
                  "column_wise": lambda i: sp.column_wise(ranks=[(i + j) % world for j in range(2)])}
    for name, gen in generators.items():
        model = torch.nn.Module()
        model.ebc = copy.deepcopy(reference)
        sharder = EmbeddingBagCollectionSharder()
        mplan = sp.construct_module_sharding_plan(model.ebc, {t.name: gen(i) for i, t in enumerate(tables)}, sharder=sharder, world_size=world, local_size=world, device_type=device.type)
        dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=ShardingPlan({"ebc": mplan}), sharders=[sharder])
        dmp.load_state_dict(reference.state_dict() if False else {f"ebc.{k}": v for k, v in reference.state_dict().items()})
        got = dmp.module.ebc(kjt.to(device)).wait().values().cpu()
        assert torch.allclose(got, want, atol=1e-5), name
        if rank == 0:
            for t, ps in mplan.items():
                where = "replicated" if ps.sharding_spec is None else ", ".join(f"{s.placement}: rows {s.shard_offsets[0]}+{s.shard_sizes[0]} cols {s.shard_offsets[1]}+{s.shard_sizes[1]}" for s in ps.sharding_spec.shards)
                print(f"{name:14s} {t:6s} -> {where}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
