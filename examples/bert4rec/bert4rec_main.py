"""Masked-item training of BERT4Rec on synthetic sessions with a sharded item table.

    python examples/bert4rec/bert4rec_main.py --num_iterations 5
    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 8 examples/bert4rec/bert4rec_main.py --sharding column_wise

(cf. ``examples/bert4rec/bert4rec_main.py`` of the reference.)"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from torchrec_b200.distributed import sharding_plan as sp  # noqa: E402
from torchrec_b200.distributed.embedding import EmbeddingCollectionSharder  # noqa: E402
from torchrec_b200.distributed.model_parallel import DistributedModelParallel  # noqa: E402
from torchrec_b200.distributed.types import ShardingEnv, ShardingPlan  # noqa: E402
from torchrec_b200.models.bert4rec import BERT4Rec  # noqa: E402
from torchrec_b200.optim.apply_optimizer_in_backward import apply_optimizer_in_backward  # noqa: E402
from torchrec_b200.optim.keyed import CombinedOptimizer, KeyedOptimizerWrapper  # noqa: E402
from torchrec_b200.optim.optimizers import in_backward_optimizer_filter  # noqa: E402
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402


def synthetic_batch(batch_size: int, max_len: int, vocab: int, mask_prob: float, gen: torch.Generator, device: torch.device):
    """Sessions with lengths in [max_len/10, max_len], Zipf-like item ids; ``mask_prob`` of the positions replaced by the mask id (vocab-1)."""
    lengths = torch.randint(max(max_len // 10, 1), max_len + 1, (batch_size,), generator=gen)
    n = int(lengths.sum())
    u = torch.rand(n, generator=gen)
    items = ((vocab - 2) ** u).long().clamp(1, vocab - 2)
    masked = torch.rand(n, generator=gen) < mask_prob
    inputs = torch.where(masked, torch.full_like(items, vocab - 1), items)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), lengths.cumsum(0)])
    row = torch.repeat_interleave(torch.arange(batch_size), lengths)
    col = torch.arange(n) - offsets[:-1][row]
    flat_pos = (row * max_len + col)[masked]
    kjt = KeyedJaggedTensor(keys=["item"], values=inputs, lengths=lengths, stride=batch_size)
    return kjt.to(device), flat_pos.to(device), items[masked].to(device)


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--vocab_size", type=int, default=20000)
    p.add_argument("--max_len", type=int, default=50)
    p.add_argument("--emb_dim", type=int, default=64)
    p.add_argument("--nhead", type=int, default=4)
    p.add_argument("--num_layers", type=int, default=2)
    p.add_argument("--batch_size", type=int, default=64)
    p.add_argument("--num_negatives", type=int, default=512)
    p.add_argument("--num_iterations", type=int, default=10)
    p.add_argument("--lr", type=float, default=1e-3)
    p.add_argument("--sharding", default="row_wise", choices=["table_wise", "row_wise", "column_wise", "data_parallel"])
    a = p.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if torch.cuda.is_available():
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
        torch.cuda.set_device(device)
        backend = "nccl"
    else:
        device, backend = torch.device("cpu"), "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29551")
        dist.init_process_group(backend, rank=rank, world_size=world)
    torch.manual_seed(0)
    model = BERT4Rec(a.vocab_size, a.max_len, a.emb_dim, a.nhead, a.num_layers).to(device)
    apply_optimizer_in_backward(torch.optim.Adam, model.history.ec.parameters(), {"lr": a.lr})
    gen_fn = {"table_wise": lambda: sp.table_wise(rank=0), "row_wise": sp.row_wise, "data_parallel": sp.data_parallel,
              "column_wise": lambda: sp.column_wise(ranks=list(range(min(world, max(a.emb_dim // 32, 1)))))}[a.sharding]
    sharder = EmbeddingCollectionSharder()
    module_plan = sp.construct_module_sharding_plan(model.history.ec, {"item_embedding": gen_fn()}, sharder=sharder, world_size=world, local_size=world, device_type=device.type)
    dmp = DistributedModelParallel(model, env=ShardingEnv.from_process_group(dist.group.WORLD), device=device, plan=ShardingPlan({"history.ec": module_plan}), sharders=[sharder])
    dense = KeyedOptimizerWrapper(dict(in_backward_optimizer_filter(dmp.named_parameters())), lambda ps: torch.optim.Adam(ps, lr=a.lr))
    opt = CombinedOptimizer([dmp.fused_optimizer, dense])
    gen = torch.Generator().manual_seed(100 + rank)
    for it in range(a.num_iterations):
        kjt, pos, targets = synthetic_batch(a.batch_size, a.max_len, a.vocab_size, 0.15, gen, device)
        negatives = torch.randint(1, a.vocab_size - 1, (a.num_negatives,), generator=gen).to(device)
        opt.zero_grad()
        logits = dmp.module.sampled_logits(kjt, pos, targets, negatives) if world == 1 else dmp(kjt).reshape(-1, a.vocab_size).index_select(0, pos)
        labels = torch.zeros(logits.shape[0], dtype=torch.long, device=device) if world == 1 else targets
        loss = torch.nn.functional.cross_entropy(logits.float(), labels)
        loss.backward()
        opt.step()
        if rank == 0:
            print(f"iter {it + 1}: masked-item loss {float(loss):.4f} ({logits.shape[0]} masked positions)", flush=True)


if __name__ == "__main__":
    main()
