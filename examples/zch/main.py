"""Managed collision in front of an embedding collection: raw ids from an unbounded space are remapped onto a small table, either
by the sort-based module (LFU eviction) or by the multi-probe zero-collision hash; the script reports how many distinct raw ids
ended up sharing a row (cf. ``examples/zch/main.py`` of the reference).

    python examples/zch/main.py --mode mpzch --num_iterations 20
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig  # noqa: E402
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from torchrec_b200.modules.hash_mc_modules import HashZchManagedCollisionModule  # noqa: E402
from torchrec_b200.modules.mc_embedding_modules import ManagedCollisionEmbeddingBagCollection  # noqa: E402
from torchrec_b200.modules.mc_modules import LFU_EvictionPolicy, ManagedCollisionCollection, MCHManagedCollisionModule  # noqa: E402
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--mode", choices=["mpzch", "sort"], default="mpzch")
    p.add_argument("--zch_size", type=int, default=4096)
    p.add_argument("--distinct_ids", type=int, default=3000)
    p.add_argument("--batch_size", type=int, default=512)
    p.add_argument("--num_iterations", type=int, default=20)
    a = p.parse_args()
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    torch.manual_seed(0)
    cfg = EmbeddingBagConfig(name="t", embedding_dim=16, num_embeddings=a.zch_size, feature_names=["f"])
    if a.mode == "mpzch":
        mc = HashZchManagedCollisionModule(zch_size=a.zch_size, device=device, total_num_buckets=4, max_probe=64)
    else:
        mc = MCHManagedCollisionModule(zch_size=a.zch_size, device=device, eviction_policy=LFU_EvictionPolicy(), eviction_interval=2)
    model = ManagedCollisionEmbeddingBagCollection(EmbeddingBagCollection(tables=[cfg], device=device), ManagedCollisionCollection({"t": mc}, [cfg]),
                                                   return_remapped_features=True)
    universe = torch.randint(0, 2 ** 40, (a.distinct_ids,))
    seen = {}
    for it in range(a.num_iterations):
        raw = universe[torch.randint(0, a.distinct_ids, (a.batch_size,))]
        kjt = KeyedJaggedTensor(keys=["f"], values=raw.to(device), lengths=torch.ones(a.batch_size, dtype=torch.int64, device=device))
        pooled, remapped = model(kjt)
        pooled.values().sum().backward()
        for r, s in zip(raw.tolist(), remapped.values().tolist()):
            seen[r] = s
    rows = {}
    for r, s in seen.items():
        rows.setdefault(s, set()).add(r)
    shared = sum(len(v) for v in rows.values() if len(v) > 1)
    print(f"{a.mode}: {len(seen)} distinct raw ids -> {len(rows)} rows of {a.zch_size}; {shared} ids share a row ({100.0 * shared / max(len(seen), 1):.2f}%)")


if __name__ == "__main__":
    main()
