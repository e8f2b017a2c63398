"""How skewed is an id stream?  Counts, per feature, the distinct ids, the share of lookups taken by the most frequent ids and the
number of ids that cover 50 / 90 / 99 % of the lookups -- the figures that decide how large a zero-collision table must be.

    python -m torchrec_b200.distributed.benchmark.benchmark_zch.count_dataset_distributions --num_batches 50

Runs on the benchmark's synthetic Zipf stream, or on any iterable of KJTs through ``count_distributions``
(``torchrec/distributed/benchmark/benchmark_zch/count_dataset_distributions.py`` of the reference does this for its datasets)."""
from __future__ import annotations

import argparse
import json
from typing import Dict, Iterable, List, Optional

import torch

from torchrec_b200.distributed.benchmark.benchmark_zch.benchmark_zch_utils import ZipfIdStream
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def count_distributions(batches: Iterable[KeyedJaggedTensor], top_k: int = 100) -> Dict[str, Dict[str, float]]:
    seen: Dict[str, List[torch.Tensor]] = {}
    for kjt in batches:
        for key, jt in kjt.to_dict().items():
            seen.setdefault(key, []).append(jt.values().cpu())
    out: Dict[str, Dict[str, float]] = {}
    for key, parts in seen.items():
        ids = torch.cat(parts)
        _, counts = torch.unique(ids, return_counts=True)
        counts, _ = torch.sort(counts, descending=True)
        cum = torch.cumsum(counts.double(), 0) / max(int(ids.numel()), 1)
        cover = {f"ids_for_{int(q * 100)}pct": int(torch.searchsorted(cum, torch.tensor(q, dtype=torch.double)).item()) + 1 for q in (0.5, 0.9, 0.99)}
        out[key] = {"lookups": int(ids.numel()), "distinct_ids": int(counts.numel()), f"top_{top_k}_share": float(cum[min(top_k, counts.numel()) - 1]), **cover}
    return out


def main(argv: Optional[List[str]] = None) -> Dict[str, Dict[str, float]]:
    p = argparse.ArgumentParser(description=__doc__)
    p.add_argument("--num_features", type=int, default=2)
    p.add_argument("--distinct_ids", type=int, default=15_000)
    p.add_argument("--zipf_alpha", type=float, default=1.05)
    p.add_argument("--batch_size", type=int, default=4096)
    p.add_argument("--num_batches", type=int, default=20)
    a = p.parse_args(argv)
    stream = ZipfIdStream(a.num_features, a.distinct_ids, a.zipf_alpha, 2 ** 50)
    batches = (KeyedJaggedTensor(keys=[f"f{i}" for i in range(a.num_features)], values=torch.cat([stream.draw(i, a.batch_size) for i in range(a.num_features)]),
                                 lengths=torch.ones(a.num_features * a.batch_size, dtype=torch.int64)) for _ in range(a.num_batches))
    res = count_distributions(batches)
    print(json.dumps(res, indent=1))
    return res


if __name__ == "__main__":
    main()
