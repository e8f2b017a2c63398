"""EmbeddingBagCollection (one ``nn.EmbeddingBag`` per table + a separate SGD) against FusedEmbeddingBagCollection (one table-batched
kernel with SGD fused into the backward) on the DLRM table set, the largest tables shrunk to fit one device.

    python benchmarks/ebc_benchmarks.py --mode ebc_comparison_dlrm
    python benchmarks/ebc_benchmarks.py --mode ebc_comparison_scaling --cpu_only

Counterpart of ``benchmarks/ebc_benchmarks.py`` of the reference; its ``fused_ebc_uvm`` mode is answered here by running the full-size
tables resident in HBM (``--mode fused_ebc_full``): 180 GB per device holds the whole DLRM table set."""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Tuple

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks.ebc_benchmarks_utils import get_random_dataset, train  # noqa: E402
from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig  # noqa: E402
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection  # noqa: E402
from torchrec_b200.modules.fused_embedding_modules import FusedEmbeddingBagCollection  # noqa: E402

DLRM_NUM_EMBEDDINGS_PER_FEATURE = [45833188, 36746, 17245, 7413, 20243, 3, 7114, 1441, 62, 29275261, 1572176, 345138, 10, 2209, 11267, 128, 4, 974, 14,
                                   48937457, 11316796, 40094537, 452104, 12606, 104, 35]


def get_shrunk_dlrm_num_embeddings(reduction_degree: int) -> List[int]:
    """Tables of 10M rows or more are divided by ``reduction_degree``."""
    return [n if n < 10_000_000 else n // reduction_degree for n in DLRM_NUM_EMBEDDINGS_PER_FEATURE]


def _tables(rows: List[int], dim: int = 128) -> List[EmbeddingBagConfig]:
    return [EmbeddingBagConfig(name=f"ebc_{i}", embedding_dim=dim, num_embeddings=n, feature_names=[f"ebc_{i}_feat_1"]) for i, n in enumerate(rows)]


def get_ebc_comparison(tables: List[EmbeddingBagConfig], device: torch.device, epochs: int = 100, batch_size: int = 64, num_batches: int = 10,
                       lr: float = 0.02) -> Tuple[float, float, float, float, float]:
    """``(ebc mean s, ebc std, fused mean s, fused std, speed-up)`` per epoch of ``num_batches`` batches."""
    data = get_random_dataset(batch_size, num_batches, 1024, tables)
    ebc = EmbeddingBagCollection(tables=tables, device=device)
    ebc_mean, ebc_std = train(ebc, torch.optim.SGD(ebc.parameters(), lr=lr), data, device, epochs)
    del ebc
    fused = FusedEmbeddingBagCollection(tables=tables, optimizer_type=torch.optim.SGD, optimizer_kwargs={"lr": lr}, device=device)
    fused_mean, fused_std = train(fused, None, data, device, epochs)
    return ebc_mean, ebc_std, fused_mean, fused_std, ebc_mean / max(fused_mean, 1e-12)


def main(argv: List[str]) -> None:
    p = argparse.ArgumentParser(description="EBC vs FusedEBC training-time benchmark")
    p.add_argument("--mode", default="ebc_comparison_dlrm", choices=["ebc_comparison_dlrm", "fused_ebc_full", "ebc_comparison_scaling"])
    p.add_argument("--cpu_only", action="store_true")
    p.add_argument("--epochs", type=int, default=100)
    p.add_argument("--reductions", default="128,64,32")
    p.add_argument("--max_tables", type=int, default=0, help="use only the first N tables (smoke runs)")
    args = p.parse_args(argv)
    device = torch.device("cuda" if torch.cuda.is_available() and not args.cpu_only else "cpu")
    cut = args.max_tables or None
    if args.mode == "ebc_comparison_dlrm":
        for k in [int(x) for x in args.reductions.split(",")]:
            e, es, f, fs, sp = get_ebc_comparison(_tables(get_shrunk_dlrm_num_embeddings(k)[:cut]), device, epochs=args.epochs)
            print(f"DLRM tables reduced {k}x: ebc_time = {e:.4f} +/- {es:.4f} s, fused_ebc_time = {f:.4f} +/- {fs:.4f} s, speedup = {sp:.1f}")
    elif args.mode == "fused_ebc_full":
        tables = _tables(DLRM_NUM_EMBEDDINGS_PER_FEATURE[:cut])
        fused = FusedEmbeddingBagCollection(tables=tables, optimizer_type=torch.optim.SGD, optimizer_kwargs={"lr": 0.02}, device=device)
        mean, std = train(fused, None, get_random_dataset(64, 10, 1024, tables), device, args.epochs)
        print(f"FusedEBC, full-size DLRM tables in device memory: {mean:.4f} +/- {std:.4f} s")
    else:
        for num_tables in (10, 100):
            for rows in (128, 1024, 8192):
                for dim in (16, 64, 128):
                    e, _, f, _, sp = get_ebc_comparison(_tables([rows] * num_tables, dim), device, epochs=min(args.epochs, 3))
                    print(f"tables = {num_tables}, rows = {rows}, dim = {dim}: ebc_time = {e:.4f} s, fused_ebc_time = {f:.4f} s, speedup = {sp:.1f}")


if __name__ == "__main__":
    main(sys.argv[1:])
