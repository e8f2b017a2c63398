"""Remap the sparse ids of the per-day ``*_sparse.npy`` files to contiguous integers, rare ids (below ``--frequency_threshold``)
to one shared id (``torchrec/datasets/scripts/contiguous_preproc_criteo.py``).

    python -m torchrec_b200.datasets.scripts.contiguous_preproc_criteo --input_dir /data/criteo_npy --output_dir /data/criteo_contig
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List

from torchrec_b200.datasets.criteo import BinaryCriteoUtils


def parse_args(argv: List[str]) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Criteo sparse ids -> contiguous ids")
    p.add_argument("--input_dir", type=str, required=True)
    p.add_argument("--output_dir", type=str, required=True)
    p.add_argument("--frequency_threshold", type=int, default=0)
    p.add_argument("--days", type=int, default=24)
    return p.parse_args(argv)


def main(argv: List[str]) -> None:
    a = parse_args(argv)
    files = [os.path.join(a.input_dir, f"day_{i}_sparse.npy") for i in range(a.days)]
    files = [f for f in files if os.path.exists(f)]
    os.makedirs(a.output_dir, exist_ok=True)
    BinaryCriteoUtils.sparse_to_contiguous(files, a.output_dir, frequency_threshold=a.frequency_threshold)


if __name__ == "__main__":  # pragma: no cover
    main(sys.argv[1:])
