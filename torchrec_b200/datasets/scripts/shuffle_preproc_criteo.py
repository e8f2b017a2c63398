"""Shuffle the rows of the first ``--days`` days jointly (labels, dense and sparse stay aligned) and write one file per kind
(``torchrec/datasets/scripts/shuffle_preproc_criteo.py``).

    python -m torchrec_b200.datasets.scripts.shuffle_preproc_criteo --input_dir_labels_and_dense /data/npy --input_dir_sparse /data/contig --output_dir_shuffled /data/shuf
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List

from torchrec_b200.datasets.criteo import BinaryCriteoUtils


def parse_args(argv: List[str]) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="shuffle preprocessed Criteo days")
    p.add_argument("--input_dir_labels_and_dense", type=str, required=True)
    p.add_argument("--input_dir_sparse", type=str, required=True)
    p.add_argument("--output_dir_shuffled", type=str, required=True)
    p.add_argument("--random_seed", type=int, default=0)
    p.add_argument("--days", type=int, default=23)
    return p.parse_args(argv)


def main(argv: List[str]) -> None:
    a = parse_args(argv)
    rows_per_day = {}
    for d in range(a.days):
        f = os.path.join(a.input_dir_labels_and_dense, f"day_{d}_labels.npy")
        if os.path.exists(f):
            rows_per_day[d] = BinaryCriteoUtils.get_shape_from_npy(f)[0]
    os.makedirs(a.output_dir_shuffled, exist_ok=True)
    BinaryCriteoUtils.shuffle(a.input_dir_labels_and_dense, a.input_dir_sparse, a.output_dir_shuffled, rows_per_day, seed=a.random_seed, days=len(rows_per_day))


if __name__ == "__main__":  # pragma: no cover
    main(sys.argv[1:])
