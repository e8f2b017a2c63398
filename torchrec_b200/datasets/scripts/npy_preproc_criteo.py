"""Convert the Criteo TSV files (``day_0`` ... ``day_23`` or ``train.txt``) into ``*_dense.npy`` / ``*_sparse.npy`` / ``*_labels.npy``
(``torchrec/datasets/scripts/npy_preproc_criteo.py``).

    python -m torchrec_b200.datasets.scripts.npy_preproc_criteo --input_dir /data/criteo_tsv --output_dir /data/criteo_npy
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List

from torchrec_b200.datasets.criteo import BinaryCriteoUtils


def parse_args(argv: List[str]) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="Criteo tsv -> npy")
    p.add_argument("--input_dir", type=str, required=True)
    p.add_argument("--output_dir", type=str, required=True)
    p.add_argument("--dataset_name", type=str, choices=["criteo_1tb", "criteo_kaggle"], default="criteo_1tb")
    return p.parse_args(argv)


def main(argv: List[str]) -> None:
    a = parse_args(argv)
    os.makedirs(a.output_dir, exist_ok=True)
    names = [f"day_{i}" for i in range(24)] if a.dataset_name == "criteo_1tb" else ["train.txt"]
    for name in names:
        src = os.path.join(a.input_dir, name)
        if not os.path.exists(src):
            continue
        out = os.path.join(a.output_dir, name)
        print(f"Processing {src}", flush=True)
        BinaryCriteoUtils.tsv_to_npys(src, out + "_dense.npy", out + "_sparse.npy", out + "_labels.npy", a.dataset_name)


if __name__ == "__main__":  # pragma: no cover
    main(sys.argv[1:])
