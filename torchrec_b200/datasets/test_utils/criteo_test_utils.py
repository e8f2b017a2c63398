"""Synthetic Criteo files for dataset tests: context managers that write a small TSV (label, 13 integer columns, 26 hex-string
categorical columns) or the three ``.npy`` arrays (dense, sparse, labels) into a temporary folder, and a sample validator.
Counterpart of ``torchrec/datasets/test_utils/criteo_test_utils.py:23-140``."""
from __future__ import annotations

import contextlib
import csv
import os
import random
import tempfile
import unittest
from typing import Any, Dict, Generator, Optional, Tuple

import numpy as np

INT_FEATURE_COUNT = 13
CAT_FEATURE_COUNT = 26
LABEL_VAL_RANGE = (0, 1)
INT_VAL_RANGE = (0, 100)
CAT_VAL_RANGE = (0, 1000)


def _hex8(rng: random.Random) -> str:
    return f"{rng.getrandbits(32):08x}"


@contextlib.contextmanager
def create_dataset_tsv(num_rows: int = 10, train: bool = True, filename: str = "criteo", seed: Optional[int] = None) -> Generator[str, None, None]:
    rng = random.Random(seed)
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, filename)
        with open(path, "w", newline="") as f:
            w = csv.writer(f, delimiter="\t")
            for _ in range(num_rows):
                row = [str(rng.randint(*LABEL_VAL_RANGE))] if train else []
                row += [str(rng.randint(*INT_VAL_RANGE)) for _ in range(INT_FEATURE_COUNT)]
                row += [_hex8(rng) for _ in range(CAT_FEATURE_COUNT)]
                w.writerow(row)
        yield path


@contextlib.contextmanager
def create_dataset_npys(num_rows: int = 10, filename: Optional[str] = None, generate_dense: bool = True, generate_sparse: bool = True,
                        generate_labels: bool = True, dense: Optional[np.ndarray] = None, sparse: Optional[np.ndarray] = None,
                        labels: Optional[np.ndarray] = None, seed: Optional[int] = None) -> Generator[Tuple[str, ...], None, None]:
    """Yields the paths of the generated ``<name>_dense.npy`` / ``_sparse.npy`` / ``_labels.npy`` files, in that order."""
    rng = np.random.default_rng(seed)
    with tempfile.TemporaryDirectory() as tmp:
        base = os.path.join(tmp, filename or "criteo")
        paths = []
        if generate_dense:
            arr = dense if dense is not None else rng.random((num_rows, INT_FEATURE_COUNT), dtype=np.float32)
            np.save(base + "_dense.npy", arr.astype(np.float32))
            paths.append(base + "_dense.npy")
        if generate_sparse:
            arr = sparse if sparse is not None else rng.integers(CAT_VAL_RANGE[0], CAT_VAL_RANGE[1] + 1, (num_rows, CAT_FEATURE_COUNT), dtype=np.int32)
            np.save(base + "_sparse.npy", arr.astype(np.int32))
            paths.append(base + "_sparse.npy")
        if generate_labels:
            arr = labels if labels is not None else rng.integers(LABEL_VAL_RANGE[0], LABEL_VAL_RANGE[1] + 1, (num_rows, 1), dtype=np.int32)
            np.save(base + "_labels.npy", arr.astype(np.int32))
            paths.append(base + "_labels.npy")
        yield tuple(paths)


def validate_sample(sample: Dict[str, Any], train: bool = True) -> None:
    """A parsed TSV row: ``label`` (train only), ``int_0..12`` within the integer range, ``cat_0..25`` 8-character hex strings."""
    assert len(sample) == INT_FEATURE_COUNT + CAT_FEATURE_COUNT + (1 if train else 0), len(sample)
    if train:
        assert LABEL_VAL_RANGE[0] <= sample["label"] <= LABEL_VAL_RANGE[1]
    for i in range(INT_FEATURE_COUNT):
        assert INT_VAL_RANGE[0] <= sample[f"int_{i}"] <= INT_VAL_RANGE[1]
    for i in range(CAT_FEATURE_COUNT):
        v = sample[f"cat_{i}"]
        assert isinstance(v, str) and len(v) == 8 and int(v, 16) >= 0


class CriteoTest(unittest.TestCase):
    """``unittest`` face of the helpers above for test classes that subclass it."""

    INT_FEATURE_COUNT, CAT_FEATURE_COUNT = INT_FEATURE_COUNT, CAT_FEATURE_COUNT
    LABEL_VAL_RANGE, INT_VAL_RANGE, CAT_VAL_RANGE = LABEL_VAL_RANGE, INT_VAL_RANGE, CAT_VAL_RANGE
    _create_dataset_tsv = staticmethod(create_dataset_tsv)
    _create_dataset_npys = staticmethod(create_dataset_npys)

    def _validate_sample(self, sample: Dict[str, Any], train: bool = True) -> None:
        validate_sample(sample, train)
