"""Command line that packages the DLRM predict factory (``torchrec/inference/dlrm_packager.py``).

    python -m torchrec_b200.inference.dlrm_packager --output_path /tmp/dlrm.pt --num_embeddings 100000
"""
from __future__ import annotations

import argparse
import sys
from typing import List

from torch.package import PackageExporter

from torchrec_b200.inference.dlrm_predict import DLRMPredictFactory
from torchrec_b200.inference.model_packager import PredictFactoryPackager


class DLRMPredictFactoryPackager(PredictFactoryPackager):
    @classmethod
    def set_extern_modules(cls, pe: PackageExporter) -> None:
        pe.extern(["torch", "torch.**", "numpy", "numpy.**", "torchrec_b200", "torchrec_b200.**", "io", "typing", "dataclasses"])

    @classmethod
    def set_mocked_modules(cls, pe: PackageExporter) -> None:
        pass


def parse_args(argv: List[str]) -> argparse.Namespace:
    p = argparse.ArgumentParser(description="DLRM model packager")
    p.add_argument("--output_path", type=str, required=True)
    return p.parse_args(argv)


def main(argv: List[str]) -> None:
    args = parse_args(argv)
    DLRMPredictFactoryPackager.save_predict_factory(DLRMPredictFactory, configs={}, output=args.output_path, extra_files={})
    print(f"Package is saved to {args.output_path}")


if __name__ == "__main__":  # pragma: no cover
    main(sys.argv[1:])
