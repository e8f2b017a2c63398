"""Build the DLRM predict module (quantized embeddings), serve it over gRPC on a local port and query it once
(cf. ``examples/prediction/predict_using_torchrec.py`` of the reference)."""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from torchrec_b200.inference.client import PredictorClient, create_request  # noqa: E402
from torchrec_b200.inference.dlrm_predict import DLRMPredictFactory, default_dlrm_config  # noqa: E402
from torchrec_b200.inference.server import PredictorServicer, serve  # noqa: E402
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor  # noqa: E402


def main() -> None:
    cfg = default_dlrm_config(num_embeddings=1000)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    factory = DLRMPredictFactory(cfg, quantize=True, device=device)
    module = factory.create_predict_module()
    server = serve(PredictorServicer(module, torch.device(device), id_list_feature_names=cfg.id_list_features_keys), "127.0.0.1:0")
    B = 4
    lengths = torch.randint(1, 4, (len(cfg.id_list_features_keys) * B,))
    kjt = KeyedJaggedTensor(keys=cfg.id_list_features_keys, values=torch.randint(0, 1000, (int(lengths.sum()),)), lengths=lengths)
    client = PredictorClient(f"127.0.0.1:{server.bound_port}")
    print("scores:", client.predict(create_request(torch.rand(B, cfg.dense_in_features), kjt))["default"].tolist())
    client.close()
    server.stop(0)


if __name__ == "__main__":
    main()
