"""Client of the prediction service: builds a request from tensors and calls ``Predict`` (``torchrec/inference/client.py:33``).

    python -m torchrec_b200.inference.client --address 127.0.0.1:50051 --batch_size 8 --num_float_features 13 --num_id_list_features 26
"""
from __future__ import annotations

import argparse
from typing import Any, Dict, Optional

import grpc
import torch

from torchrec_b200.inference import predictor_pb as pb
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


def create_training_batch(args: argparse.Namespace) -> Any:
    """One random Criteo-shaped batch (13 dense features, the 26 categorical ones with one id each) of ``args.batch_size`` samples
    with ids below ``args.num_embedding_features``: what the example client sends (``torchrec/inference/client.py:19-30``)."""
    from torchrec_b200.datasets.criteo import DEFAULT_CAT_NAMES, DEFAULT_INT_NAMES
    from torchrec_b200.datasets.random import RandomRecDataset

    return next(iter(RandomRecDataset(keys=DEFAULT_CAT_NAMES, batch_size=args.batch_size, hash_size=args.num_embedding_features, ids_per_feature=1,
                                      num_dense=len(DEFAULT_INT_NAMES))))


def to_bytes(t: torch.Tensor) -> bytes:
    return t.detach().cpu().contiguous().numpy().tobytes()


def create_request(float_features: torch.Tensor, id_list_features: Optional[KeyedJaggedTensor] = None, id_score_list_features: Optional[KeyedJaggedTensor] = None) -> Any:
    B = float_features.shape[0]
    req = pb.PredictionRequest()
    req.batch_size = B
    req.float_features.num_features = float_features.shape[1]
    req.float_features.values = to_bytes(float_features.float())
    for name, kjt in (("id_list_features", id_list_features), ("id_score_list_features", id_score_list_features)):
        if kjt is None:
            continue
        sf = getattr(req, name)
        sf.num_features = len(kjt.keys())
        sf.lengths = to_bytes(kjt.lengths().int())
        sf.values = to_bytes(kjt.values().int())
        if kjt.weights_or_none() is not None:
            sf.weights = to_bytes(kjt.weights().float())
    return req


class PredictorClient:
    def __init__(self, address: str) -> None:
        self._channel = grpc.insecure_channel(address)
        self._predict = self._channel.unary_unary(pb.PREDICT_METHOD, request_serializer=lambda m: m.SerializeToString(), response_deserializer=pb.PredictionResponse.FromString)

    def predict(self, request: Any, timeout: float = 30.0) -> Dict[str, torch.Tensor]:
        resp = self._predict(request, timeout=timeout)
        return {k: torch.tensor(list(v.data)) for k, v in resp.predictions.items()}

    def close(self) -> None:
        self._channel.close()


def main() -> None:  # pragma: no cover
    p = argparse.ArgumentParser()
    p.add_argument("--address", default="127.0.0.1:50051")
    p.add_argument("--batch_size", type=int, default=8)
    p.add_argument("--num_float_features", type=int, default=13)
    p.add_argument("--num_id_list_features", type=int, default=26)
    p.add_argument("--num_embeddings", type=int, default=100)
    a = p.parse_args()
    client = PredictorClient(a.address)
    if a.num_float_features == 13 and a.num_id_list_features == 26:
        a.num_embedding_features = a.num_embeddings
        batch = create_training_batch(a)
        print(client.predict(create_request(batch.dense_features, batch.sparse_features)))
        return
    lengths = torch.randint(0, 4, (a.num_id_list_features * a.batch_size,))
    kjt = KeyedJaggedTensor(keys=[f"cat_{i}" for i in range(a.num_id_list_features)], values=torch.randint(0, a.num_embeddings, (int(lengths.sum()),)), lengths=lengths)
    print(client.predict(create_request(torch.rand(a.batch_size, a.num_float_features), kjt)))


if __name__ == "__main__":  # pragma: no cover
    main()
