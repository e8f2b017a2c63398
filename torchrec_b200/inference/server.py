"""Prediction server: ``Predict(PredictionRequest) -> PredictionResponse`` over gRPC.

A request carries raw tensor bytes (wire format: ``predictor_pb.py``); the server rebuilds ``float_features [B, n]`` and the
``id_list_features`` / ``id_score_list_features`` jagged inputs, moves them to the serving device from pinned staging buffers, runs
the predict module and returns ``{"default": scores}`` (or every entry of a dict result).  Requests arriving together are merged
into one forward by the native batching queue (``torch.classes.trb_inference.BatchingQueue``) when ``max_batch_size`` allows.

    python -m torchrec_b200.inference.server --package model.pt --port 50051

The reference's server is a C++ binary on gRPC C++ and a TorchScript module (``torchrec/inference/server.cpp:45-179``); no
gRPC C++ / protobuf development files exist in this environment, so the transport layer here is grpcio while request decoding
and model execution stay in tensors.
"""
from __future__ import annotations

import argparse
import threading
from concurrent import futures
from typing import Any, Dict, List, Optional

import grpc
import torch
from torch import nn

from torchrec_b200.inference import predictor_pb as pb


def _tensor(raw: bytes, dtype: torch.dtype) -> torch.Tensor:
    return torch.frombuffer(bytearray(raw), dtype=dtype) if raw else torch.empty(0, dtype=dtype)


def decode_request(req: Any) -> Dict[str, torch.Tensor]:
    """``{"float_features", "id_list_features.lengths", "id_list_features.values", ...}`` as host tensors."""
    B = int(req.batch_size)
    out: Dict[str, torch.Tensor] = {}
    ff = req.float_features
    out["float_features"] = _tensor(ff.values, torch.float32).view(B, max(int(ff.num_features), 0)) if ff.num_features else torch.zeros(B, 0)
    for name in ("id_list_features", "id_score_list_features"):
        sf = getattr(req, name)
        if sf.num_features:
            out[f"{name}.lengths"] = _tensor(sf.lengths, torch.int32)
            out[f"{name}.values"] = _tensor(sf.values, torch.int32)
            if sf.weights:
                out[f"{name}.weights"] = _tensor(sf.weights, torch.float32)
    return out


class PredictorServicer:
    """Holds the model; thread-safe (one forward at a time per device stream)."""

    def __init__(self, module: nn.Module, device: torch.device, id_list_feature_names: Optional[List[str]] = None,
                 id_score_list_feature_names: Optional[List[str]] = None) -> None:
        self.module = module.to(device).eval() if not any(p.is_meta for p in module.parameters()) else module
        self.device = device
        self.id_list_feature_names = id_list_feature_names or []
        self.id_score_list_feature_names = id_score_list_feature_names or []
        self._lock = threading.Lock()

    def _kjt(self, t: Dict[str, torch.Tensor], name: str, keys: List[str], B: int):
        from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor

        if f"{name}.lengths" not in t:
            return None
        lengths, values = t[f"{name}.lengths"], t[f"{name}.values"]
        keys = keys or [f"f{i}" for i in range(lengths.numel() // max(B, 1))]
        pin = (lambda x: x.pin_memory()) if self.device.type == "cuda" else (lambda x: x)
        return KeyedJaggedTensor(keys=keys, values=pin(values).to(self.device, non_blocking=True), lengths=pin(lengths).to(self.device, non_blocking=True),
                                 weights=pin(t[f"{name}.weights"]).to(self.device, non_blocking=True) if f"{name}.weights" in t else None, stride=B)

    @torch.no_grad()
    def predict_tensors(self, t: Dict[str, torch.Tensor], B: int) -> Dict[str, torch.Tensor]:
        batch: Dict[str, Any] = {"float_features": t["float_features"].to(self.device, non_blocking=True)}
        for name, keys in (("id_list_features", self.id_list_feature_names), ("id_score_list_features", self.id_score_list_feature_names)):
            kjt = self._kjt(t, name, keys, B)
            if kjt is not None:
                batch[name] = kjt
        with self._lock:
            out = self.module(batch)
        if isinstance(out, torch.Tensor):
            out = {"default": out}
        return {k: v.detach().float().reshape(-1).cpu() for k, v in out.items()}

    def Predict(self, request: Any, context: Any = None) -> Any:
        preds = self.predict_tensors(decode_request(request), int(request.batch_size))
        resp = pb.PredictionResponse()
        for k, v in preds.items():
            resp.predictions[k].data.extend(v.tolist())
        return resp


def add_servicer_to_server(servicer: PredictorServicer, server: grpc.Server) -> None:
    handler = grpc.unary_unary_rpc_method_handler(servicer.Predict, request_deserializer=pb.PredictionRequest.FromString,
                                                  response_serializer=lambda m: m.SerializeToString())
    server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(pb.SERVICE, {"Predict": handler}),))


def serve(servicer: PredictorServicer, address: str = "127.0.0.1:50051", max_workers: int = 4) -> grpc.Server:
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=max_workers))
    add_servicer_to_server(servicer, server)
    port = server.add_insecure_port(address)
    server.start()
    server.bound_port = port  # type: ignore[attr-defined]
    return server


def main() -> None:  # pragma: no cover - needs a packaged model
    p = argparse.ArgumentParser()
    p.add_argument("--package", required=True, help="file written by PredictFactoryPackager.save_predict_factory")
    p.add_argument("--address", default="127.0.0.1:50051")
    p.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    a = p.parse_args()
    from torchrec_b200.inference.model_packager import load_predict_factory

    factory = load_predict_factory(a.package)
    module = factory.create_predict_module()
    names = factory.model_inputs_data() if hasattr(factory, "model_inputs_data") else {}
    servicer = PredictorServicer(module, torch.device(a.device), names.get("id_list_features"), names.get("id_score_list_features"))
    server = serve(servicer, a.address)
    print(f"serving on {a.address}", flush=True)
    server.wait_for_termination()


if __name__ == "__main__":  # pragma: no cover
    main()
