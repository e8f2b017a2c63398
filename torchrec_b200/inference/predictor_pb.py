"""Messages of the prediction service, built at import time from a descriptor written in code (no protobuf compiler at build or
run time).  Package ``predictor``; service ``Predictor`` with one unary method ``Predict(PredictionRequest) -> PredictionResponse``.

Wire format (field numbers in brackets; the same numbers as the reference's ``torchrec/inference/protos/predictor.proto``, so
clients of either server interoperate).  Tensors travel as raw little-endian bytes.

* ``PredictionRequest``: batch_size [1] int32; float_features [2] ``FloatFeatures``; id_list_features [3], id_score_list_features [4]
  and unary_features [6] ``SparseFeatures``; embedding_features [5] ``FloatFeatures``.
* ``FloatFeatures``: num_features [1] int32; values [2] bytes = fp32 ``[batch, num_features]``.
* ``SparseFeatures``: num_features [1] int32; lengths [2] bytes = int32 ``[num_features, batch]``; values [3] bytes = int32 ids,
  jagged, feature-major; weights [4] bytes = fp32, one per id (score lists only).
* ``PredictionResponse``: predictions [1] map from task name to ``FloatVec`` (data [1] repeated float).
"""
from __future__ import annotations

from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

_T = descriptor_pb2.FieldDescriptorProto


def _field(msg, name: str, number: int, ftype: int, label: int = _T.LABEL_OPTIONAL, type_name: str = "") -> None:
    f = msg.field.add()
    f.name, f.number, f.type, f.label = name, number, ftype, label
    if type_name:
        f.type_name = type_name


def _build():
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = "torchrec_b200/inference/protos/predictor.proto"
    fd.package = "predictor"
    fd.syntax = "proto3"
    m = fd.message_type.add()
    m.name = "SparseFeatures"
    _field(m, "num_features", 1, _T.TYPE_INT32)
    _field(m, "lengths", 2, _T.TYPE_BYTES)
    _field(m, "values", 3, _T.TYPE_BYTES)
    _field(m, "weights", 4, _T.TYPE_BYTES)
    m = fd.message_type.add()
    m.name = "FloatFeatures"
    _field(m, "num_features", 1, _T.TYPE_INT32)
    _field(m, "values", 2, _T.TYPE_BYTES)
    m = fd.message_type.add()
    m.name = "PredictionRequest"
    _field(m, "batch_size", 1, _T.TYPE_INT32)
    _field(m, "float_features", 2, _T.TYPE_MESSAGE, type_name=".predictor.FloatFeatures")
    _field(m, "id_list_features", 3, _T.TYPE_MESSAGE, type_name=".predictor.SparseFeatures")
    _field(m, "id_score_list_features", 4, _T.TYPE_MESSAGE, type_name=".predictor.SparseFeatures")
    _field(m, "embedding_features", 5, _T.TYPE_MESSAGE, type_name=".predictor.FloatFeatures")
    _field(m, "unary_features", 6, _T.TYPE_MESSAGE, type_name=".predictor.SparseFeatures")
    m = fd.message_type.add()
    m.name = "FloatVec"
    _field(m, "data", 1, _T.TYPE_FLOAT, label=_T.LABEL_REPEATED)
    m = fd.message_type.add()
    m.name = "PredictionResponse"
    entry = m.nested_type.add()
    entry.name = "PredictionsEntry"
    entry.options.map_entry = True
    _field(entry, "key", 1, _T.TYPE_STRING)
    _field(entry, "value", 2, _T.TYPE_MESSAGE, type_name=".predictor.FloatVec")
    _field(m, "predictions", 1, _T.TYPE_MESSAGE, label=_T.LABEL_REPEATED, type_name=".predictor.PredictionResponse.PredictionsEntry")
    svc = fd.service.add()
    svc.name = "Predictor"
    rpc = svc.method.add()
    rpc.name, rpc.input_type, rpc.output_type = "Predict", ".predictor.PredictionRequest", ".predictor.PredictionResponse"
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = lambda n: message_factory.GetMessageClass(pool.FindMessageTypeByName(f"predictor.{n}"))
    return {n: get(n) for n in ("SparseFeatures", "FloatFeatures", "PredictionRequest", "FloatVec", "PredictionResponse")}


_CLASSES = _build()
SparseFeatures = _CLASSES["SparseFeatures"]
FloatFeatures = _CLASSES["FloatFeatures"]
PredictionRequest = _CLASSES["PredictionRequest"]
FloatVec = _CLASSES["FloatVec"]
PredictionResponse = _CLASSES["PredictionResponse"]
SERVICE = "predictor.Predictor"
PREDICT_METHOD = f"/{SERVICE}/Predict"
