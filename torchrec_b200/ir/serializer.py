"""JSON serializers of the embedding modules (``torchrec/ir/serializer.py:160-460``): ``EmbeddingBagCollection``,
``FeatureProcessedEmbeddingBagCollection``, ``PositionWeightedModule(Collection)`` and ``KTRegroupAsDict``."""
from __future__ import annotations

import json
import types
from typing import Any, Dict, List, Optional, Type

import torch
from torch import nn

from torchrec_b200.ir.schema import (
    EBCMetadata,
    EmbeddingBagConfigMetadata,
    FPEBCMetadata,
    KTRegroupAsDictMetadata,
    PositionWeightedModuleCollectionMetadata,
    PositionWeightedModuleMetadata,
)
from torchrec_b200.ir.types import SerializerInterface
from torchrec_b200.ir.utils import qualname
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingBagConfig, PoolingType
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.feature_processor_ import FeatureProcessor, FeatureProcessorsCollection, PositionWeightedModule, PositionWeightedModuleCollection
from torchrec_b200.modules.fp_embedding_modules import FeatureProcessedEmbeddingBagCollection
from torchrec_b200.modules.regroup import KTRegroupAsDict
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


def embedding_bag_config_to_metadata(c: EmbeddingBagConfig) -> EmbeddingBagConfigMetadata:
    return EmbeddingBagConfigMetadata(num_embeddings=c.num_embeddings, embedding_dim=c.embedding_dim, name=c.name, data_type=c.data_type.value,
                                      feature_names=list(c.feature_names), weight_init_max=c.weight_init_max, weight_init_min=c.weight_init_min,
                                      need_pos=c.need_pos, pooling=c.pooling.value)


def embedding_metadata_to_config(t: EmbeddingBagConfigMetadata) -> EmbeddingBagConfig:
    return EmbeddingBagConfig(num_embeddings=t.num_embeddings, embedding_dim=t.embedding_dim, name=t.name, data_type=DataType(t.data_type), feature_names=t.feature_names,
                              weight_init_max=t.weight_init_max, weight_init_min=t.weight_init_min, need_pos=t.need_pos, pooling=PoolingType(t.pooling))


def get_deserialized_device(config_device: Optional[str], device: Optional[torch.device]) -> Optional[torch.device]:
    if config_device is None or device is None:
        return device if device is not None else (torch.device(config_device) if config_device else None)
    original = torch.device(config_device)
    return original if original.type == device.type else device


def _kjt_tensors(features: KeyedJaggedTensor) -> List[Optional[torch.Tensor]]:
    return [features._values, features._weights, features._lengths, features._offsets]


def ebc_meta_forward(ebc: EmbeddingBagCollection, features: KeyedJaggedTensor) -> KeyedTensor:
    dims = [c.embedding_dim for c in ebc._embedding_bag_configs for _ in c.feature_names]
    if features.variable_stride_per_key():
        outs = torch.ops.trb200_ir.dynamic_batch_emb_lookup(_kjt_tensors(features), features.stride(), dims)
    else:
        outs = torch.ops.trb200_ir.emb_lookup(_kjt_tensors(features), features.stride(), dims)
    return KeyedTensor(keys=ebc._embedding_names, values=torch.cat(outs, dim=1), length_per_key=dims)


def fpebc_meta_forward(fpebc: FeatureProcessedEmbeddingBagCollection, features: KeyedJaggedTensor) -> KeyedTensor:
    ebc = fpebc._embedding_bag_collection
    dims = [c.embedding_dim for c in ebc._embedding_bag_configs for _ in c.feature_names]
    fp = fpebc._feature_processors
    weights = list(fp.position_weights.values()) if hasattr(fp, "position_weights") else [p for p in fp.parameters()]
    outs = torch.ops.trb200_ir.emb_lookup(_kjt_tensors(features) + weights, features.stride(), dims)
    return KeyedTensor(keys=ebc._embedding_names, values=torch.cat(outs, dim=1), length_per_key=dims)


def kt_regroup_meta_forward(op: KTRegroupAsDict, keyed_tensors: List[KeyedTensor]) -> Dict[str, torch.Tensor]:
    lengths = {k: l for kt in keyed_tensors for k, l in zip(kt.keys(), kt.length_per_key())}
    dims = [sum(lengths[k] for k in g) for g in op._groups]
    arg = [kt.values() for kt in keyed_tensors]
    dtype = op._emb_dtype if op._emb_dtype is not None else arg[0].dtype
    outs = torch.ops.trb200_ir.kt_regroup(arg, keyed_tensors[0].values().size(0), dims, dtype)
    return dict(zip(op._keys, outs))


class JsonSerializer(SerializerInterface):
    _module_cls: Optional[Type[nn.Module]] = None
    _children: Optional[List[str]] = None

    @classmethod
    def children(cls, module: nn.Module) -> List[str]:
        return [] if cls._children is None else cls._children

    @classmethod
    def serialize_to_dict(cls, module: nn.Module) -> Dict[str, Any]:
        raise NotImplementedError

    @classmethod
    def deserialize_from_dict(cls, metadata_dict: Dict[str, Any], device: Optional[torch.device] = None, unflatten_ep: Optional[nn.Module] = None) -> nn.Module:
        raise NotImplementedError

    @classmethod
    def swap_meta_forward(cls, module: nn.Module) -> None:
        pass

    @classmethod
    def encapsulate_module(cls, module: nn.Module) -> List[str]:
        typename = qualname(module)
        ser = cls.module_to_serializer_cls.get(typename)
        if ser is None:
            raise ValueError(f"no serializer for {typename}")
        assert issubclass(ser, JsonSerializer)
        assert ser._module_cls is not None and isinstance(module, ser._module_cls)
        payload = {"__typename": typename, **ser.serialize_to_dict(module)}
        raw = json.dumps(payload).encode("utf-8")
        module.register_buffer("ir_metadata", torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone(), persistent=False)
        ser.swap_meta_forward(module)
        return ser.children(module)

    @classmethod
    def decapsulate_module(cls, module: nn.Module, device: Optional[torch.device] = None) -> nn.Module:
        raw = module.get_buffer("ir_metadata")
        payload = json.loads(bytes(raw.cpu().numpy().tobytes()).decode("utf-8"))
        typename = payload.pop("__typename")
        ser = cls.module_to_serializer_cls.get(typename)
        if ser is None:
            raise ValueError(f"no deserializer for {typename}")
        assert issubclass(ser, JsonSerializer)
        return ser.deserialize_from_dict(payload, device, module)

    module_to_serializer_cls: Dict[str, Type["JsonSerializer"]] = {}


def _asdict(obj: Any) -> Any:
    import dataclasses

    return dataclasses.asdict(obj)


class EBCJsonSerializer(JsonSerializer):
    _module_cls = EmbeddingBagCollection

    @classmethod
    def swap_meta_forward(cls, module: nn.Module) -> None:
        module.forward = types.MethodType(ebc_meta_forward, module)

    @classmethod
    def serialize_to_dict(cls, module: nn.Module) -> Dict[str, Any]:
        assert isinstance(module, EmbeddingBagCollection)
        dev = getattr(module, "device", None)
        return _asdict(EBCMetadata(tables=[embedding_bag_config_to_metadata(c) for c in module.embedding_bag_configs()], is_weighted=module.is_weighted(),
                                   device=str(dev) if dev is not None else None))

    @classmethod
    def deserialize_from_dict(cls, metadata_dict: Dict[str, Any], device: Optional[torch.device] = None, unflatten_ep: Optional[nn.Module] = None) -> nn.Module:
        tables = [embedding_metadata_to_config(EmbeddingBagConfigMetadata(**t)) for t in metadata_dict["tables"]]
        return EmbeddingBagCollection(tables=tables, is_weighted=metadata_dict["is_weighted"], device=get_deserialized_device(metadata_dict.get("device"), device))


class PWMJsonSerializer(JsonSerializer):
    _module_cls = PositionWeightedModule

    @classmethod
    def serialize_to_dict(cls, module: nn.Module) -> Dict[str, Any]:
        return _asdict(PositionWeightedModuleMetadata(max_feature_length=module.position_weight.shape[0]))

    @classmethod
    def deserialize_from_dict(cls, metadata_dict: Dict[str, Any], device: Optional[torch.device] = None, unflatten_ep: Optional[nn.Module] = None) -> nn.Module:
        return PositionWeightedModule(max_feature_length=metadata_dict["max_feature_length"], device=device)


class PWMCJsonSerializer(JsonSerializer):
    _module_cls = PositionWeightedModuleCollection

    @classmethod
    def serialize_to_dict(cls, module: nn.Module) -> Dict[str, Any]:
        return _asdict(PositionWeightedModuleCollectionMetadata(max_feature_lengths=[(k, v) for k, v in module.max_feature_lengths.items()]))

    @classmethod
    def deserialize_from_dict(cls, metadata_dict: Dict[str, Any], device: Optional[torch.device] = None, unflatten_ep: Optional[nn.Module] = None) -> nn.Module:
        return PositionWeightedModuleCollection({k: v for k, v in metadata_dict["max_feature_lengths"]}, device=device)


class FPEBCJsonSerializer(JsonSerializer):
    _module_cls = FeatureProcessedEmbeddingBagCollection
    _children = ["_feature_processors", "_embedding_bag_collection"]

    @classmethod
    def swap_meta_forward(cls, module: nn.Module) -> None:
        module.forward = types.MethodType(fpebc_meta_forward, module)

    @classmethod
    def serialize_to_dict(cls, module: nn.Module) -> Dict[str, Any]:
        if isinstance(module._feature_processors, FeatureProcessorsCollection):
            meta = FPEBCMetadata(is_fp_collection=True, features=[])
        else:
            meta = FPEBCMetadata(is_fp_collection=False, features=list(module._feature_processors.keys()))
        return _asdict(meta)

    @classmethod
    def children(cls, module: nn.Module) -> List[str]:
        if isinstance(module._feature_processors, FeatureProcessorsCollection):
            return ["_feature_processors", "_embedding_bag_collection"]
        return [f"_feature_processors.{k}" for k in module._feature_processors.keys()] + ["_embedding_bag_collection"]

    @classmethod
    def deserialize_from_dict(cls, metadata_dict: Dict[str, Any], device: Optional[torch.device] = None, unflatten_ep: Optional[nn.Module] = None) -> nn.Module:
        assert unflatten_ep is not None
        if metadata_dict["is_fp_collection"]:
            fps = unflatten_ep._feature_processors
            assert isinstance(fps, FeatureProcessorsCollection)
        else:
            fps = {}
            for f in metadata_dict["features"]:
                fp = getattr(unflatten_ep._feature_processors, f)
                assert isinstance(fp, FeatureProcessor)
                fps[f] = fp
        ebc = unflatten_ep._embedding_bag_collection
        assert isinstance(ebc, EmbeddingBagCollection)
        return FeatureProcessedEmbeddingBagCollection(ebc, fps)


class KTRegroupAsDictJsonSerializer(JsonSerializer):
    _module_cls = KTRegroupAsDict

    @classmethod
    def swap_meta_forward(cls, module: nn.Module) -> None:
        module.forward = types.MethodType(kt_regroup_meta_forward, module)

    @classmethod
    def serialize_to_dict(cls, module: nn.Module) -> Dict[str, Any]:
        dt = module._emb_dtype
        return _asdict(KTRegroupAsDictMetadata(groups=module._groups, keys=module._keys, emb_dtype=None if dt is None else str(dt).split(".")[-1]))

    @classmethod
    def deserialize_from_dict(cls, metadata_dict: Dict[str, Any], device: Optional[torch.device] = None, unflatten_ep: Optional[nn.Module] = None) -> nn.Module:
        dt = metadata_dict.get("emb_dtype")
        return KTRegroupAsDict(groups=metadata_dict["groups"], keys=metadata_dict["keys"], emb_dtype=None if dt is None else getattr(torch, dt))


JsonSerializer.module_to_serializer_cls = {
    qualname(EmbeddingBagCollection): EBCJsonSerializer,
    qualname(PositionWeightedModule): PWMJsonSerializer,
    qualname(PositionWeightedModuleCollection): PWMCJsonSerializer,
    qualname(FeatureProcessedEmbeddingBagCollection): FPEBCJsonSerializer,
    qualname(KTRegroupAsDict): KTRegroupAsDictJsonSerializer,
}
