"""Helpers shared by the embedding modules (``torchrec/modules/utils.py``): output-dimension checks, module-list construction,
jagged-tensor assembly of unpooled lookups, deterministic de-duplication."""
from __future__ import annotations

import copy
from collections import defaultdict
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple, Union

import torch
from torch import nn

from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor
from torchrec_b200.streamable import Multistreamable


@dataclass
class SequenceVBEContext(Multistreamable):
    """What a sequence lookup needs to undo variable-batch padding: the recat, the unpadded lengths and the re-indexed lengths."""

    recat: torch.Tensor
    unpadded_lengths: torch.Tensor
    reindexed_lengths: torch.Tensor
    reindexed_length_per_key: List[int]
    reindexed_values: Optional[torch.Tensor] = None

    def record_stream(self, stream: torch.Stream) -> None:
        for t in (self.recat, self.unpadded_lengths, self.reindexed_lengths, self.reindexed_values):
            if t is not None:
                t.record_stream(stream)


def extract_module_or_tensor_callable(module_or_callable: Union[Callable[[], nn.Module], nn.Module, Callable[[torch.Tensor], torch.Tensor]]):
    """A zero-argument factory is called; modules and tensor callables pass through."""
    try:
        out = module_or_callable()  # type: ignore[call-arg]
        if isinstance(out, nn.Module):
            return out
        raise ValueError("Expected a callable that takes no input to return a torch.nn.Module, but got: {}".format(type(out)))
    except TypeError as e:
        if "required positional argument" in str(e) or "missing" in str(e):
            return module_or_callable
        raise


def get_module_output_dimension(module: Union[Callable[[torch.Tensor], torch.Tensor], nn.Module], in_features: int) -> int:
    return int(module(torch.zeros(1, in_features)).size(-1))


def check_module_output_dimension(module: Union[Iterable[nn.Module], nn.Module], in_features: int, out_features: int) -> bool:
    if isinstance(module, (list, nn.ModuleList)):
        return all(check_module_output_dimension(m, in_features, out_features) for m in module)
    return get_module_output_dimension(module, in_features) == out_features  # type: ignore[arg-type]


def init_mlp_weights_xavier_uniform(m: nn.Module) -> None:
    if isinstance(m, nn.Linear):
        nn.init.xavier_uniform_(m.weight)
        m.bias.data.fill_(0.0)


def construct_modulelist_from_single_module(module: nn.Module, sizes: Tuple[int, ...]) -> nn.Module:
    """Nested ``ModuleList`` of deep copies of ``module`` with the given shape, each copy re-initialised."""
    if len(sizes) == 1:
        return nn.ModuleList([copy.deepcopy(module).apply(init_mlp_weights_xavier_uniform) for _ in range(sizes[0])])
    return nn.ModuleList([construct_modulelist_from_single_module(module, sizes[1:]) for _ in range(sizes[0])])


def convert_list_of_modules_to_modulelist(modules: Iterable[nn.Module], sizes: Tuple[int, ...]) -> nn.Module:
    modules = list(modules)
    assert len(modules) == sizes[0], f"the counts of modules ({len(modules)}) do not match the requested size {sizes[0]}"
    if len(sizes) == 1:
        return nn.ModuleList(modules)
    assert all(isinstance(m, (list, nn.ModuleList)) for m in modules), "nested sizes need nested lists of modules"
    return nn.ModuleList([convert_list_of_modules_to_modulelist(m, sizes[1:]) for m in modules])  # type: ignore[arg-type]


def _permute_tensor_by_segments(tensor: torch.Tensor, segment_sizes: torch.Tensor, recat: torch.Tensor, weights: Optional[torch.Tensor] = None,
                                output_size: Optional[int] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Reorder the variable-length segments of a 1-D tensor."""
    _, out, out_w = sops.permute_1D_sparse_data(recat, segment_sizes, tensor, weights, output_size)
    return out, out_w


def _vbe_reindex(embeddings: torch.Tensor, seq_vbe_ctx: SequenceVBEContext) -> Tuple[torch.Tensor, torch.Tensor, List[int], Optional[torch.Tensor]]:
    """Bring the rows of a variable-batch sequence lookup from rank-major back to key-major order."""
    dim = embeddings.shape[1]
    out, _ = _permute_tensor_by_segments(embeddings.flatten(), seq_vbe_ctx.unpadded_lengths * dim, seq_vbe_ctx.recat, None, embeddings.numel())
    return out.view(-1, dim), seq_vbe_ctx.reindexed_lengths, seq_vbe_ctx.reindexed_length_per_key, seq_vbe_ctx.reindexed_values


def construct_jagged_tensors(embeddings: torch.Tensor, features: KeyedJaggedTensor, embedding_names: List[str], need_indices: bool = False,
                             features_to_permute_indices: Optional[Dict[str, List[int]]] = None, original_features: Optional[KeyedJaggedTensor] = None,
                             reverse_indices: Optional[torch.Tensor] = None, seq_vbe_ctx: Optional[SequenceVBEContext] = None) -> Dict[str, JaggedTensor]:
    """``embeddings [sum L, D]`` (key-major like ``features``) -> one ``JaggedTensor`` per embedding name; column shards of one
    name are concatenated along dim 1."""
    if original_features is not None:
        features = original_features
    if reverse_indices is not None:
        embeddings = torch.index_select(embeddings, 0, reverse_indices.to(torch.int64))
    if seq_vbe_ctx is not None:
        embeddings, lengths, length_per_key, values = _vbe_reindex(embeddings, seq_vbe_ctx)
        stride = lengths.numel() // max(len(features.keys()), 1)
    else:
        lengths, length_per_key, values, stride = features.lengths(), features.length_per_key(), features.values(), features.stride()
    lengths_tuple = torch.unbind(lengths.view(-1, stride), dim=0)
    embeddings_list = torch.split(embeddings, length_per_key, dim=0)
    values_list = torch.split(values, length_per_key) if need_indices and values is not None else None
    key_indices: Dict[str, List[int]] = defaultdict(list)
    for i, key in enumerate(embedding_names):
        key_indices[key].append(i)
    ret: Dict[str, JaggedTensor] = {}
    for key, indices in key_indices.items():
        if features_to_permute_indices and key in features_to_permute_indices:
            indices = _permute_indices(indices, features_to_permute_indices[key])
        ret[key] = JaggedTensor(lengths=lengths_tuple[indices[0]],
                                values=embeddings_list[indices[0]] if len(indices) == 1 else torch.cat([embeddings_list[i] for i in indices], dim=1),
                                weights=values_list[indices[0]] if values_list is not None else None)
    return ret


def construct_jagged_tensors_inference(embeddings: torch.Tensor, lengths: torch.Tensor, values: torch.Tensor, embedding_names: List[str], need_indices: bool = False,
                                       features_to_permute_indices: Optional[Dict[str, List[int]]] = None, reverse_indices: Optional[torch.Tensor] = None,
                                       remove_padding: bool = False) -> Dict[str, JaggedTensor]:
    """Inference form: ``lengths [F, B]`` and ``values`` are passed as plain tensors (no KJT caches, no host sync besides the split sizes)."""
    if reverse_indices is not None:
        embeddings = torch.index_select(embeddings, 0, reverse_indices.to(torch.int64))
    elif remove_padding:
        embeddings = embeddings[: int(lengths.sum())]
    lengths = lengths.view(len(embedding_names), -1)
    per_key = lengths.sum(dim=1).tolist()
    kjt = KeyedJaggedTensor(keys=[str(i) for i in range(len(embedding_names))], values=values, lengths=lengths.reshape(-1), length_per_key=per_key)
    return construct_jagged_tensors(embeddings, kjt, embedding_names, need_indices, features_to_permute_indices)


def _permute_indices(indices: List[int], permute: List[int]) -> List[int]:
    return [indices[p] for p in permute] if len(permute) == len(indices) else indices


def jagged_index_select_with_empty(values: torch.Tensor, ids: torch.Tensor, offsets: torch.Tensor, output_offsets: torch.Tensor) -> torch.Tensor:
    """Select the segments ``ids`` of a jagged 2-D tensor; an empty ``values`` gives an empty result."""
    if values.numel() == 0:
        return torch.empty(0, device=values.device, dtype=values.dtype)
    lengths = offsets[1:] - offsets[:-1]
    out, _ = sops.jagged_index_select(values, lengths, ids)
    return out


def deterministic_dedup(ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(sorted unique ids, index of the last occurrence of each)`` -- a stable sort makes the chosen occurrence reproducible,
    which scatter-based de-duplication does not guarantee."""
    sorted_ids, sorted_idx = ids.sort(stable=True)
    last = torch.cat([sorted_ids[1:] != sorted_ids[:-1], torch.ones(1, dtype=torch.bool, device=ids.device)]) if ids.numel() else torch.empty(0, dtype=torch.bool, device=ids.device)
    return sorted_ids[last], sorted_idx[last]


def reset_module_states_post_sharding(module: nn.Module) -> None:
    """Modules that cache sharding-dependent state expose ``reset_inference_mode`` / ``_has_uninitialized_*`` hooks: reset them."""
    for m in module.modules():
        if hasattr(m, "reset_inference_mode") and getattr(m, "_is_inference", False):
            m.reset_inference_mode()


def _get_batching_hinted_output(lengths: torch.Tensor, output: torch.Tensor) -> torch.Tensor:
    """Identity that keeps ``lengths`` alive next to ``output`` for tracers that would otherwise drop the dependency."""
    return output


def _fx_trec_get_feature_length(features: KeyedJaggedTensor, embedding_names: List[str]) -> torch.Tensor:
    torch._assert(len(embedding_names) == len(features.keys()), "embedding output and features mismatch")
    return features.lengths()
