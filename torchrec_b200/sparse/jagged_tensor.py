"""Sparse data types: ``JaggedTensor``, ``KeyedJaggedTensor``, ``KeyedTensor``.

Behavioural counterpart of the reference's ``torchrec/sparse/jagged_tensor.py``
(``JaggedTensor`` ``:562``, ``KeyedJaggedTensor`` ``:1679``, ``KeyedTensor`` ``:3145``).
The layout conventions are the same -- a KJT stores ``values [sum L]`` and
``lengths [F * B]`` key-major -- but the implementation is organised around the ops in
``torchrec_b200.ops.sparse_ops`` (composite torch on CPU, sm_100a kernels on CUDA) and
keeps host-side caches (``length_per_key`` ...) lazy so that the fused device paths never
force a device-to-host sync unless a caller asks for a Python list.
"""
from __future__ import annotations

import abc
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch
from torch.utils import _pytree as pytree

from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.streamable import Pipelineable


def _cumsum_list(o: List[int]) -> List[int]:
    out = [0] * (len(o) + 1)
    for i, v in enumerate(o):
        out[i + 1] = out[i] + v
    return out


def _to_offsets(lengths: torch.Tensor) -> torch.Tensor:
    return sops.asynchronous_complete_cumsum(lengths)


def _to_lengths(offsets: torch.Tensor) -> torch.Tensor:
    return offsets[1:] - offsets[:-1]


def _maybe_compute_lengths(lengths: Optional[torch.Tensor], offsets: Optional[torch.Tensor]) -> torch.Tensor:
    if lengths is None:
        assert offsets is not None
        lengths = _to_lengths(offsets)
    return lengths


def _maybe_compute_offsets(lengths: Optional[torch.Tensor], offsets: Optional[torch.Tensor]) -> torch.Tensor:
    if offsets is None:
        assert lengths is not None
        offsets = _to_offsets(lengths)
    return offsets


def _get_weights_or_throw(weights: Optional[torch.Tensor]) -> torch.Tensor:
    assert weights is not None, "This (Keyed)JaggedTensor doesn't have weights."
    return weights


def _get_lengths_offset_per_key_or_throw(x: Optional[List[int]]) -> List[int]:
    assert x is not None, "This (Keyed)JaggedTensor doesn't have lengths_offset_per_key."
    return x


def _get_stride_per_key_or_throw(x: Optional[List[int]]) -> List[int]:
    assert x is not None, "This (Keyed)JaggedTensor doesn't have stride_per_key."
    return x


def _get_inverse_indices_or_throw(x: Optional[Tuple[List[str], torch.Tensor]]) -> Tuple[List[str], torch.Tensor]:
    assert x is not None, "This KJT doesn't have inverse indices."
    return x


def _assert_offsets_or_lengths_is_provided(offsets: Optional[torch.Tensor], lengths: Optional[torch.Tensor]) -> None:
    assert offsets is not None or lengths is not None, "Must provide lengths or offsets"


def _assert_tensor_has_no_elements_or_has_integers(tensor: Optional[torch.Tensor], name: str) -> None:
    if tensor is None or tensor.numel() == 0:
        return
    assert tensor.dtype in (torch.long, torch.int, torch.short, torch.int8, torch.uint8), (
        f"{name} must be of integer type, but got {tensor.dtype}"
    )


def _optional_mask(t: Optional[torch.Tensor], mask: torch.Tensor) -> Optional[torch.Tensor]:
    return t[mask] if t is not None else None


def _arange(*args, **kwargs) -> torch.Tensor:
    return torch.arange(*args, **kwargs)


def _permute_tensor_by_segments(
    tensor: torch.Tensor,
    segment_sizes: torch.Tensor,
    recat: torch.Tensor,
    weights: Optional[torch.Tensor] = None,
    output_size: Optional[int] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Reorder contiguous segments of a 1-D tensor (and matching weights) by ``recat``."""
    _, out_t, out_w = sops.permute_1D_sparse_data(recat, segment_sizes, tensor, weights, output_size)
    return out_t, out_w


def _jagged_values_string(values: torch.Tensor, offsets: torch.Tensor, offset_start: int, offset_end: int) -> str:
    off = offsets.tolist()
    return "[" + ", ".join(
        str(values[off[i]: off[i + 1]].tolist()) for i in range(offset_start, offset_end)
    ) + "]"


class JaggedTensorMeta(abc.ABCMeta):
    pass


class JaggedTensor(Pipelineable, metaclass=JaggedTensorMeta):
    """Values of ONE feature with a variable number of entries per sample.

    ``values [N(, D)]`` plus either ``lengths [B]`` or ``offsets [B+1]`` and optional
    per-value ``weights``.  Whichever of lengths/offsets is missing is computed on demand.
    """

    _fields = ["_values", "_weights", "_lengths", "_offsets"]

    def __init__(
        self,
        values: torch.Tensor,
        weights: Optional[torch.Tensor] = None,
        lengths: Optional[torch.Tensor] = None,
        offsets: Optional[torch.Tensor] = None,
    ) -> None:
        _assert_offsets_or_lengths_is_provided(offsets, lengths)
        for name, t in (("offsets", offsets), ("lengths", lengths)):
            if t is not None:
                _assert_tensor_has_no_elements_or_has_integers(t, name)
        self._values, self._weights = values, weights
        self._lengths, self._offsets = lengths, offsets

    @staticmethod
    def empty(
        is_weighted: bool = False,
        device: Optional[torch.device] = None,
        values_dtype: Optional[torch.dtype] = None,
        weights_dtype: Optional[torch.dtype] = None,
        lengths_dtype: torch.dtype = torch.int32,
    ) -> "JaggedTensor":
        weights = torch.empty(0, dtype=weights_dtype, device=device) if is_weighted else None
        return JaggedTensor(
            values=torch.empty(0, dtype=values_dtype, device=device),
            offsets=torch.empty(0, dtype=lengths_dtype, device=device),
            lengths=torch.empty(0, dtype=lengths_dtype, device=device),
            weights=weights,
        )

    @staticmethod
    def from_dense_lengths(
        values: torch.Tensor, lengths: torch.Tensor, weights: Optional[torch.Tensor] = None
    ) -> "JaggedTensor":
        """Build from a padded ``[B, L(, D)]`` tensor and the valid length of every row."""
        mask2d = _arange(end=values.size(1), device=values.device).expand(values.size(0), -1) < lengths.unsqueeze(-1)
        return JaggedTensor(values=values[mask2d], weights=_optional_mask(weights, mask2d), lengths=lengths)

    @staticmethod
    def from_dense(values: List[torch.Tensor], weights: Optional[List[torch.Tensor]] = None) -> "JaggedTensor":
        """Build from a list of per-sample 1-D tensors."""
        values_tensor = torch.cat(values, dim=0)
        lengths = torch.tensor([v.size(0) for v in values], dtype=torch.int32, device=values_tensor.device)
        weights_tensor = torch.cat(weights, dim=0) if weights is not None else None
        return JaggedTensor(values=values_tensor, weights=weights_tensor, lengths=lengths)

    def to_dense(self) -> List[torch.Tensor]:
        off = self.offsets().tolist()
        return [self._values[off[i]: off[i + 1]] for i in range(len(off) - 1)]

    def to_dense_weights(self) -> Optional[List[torch.Tensor]]:
        if self._weights is None:
            return None
        off = self.offsets().tolist()
        return [self._weights[off[i]: off[i + 1]] for i in range(len(off) - 1)]

    def to_padded_dense(self, desired_length: Optional[int] = None, padding_value: float = 0.0) -> torch.Tensor:
        """``[B, desired_length(, D)]``; long rows are truncated, short rows padded."""
        if desired_length is None:
            N = int(self.lengths().max().item()) if self.lengths().numel() else 0
        else:
            N = desired_length
        return sops.jagged_to_padded_dense(self._values, self.offsets(), N, padding_value)

    def to_padded_dense_weights(self, desired_length: Optional[int] = None, padding_value: float = 0.0):
        if self._weights is None:
            return None
        if desired_length is None:
            N = int(self.lengths().max().item()) if self.lengths().numel() else 0
        else:
            N = desired_length
        return sops.jagged_to_padded_dense(self._weights, self.offsets(), N, padding_value)

    def device(self) -> torch.device:
        return self._values.device

    def lengths(self) -> torch.Tensor:
        self._lengths = _maybe_compute_lengths(self._lengths, self._offsets)
        return self._lengths

    def lengths_or_none(self) -> Optional[torch.Tensor]:
        return self._lengths

    def offsets(self) -> torch.Tensor:
        self._offsets = _maybe_compute_offsets(self._lengths, self._offsets)
        return self._offsets

    def offsets_or_none(self) -> Optional[torch.Tensor]:
        return self._offsets

    def values(self) -> torch.Tensor:
        return self._values

    def weights(self) -> torch.Tensor:
        return _get_weights_or_throw(self._weights)

    def weights_or_none(self) -> Optional[torch.Tensor]:
        return self._weights

    def to(self, device: torch.device, non_blocking: bool = False) -> "JaggedTensor":
        return JaggedTensor(
            values=self._values.to(device, non_blocking=non_blocking),
            weights=None if self._weights is None else self._weights.to(device, non_blocking=non_blocking),
            lengths=None if self._lengths is None else self._lengths.to(device, non_blocking=non_blocking),
            offsets=None if self._offsets is None else self._offsets.to(device, non_blocking=non_blocking),
        )

    @torch.jit.unused
    def record_stream(self, stream: torch.Stream) -> None:
        for t in (self._values, self._weights, self._lengths, self._offsets):
            if t is not None and t.is_cuda:
                t.record_stream(stream)

    def __str__(self) -> str:
        offsets = self.offsets()
        if self._weights is None:
            return "JaggedTensor({\n    " + _jagged_values_string(self._values, offsets, 0, len(offsets) - 1) + "\n})\n"
        return (
            "JaggedTensor({\n"
            + '    "values": ' + _jagged_values_string(self._values, offsets, 0, len(offsets) - 1)
            + ',\n    "weights": ' + _jagged_values_string(self._weights, offsets, 0, len(offsets) - 1)
            + "\n})\n"
        )


def _jt_flatten(t: JaggedTensor):
    return [getattr(t, a) for a in JaggedTensor._fields], None


def _jt_unflatten(values, context) -> JaggedTensor:
    return JaggedTensor(*values)


def _jt_flatten_with_keys(t: JaggedTensor):
    values, context = _jt_flatten(t)
    return [(pytree.GetAttrKey(k), v) for k, v in zip(JaggedTensor._fields, values)], context


pytree.register_pytree_node(
    JaggedTensor, _jt_flatten, _jt_unflatten, flatten_with_keys_fn=_jt_flatten_with_keys,
    serialized_type_name="torchrec_b200.sparse.jagged_tensor.JaggedTensor"
)


# --------------------------------------------------------------------------------------
# helpers for KJT caches
# --------------------------------------------------------------------------------------
def _maybe_compute_index_per_key(keys: List[str], index_per_key: Optional[Dict[str, int]]) -> Dict[str, int]:
    if index_per_key is None:
        index_per_key = {key: i for i, key in enumerate(keys)}
    return index_per_key


def _sum_by_splits(input_list: List[int], splits: List[int]) -> List[int]:
    out, s = [], 0
    for sp in splits:
        out.append(sum(input_list[s: s + sp]))
        s += sp
    return out


def _length_per_key_from_stride_per_key(lengths: torch.Tensor, stride_per_key: List[int]) -> List[int]:
    """Total ids per key when every key has its own batch size."""
    if lengths.numel() == 0:
        return [0] * len(stride_per_key)
    csr = torch.tensor(_cumsum_list(stride_per_key), dtype=torch.int64, device=lengths.device)
    return sops.segment_sum_csr(1, csr, lengths.to(torch.int64)).tolist()


def _maybe_compute_stride_kjt(
    keys: List[str],
    stride: Optional[int],
    lengths: Optional[torch.Tensor],
    offsets: Optional[torch.Tensor],
    stride_per_key_per_rank: Optional[torch.Tensor],
) -> int:
    if stride is None:
        if len(keys) == 0:
            stride = 0
        elif stride_per_key_per_rank is not None and stride_per_key_per_rank.numel() > 0:
            stride = int(stride_per_key_per_rank.sum(dim=1).max().item())
        elif offsets is not None and offsets.numel() > 0:
            stride = (offsets.numel() - 1) // len(keys)
        elif lengths is not None:
            stride = lengths.numel() // len(keys)
        else:
            stride = 0
    return stride


def _kjt_empty_like(kjt: "KeyedJaggedTensor") -> "KeyedJaggedTensor":
    stride, stride_per_key_per_rank = (
        (None, kjt._stride_per_key_per_rank) if kjt.variable_stride_per_key() else (kjt.stride(), None)
    )
    return KeyedJaggedTensor(
        keys=[],
        values=torch.empty(0, device=kjt.device(), dtype=kjt.values().dtype),
        weights=None if kjt.weights_or_none() is None else torch.empty(0, device=kjt.device(), dtype=kjt.weights().dtype),
        lengths=torch.empty(0, device=kjt.device(), dtype=kjt.lengths().dtype),
        stride=stride,
        stride_per_key_per_rank=stride_per_key_per_rank,
    )


def _regroup_keyed_tensors(keyed_tensors: List["KeyedTensor"], groups: List[List[str]]) -> List[torch.Tensor]:
    in_keys = [kt.keys() for kt in keyed_tensors]
    in_lengths = [kt.length_per_key() for kt in keyed_tensors]
    key_dim = keyed_tensors[0].key_dim()
    values = [kt.values() for kt in keyed_tensors]
    if key_dim != 1:
        values = [v.transpose(key_dim, 1) for v in values]
    outs = sops.permute_multi_embedding(values, in_lengths, in_keys, groups)
    if key_dim != 1:
        outs = [o.transpose(key_dim, 1) for o in outs]
    return outs


class KeyedJaggedTensor(Pipelineable, metaclass=JaggedTensorMeta):
    """Jagged values of several features (keys) over one batch.

    Layout: ``lengths`` has one entry per (key, sample) in key-major order, so the bags
    of key ``k`` are ``lengths[k*B:(k+1)*B]`` and its ids are one contiguous slice of
    ``values``.  With ``stride_per_key_per_rank`` every key may have its own batch size
    (variable batch per feature); ``inverse_indices`` then maps the deduplicated bags back
    to the full batch.
    """

    _fields = ["_values", "_weights", "_lengths", "_offsets"]

    def __init__(
        self,
        keys: List[str],
        values: torch.Tensor,
        weights: Optional[torch.Tensor] = None,
        lengths: Optional[torch.Tensor] = None,
        offsets: Optional[torch.Tensor] = None,
        stride: Optional[int] = None,
        stride_per_key_per_rank: Optional[Union[torch.Tensor, List[List[int]]]] = None,
        stride_per_key: Optional[List[int]] = None,
        length_per_key: Optional[List[int]] = None,
        lengths_offset_per_key: Optional[List[int]] = None,
        offset_per_key: Optional[List[int]] = None,
        index_per_key: Optional[Dict[str, int]] = None,
        jt_dict: Optional[Dict[str, JaggedTensor]] = None,
        inverse_indices: Optional[Tuple[List[str], torch.Tensor]] = None,
    ) -> None:
        _assert_offsets_or_lengths_is_provided(offsets, lengths)
        # the data: ids (+ weights) of all keys back to back, and how they split into bags
        self._keys, self._values, self._weights = keys, values, weights
        self._lengths, self._offsets, self._stride = lengths, offsets, stride
        if stride_per_key_per_rank is not None and not isinstance(stride_per_key_per_rank, torch.Tensor):
            rows = len(stride_per_key_per_rank)
            stride_per_key_per_rank = torch.tensor(stride_per_key_per_rank, dtype=torch.int64, device="cpu").view(rows, -1)
        self._stride_per_key_per_rank = stride_per_key_per_rank
        self._inverse_indices = inverse_indices
        # host-side caches: computed lazily, or handed over by a producer that already knows them (split, permute, dist)
        self._stride_per_key, self._index_per_key, self._jt_dict = stride_per_key, index_per_key, jt_dict
        self._length_per_key, self._offset_per_key, self._lengths_offset_per_key = length_per_key, offset_per_key, lengths_offset_per_key

    # ---- constructors ---------------------------------------------------------------
    @staticmethod
    def from_offsets_sync(
        keys: List[str],
        values: torch.Tensor,
        offsets: torch.Tensor,
        weights: Optional[torch.Tensor] = None,
        stride: Optional[int] = None,
        stride_per_key_per_rank: Optional[List[List[int]]] = None,
        inverse_indices: Optional[Tuple[List[str], torch.Tensor]] = None,
    ) -> "KeyedJaggedTensor":
        return KeyedJaggedTensor(
            keys=keys, values=values, weights=weights, offsets=offsets, stride=stride,
            stride_per_key_per_rank=stride_per_key_per_rank, inverse_indices=inverse_indices,
        ).sync()

    @staticmethod
    def from_lengths_sync(
        keys: List[str],
        values: torch.Tensor,
        lengths: torch.Tensor,
        weights: Optional[torch.Tensor] = None,
        stride: Optional[int] = None,
        stride_per_key_per_rank: Optional[List[List[int]]] = None,
        inverse_indices: Optional[Tuple[List[str], torch.Tensor]] = None,
    ) -> "KeyedJaggedTensor":
        return KeyedJaggedTensor(
            keys=keys, values=values, weights=weights, lengths=lengths, stride=stride,
            stride_per_key_per_rank=stride_per_key_per_rank, inverse_indices=inverse_indices,
        ).sync()

    @staticmethod
    def concat(kjt_list: List["KeyedJaggedTensor"]) -> "KeyedJaggedTensor":
        """Concatenate along the key dimension (all inputs share the batch)."""
        if not kjt_list:
            raise ValueError("Can't concat empty KJT list")
        first = kjt_list[0]
        weighted = first.weights_or_none() is not None
        variable = any(k.variable_stride_per_key() for k in kjt_list)
        known = [k._length_per_key for k in kjt_list]  # the cached per-key totals survive only if every input has them
        return KeyedJaggedTensor(
            keys=[key for k in kjt_list for key in k.keys()],
            values=torch.cat([k.values() for k in kjt_list], dim=0),
            weights=torch.cat([k.weights() for k in kjt_list], dim=0) if weighted else None,
            lengths=torch.cat([k.lengths() for k in kjt_list], dim=0),
            stride=None if variable else first.stride(),
            stride_per_key_per_rank=torch.cat([k.stride_per_key_per_rank_tensor() for k in kjt_list], dim=0) if variable else None,
            length_per_key=[n for per in known for n in per] if all(per is not None for per in known) else None,
        )

    @staticmethod
    def empty(
        is_weighted: bool = False,
        device: Optional[torch.device] = None,
        values_dtype: Optional[torch.dtype] = None,
        weights_dtype: Optional[torch.dtype] = None,
        lengths_dtype: torch.dtype = torch.int32,
    ) -> "KeyedJaggedTensor":
        weights = torch.empty(0, dtype=weights_dtype, device=device) if is_weighted else None
        return KeyedJaggedTensor(
            keys=[], values=torch.empty(0, dtype=values_dtype, device=device), weights=weights,
            lengths=torch.empty(0, dtype=lengths_dtype, device=device), stride=0,
        )

    @staticmethod
    def empty_like(kjt: "KeyedJaggedTensor") -> "KeyedJaggedTensor":
        return _kjt_empty_like(kjt)

    @staticmethod
    def from_jt_dict(jt_dict: Dict[str, JaggedTensor]) -> "KeyedJaggedTensor":
        """Build from per-key ``JaggedTensor``s that all have the same batch size."""
        jts = list(jt_dict.values())
        batch_sizes = [jt.lengths().numel() for jt in jts]
        uniform = len(set(batch_sizes)) <= 1
        weights = [jt.weights() for jt in jts if jt.weights_or_none() is not None]
        return KeyedJaggedTensor(
            keys=list(jt_dict.keys()),
            values=torch.cat([jt.values() for jt in jts]),
            weights=torch.cat(weights) if weights else None,
            lengths=torch.cat([jt.lengths() for jt in jts]),
            stride=(batch_sizes[0] if batch_sizes else 0) if uniform else None,
            stride_per_key_per_rank=None if uniform else [[b] for b in batch_sizes],
        ).sync()

    # ---- caches ---------------------------------------------------------------------
    def sync(self) -> "KeyedJaggedTensor":
        """Materialise the host-side per-key caches (one device-to-host copy)."""
        if not torch.jit.is_scripting():
            self.length_per_key()
            self.offset_per_key()
        return self

    def unsync(self) -> "KeyedJaggedTensor":
        self._length_per_key = None
        self._offset_per_key = None
        return self

    def device(self) -> torch.device:
        return self._values.device

    def lengths(self) -> torch.Tensor:
        self._lengths = _maybe_compute_lengths(self._lengths, self._offsets)
        return self._lengths

    def lengths_or_none(self) -> Optional[torch.Tensor]:
        return self._lengths

    def offsets(self) -> torch.Tensor:
        self._offsets = _maybe_compute_offsets(self._lengths, self._offsets)
        return self._offsets

    def offsets_or_none(self) -> Optional[torch.Tensor]:
        return self._offsets

    def keys(self) -> List[str]:
        return self._keys

    def values(self) -> torch.Tensor:
        return self._values

    def weights(self) -> torch.Tensor:
        return _get_weights_or_throw(self._weights)

    def weights_or_none(self) -> Optional[torch.Tensor]:
        return self._weights

    def stride(self) -> int:
        self._stride = _maybe_compute_stride_kjt(
            self._keys, self._stride, self._lengths, self._offsets, self._stride_per_key_per_rank
        )
        return self._stride

    def stride_per_key(self) -> List[int]:
        if self._stride_per_key is None:
            if self._stride_per_key_per_rank is not None:
                self._stride_per_key = self._stride_per_key_per_rank.sum(dim=1).tolist()
            else:
                self._stride_per_key = [self.stride()] * len(self._keys)
        return _get_stride_per_key_or_throw(self._stride_per_key)

    def stride_per_key_per_rank(self) -> List[List[int]]:
        if self._stride_per_key_per_rank is None:
            return []
        return self._stride_per_key_per_rank.tolist()

    def stride_per_key_per_rank_tensor(self) -> torch.Tensor:
        if self._stride_per_key_per_rank is None:
            return torch.tensor([[self.stride()]] * len(self._keys), dtype=torch.int64).view(len(self._keys), -1)
        return self._stride_per_key_per_rank

    def variable_stride_per_key(self) -> bool:
        return self._stride_per_key_per_rank is not None

    def inverse_indices(self) -> Tuple[List[str], torch.Tensor]:
        return _get_inverse_indices_or_throw(self._inverse_indices)

    def inverse_indices_or_none(self) -> Optional[Tuple[List[str], torch.Tensor]]:
        return self._inverse_indices

    def _key_indices(self) -> Dict[str, int]:
        self._index_per_key = _maybe_compute_index_per_key(self._keys, self._index_per_key)
        return self._index_per_key

    def length_per_key(self) -> List[int]:
        if self._length_per_key is None:
            if len(self._keys) == 0:
                self._length_per_key = []
            elif self.variable_stride_per_key():
                self._length_per_key = _length_per_key_from_stride_per_key(self.lengths(), self.stride_per_key())
            else:
                B = self.stride()
                if B == 0 or self.lengths().numel() == 0:
                    self._length_per_key = [0] * len(self._keys)
                else:
                    self._length_per_key = self.lengths().view(len(self._keys), B).sum(dim=1).tolist()
        return self._length_per_key

    def length_per_key_or_none(self) -> Optional[List[int]]:
        return self._length_per_key

    def offset_per_key(self) -> List[int]:
        if self._offset_per_key is None:
            self._offset_per_key = _cumsum_list(self.length_per_key())
        return self._offset_per_key

    def offset_per_key_or_none(self) -> Optional[List[int]]:
        return self._offset_per_key

    def lengths_offset_per_key(self) -> List[int]:
        if self._lengths_offset_per_key is None:
            self._lengths_offset_per_key = _cumsum_list(self.stride_per_key())
        return _get_lengths_offset_per_key_or_throw(self._lengths_offset_per_key)

    def index_per_key(self) -> Dict[str, int]:
        return self._key_indices()

    # ---- restructuring --------------------------------------------------------------
    def split(self, segments: List[int]) -> List["KeyedJaggedTensor"]:
        """Split along keys into consecutive groups of ``segments[i]`` keys."""
        n_keys = len(self._keys)
        totals, id_bounds = self.length_per_key(), self.offset_per_key()
        strides = self._stride_per_key_per_rank
        bag_bounds = self.lengths_offset_per_key() if self.variable_stride_per_key() else [k * self.stride() for k in range(n_keys + 1)]

        def empty_like_me(dtype: torch.dtype) -> torch.Tensor:
            return torch.empty(0, device=self.device(), dtype=dtype)

        pieces: List[KeyedJaggedTensor] = []
        k0 = 0
        for width in segments:
            k1 = k0 + width
            sub_strides = None if strides is None else strides[k0:k1, :]
            if width == n_keys:  # the whole thing: no copy, caches kept
                pieces.append(self)
            elif width == 0:
                bag_dtype = self.lengths().dtype
                pieces.append(KeyedJaggedTensor(
                    keys=[], values=empty_like_me(self._values.dtype), weights=None if self._weights is None else empty_like_me(self._weights.dtype),
                    lengths=empty_like_me(bag_dtype), offsets=empty_like_me(bag_dtype), stride=self._stride, stride_per_key_per_rank=sub_strides))
            else:
                ids = slice(id_bounds[k0], id_bounds[k1])
                pieces.append(KeyedJaggedTensor(
                    keys=self._keys[k0:k1], values=self._values[ids], weights=None if self._weights is None else self._weights[ids],
                    lengths=self.lengths()[bag_bounds[k0]: bag_bounds[k1]], stride=self._stride, stride_per_key_per_rank=sub_strides,
                    length_per_key=totals[k0:k1]))
            k0 = k1
        return pieces

    def permute(self, indices: List[int], indices_tensor: Optional[torch.Tensor] = None) -> "KeyedJaggedTensor":
        """Reorder (or repeat / drop) keys."""
        if indices_tensor is None:
            indices_tensor = torch.tensor(indices, dtype=torch.int32, device=self.device())
        length_per_key = self.length_per_key()
        permuted_keys = [self._keys[i] for i in indices]
        permuted_length_per_key = [length_per_key[i] for i in indices]
        permuted_length_per_key_sum = sum(permuted_length_per_key)
        spkpr = self._stride_per_key_per_rank
        if self.variable_stride_per_key():
            assert spkpr is not None
            permuted_spkpr = spkpr[list(indices), :] if len(indices) else spkpr[:0, :]
            spk = self.stride_per_key()
            lopk = self.lengths_offset_per_key()
            # bag-level permutation: expand the key permutation over each key's own batch
            seg = torch.tensor(spk, dtype=torch.int64, device=self.device())
            permuted_lengths, _ = _permute_tensor_by_segments(self.lengths(), seg, indices_tensor, None)
            lpk = torch.tensor(length_per_key, dtype=torch.int64, device=self.device())
            permuted_values, permuted_weights = _permute_tensor_by_segments(
                self.values(), lpk, indices_tensor, self.weights_or_none(), permuted_length_per_key_sum
            )
            del lopk
            stride = None
        else:
            permuted_spkpr = None
            stride = self._stride
            if self.stride() == 0 or len(self._keys) == 0:
                permuted_lengths = self.lengths().new_empty(len(indices) * self.stride())
                permuted_values = self._values[:0]
                permuted_weights = None if self._weights is None else self._weights[:0]
            else:
                permuted_lengths, permuted_values, permuted_weights = sops.permute_2D_sparse_data(
                    indices_tensor,
                    self.lengths().view(len(self._keys), -1),
                    self.values(),
                    self.weights_or_none(),
                    permuted_length_per_key_sum,
                )
        return KeyedJaggedTensor(
            keys=permuted_keys,
            values=permuted_values,
            weights=permuted_weights,
            lengths=permuted_lengths.view(-1),
            stride=stride,
            stride_per_key_per_rank=permuted_spkpr,
            length_per_key=permuted_length_per_key if len(permuted_keys) > 0 else None,
            inverse_indices=None,
        )

    def flatten_lengths(self) -> "KeyedJaggedTensor":
        stride, spkpr = (
            (None, self._stride_per_key_per_rank) if self.variable_stride_per_key() else (self._stride, None)
        )
        return KeyedJaggedTensor(
            keys=self._keys, values=self._values, weights=self._weights, lengths=self.lengths().view(-1),
            stride=stride, stride_per_key_per_rank=spkpr, length_per_key=self.length_per_key(),
        )

    def __getitem__(self, key: str) -> JaggedTensor:
        k = self._key_indices()[key]
        id_bounds, bag_bounds = self.offset_per_key(), self.lengths_offset_per_key()
        ids = slice(id_bounds[k], id_bounds[k + 1]) if k + 1 < len(id_bounds) else slice(id_bounds[k], id_bounds[k])
        return JaggedTensor(values=self._values[ids], weights=None if self._weights is None else self._weights[ids],
                            lengths=self.lengths()[bag_bounds[k]: bag_bounds[k + 1]])

    def to_dict(self) -> Dict[str, JaggedTensor]:
        if self._jt_dict is None:
            self._jt_dict = {k: self[k] for k in self._keys}
        return self._jt_dict

    @torch.jit.unused
    def record_stream(self, stream: torch.Stream) -> None:
        for t in (self._values, self._weights, self._lengths, self._offsets):
            if t is not None and t.is_cuda:
                t.record_stream(stream)
        if self._inverse_indices is not None and self._inverse_indices[1].is_cuda:
            self._inverse_indices[1].record_stream(stream)

    def to(self, device: torch.device, non_blocking: bool = False, dtype: Optional[torch.dtype] = None) -> "KeyedJaggedTensor":
        weights = self._weights
        if weights is not None:
            weights = weights.to(device, non_blocking=non_blocking, dtype=dtype) if dtype is not None else weights.to(device, non_blocking=non_blocking)
        inv = self._inverse_indices
        if inv is not None:
            inv = (inv[0], inv[1].to(device, non_blocking=non_blocking))
        stride, spkpr = (
            (None, self._stride_per_key_per_rank) if self.variable_stride_per_key() else (self._stride, None)
        )
        return KeyedJaggedTensor(
            keys=self._keys,
            values=self._values.to(device, non_blocking=non_blocking),
            weights=weights,
            lengths=None if self._lengths is None else self._lengths.to(device, non_blocking=non_blocking),
            offsets=None if self._offsets is None else self._offsets.to(device, non_blocking=non_blocking),
            stride=stride,
            stride_per_key_per_rank=spkpr,
            stride_per_key=self._stride_per_key,
            length_per_key=self._length_per_key,
            lengths_offset_per_key=self._lengths_offset_per_key,
            offset_per_key=self._offset_per_key,
            index_per_key=self._index_per_key,
            jt_dict=None,
            inverse_indices=inv,
        )

    def pin_memory(self) -> "KeyedJaggedTensor":
        stride, spkpr = (
            (None, self._stride_per_key_per_rank) if self.variable_stride_per_key() else (self._stride, None)
        )
        inv = self._inverse_indices
        if inv is not None:
            inv = (inv[0], inv[1].pin_memory())
        return KeyedJaggedTensor(
            keys=self._keys,
            values=self._values.pin_memory(),
            weights=None if self._weights is None else self._weights.pin_memory(),
            lengths=None if self._lengths is None else self._lengths.pin_memory(),
            offsets=None if self._offsets is None else self._offsets.pin_memory(),
            stride=stride, stride_per_key_per_rank=spkpr,
            length_per_key=self._length_per_key, offset_per_key=self._offset_per_key,
            inverse_indices=inv,
        )

    def __str__(self) -> str:
        if len(self._keys) == 0 or (self._offsets is None and self._lengths is None):
            return "KeyedJaggedTensor()\n"
        offsets = self.offsets()
        lopk = self.lengths_offset_per_key()
        out = "KeyedJaggedTensor({\n"
        for i, key in enumerate(self._keys):
            a, b = lopk[i], lopk[i + 1]
            if self._weights is None:
                out += f'    "{key}": ' + _jagged_values_string(self._values, offsets, a, b)
            else:
                out += (
                    f'    "{key}": {{\n        "values": ' + _jagged_values_string(self._values, offsets, a, b)
                    + ',\n        "weights": ' + _jagged_values_string(self._weights, offsets, a, b) + "\n    }"
                )
            out += ",\n" if i + 1 < len(self._keys) else "\n"
        return out + "})\n"

    # ---- distributed protocol -------------------------------------------------------
    def _dist_parts(self) -> List[str]:
        """What travels in the input all-to-all, in order: bag lengths and ids always; per-key batch sizes when every key has
        its own; per-id weights when present."""
        optional = (("strides", self.variable_stride_per_key()), ("weights", self.weights_or_none() is not None))
        return ["lengths", "values"] + [name for name, present in optional if present]

    def dist_labels(self) -> List[str]:
        return self._dist_parts()

    def dist_splits(self, key_splits: List[int]) -> List[List[int]]:
        """Per part of :meth:`dist_labels`, how many elements go to every destination."""
        bags = _sum_by_splits(self.stride_per_key(), key_splits)
        ids = _sum_by_splits(self.length_per_key(), key_splits)
        per_part = {"lengths": bags, "values": ids, "strides": key_splits, "weights": ids}
        return [per_part[name] for name in self._dist_parts()]

    def dist_tensors(self) -> List[torch.Tensor]:
        def strides_on_device() -> torch.Tensor:
            return torch.tensor(self.stride_per_key(), dtype=torch.int64).to(self.device(), non_blocking=True)

        per_part = {"lengths": self.lengths, "values": self.values, "strides": strides_on_device, "weights": self.weights}
        return [per_part[name]() for name in self._dist_parts()]

    @staticmethod
    def dist_init(
        keys: List[str],
        tensors: List[torch.Tensor],
        variable_stride_per_key: bool,
        num_workers: int,
        recat: Optional[torch.Tensor],
        stride_per_rank: Optional[List[int]],
        stagger: int = 1,
    ) -> "KeyedJaggedTensor":
        """Assemble the KJT a rank owns after the input all-to-all.

        Received data is (source-rank, key)-major; ``recat`` reorders it to key-major so
        that each key's bags from all ranks are contiguous.
        """
        assert len(tensors) in (2, 3, 4)
        parts = ["lengths", "values"] + (["strides"] if variable_stride_per_key else [])
        named = dict(zip(parts + ["weights"], tensors))  # weights, when sent, come last
        lengths, values, weights = named["lengths"], named["values"], named.get("weights")
        if variable_stride_per_key:
            sent_strides = named["strides"]  # (source rank, key)-major batch sizes
            matrix = sent_strides.view(num_workers, len(keys)).T.cpu()
            if recat is not None:
                bag_bounds = sops.asynchronous_complete_cumsum(sent_strides).to(torch.int64)
                id_prefix = sops.asynchronous_complete_cumsum(lengths)
                ids_per_segment = id_prefix[bag_bounds[1:]] - id_prefix[bag_bounds[:-1]]
                lengths, _ = _permute_tensor_by_segments(lengths, sent_strides, recat, None)
                values, weights = _permute_tensor_by_segments(values, ids_per_segment, recat, weights)
            if matrix.numel() == 0:
                matrix = torch.zeros((len(keys), 1), device="cpu", dtype=torch.int64)
            if stagger > 1:
                matrix = matrix[:, torch.arange(num_workers).view(stagger, -1).T.reshape(-1)]
            return KeyedJaggedTensor(keys=keys, values=values, weights=weights, lengths=lengths, stride_per_key_per_rank=matrix).sync()
        assert stride_per_rank is not None
        if recat is not None:
            same_batch_everywhere = len(set(stride_per_rank)) <= 1
            if not same_batch_everywhere:
                lengths, values, weights = sops.permute_1D_sparse_data(recat, lengths.view(-1), values, weights, values.numel())
            elif stride_per_rank and stride_per_rank[0] > 0:
                rows = lengths.view(-1, stride_per_rank[0])
                rows, values, weights = sops.permute_2D_sparse_data(recat, rows, values, weights, values.numel())
                lengths = rows.view(-1)
        return KeyedJaggedTensor(keys=keys, values=values, weights=weights, lengths=lengths, stride=sum(stride_per_rank)).sync()


def _kjt_flatten(t: KeyedJaggedTensor):
    return [getattr(t, a) for a in KeyedJaggedTensor._fields], (t._keys, t._stride_per_key_per_rank)


def _kjt_unflatten(values, context) -> KeyedJaggedTensor:
    keys, spkpr = context
    return KeyedJaggedTensor(keys, *values, stride_per_key_per_rank=spkpr)


def _kjt_flatten_with_keys(t: KeyedJaggedTensor):
    values, context = _kjt_flatten(t)
    return [(pytree.GetAttrKey(k), v) for k, v in zip(KeyedJaggedTensor._fields, values)], context


pytree.register_pytree_node(
    KeyedJaggedTensor, _kjt_flatten, _kjt_unflatten, flatten_with_keys_fn=_kjt_flatten_with_keys,
    serialized_type_name="torchrec_b200.sparse.jagged_tensor.KeyedJaggedTensor",
)


def jt_is_equal(jt_1: "JaggedTensor", jt_2: "JaggedTensor") -> bool:
    """Equality of two jagged tensors: values and weights (close, for floats), and the same bag boundaries whether either side
    stores them as lengths or as offsets.  Anything that is not a ``JaggedTensor`` compares unequal."""
    if not isinstance(jt_1, JaggedTensor) or not isinstance(jt_2, JaggedTensor):
        return False
    if (jt_1.weights_or_none() is None) != (jt_2.weights_or_none() is None):
        return False
    pairs = [(jt_1.values(), jt_2.values()), (jt_1.lengths(), jt_2.lengths())]
    if jt_1.weights_or_none() is not None:
        pairs.append((jt_1.weights(), jt_2.weights()))
    for a, b in pairs:
        if a.shape != b.shape:
            return False
        same = torch.allclose(a, b.to(a.dtype)) if a.is_floating_point() or b.is_floating_point() else torch.equal(a.to(b.dtype), b)
        if not same:
            return False
    return True


def regroup_kts(keyed_tensors: List["KeyedTensor"], groups: List[List[str]]) -> List[torch.Tensor]:
    """``groups[i]`` names the keys (from any of ``keyed_tensors``) whose columns form output ``i``, in that order; one kernel moves
    every column (``permute_multi_embedding``).  Same result as ``KeyedTensor.regroup``."""
    return _regroup_keyed_tensors(keyed_tensors, groups)


def kjt_is_equal(kjt_1: "KeyedJaggedTensor", kjt_2: "KeyedJaggedTensor") -> bool:
    """Field-by-field equality of two KJTs (keys order included)."""
    if not isinstance(kjt_1, KeyedJaggedTensor) or not isinstance(kjt_2, KeyedJaggedTensor):
        return False
    if kjt_1.keys() != kjt_2.keys():
        return False
    if (kjt_1.weights_or_none() is None) != (kjt_2.weights_or_none() is None):
        return False
    if kjt_1.variable_stride_per_key() != kjt_2.variable_stride_per_key():
        return False
    if kjt_1.variable_stride_per_key() and kjt_1.stride_per_key_per_rank() != kjt_2.stride_per_key_per_rank():
        return False
    pairs = [(kjt_1.lengths(), kjt_2.lengths()), (kjt_1.values(), kjt_2.values())]
    if kjt_1.weights_or_none() is not None:
        pairs.append((kjt_1.weights(), kjt_2.weights()))
    for a, b in pairs:
        if a.shape != b.shape or not torch.equal(a.to(b.dtype) if a.dtype != b.dtype else a, b):
            return False
    return True


class ComputeKJTToJTDict(torch.nn.Module):
    """Module form of ``KeyedJaggedTensor.to_dict`` (traceable leaf)."""

    def forward(self, keyed_jagged_tensor: "KeyedJaggedTensor") -> Dict[str, JaggedTensor]:
        return {k: keyed_jagged_tensor[k] for k in keyed_jagged_tensor.keys()}


class ComputeJTDictToKJT(torch.nn.Module):
    def forward(self, jt_dict: Dict[str, JaggedTensor]) -> KeyedJaggedTensor:
        return KeyedJaggedTensor.from_jt_dict(jt_dict)


# --------------------------------------------------------------------------------------
# KeyedTensor
# --------------------------------------------------------------------------------------
def _keyed_values_string(values: torch.Tensor) -> str:
    return "[" + ", ".join([str(v.tolist()) for v in values]) + "]"


class KeyedTensor(Pipelineable, metaclass=JaggedTensorMeta):
    """Dense tensor whose ``key_dim`` is a concatenation of named blocks.

    The pooled output of an ``EmbeddingBagCollection`` is a ``KeyedTensor`` with
    ``values [B, sum(D)]`` and one block of width ``D_k`` per feature.
    """

    def __init__(
        self,
        keys: List[str],
        length_per_key: List[int],
        values: torch.Tensor,
        key_dim: int = 1,
        offset_per_key: Optional[List[int]] = None,
        index_per_key: Optional[Dict[str, int]] = None,
    ) -> None:
        self._keys = keys
        self._length_per_key = length_per_key
        self._values = values
        self._key_dim = key_dim
        self._offset_per_key: Optional[List[int]] = offset_per_key
        self._index_per_key: Optional[Dict[str, int]] = index_per_key

    @staticmethod
    def from_tensor_list(keys: List[str], tensors: List[torch.Tensor], key_dim: int = 1, cat_dim: int = 1) -> "KeyedTensor":
        length_per_key = [t.shape[key_dim] for t in tensors]
        return KeyedTensor(keys=keys, length_per_key=length_per_key, values=torch.cat(tensors, dim=cat_dim), key_dim=key_dim)

    def keys(self) -> List[str]:
        return self._keys

    def values(self) -> torch.Tensor:
        return self._values

    def key_dim(self) -> int:
        return self._key_dim

    def device(self) -> torch.device:
        return self._values.device

    def offset_per_key(self) -> List[int]:
        if self._offset_per_key is None:
            self._offset_per_key = _cumsum_list(self._length_per_key)
        return self._offset_per_key

    def length_per_key(self) -> List[int]:
        return self._length_per_key

    def _key_indices(self) -> Dict[str, int]:
        self._index_per_key = _maybe_compute_index_per_key(self._keys, self._index_per_key)
        return self._index_per_key

    def __getitem__(self, key: str) -> torch.Tensor:
        index = self._key_indices()[key]
        start = self.offset_per_key()[index]
        return self._values.narrow(self._key_dim, start, self._length_per_key[index])

    def to_dict(self) -> Dict[str, torch.Tensor]:
        split_values = self._values.split(self._length_per_key, dim=self._key_dim)
        return {key: split_values[i] for i, key in enumerate(self._keys)}

    @staticmethod
    def regroup(keyed_tensors: List["KeyedTensor"], groups: List[List[str]]) -> List[torch.Tensor]:
        """Build one dense tensor per group of keys, drawing blocks from several KTs."""
        return _regroup_keyed_tensors(keyed_tensors, groups)

    @staticmethod
    def regroup_as_dict(keyed_tensors: List["KeyedTensor"], groups: List[List[str]], keys: List[str]) -> Dict[str, torch.Tensor]:
        assert len(groups) == len(keys), "Groups and keys should have same length"
        tensor_list = _regroup_keyed_tensors(keyed_tensors, groups)
        return {key: tensor_list[i] for i, key in enumerate(keys)}

    @torch.jit.unused
    def record_stream(self, stream: torch.Stream) -> None:
        if self._values.is_cuda:
            self._values.record_stream(stream)

    def to(self, device: torch.device, non_blocking: bool = False) -> "KeyedTensor":
        return KeyedTensor(
            keys=self._keys, length_per_key=self._length_per_key,
            values=self._values.to(device, non_blocking=non_blocking), key_dim=self._key_dim,
            offset_per_key=self._offset_per_key, index_per_key=self._index_per_key,
        )

    def __str__(self) -> str:
        if len(self._keys) == 0:
            return "KeyedTensor()\n"
        return (
            "KeyedTensor({\n"
            + "".join(f'    "{key}": ' + _keyed_values_string(self[key]) + "\n" for key in self._keys)
            + "})\n"
        )


def _kt_flatten(kt: KeyedTensor):
    return [kt._values], (kt._keys, kt._length_per_key, kt._key_dim)


def _kt_unflatten(values, context) -> KeyedTensor:
    keys, lpk, key_dim = context
    return KeyedTensor(keys, lpk, values[0], key_dim)


def _kt_flatten_with_keys(kt: KeyedTensor):
    values, context = _kt_flatten(kt)
    return [(pytree.GetAttrKey("_values"), values[0])], context


pytree.register_pytree_node(
    KeyedTensor, _kt_flatten, _kt_unflatten, flatten_with_keys_fn=_kt_flatten_with_keys,
    serialized_type_name="torchrec_b200.sparse.jagged_tensor.KeyedTensor"
)


def flatten_kjt_list(kjt_arr: List[KeyedJaggedTensor]) -> Tuple[List[Optional[torch.Tensor]], List[Any]]:
    flat, ctx = [], []
    for k in kjt_arr:
        v, c = _kjt_flatten(k)
        flat.extend(v)
        ctx.append(c)
    return flat, ctx


def unflatten_kjt_list(values: List[Optional[torch.Tensor]], contexts: List[Any]) -> List[KeyedJaggedTensor]:
    n = len(KeyedJaggedTensor._fields)
    return [_kjt_unflatten(values[i * n: (i + 1) * n], contexts[i]) for i in range(len(contexts))]
