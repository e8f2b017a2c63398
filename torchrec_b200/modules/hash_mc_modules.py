"""Multi-probe zero-collision hash (MPZCH) as a managed-collision module.

Unbounded ids are mapped onto the rows of a bounded table so that, while the table has room, two ids never share a row: the id
is hashed into its bucket of the slot table and takes the first free slot among the next ``max_probe`` ones; when none is free it
may replace an id whose time-to-live ran out (or the least recently used probed one), else it shares the row at its hash position.
The slot table (``_hash_zch_identities``) and the eviction scores (``_hash_zch_metadata``) are the module's checkpointed state.
Buckets make the state reshardable: bucket ``b`` owns the slots ``[segments[b], segments[b+1])`` and ids are dealt to buckets by
the same rule the row-wise input distribution uses, so a rank that owns buckets ``[start, end)`` sees exactly their ids.

Lookup, insertion, eviction and the bucket arithmetic run in one op (``ops.sparse_ops.zch_probe``; device kernels in
``csrc/cuda/misc_kernels.cu``).  Counterpart of ``torchrec/modules/hash_mc_modules.py`` (``HashZchManagedCollisionModule`` ``:155``,
``remap`` ``:469``).  Opt-in admission (``opt_in_prob``, ``percent_reserved_slots``): an id without a slot may claim one only with the
given probability per occurrence; until then it shares one of the reserved rows at the end of its bucket, which no id can claim.
"""
from __future__ import annotations

import logging
import math
from typing import Any, Dict, Iterator, List, Optional, Tuple

import torch

from torchrec_b200.modules.hash_mc_evictions import HashZchEvictionConfig, HashZchEvictionModule, HashZchEvictionPolicyName, get_kernel_from_policy
from torchrec_b200.modules.hash_mc_metrics import ScalarLogger
from torchrec_b200.modules.mc_modules import ManagedCollisionModule
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import JaggedTensor

logger: logging.Logger = logging.getLogger(__name__)


def create_zch_buffer(size: int, support_evict: bool, device: torch.device) -> Tuple[torch.Tensor, torch.Tensor]:
    """Empty slot table ``[size, 1]`` (-1 everywhere) and its score table (``[size, 1]``, or ``[0, 1]`` without eviction)."""
    identities = torch.full((size, 1), -1, dtype=torch.int64, device=device)
    metadata = torch.full((size if support_evict else 0, 1), sops.ZCH_EMPTY_SCORE, dtype=torch.int32, device=device)
    return identities, metadata


class TrainInputMapper(torch.nn.Module):
    """Where every id of an inference input would have gone at training time.  At inference the slot tables of all training ranks
    are merged into one; an id must still be probed inside the chunk of the rank that owned it.  ``forward(values, output_offset)``
    returns, per id: the id as that rank saw it (divided by, or reduced modulo, the dealing rule when
    ``inference_dispatch_div_train_world_size``), the size of the owning chunk, and the chunk's first row (minus ``output_offset``).
    Ids are dealt to ``total_num_buckets`` chunks by ``id % buckets`` when ``input_hash_size`` is 0, else by contiguous blocks of
    ``ceil(input_hash_size / buckets)`` ids - the rule of the row-wise input distribution.
    Counterpart of ``torchrec/modules/hash_mc_modules.py:44-147``."""

    def __init__(self, input_hash_size: int, total_num_buckets: int, size_per_rank: torch.Tensor, train_rank_offsets: torch.Tensor,
                 inference_dispatch_div_train_world_size: bool = False, name: Optional[str] = None) -> None:
        super().__init__()
        assert total_num_buckets > 0, f"{total_num_buckets=} must be positive"
        self._input_hash_size = input_hash_size
        self._buckets = total_num_buckets
        self._inference_dispatch_div_train_world_size = inference_dispatch_div_train_world_size
        self._name = name
        self.register_buffer("_zch_size_per_training_rank", size_per_rank, persistent=False)
        self.register_buffer("_train_rank_offsets", train_rank_offsets, persistent=False)

    def forward(self, values: torch.Tensor, output_offset: Optional[torch.Tensor] = None
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
        sizes = self._zch_size_per_training_rank.to(values.device)
        starts = self._train_rank_offsets.to(values.device)
        if self._input_hash_size == 0:
            owner = values % self._buckets
            seen = values // self._buckets if self._inference_dispatch_div_train_world_size else values
        else:
            block = -(-self._input_hash_size // self._buckets)
            owner = values // block
            seen = values % block if self._inference_dispatch_div_train_world_size else values
        offsets = starts.index_select(0, owner)
        if output_offset is not None:
            offsets = offsets - output_offset
        return seen, sizes.index_select(0, owner), offsets


class HashZchManagedCollisionModule(ManagedCollisionModule):
    IDENTITY_BUFFER: str = "_hash_zch_identities"
    METADATA_BUFFER: str = "_hash_zch_metadata"

    def __init__(
        self,
        zch_size: int,
        device: torch.device,
        total_num_buckets: int,
        max_probe: int = 128,
        input_hash_size: int = 0,
        output_segments: Optional[List[int]] = None,
        is_inference: bool = False,
        name: Optional[str] = None,
        tb_logging_frequency: int = 0,
        eviction_policy_name: Optional[HashZchEvictionPolicyName] = None,
        eviction_config: Optional[HashZchEvictionConfig] = None,
        inference_dispatch_div_train_world_size: bool = False,
        start_bucket: int = 0,
        end_bucket: Optional[int] = None,
        opt_in_prob: int = -1,
        percent_reserved_slots: float = 0,
        disable_fallback: bool = False,
    ) -> None:
        if output_segments is None:
            assert zch_size % total_num_buckets == 0, f"pass output_segments when buckets are not uniform ({zch_size=}, {total_num_buckets=})"
            output_segments = [(zch_size // total_num_buckets) * b for b in range(total_num_buckets + 1)]
        super().__init__(device=device if device.type != "meta" else torch.device("cpu"), output_segments=output_segments, skip_state_validation=True)
        assert 0 <= percent_reserved_slots < 100, "percent_reserved_slots must be in [0, 100)"
        assert opt_in_prob == -1 or 0 <= opt_in_prob <= 100, "opt_in_prob is a percentage (or -1: every id is admitted)"
        assert opt_in_prob == -1 or percent_reserved_slots > 0, "percent_reserved_slots must be positive when opt_in_prob is set"
        self._opt_in_prob, self._percent_reserved_slots = int(opt_in_prob), float(percent_reserved_slots)
        self._device = device
        self._zch_size = zch_size
        self._output_segments = list(output_segments)
        self._buckets = total_num_buckets
        self._start_bucket = start_bucket
        self._end_bucket = end_bucket if end_bucket is not None else total_num_buckets
        self._output_global_offset = int(output_segments[start_bucket])
        self._input_hash_size = input_hash_size
        self._max_probe = max_probe
        self._is_inference = is_inference
        self._name = name
        self._inference_dispatch_div_train_world_size = inference_dispatch_div_train_world_size
        self._disable_fallback = disable_fallback
        self._tb_logging_frequency = 0 if (is_inference or name is None) else tb_logging_frequency
        self._eviction_policy_name = eviction_policy_name
        self._eviction_policy_name_copy = eviction_policy_name
        self._eviction_config = eviction_config
        self._eviction_module: Optional[HashZchEvictionModule] = (
            HashZchEvictionModule(eviction_policy_name, device, eviction_config) if eviction_policy_name is not None else None)
        self._scalar_logger: Optional[ScalarLogger] = (
            ScalarLogger(name=name or "", zch_size=zch_size, frequency=self._tb_logging_frequency, start_bucket=start_bucket, disable_fallback=disable_fallback)
            if self._tb_logging_frequency > 0 and device.type != "meta" else None)
        identities, metadata = create_zch_buffer(zch_size, self._eviction_module is not None, device)
        self._hash_zch_identities = torch.nn.Parameter(identities, requires_grad=False)
        self.register_buffer(self.METADATA_BUFFER, metadata)
        self._evicted_indices: List[torch.Tensor] = []
        self.table_name_on_device_remapped_ids_dict: Dict[str, torch.Tensor] = {}
        self.table_name_on_device_input_ids_dict: Dict[str, torch.Tensor] = {}
        if is_inference:
            self.reset_inference_mode()

    # ---- state -------------------------------------------------------------------------------------
    @property
    def device(self) -> torch.device:
        return self._hash_zch_identities.device

    def buckets(self) -> int:
        return self._buckets

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True) -> Iterator[Tuple[str, torch.Tensor]]:
        yield from super().named_buffers(prefix, recurse, remove_duplicate)
        yield (f"{prefix}.{self.IDENTITY_BUFFER}" if prefix else self.IDENTITY_BUFFER, self._hash_zch_identities.data)

    def validate_state(self) -> None:
        ids = self._hash_zch_identities.data.view(-1)
        stored = ids[ids != -1]
        assert stored.unique().numel() == stored.numel(), "an id is stored in two slots"

    def _set_eval_mode_impl(self) -> None:
        self.eval()
        self._is_inference = True
        self._evicted_indices = []
        self._eviction_policy_name = None
        self._eviction_module = None

    def reset_inference_mode(self) -> None:
        self._set_eval_mode_impl()
        self._hash_zch_metadata = None

        def drop_metadata(module: "HashZchManagedCollisionModule", state_dict: Dict[str, Any], prefix: str, *args: Any) -> None:
            if module._is_inference:
                state_dict.pop(prefix + self.METADATA_BUFFER, None)

        self._register_load_state_dict_pre_hook(drop_metadata, with_module=True)

    def reset_intrainer_bulk_eval_mode(self) -> None:
        self._set_eval_mode_impl()

    def reset_training_mode(self) -> None:
        self._is_inference = False
        self.train()
        self._eviction_policy_name = self._eviction_policy_name_copy
        self._eviction_module = (HashZchEvictionModule(self._eviction_policy_name, self._device, self._eviction_config)
                                 if self._eviction_policy_name is not None else None)

    # ---- interface -----------------------------------------------------------------------------------
    def preprocess(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        return features

    def profile(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        return features

    def evict(self) -> Optional[torch.Tensor]:
        if not self._evicted_indices:
            return None
        out = torch.unique(torch.cat(self._evicted_indices))
        self._evicted_indices = []
        return out + self._output_global_offset

    def get_reserved_slots_per_bucket(self) -> int:
        """With opt-in admission, the number of slots at the end of every bucket that no id may claim (the shared rows of the ids that
        were not admitted); -1 when admission is off."""
        if self._opt_in_prob == -1:
            return -1
        return math.floor(self._zch_size * self._percent_reserved_slots / 100 / (self._end_bucket - self._start_bucket))

    def _dispatch_ids(self, values: torch.Tensor) -> torch.Tensor:
        """Ids as the training ranks saw them: at inference the merged table receives raw ids, while a training rank received the
        row-wise-bucketized local id when ``inference_dispatch_div_train_world_size`` is set."""
        return values

    @torch.no_grad()
    def remap(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        readonly = not self.training
        metadata = getattr(self, self.METADATA_BUFFER, None) if self.training else None
        if metadata is not None and metadata.numel() == 0:
            metadata = None
        identities = self._hash_zch_identities.data.view(-1)
        segments = self._output_segments_tensor
        out: Dict[str, JaggedTensor] = {}
        for name, feature in features.items():
            values = feature.values()
            orig_device = values.device
            score, threshold = (self._eviction_module(feature) if (self._eviction_module is not None and self.training) else (None, -1))
            ids = values.to(self.device)
            before = identities.clone() if self._scalar_logger is not None else None
            # opt-in admission: while training, an id that has no slot yet may claim one only if its draw (a percentage) falls below opt_in_prob
            admit = None
            if self._opt_in_prob != -1 and self.training:
                admit = (torch.rand(ids.shape, device=ids.device) * 100).to(torch.int32) < self._opt_in_prob
            slots, evicted = sops.zch_probe(
                ids, identities, None if metadata is None else metadata.view(-1), segments, input_hash_size=self._input_hash_size,
                out_offset=self._output_global_offset, max_probe=self._max_probe, readonly=readonly, disable_fallback=self._disable_fallback,
                input_metadata=score, eviction_threshold=threshold, eviction_policy=get_kernel_from_policy(self._eviction_policy_name) if self.training else sops.ZCH_NO_EVICT,
                reserved_slots=max(self.get_reserved_slots_per_bucket(), 0), admit=admit)
            self.table_name_on_device_input_ids_dict[name] = ids
            self.table_name_on_device_remapped_ids_dict[name] = slots
            if self._scalar_logger is not None and before is not None:
                self._scalar_logger.update(identities_0=before, identities_1=identities, values=ids, remapped_ids=slots, evicted_emb_indices=evicted)
            lengths = feature.lengths()
            offsets = feature.offsets()
            weights = feature.weights_or_none()
            if self._disable_fallback:
                # ids without a slot are dropped from their bags
                keep = slots >= 0
                seg = torch.repeat_interleave(torch.arange(lengths.numel(), device=slots.device), lengths.to(slots.device))
                lengths = torch.zeros_like(lengths).scatter_add_(0, seg[keep].to(lengths.device), torch.ones(int(keep.sum()), dtype=lengths.dtype, device=lengths.device))
                slots = slots[keep]
                weights = None if weights is None else weights[keep.to(weights.device)]
                offsets = None
            ev = evicted[evicted >= 0]
            if ev.numel() > 0:
                self._evicted_indices.append(ev)
            out[name] = JaggedTensor(values=(slots + self._output_global_offset).to(orig_device), lengths=lengths, offsets=offsets, weights=weights)
        if self._scalar_logger is not None:
            self._scalar_logger(run_type="train" if self.training else "eval", identities=identities)
        return out

    def forward(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        return self.remap(features)

    def output_size(self) -> int:
        return self._zch_size

    def input_size(self) -> int:
        return self._input_hash_size

    def open_slots(self) -> torch.Tensor:
        return (self._hash_zch_identities.data.view(-1) == -1).sum().view(1)

    def rebuild_with_output_id_range(self, output_id_range: Tuple[int, int], output_segments: Optional[List[int]] = None,
                                     device: Optional[torch.device] = None) -> "HashZchManagedCollisionModule":
        try:
            start = self._output_segments.index(output_id_range[0])
            end = self._output_segments.index(output_id_range[1])
        except ValueError:
            raise RuntimeError(f"the shard {output_id_range} does not lie on bucket boundaries; total_num_buckets={self._buckets} must be a multiple of the world size")
        return type(self)(
            zch_size=output_id_range[1] - output_id_range[0], device=device or self.device, total_num_buckets=self._buckets, max_probe=self._max_probe,
            input_hash_size=self._input_hash_size, output_segments=self._output_segments, is_inference=self._is_inference, name=self._name,
            tb_logging_frequency=self._tb_logging_frequency, eviction_policy_name=self._eviction_policy_name, eviction_config=self._eviction_config,
            inference_dispatch_div_train_world_size=self._inference_dispatch_div_train_world_size, start_bucket=start, end_bucket=end, opt_in_prob=self._opt_in_prob, percent_reserved_slots=self._percent_reserved_slots,
            disable_fallback=self._disable_fallback)
