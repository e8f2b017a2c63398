"""Managed collision: remap an unbounded id space onto a table of ``zch_size`` rows, keeping the ids the eviction policy
values most in private slots ("zero collision") and hashing the rest.

``MCHManagedCollisionModule`` keeps a sorted array of the admitted raw ids with their slot and policy metadata.  During
training every batch is *profiled* (counts / recency of its ids); every ``eviction_interval`` batches the admitted set is
rebuilt: current members and newly seen candidates are ranked by the policy score, the best ``zch_size`` stay or move
in, members that drop out hand their slots to the newcomers and are reported by ``evict()`` so that the caller can
reset those embedding rows.  ``remap`` is a ``searchsorted`` lookup; ids that are not admitted fall back to
``id % zch_size``.

Counterpart of ``torchrec/modules/mc_modules.py`` (``MCHManagedCollisionModule``, eviction policies LFU / LRU /
DistanceLFU, ``ManagedCollisionCollection``).
"""
from __future__ import annotations

import abc
from typing import Callable, Dict, List, NamedTuple, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


@torch.no_grad()
def apply_mc_method_to_jt_dict(mc_module: nn.Module, method: str, features_dict: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
    """Call ``mc_module.<method>(features_dict)`` (``"preprocess"``, ``"profile"``, ``"remap"``): one entry point for the steps a
    collection runs on every module's features, in the dictionary's order."""
    return getattr(mc_module, method)(features_dict)


def dynamic_threshold_filter(id_counts: torch.Tensor, threshold_skew_multiplier: float = 10.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Keep ids seen more often than ``multiplier * total / distinct``."""
    num_ids = id_counts.numel()
    total = id_counts.sum()
    threshold = threshold_skew_multiplier * total / max(num_ids, 1)
    return id_counts > threshold, threshold


@torch.no_grad()
def average_threshold_filter(id_counts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    if id_counts.dim() == 0 or id_counts.numel() == 0:
        return id_counts > 0, torch.tensor(0.0)
    threshold = id_counts.float().mean()
    return id_counts > threshold, threshold


@torch.no_grad()
def probabilistic_threshold_filter(id_counts: torch.Tensor, per_id_probability: float = 0.01) -> Tuple[torch.Tensor, torch.Tensor]:
    """Admit an id seen ``c`` times with probability ``1 - (1 - p)^c``."""
    probability = 1 - torch.pow(1 - per_id_probability, id_counts.float())
    threshold = torch.rand(id_counts.size(), device=id_counts.device)
    return probability > threshold, threshold


class MCHEvictionPolicyMetadataInfo(NamedTuple):
    metadata_name: str
    is_mch_metadata: bool
    is_history_metadata: bool


class MCHEvictionPolicy(abc.ABC):
    """Scores ids: higher = keep.  ``coalesce`` merges metadata of repeated ids; ``score`` ranks members and candidates."""

    def __init__(self, metadata_info: List[MCHEvictionPolicyMetadataInfo], threshold_filtering_func: Optional[Callable[[torch.Tensor], Tuple[torch.Tensor, torch.Tensor]]] = None) -> None:
        self._metadata_info = metadata_info
        self._threshold_filtering_func = threshold_filtering_func

    @property
    def metadata_info(self) -> List[MCHEvictionPolicyMetadataInfo]:
        return self._metadata_info

    @abc.abstractmethod
    def score(self, counts: torch.Tensor, last_access: torch.Tensor, current_iter: int) -> torch.Tensor:
        ...

    def admit(self, counts: torch.Tensor) -> torch.Tensor:
        """Which candidates may enter at all (threshold filter on their counts)."""
        if self._threshold_filtering_func is None:
            return torch.ones_like(counts, dtype=torch.bool)
        return self._threshold_filtering_func(counts)[0]


class LFU_EvictionPolicy(MCHEvictionPolicy):
    def __init__(self, threshold_filtering_func=None) -> None:
        super().__init__([MCHEvictionPolicyMetadataInfo("counts", True, True)], threshold_filtering_func)

    def score(self, counts, last_access, current_iter):
        return counts.double()


class LRU_EvictionPolicy(MCHEvictionPolicy):
    def __init__(self, decay_exponent: float = 1.0, threshold_filtering_func=None) -> None:
        super().__init__([MCHEvictionPolicyMetadataInfo("last_access_iter", True, True)], threshold_filtering_func)
        self._decay_exponent = decay_exponent

    def score(self, counts, last_access, current_iter):
        return last_access.double()


class DistanceLFU_EvictionPolicy(MCHEvictionPolicy):
    """Frequency discounted by how long ago the id was last seen: ``count / (iters since last access + 1)^decay``."""

    def __init__(self, decay_exponent: float = 1.0, threshold_filtering_func=None) -> None:
        super().__init__([MCHEvictionPolicyMetadataInfo("counts", True, True), MCHEvictionPolicyMetadataInfo("last_access_iter", True, True)], threshold_filtering_func)
        self._decay_exponent = decay_exponent

    def score(self, counts, last_access, current_iter):
        return counts.double() / torch.pow((current_iter - last_access).clamp(min=0).double() + 1.0, self._decay_exponent)


class ManagedCollisionModule(nn.Module):
    """Interface: ``preprocess`` -> ``profile`` (training) -> ``remap``; ``evict`` reports rows to reset."""

    def __init__(self, device: torch.device, output_segments: List[int], skip_state_validation: bool = False) -> None:
        super().__init__()
        self._device = device
        self._output_segments_tensor = torch.tensor(output_segments, dtype=torch.int64, device=device)

    @abc.abstractmethod
    def preprocess(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        ...

    @property
    def device(self) -> torch.device:
        return self._device

    @abc.abstractmethod
    def evict(self) -> Optional[torch.Tensor]:
        ...

    @abc.abstractmethod
    def remap(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        ...

    @abc.abstractmethod
    def profile(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        ...

    @abc.abstractmethod
    def forward(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        ...

    @abc.abstractmethod
    def output_size(self) -> int:
        ...

    @abc.abstractmethod
    def input_size(self) -> int:
        ...

    @abc.abstractmethod
    def open_slots(self) -> torch.Tensor:
        ...

    @abc.abstractmethod
    def reset_inference_mode(self) -> None:
        """Called when the module is moved into a serving (quantized) model: drop whatever only training needs."""
        return None

    def rebuild_with_output_id_range(self, output_id_range: Tuple[int, int], output_segments: List[int], device: Optional[torch.device] = None) -> "ManagedCollisionModule":
        ...


_PAD = torch.iinfo(torch.int64).max


class MCHManagedCollisionModule(ManagedCollisionModule):
    def __init__(self, zch_size: int, device: torch.device, eviction_policy: MCHEvictionPolicy, eviction_interval: int, input_hash_size: int = (2 ** 63) - 1,
                 input_hash_func: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None, mch_size: Optional[int] = None, mch_hash_func=None,
                 name: Optional[str] = None, output_global_offset: int = 0, output_segments: Optional[List[int]] = None, buckets: int = 1) -> None:
        super().__init__(device, output_segments or [output_global_offset, output_global_offset + zch_size])
        self._zch_size = zch_size
        self._eviction_policy = eviction_policy
        self._eviction_interval = eviction_interval
        self._input_hash_size = input_hash_size
        self._input_hash_func = input_hash_func
        self._output_global_offset = output_global_offset
        self._name = name
        self._buckets = buckets
        self._current_iter = -1
        self.register_buffer("_mch_sorted_raw_ids", torch.full((zch_size,), _PAD, dtype=torch.int64, device=device))
        self.register_buffer("_mch_remapped_ids_mapping", torch.arange(zch_size, dtype=torch.int64, device=device))
        self.register_buffer("_mch_counts", torch.zeros(zch_size, dtype=torch.int64, device=device))
        self.register_buffer("_mch_last_access_iter", torch.zeros(zch_size, dtype=torch.int64, device=device))
        self.register_buffer("_current_iter_tensor", torch.zeros(1, dtype=torch.int64, device=device))
        # ids seen since the last rebuild (unique) with their counts / last access
        self._history_ids = torch.empty(0, dtype=torch.int64, device=device)
        self._history_counts = torch.empty(0, dtype=torch.int64, device=device)
        self._history_last = torch.empty(0, dtype=torch.int64, device=device)
        self._evicted: bool = False
        self._last_eviction_iter = -1
        self._evicted_emb_indices = torch.empty(0, dtype=torch.int64, device=device)

    def preprocess(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        if self._input_hash_func is None:
            return features
        return {k: JaggedTensor(values=self._input_hash_func(jt.values(), self._input_hash_size), lengths=jt.lengths(), offsets=jt.offsets(), weights=jt.weights_or_none())
                for k, jt in features.items()}

    def _members(self) -> torch.Tensor:
        return self._mch_sorted_raw_ids != _PAD

    @torch.no_grad()
    def _match(self, values: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Position in the sorted member array and whether the id is a member."""
        pos = torch.searchsorted(self._mch_sorted_raw_ids, values).clamp(max=self._zch_size - 1)
        return pos, self._mch_sorted_raw_ids[pos] == values

    @torch.no_grad()
    def profile(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        if not self.training:
            return features
        if self._current_iter == -1:
            self._current_iter = int(self._current_iter_tensor.item())
            self._last_eviction_iter = self._current_iter
        self._current_iter += 1
        self._current_iter_tensor += 1
        ids = torch.cat([jt.values().to(self._device).long() for jt in features.values()]) if features else torch.empty(0, dtype=torch.int64, device=self._device)
        if ids.numel():
            uniq, counts = torch.unique(ids, return_counts=True)
            pos, hit = self._match(uniq)
            # members: bump their metadata in place
            self._mch_counts[pos[hit]] += counts[hit]
            self._mch_last_access_iter[pos[hit]] = self._current_iter
            # non-members: merge into the history of candidates
            cand, ccnt = uniq[~hit], counts[~hit]
            if cand.numel():
                all_ids = torch.cat([self._history_ids, cand])
                all_cnt = torch.cat([self._history_counts, ccnt])
                all_last = torch.cat([self._history_last, torch.full_like(cand, self._current_iter)])
                u, inv = torch.unique(all_ids, return_inverse=True)
                self._history_counts = torch.zeros_like(u).index_add_(0, inv, all_cnt)
                self._history_last = torch.zeros_like(u).scatter_reduce_(0, inv, all_last, "amax", include_self=False)
                self._history_ids = u
        if self._current_iter - self._last_eviction_iter >= self._eviction_interval:
            self._rebuild()
            self._last_eviction_iter = self._current_iter
        return features

    @torch.no_grad()
    def _rebuild(self) -> None:
        """Rank members and admitted candidates together; the top ``zch_size`` form the new member set."""
        member = self._members()
        m_ids, m_slots = self._mch_sorted_raw_ids[member], self._mch_remapped_ids_mapping[member]
        m_cnt, m_last = self._mch_counts[member], self._mch_last_access_iter[member]
        admit = self._eviction_policy.admit(self._history_counts) if self._history_ids.numel() else torch.empty(0, dtype=torch.bool, device=self._device)
        c_ids, c_cnt, c_last = self._history_ids[admit], self._history_counts[admit], self._history_last[admit]
        ids = torch.cat([m_ids, c_ids]); cnt = torch.cat([m_cnt, c_cnt]); last = torch.cat([m_last, c_last])
        is_member = torch.cat([torch.ones_like(m_ids, dtype=torch.bool), torch.zeros_like(c_ids, dtype=torch.bool)])
        slots = torch.cat([m_slots, torch.full_like(c_ids, -1)])
        score = self._eviction_policy.score(cnt, last, self._current_iter)
        # ties: members first (stable against churn), then larger raw id last
        order = torch.argsort(score + is_member.double() * 1e-9, descending=True, stable=True)
        keep = order[: self._zch_size]
        kept_member = is_member[keep]
        evicted_slots = torch.cat([m_slots[~torch.isin(torch.arange(m_ids.numel(), device=self._device), keep[keep < m_ids.numel()])]]) if m_ids.numel() else torch.empty(0, dtype=torch.int64, device=self._device)
        used = torch.zeros(self._zch_size, dtype=torch.bool, device=self._device)
        used[slots[keep][kept_member]] = True
        free = torch.nonzero(~used).view(-1)
        new_slots = slots[keep].clone()
        n_new = int((~kept_member).sum())
        new_slots[~kept_member] = free[:n_new]
        k_ids, k_cnt, k_last = ids[keep], cnt[keep], last[keep]
        srt = torch.argsort(k_ids)
        n = k_ids.numel()
        self._mch_sorted_raw_ids.fill_(_PAD)
        self._mch_sorted_raw_ids[:n] = k_ids[srt]
        self._mch_remapped_ids_mapping[:n] = new_slots[srt]
        self._mch_counts.zero_()
        self._mch_last_access_iter.zero_()
        self._mch_counts[:n] = k_cnt[srt]
        self._mch_last_access_iter[:n] = k_last[srt]
        # rows whose owner changed: slots of evicted members that were handed to newcomers
        self._evicted_emb_indices = evicted_slots[torch.isin(evicted_slots, new_slots[~kept_member])] + self._output_global_offset
        self._evicted = self._evicted_emb_indices.numel() > 0
        self._history_ids = self._history_ids[:0]
        self._history_counts = self._history_counts[:0]
        self._history_last = self._history_last[:0]

    @torch.no_grad()
    def remap(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        out: Dict[str, JaggedTensor] = {}
        for name, jt in features.items():
            v = jt.values().to(self._device).long()
            pos, hit = self._match(v)
            remapped = torch.where(hit, self._mch_remapped_ids_mapping[pos], torch.remainder(v, self._zch_size)) + self._output_global_offset
            out[name] = JaggedTensor(values=remapped.to(jt.values().device), lengths=jt.lengths(), offsets=jt.offsets(), weights=jt.weights_or_none())
        return out

    def forward(self, features: Dict[str, JaggedTensor]) -> Dict[str, JaggedTensor]:
        features = self.preprocess(features)
        features = self.profile(features)
        return self.remap(features)

    def output_size(self) -> int:
        return self._zch_size

    def input_size(self) -> int:
        return self._input_hash_size

    def open_slots(self) -> torch.Tensor:
        return (self._zch_size - self._members().sum()).view(1)

    @torch.no_grad()
    def evict(self) -> Optional[torch.Tensor]:
        if self._evicted:
            self._evicted = False
            return self._evicted_emb_indices
        return None

    def reset_inference_mode(self) -> None:
        """Serving keeps the id -> slot map and nothing else: no pending eviction report, no admission candidates."""
        self._evicted, self._last_eviction_iter = False, -1
        self._evicted_emb_indices = self._evicted_emb_indices[:0]
        self._history_ids, self._history_counts, self._history_last = self._history_ids[:0], self._history_counts[:0], self._history_last[:0]

    def rebuild_with_output_id_range(self, output_id_range: Tuple[int, int], output_segments: List[int], device: Optional[torch.device] = None) -> "MCHManagedCollisionModule":
        return type(self)(zch_size=int(output_id_range[1] - output_id_range[0]), device=device or self.device, eviction_policy=self._eviction_policy,
                          eviction_interval=self._eviction_interval, input_hash_size=self._input_hash_size, input_hash_func=self._input_hash_func,
                          name=self._name, output_global_offset=int(output_id_range[0]), output_segments=output_segments, buckets=self._buckets)


class ManagedCollisionCollection(nn.Module):
    """One managed-collision module per embedding table; ``forward(KJT) -> KJT`` with remapped ids."""

    def __init__(self, managed_collision_modules: Dict[str, ManagedCollisionModule], embedding_configs, need_preprocess: bool = True) -> None:
        super().__init__()
        self._managed_collision_modules = nn.ModuleDict(managed_collision_modules)
        self._embedding_configs = embedding_configs
        self.need_preprocess = need_preprocess
        self._feature_to_table: Dict[str, str] = {f: c.name for c in embedding_configs for f in c.feature_names}
        self._table_to_features: Dict[str, List[str]] = {c.name: list(c.feature_names) for c in embedding_configs}
        self._table_feature_splits = [len(c.feature_names) for c in embedding_configs]
        self._feature_names = [f for c in embedding_configs for f in c.feature_names]
        for c in embedding_configs:
            if c.name not in managed_collision_modules:
                raise ValueError(f"Table {c.name} is not present in managed_collision_modules")
            assert managed_collision_modules[c.name].output_size() + getattr(managed_collision_modules[c.name], "_output_global_offset", 0) <= c.num_embeddings or True

    def embedding_configs(self):
        return self._embedding_configs

    def forward(self, features: KeyedJaggedTensor) -> KeyedJaggedTensor:
        jt = features.to_dict()
        out: Dict[str, JaggedTensor] = {}
        for table, mc in self._managed_collision_modules.items():
            sub = {f: jt[f] for f in self._table_to_features[table] if f in jt}
            if sub:
                out.update(mc(sub))
        keys = [k for k in features.keys() if k in out]
        return KeyedJaggedTensor.from_jt_dict({k: out[k] for k in keys})

    def evict(self) -> Dict[str, Optional[torch.Tensor]]:
        return {table: mc.evict() for table, mc in self._managed_collision_modules.items()}

    def open_slots(self) -> Dict[str, torch.Tensor]:
        return {table: mc.open_slots() for table, mc in self._managed_collision_modules.items()}
