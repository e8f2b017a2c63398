"""Eviction scoring for the multi-probe zero-collision hash.

A policy turns a feature's ids into the score written beside every id that is stored or seen again, and the threshold below
which a stored id may be replaced: with time-to-live policies the score is the hour at which the id expires and the threshold
is the current hour; with LRU the score is the current hour and the oldest probed slot loses.
Counterpart of ``torchrec/modules/hash_mc_evictions.py`` (policies ``:23``, scorers ``:54-108``, module ``:219``).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from enum import Enum, unique
from typing import List, Optional, Tuple

import torch

from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import JaggedTensor


@unique
class HashZchEvictionPolicyName(Enum):
    SINGLE_TTL_EVICTION = "SINGLE_TTL_EVICTION"
    PER_FEATURE_TTL_EVICTION = "PER_FEATURE_TTL_EVICTION"
    LRU_EVICTION = "LRU_EVICTION"


@dataclass
class HashZchEvictionConfig:
    features: List[str]
    single_ttl: Optional[int] = None
    per_feature_ttl: Optional[List[int]] = None


def get_kernel_from_policy(policy_name: Optional[HashZchEvictionPolicyName]) -> int:
    """Policy code of the probe kernel."""
    if policy_name is None:
        return sops.ZCH_NO_EVICT
    return sops.ZCH_LRU if policy_name == HashZchEvictionPolicyName.LRU_EVICTION else sops.ZCH_TTL


def current_hour() -> int:
    return int(time.time() / 3600)


class HashZchEvictionScorer:
    def __init__(self, config: HashZchEvictionConfig) -> None:
        self._config = config

    def gen_score(self, feature: JaggedTensor, device: torch.device) -> torch.Tensor:
        raise NotImplementedError

    def gen_threshold(self) -> int:
        return current_hour()


class HashZchSingleTtlScorer(HashZchEvictionScorer):
    def gen_score(self, feature: JaggedTensor, device: torch.device) -> torch.Tensor:
        ttl = self._config.single_ttl
        assert ttl is not None and ttl > 0, "SINGLE_TTL_EVICTION needs a positive single_ttl"
        return torch.full_like(feature.values(), ttl + current_hour(), dtype=torch.int32, device=device)


class HashZchPerFeatureTtlScorer(HashZchEvictionScorer):
    """The jagged tensor holds the features of one table back to back; ``feature.weights()`` is not used, the split per
    feature comes from ``feature.lengths()`` laid out ``[F, B]``."""

    def __init__(self, config: HashZchEvictionConfig) -> None:
        super().__init__(config)
        ttls = config.per_feature_ttl
        assert ttls is not None and len(ttls) == len(config.features), "PER_FEATURE_TTL_EVICTION needs one ttl per feature"
        self._per_feature_ttl = torch.tensor(ttls, dtype=torch.int32)

    def gen_score(self, feature: JaggedTensor, device: torch.device) -> torch.Tensor:
        F = self._per_feature_ttl.numel()
        per_feature = feature.lengths().view(F, -1).sum(dim=1)
        return (self._per_feature_ttl.to(device).repeat_interleave(per_feature.to(device)) + current_hour()).to(torch.int32)


class HashZchLruScorer(HashZchEvictionScorer):
    def gen_score(self, feature: JaggedTensor, device: torch.device) -> torch.Tensor:
        return torch.full_like(feature.values(), current_hour(), dtype=torch.int32, device=device)

    def gen_threshold(self) -> int:
        return -1  # the kernel compares the probed slots with each other


def get_eviction_scorer(policy_name: HashZchEvictionPolicyName, config: HashZchEvictionConfig) -> HashZchEvictionScorer:
    if policy_name == HashZchEvictionPolicyName.SINGLE_TTL_EVICTION:
        return HashZchSingleTtlScorer(config)
    if policy_name == HashZchEvictionPolicyName.PER_FEATURE_TTL_EVICTION:
        return HashZchPerFeatureTtlScorer(config)
    if policy_name == HashZchEvictionPolicyName.LRU_EVICTION:
        return HashZchLruScorer(config)
    raise ValueError(f"unsupported eviction policy {policy_name}")


_SCORED_POLICIES = (HashZchEvictionPolicyName.SINGLE_TTL_EVICTION, HashZchEvictionPolicyName.PER_FEATURE_TTL_EVICTION, HashZchEvictionPolicyName.LRU_EVICTION)


class HashZchThresholdEvictionModule(torch.nn.Module):
    """Policies that score every id (expiry hour or last access) and give the lookup a threshold below which a slot may be taken over:
    ``forward(feature, device) -> (score per id, threshold)``."""

    def __init__(self, policy_name: HashZchEvictionPolicyName, config: HashZchEvictionConfig) -> None:
        super().__init__()
        self._policy_name, self._config = policy_name, config
        self._eviction_scorer = get_eviction_scorer(policy_name, config)

    def forward(self, feature: JaggedTensor, device: torch.device) -> Tuple[torch.Tensor, int]:
        return self._eviction_scorer.gen_score(feature, device), self._eviction_scorer.gen_threshold()


class HashZchOptEvictionModule(torch.nn.Module):
    """A policy that needs no per-id score (slots are only claimed while free): ``forward -> (None, -1)``."""

    def __init__(self, policy_name: HashZchEvictionPolicyName) -> None:
        super().__init__()
        self._policy_name = policy_name

    def forward(self, feature: JaggedTensor, device: torch.device) -> Tuple[None, int]:
        return None, -1


def get_eviction_module(policy_name: HashZchEvictionPolicyName, config: Optional[HashZchEvictionConfig]) -> torch.nn.Module:
    if policy_name in _SCORED_POLICIES:
        assert config is not None, "a scored eviction policy needs its config"
        return HashZchThresholdEvictionModule(policy_name, config)
    return HashZchOptEvictionModule(policy_name)


class HashZchEvictionModule(torch.nn.Module):
    """``forward(feature) -> (score per id or None, threshold or -1)`` of the configured policy, on the module's device."""

    def __init__(self, policy_name: HashZchEvictionPolicyName, device: torch.device, config: Optional[HashZchEvictionConfig]) -> None:
        super().__init__()
        self._policy_name = policy_name
        self._device = device
        self._eviction_module = get_eviction_module(policy_name, config)

    def forward(self, feature: JaggedTensor) -> Tuple[Optional[torch.Tensor], int]:
        return self._eviction_module(feature, self._device)
