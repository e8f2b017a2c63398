"""DLRM model family (counterpart of ``torchrec/models/dlrm.py:38-933``).

``DLRM`` (dot interaction), ``DLRM_Projection`` and ``DLRM_DCN`` (DCN-v2 low-rank cross
interaction), plus ``DLRMTrain`` which adds the BCE-with-logits loss.  Submodule and
parameter names match the reference so that checkpoints are interchangeable.  On CUDA in
bf16 dense mode the towers run through the fused tcgen05 layers of
``torchrec_b200.ops.dense_ops``; the math on CPU / fp32 is plain torch.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple, Union

import torch
from torch import nn

from torchrec_b200.datasets.utils import Batch
from torchrec_b200.modules.crossnet import LowRankCrossNet
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.mlp import MLP
from torchrec_b200.ops import dense_ops
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor


def choose(n: int, k: int) -> int:
    """Binomial coefficient."""
    if 0 <= k <= n:
        ntok, ktok = 1, 1
        for t in range(1, min(k, n - k) + 1):
            ntok *= n
            ktok *= t
            n -= 1
        return ntok // ktok
    return 0


class SparseArch(nn.Module):
    """EBC lookup reshaped to ``[B, F, D]`` in feature order."""

    def __init__(self, embedding_bag_collection: EmbeddingBagCollection) -> None:
        super().__init__()
        configs = embedding_bag_collection.embedding_bag_configs()
        assert configs, "Embedding bag collection cannot be empty!"
        self.embedding_bag_collection = embedding_bag_collection
        self._sparse_feature_names: List[str] = [feature for cfg in configs for feature in cfg.feature_names]
        self.F, self.D = len(self._sparse_feature_names), int(configs[0].embedding_dim)

    def forward(self, features: KeyedJaggedTensor) -> torch.Tensor:
        pooled: KeyedTensor = self.embedding_bag_collection(features)
        values = pooled.values()
        if pooled.keys() != self._sparse_feature_names:  # rare: put the blocks in feature order (one gathering copy)
            by_key = pooled.to_dict()
            values = torch.cat([by_key[name] for name in self._sparse_feature_names], dim=1)
        return values.reshape(-1, self.F, self.D)

    @property
    def sparse_feature_names(self) -> List[str]:
        return self._sparse_feature_names


class DenseArch(nn.Module):
    """Bottom MLP over the dense features."""

    def __init__(self, in_features: int, layer_sizes: List[int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.model: nn.Module = MLP(in_features, layer_sizes, bias=True, activation="relu", device=device)

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        return self.model(features)


class InteractionArch(nn.Module):
    """Pairwise dot products of the dense vector and all sparse embeddings -> ``[B, D + F + C(F,2)]``."""

    def __init__(self, num_sparse_features: int) -> None:
        super().__init__()
        self.F: int = num_sparse_features
        self.register_buffer(
            "triu_indices", torch.triu_indices(self.F + 1, self.F + 1, offset=1), persistent=False,
        )

    def forward(self, dense_features: torch.Tensor, sparse_features: torch.Tensor) -> torch.Tensor:
        if self.F <= 0:
            return dense_features
        return dense_ops.dot_interaction(dense_features, sparse_features)


def _dense_and_sparse_flat(dense_features: torch.Tensor, sparse_features: torch.Tensor) -> torch.Tensor:
    """``[B, D]`` and ``[B, F, D]`` side by side as one ``[B, (F + 1) * D]`` row per sample, dense block first."""
    return torch.cat((dense_features, sparse_features.to(dense_features.dtype).flatten(1)), dim=1)


class InteractionDCNArch(nn.Module):
    """Cross-network interaction over the flattened ``[dense, sparse]`` vector -> ``[B, (F+1)*D]``."""

    def __init__(self, num_sparse_features: int, crossnet: nn.Module) -> None:
        super().__init__()
        self.F: int = num_sparse_features
        self.crossnet = crossnet

    def forward(self, dense_features: torch.Tensor, sparse_features: torch.Tensor) -> torch.Tensor:
        return self.crossnet(_dense_and_sparse_flat(dense_features, sparse_features)) if self.F > 0 else dense_features


class InteractionProjectionArch(nn.Module):
    """Interaction between two learned projections of the features -> ``[B, D + F1*F2]``."""

    def __init__(self, num_sparse_features: int, interaction_branch1: nn.Module, interaction_branch2: nn.Module) -> None:
        super().__init__()
        self.F: int = num_sparse_features
        self.interaction_branch1 = interaction_branch1
        self.interaction_branch2 = interaction_branch2

    def forward(self, dense_features: torch.Tensor, sparse_features: torch.Tensor) -> torch.Tensor:
        if self.F <= 0:
            return dense_features
        B, D = dense_features.shape
        flat = _dense_and_sparse_flat(dense_features, sparse_features)
        left = self.interaction_branch1(flat).view(B, -1, D)    # [B, F1, D]
        right = self.interaction_branch2(flat).view(B, D, -1)   # [B, D, F2]
        pairwise = torch.bmm(left, right).flatten(1).to(dense_features.dtype)
        return torch.cat((dense_features, pairwise), dim=1)


class OverArch(nn.Module):
    """Top MLP; the last layer is a plain linear producing logits."""

    def __init__(self, in_features: int, layer_sizes: List[int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        if len(layer_sizes) <= 1:
            raise ValueError("OverArch must have multiple layers.")
        self.model: nn.Module = nn.Sequential(
            MLP(in_features, layer_sizes[:-1], bias=True, activation="relu", device=device),
            nn.Linear(layer_sizes[-2], layer_sizes[-1], bias=True, device=device),
        )

    def forward(self, features: torch.Tensor) -> torch.Tensor:
        h = self.model[0](features)
        last = self.model[1]
        if dense_ops.fused_dense_enabled(h):
            return dense_ops.linear_small_out(h, last.weight, last.bias)
        return last(h)


def _check_ebc(embedding_bag_collection, dense_arch_layer_sizes) -> int:
    cfgs = embedding_bag_collection.embedding_bag_configs()
    assert len(cfgs) > 0, "At least one embedding bag is required"
    for i in range(1, len(cfgs)):
        assert cfgs[i - 1].embedding_dim == cfgs[i].embedding_dim, "All EmbeddingBagConfigs must have the same dimension"
    embedding_dim = cfgs[0].embedding_dim
    if dense_arch_layer_sizes[-1] != embedding_dim:
        raise ValueError(
            f"embedding_bag_collection dimension ({embedding_dim}) and final dense "
            f"arch layer size ({dense_arch_layer_sizes[-1]}) must match."
        )
    return embedding_dim


class DLRM(nn.Module):
    """Deep Learning Recommendation Model with dot-product interaction."""

    def __init__(
        self,
        embedding_bag_collection: EmbeddingBagCollection,
        dense_in_features: int,
        dense_arch_layer_sizes: List[int],
        over_arch_layer_sizes: List[int],
        dense_device: Optional[torch.device] = None,
    ) -> None:
        super().__init__()
        embedding_dim = _check_ebc(embedding_bag_collection, dense_arch_layer_sizes)
        self.sparse_arch: SparseArch = SparseArch(embedding_bag_collection)
        num_sparse_features = len(self.sparse_arch.sparse_feature_names)
        self.dense_arch = DenseArch(dense_in_features, dense_arch_layer_sizes, device=dense_device)
        self.inter_arch = InteractionArch(num_sparse_features=num_sparse_features)
        over_in_features = embedding_dim + choose(num_sparse_features, 2) + num_sparse_features
        self.over_arch = OverArch(over_in_features, over_arch_layer_sizes, device=dense_device)

    def forward(self, dense_features: torch.Tensor, sparse_features: KeyedJaggedTensor) -> torch.Tensor:
        embedded_dense = self.dense_arch(dense_features)
        embedded_sparse = self.sparse_arch(sparse_features)
        concatenated_dense = self.inter_arch(dense_features=embedded_dense, sparse_features=embedded_sparse)
        return self.over_arch(concatenated_dense)


class DLRM_Projection(DLRM):
    """DLRM whose interaction is computed between two projected feature sets."""

    def __init__(
        self,
        embedding_bag_collection: EmbeddingBagCollection,
        dense_in_features: int,
        dense_arch_layer_sizes: List[int],
        over_arch_layer_sizes: List[int],
        interaction_branch1_layer_sizes: List[int],
        interaction_branch2_layer_sizes: List[int],
        dense_device: Optional[torch.device] = None,
    ) -> None:
        super().__init__(embedding_bag_collection, dense_in_features, dense_arch_layer_sizes, over_arch_layer_sizes, dense_device)
        embedding_dim = embedding_bag_collection.embedding_bag_configs()[0].embedding_dim
        num_sparse_features = len(self.sparse_arch.sparse_feature_names)
        if interaction_branch1_layer_sizes[-1] % embedding_dim != 0:
            raise ValueError(
                f"Final interaction branch1 layer size ({interaction_branch1_layer_sizes[-1]}) is not a multiple "
                f"of embedding size ({embedding_dim})"
            )
        projected_b1 = interaction_branch1_layer_sizes[-1] // embedding_dim
        if interaction_branch2_layer_sizes[-1] % embedding_dim != 0:
            raise ValueError(
                f"Final interaction branch2 layer size ({interaction_branch2_layer_sizes[-1]}) is not a multiple "
                f"of embedding size ({embedding_dim})"
            )
        projected_b2 = interaction_branch2_layer_sizes[-1] // embedding_dim
        self.inter_arch = InteractionProjectionArch(
            num_sparse_features=num_sparse_features,
            interaction_branch1=DenseArch((num_sparse_features + 1) * embedding_dim, interaction_branch1_layer_sizes, dense_device),
            interaction_branch2=DenseArch((num_sparse_features + 1) * embedding_dim, interaction_branch2_layer_sizes, dense_device),
        )
        self.over_arch = OverArch(embedding_dim + projected_b1 * projected_b2, over_arch_layer_sizes, device=dense_device)


class DLRM_DCN(DLRM):
    """DLRM with a DCN-v2 low-rank cross network as the interaction (the MLPerf DLRM-DCNv2 model)."""

    def __init__(
        self,
        embedding_bag_collection: EmbeddingBagCollection,
        dense_in_features: int,
        dense_arch_layer_sizes: List[int],
        over_arch_layer_sizes: List[int],
        dcn_num_layers: int,
        dcn_low_rank_dim: int,
        dense_device: Optional[torch.device] = None,
    ) -> None:
        super().__init__(embedding_bag_collection, dense_in_features, dense_arch_layer_sizes, over_arch_layer_sizes, dense_device)
        embedding_dim = embedding_bag_collection.embedding_bag_configs()[0].embedding_dim
        num_sparse_features = len(self.sparse_arch.sparse_feature_names)
        crossnet = LowRankCrossNet(
            in_features=(num_sparse_features + 1) * embedding_dim, num_layers=dcn_num_layers, low_rank=dcn_low_rank_dim,
        )
        if dense_device is not None:
            crossnet = crossnet.to(dense_device)
        self.inter_arch = InteractionDCNArch(num_sparse_features=num_sparse_features, crossnet=crossnet)
        self.over_arch = OverArch((num_sparse_features + 1) * embedding_dim, over_arch_layer_sizes, device=dense_device)


class DLRMTrain(nn.Module):
    """Training wrapper: ``forward(batch) -> (loss, (loss.detach(), logits.detach(), labels))``."""

    def __init__(self, dlrm_module: DLRM) -> None:
        super().__init__()
        self.model = dlrm_module
        self.loss_fn: nn.Module = nn.BCEWithLogitsLoss()

    def forward(self, batch: Batch) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
        logits = self.model(batch.dense_features, batch.sparse_features)
        logits = logits.squeeze(-1)
        if logits.is_cuda and type(self.loss_fn) is nn.BCEWithLogitsLoss and self.loss_fn.weight is None and self.loss_fn.pos_weight is None and self.loss_fn.reduction == "mean":
            loss = dense_ops.bce_with_logits_mean(logits, batch.labels)  # loss and its gradient in one kernel
        else:
            loss = self.loss_fn(logits.float(), batch.labels.float())
        return loss, (loss.detach(), logits.detach(), batch.labels.detach())


class DLRMWrapper(DLRM):
    """DLRM taking a ``ModelInput``-like object (``float_features``, ``idlist_features``, ``label``)."""

    def forward(self, model_input) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:  # type: ignore[override]
        pred = super().forward(dense_features=model_input.float_features, sparse_features=model_input.idlist_features)
        if self.training:
            loss = torch.nn.functional.binary_cross_entropy_with_logits(pred.squeeze().float(), model_input.label.float())
            return (loss, pred)
        return pred
