"""Two-tower retrieval model: a query tower and a candidate tower, each an embedding lookup followed by an MLP, trained so that
the dot product of the two tower outputs predicts the label; at serving time the candidate side becomes a top-k search over the
item embeddings (brute force on the device here: one GEMM against the whole item matrix, which a B200 does for tens of millions
of items in milliseconds; an approximate index can replace ``TopKIndex``).
Counterpart of ``examples/retrieval/modules/two_tower.py`` of the reference."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.mlp import MLP
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor


class TwoTower(nn.Module):
    """``embedding_bag_collection`` holds exactly two tables: the first is the query side, the second the candidate side."""

    def __init__(self, embedding_bag_collection: EmbeddingBagCollection, layer_sizes: List[int], device: Optional[torch.device] = None) -> None:
        super().__init__()
        cfgs = embedding_bag_collection.embedding_bag_configs()
        assert len(cfgs) == 2, "expected two embedding tables (query, candidate)"
        assert cfgs[0].embedding_dim == cfgs[1].embedding_dim, "both towers must share the embedding dimension"
        self._feature_names_query: List[str] = list(cfgs[0].feature_names)
        self._candidate_feature_names: List[str] = list(cfgs[1].feature_names)
        self.ebc = embedding_bag_collection
        dim = cfgs[0].embedding_dim
        # the last layer is linear: a ReLU there would make every score non-negative and the towers collapse to zero
        # under mostly-negative labels

        def tower(in_size: int) -> nn.Module:
            if len(layer_sizes) == 1:
                return nn.Linear(in_size, layer_sizes[0], device=device)
            return nn.Sequential(MLP(in_size=in_size, layer_sizes=layer_sizes[:-1], device=device), nn.Linear(layer_sizes[-2], layer_sizes[-1], device=device))

        self.query_proj = tower(dim * len(self._feature_names_query))
        self.candidate_proj = tower(dim * len(self._candidate_feature_names))

    def forward(self, kjt: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        pooled = self.ebc(kjt)
        if hasattr(pooled, "wait"):
            pooled = pooled.wait()
        q = self.query_proj(torch.cat([pooled[f] for f in self._feature_names_query], dim=1))
        c = self.candidate_proj(torch.cat([pooled[f] for f in self._candidate_feature_names], dim=1))
        return q, c


class TwoTowerTrainTask(nn.Module):
    def __init__(self, two_tower: TwoTower) -> None:
        super().__init__()
        self.two_tower = two_tower
        self.loss_fn = nn.BCEWithLogitsLoss()
        # a learned offset absorbs the base rate of the labels
        self.bias = nn.Parameter(torch.zeros(1))

    def forward(self, batch) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
        q, c = self.two_tower(batch.sparse_features)
        logits = (q * c).sum(dim=1) + self.bias
        loss = self.loss_fn(logits, batch.labels.float())
        return loss, (loss.detach(), logits.detach(), batch.labels.detach())


class TopKIndex(nn.Module):
    """Exact maximum-inner-product search over ``item_embeddings [N, D]`` by one matrix product per query batch."""

    def __init__(self, item_embeddings: torch.Tensor) -> None:
        super().__init__()
        self.register_buffer("items", item_embeddings)

    def forward(self, queries: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
        scores = queries.to(self.items.dtype) @ self.items.t()
        top = torch.topk(scores, k=min(k, self.items.shape[0]), dim=1)
        return top.values, top.indices


class TwoTowerRetrieval(nn.Module):
    """Serving form: the query tower plus an index over the projected candidate embeddings of every item."""

    def __init__(self, two_tower: TwoTower, num_items: int, k: int = 10, batch: int = 65536) -> None:
        super().__init__()
        self.two_tower = two_tower
        self.k = k
        feature = two_tower._candidate_feature_names[0]
        cand_table = [c for c in two_tower.ebc.embedding_bag_configs() if feature in c.feature_names][0]
        weight = two_tower.ebc.embedding_bags[cand_table.name].weight
        chunks = []
        with torch.no_grad():
            for lo in range(0, num_items, batch):
                chunks.append(two_tower.candidate_proj(weight[lo: min(lo + batch, num_items)]))
        self.index = TopKIndex(torch.cat(chunks))
        # the query side alone: a collection over the query table that shares its weights
        q_cfgs = [c for c in two_tower.ebc.embedding_bag_configs() if any(f in c.feature_names for f in two_tower._feature_names_query)]
        self.query_ebc = EmbeddingBagCollection(tables=q_cfgs, device=weight.device)
        for c in q_cfgs:
            self.query_ebc.embedding_bags[c.name].weight = two_tower.ebc.embedding_bags[c.name].weight

    @torch.no_grad()
    def forward(self, query_kjt: KeyedJaggedTensor) -> torch.Tensor:
        pooled = self.query_ebc(query_kjt)
        q = self.two_tower.query_proj(torch.cat([pooled[f] for f in self.two_tower._feature_names_query], dim=1))
        return self.index(q, self.k)[1]
