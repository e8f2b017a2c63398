"""Table-set generator for tests and benchmarks: ``N`` unweighted and ``M`` weighted single-feature tables of one width, plus extra
tables given as plain dictionaries (``torchrec/distributed/test_utils/test_tables.py:17-100``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List

from torchrec_b200.modules.embedding_configs import EmbeddingBagConfig


def _rows(i: int) -> int:
    return max(i + 1, 100) * 1000


@dataclass
class EmbeddingTablesConfig:
    __test__ = False
    num_unweighted_features: int = 100
    num_weighted_features: int = 100
    embedding_feature_dim: int = 128
    # additional_tables[g] is a list of EmbeddingBagConfig keyword dictionaries for group g: group 0 extends the unweighted
    # tables, group 1 the weighted ones, later groups are returned as further lists
    additional_tables: List[List[Dict[str, Any]]] = field(default_factory=list)

    def generate_tables(self) -> List[List[EmbeddingBagConfig]]:
        """``[unweighted tables, weighted tables, *extra groups]``; table ``i`` has ``max(i + 1, 100) * 1000`` rows."""
        groups: List[List[EmbeddingBagConfig]] = [
            [EmbeddingBagConfig(num_embeddings=_rows(i), embedding_dim=self.embedding_feature_dim, name=f"table_{i}", feature_names=[f"feature_{i}"])
             for i in range(self.num_unweighted_features)],
            [EmbeddingBagConfig(num_embeddings=_rows(i), embedding_dim=self.embedding_feature_dim, name=f"weighted_table_{i}", feature_names=[f"weighted_feature_{i}"])
             for i in range(self.num_weighted_features)],
        ]
        for g, extra in enumerate(self.additional_tables):
            while len(groups) <= g:
                groups.append([])
            groups[g].extend(EmbeddingBagConfig(**kw) for kw in extra)
        return groups
