"""BERT4Rec: a bidirectional transformer over a user's item sequence whose item embeddings come from an
``EmbeddingCollection`` (so they can be sharded column-/row-/table-wise), trained with masked-item prediction.

The jagged item sequences (a ``KeyedJaggedTensor`` with one feature) are looked up unpooled, padded to ``max_len`` with the
jagged-to-padded kernel, combined with learned position embeddings and run through ``num_layers`` encoder blocks; the output
layer scores every position against the vocabulary (or against sampled negatives for large vocabularies).
Counterpart of ``examples/bert4rec/models/bert4rec.py`` of the reference.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from torchrec_b200.modules.embedding_configs import EmbeddingConfig
from torchrec_b200.modules.embedding_modules import EmbeddingCollection
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


class HistoryArch(nn.Module):
    """Item + position embeddings of the padded history: ``KJT -> [B, max_len, D]`` and the padding mask ``[B, max_len]``."""

    def __init__(self, vocab_size: int, history_len: int, emb_dim: int, dropout: float = 0.1, device: Optional[torch.device] = None,
                 feature_name: str = "item") -> None:
        super().__init__()
        self.emb_dim = emb_dim
        self.history_len = history_len
        self.feature_name = feature_name
        self.ec = EmbeddingCollection(tables=[EmbeddingConfig(name="item_embedding", embedding_dim=emb_dim, num_embeddings=vocab_size, feature_names=[feature_name])], device=device)
        self.positional = nn.Parameter(torch.randn(history_len, emb_dim, device=device if device is not None and device.type != "meta" else None) * 0.02)
        self.layernorm = nn.LayerNorm(emb_dim)
        self.dropout = nn.Dropout(p=dropout)

    def forward(self, id_list_features: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        jt_dict = self.ec(id_list_features)
        if hasattr(jt_dict, "wait"):
            jt_dict = jt_dict.wait()
        jt: JaggedTensor = jt_dict[self.feature_name]
        padded = sops.jagged_to_padded_dense(jt.values(), jt.offsets(), self.history_len, 0.0)  # [B, L, D]
        lengths = jt.lengths().clamp(max=self.history_len)
        mask = torch.arange(self.history_len, device=padded.device).unsqueeze(0) < lengths.unsqueeze(1)
        x = padded + self.positional.unsqueeze(0).to(padded.dtype)
        return self.dropout(self.layernorm(x)), mask


class BERT4Rec(nn.Module):
    def __init__(self, vocab_size: int, max_len: int, emb_dim: int, nhead: int, num_layers: int, dim_feedforward: Optional[int] = None, dropout: float = 0.1,
                 device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.vocab_size = vocab_size
        self.max_len = max_len
        self.history = HistoryArch(vocab_size, max_len, emb_dim, dropout, device)
        layer = nn.TransformerEncoderLayer(d_model=emb_dim, nhead=nhead, dim_feedforward=dim_feedforward or 4 * emb_dim, dropout=dropout, activation="gelu",
                                           batch_first=True, norm_first=True)
        self.encoder = nn.TransformerEncoder(layer, num_layers=num_layers, enable_nested_tensor=False)
        self.out = nn.Linear(emb_dim, vocab_size)

    def encode(self, input: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x, mask = self.history(input)
        h = self.encoder(x, src_key_padding_mask=~mask)
        return h, mask

    def forward(self, input: KeyedJaggedTensor) -> torch.Tensor:
        """Logits ``[B, max_len, vocab]`` over the full vocabulary."""
        h, _ = self.encode(input)
        return self.out(h)

    def sampled_logits(self, input: KeyedJaggedTensor, positions: torch.Tensor, targets: torch.Tensor, negatives: torch.Tensor) -> torch.Tensor:
        """Scores of the hidden states at flat ``positions`` (into ``[B*max_len]``) against their target item and a shared set of
        sampled negatives: ``[P, 1 + N]`` (column 0 is the positive)."""
        h, _ = self.encode(input)
        hp = h.reshape(-1, h.shape[-1]).index_select(0, positions)
        w = self.out.weight
        pos = (hp * w.index_select(0, targets)).sum(-1, keepdim=True) + self.out.bias.index_select(0, targets).unsqueeze(1)
        neg = hp @ w.index_select(0, negatives).t() + self.out.bias.index_select(0, negatives).unsqueeze(0)
        return torch.cat([pos, neg], dim=1)
