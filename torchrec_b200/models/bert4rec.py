"""BERT4Rec: a bidirectional transformer over a user's item sequence whose item embeddings come from an
``EmbeddingCollection`` (so they can be sharded column-/row-/table-wise), trained with masked-item prediction.

The jagged item sequences (a ``KeyedJaggedTensor``) are looked up unpooled, padded to ``max_len`` with the jagged-to-padded
kernel, combined with learned position embeddings and run through ``num_layers`` encoder blocks.  Two heads:

* ``BERT4Rec`` scores every position against the whole vocabulary with a dense projection (small vocabularies);
* ``BERT4RecSampled`` scores the masked positions against their target and a shared set of sampled negatives whose *output*
  embeddings are a second table of the same collection, looked up through the feature ``"cand"`` -- the output layer of a
  20M-item vocabulary is then as sparse as the input layer: no dense ``[vocab, D]`` gradient and a fused sparse optimizer.

Counterpart of ``examples/bert4rec/models/bert4rec.py`` of the reference.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.modules import jagged_transformer
from torchrec_b200.modules.embedding_configs import DataType, EmbeddingConfig
from torchrec_b200.modules.embedding_modules import EmbeddingCollection
from torchrec_b200.ops.transformer_ops import residual_layer_norm
from torchrec_b200.ops import dense_ops
from torchrec_b200.ops import sparse_ops as sops
from torchrec_b200.sparse.jagged_tensor import JaggedTensor, KeyedJaggedTensor


class HistoryArch(nn.Module):
    """Item + position embeddings of the padded history: ``KJT -> [B, max_len, D]``, the padding mask ``[B, max_len]`` and the
    looked-up jagged tensors of every feature."""

    def __init__(self, vocab_size: int, history_len: int, emb_dim: int, dropout: float = 0.1, device: Optional[torch.device] = None,
                 feature_name: str = "item", embedding_device: Optional[torch.device] = None, data_type: DataType = DataType.FP32,
                 output_table_feature: Optional[str] = None) -> None:
        super().__init__()
        self.emb_dim = emb_dim
        self.history_len = history_len
        self.feature_name = feature_name
        tables = [EmbeddingConfig(name="item_embedding", embedding_dim=emb_dim, num_embeddings=vocab_size, feature_names=[feature_name], data_type=data_type)]
        if output_table_feature is not None:
            tables.append(EmbeddingConfig(name="item_output_embedding", embedding_dim=emb_dim, num_embeddings=vocab_size, feature_names=[output_table_feature], data_type=data_type))
        self.ec = EmbeddingCollection(tables=tables, device=embedding_device if embedding_device is not None else device)
        self.positional = nn.Parameter(torch.randn(history_len, emb_dim, device=device if device is not None and device.type != "meta" else None) * 0.02)
        self.layernorm = nn.LayerNorm(emb_dim, device=device)
        self.dropout = nn.Dropout(p=dropout)

    def forward(self, id_list_features: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor, Dict[str, JaggedTensor]]:
        jt_dict = self.ec(id_list_features)
        if hasattr(jt_dict, "wait"):
            jt_dict = jt_dict.wait()
        jt: JaggedTensor = jt_dict[self.feature_name]
        padded = sops.jagged_to_padded_dense(jt.values(), jt.offsets(), self.history_len, 0.0)  # [B, L, D]
        lengths = jt.lengths().clamp(max=self.history_len)
        mask = torch.arange(self.history_len, device=padded.device).unsqueeze(0) < lengths.unsqueeze(1)
        x = padded + self.positional.unsqueeze(0).to(padded.dtype)
        return self.dropout(self.layernorm(x)), mask, jt_dict

    def forward_packed(self, id_list_features: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor, Dict[str, JaggedTensor]]:
        """The same embedding stage without padding: ``[T, D]`` rows of all histories back to back, their ``offsets [B + 1]``, and
        the looked-up jagged tensors.  Histories are expected to hold at most ``history_len`` items."""
        jt_dict = self.ec(id_list_features)
        if hasattr(jt_dict, "wait"):
            jt_dict = jt_dict.wait()
        jt: JaggedTensor = jt_dict[self.feature_name]
        rows, lengths, offsets = jt.values(), jt.lengths(), jt.offsets()
        T = rows.shape[0]
        first = torch.repeat_interleave(offsets[:-1].to(torch.int64), lengths.to(torch.int64), output_size=T)
        position = (torch.arange(T, device=rows.device) - first).clamp_(max=self.history_len - 1)
        if dense_ops.fused_dense_enabled(rows):  # the packed encoder keeps its activations in bf16 from here on
            rows = rows.to(torch.bfloat16)
        x = rows + self.positional.to(rows.dtype).index_select(0, position)
        _, y = residual_layer_norm(None, x.contiguous(), self.layernorm.weight, self.layernorm.bias, 0.0, self.training, self.layernorm.eps)
        return self.dropout(y), offsets, jt_dict


def _encoder(emb_dim: int, nhead: int, num_layers: int, dim_feedforward: Optional[int], dropout: float, device: Optional[torch.device]) -> nn.TransformerEncoder:
    layer = nn.TransformerEncoderLayer(d_model=emb_dim, nhead=nhead, dim_feedforward=dim_feedforward or 4 * emb_dim, dropout=dropout, activation="gelu",
                                       batch_first=True, norm_first=True, device=device)
    return nn.TransformerEncoder(layer, num_layers=num_layers, enable_nested_tensor=False)


def _packed_positions(positions: torch.Tensor, offsets: torch.Tensor, max_len: int) -> torch.Tensor:
    """Flat positions into the padded ``[B * max_len]`` layout -> row indices of the packed ``[T]`` layout."""
    sample = torch.div(positions, max_len, rounding_mode="floor")
    return offsets.to(torch.int64).index_select(0, sample) + (positions - sample * max_len)


class BERT4Rec(nn.Module):
    def __init__(self, vocab_size: int, max_len: int, emb_dim: int, nhead: int, num_layers: int, dim_feedforward: Optional[int] = None, dropout: float = 0.1,
                 device: Optional[torch.device] = None) -> None:
        super().__init__()
        self.vocab_size = vocab_size
        self.max_len = max_len
        self.history = HistoryArch(vocab_size, max_len, emb_dim, dropout, device)
        self.encoder = _encoder(emb_dim, nhead, num_layers, dim_feedforward, dropout, device)
        self.out = nn.Linear(emb_dim, vocab_size, device=device)

    def encode(self, input: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        x, mask, _ = self.history(input)
        h = self.encoder(x, src_key_padding_mask=~mask)
        return h, mask

    def encode_packed(self, input: KeyedJaggedTensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Hidden states of the real tokens only, ``[T, D]`` with the sequence ``offsets`` (no padding position is computed)."""
        x, offsets, _ = self.history.forward_packed(input)
        return jagged_transformer.jagged_encoder_forward(self.encoder, x, offsets, self.max_len), offsets

    def forward(self, input: KeyedJaggedTensor, positions: Optional[torch.Tensor] = None, targets: Optional[torch.Tensor] = None,
                negatives: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Logits ``[B, max_len, vocab]`` over the full vocabulary; with ``positions`` / ``targets`` / ``negatives`` the sampled
        scores of :meth:`sampled_logits` instead (through ``forward`` so that a data-parallel wrapper sees the call)."""
        if positions is not None:
            assert targets is not None and negatives is not None
            return self.sampled_logits(input, positions, targets, negatives)
        h, _ = self.encode(input)
        return self.out(h)

    def sampled_logits(self, input: KeyedJaggedTensor, positions: torch.Tensor, targets: torch.Tensor, negatives: torch.Tensor) -> torch.Tensor:
        """Scores of the hidden states at flat ``positions`` (into ``[B*max_len]``) against their target item and a shared set of
        sampled negatives: ``[P, 1 + N]`` (column 0 is the positive)."""
        if jagged_transformer.supports(self.encoder):
            h, offsets = self.encode_packed(input)
            hp = h.index_select(0, _packed_positions(positions, offsets, self.max_len)).to(self.out.weight.dtype)
        else:
            h, _ = self.encode(input)
            hp = h.reshape(-1, h.shape[-1]).index_select(0, positions)
        w = self.out.weight
        pos = (hp * w.index_select(0, targets)).sum(-1, keepdim=True) + self.out.bias.index_select(0, targets).unsqueeze(1)
        neg = hp @ w.index_select(0, negatives).t() + self.out.bias.index_select(0, negatives).unsqueeze(0)
        return torch.cat([pos, neg], dim=1)


class BERT4RecSampled(nn.Module):
    """Sampled-softmax BERT4Rec with a sparse output layer.

    ``forward(kjt, positions)``: ``kjt`` has the features ``"item"`` (the masked histories) and ``"cand"`` (sample 0 holds the ``P``
    target ids of the masked positions followed by the ``N`` shared negatives, the other samples are empty); ``positions [P]`` are
    the flat indices of the masked positions in ``[B * max_len]``.  Returns ``[P, 1 + N]`` scores, column 0 the positive; with
    ``loss=True`` the mean sampled-softmax cross entropy instead (the scores then never leave bf16 and are read once).
    """

    def __init__(self, vocab_size: int, max_len: int, emb_dim: int, nhead: int, num_layers: int, dim_feedforward: Optional[int] = None, dropout: float = 0.1,
                 device: Optional[torch.device] = None, embedding_device: Optional[torch.device] = None, data_type: DataType = DataType.FP32) -> None:
        super().__init__()
        self.vocab_size, self.max_len = vocab_size, max_len
        self.history = HistoryArch(vocab_size, max_len, emb_dim, dropout, device, embedding_device=embedding_device, data_type=data_type, output_table_feature="cand")
        self.encoder = _encoder(emb_dim, nhead, num_layers, dim_feedforward, dropout, device)
        self.packed = True  # run the encoder over the real tokens only (False: padded [B, max_len, D] through the library modules)

    @staticmethod
    def make_input(items: torch.Tensor, lengths: torch.Tensor, targets: torch.Tensor, negatives: torch.Tensor) -> KeyedJaggedTensor:
        B = lengths.numel()
        cand_len = torch.zeros(B, dtype=lengths.dtype)
        cand_len[0] = targets.numel() + negatives.numel()
        return KeyedJaggedTensor(keys=["item", "cand"], values=torch.cat([items, targets, negatives]), lengths=torch.cat([lengths, cand_len]), stride=B)

    def forward(self, input: KeyedJaggedTensor, positions: torch.Tensor, loss: bool = False) -> torch.Tensor:
        if self.packed and jagged_transformer.supports(self.encoder):
            x, offsets, jts = self.history.forward_packed(input)
            h = jagged_transformer.jagged_encoder_forward(self.encoder, x, offsets, self.max_len)
            hp = h.index_select(0, _packed_positions(positions, offsets, self.max_len))
        else:
            x, mask, jts = self.history(input)
            h = self.encoder(x, src_key_padding_mask=~mask)
            hp = h.reshape(-1, h.shape[-1]).index_select(0, positions)
        P = positions.numel()
        if loss:
            from torchrec_b200.ops.transformer_ops import sampled_softmax_loss

            cand = jts["cand"].values()
            return sampled_softmax_loss(hp, cand[:P], cand[P:])
        cand = jts["cand"].values().to(hp.dtype)
        pos = (hp * cand[:P]).sum(-1, keepdim=True)
        neg = hp @ cand[P:].t()
        return torch.cat([pos, neg], dim=1)
