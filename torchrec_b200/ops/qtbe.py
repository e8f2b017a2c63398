"""Quantized table-batched embedding lookup for inference: several row-wise quantized tables in one byte buffer, one
kernel launch per lookup (CUDA: ``qtbe_forward``; CPU: dequantize + ``embedding_bag``, which is also the test oracle)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.modules.embedding_configs import PoolingMode
from torchrec_b200.ops import _ext
from torchrec_b200.ops.quant_ops import dequantize_rowwise_nbit, row_bytes

_OUT_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


class QuantTableBatchedEmbeddingBags(nn.Module):
    """``embedding_specs``: ``(rows, dim, bits)`` per table, bits in {32, 16, 8, 4, 2}."""

    def __init__(self, embedding_specs: List[Tuple[int, int, int]], feature_table_map: Optional[List[int]] = None,
                 pooling_mode: PoolingMode = PoolingMode.SUM, output_dtype: torch.dtype = torch.float32, device: Optional[torch.device] = None,
                 persistent_weights: bool = True) -> None:
        super().__init__()
        self.embedding_specs = [(int(r), int(d), int(b)) for r, d, b in embedding_specs]
        T = len(self.embedding_specs)
        self.feature_table_map = list(feature_table_map) if feature_table_map is not None else list(range(T))
        self.pooling_mode = PoolingMode(int(pooling_mode))
        self.output_dtype = output_dtype
        for _, d, b in self.embedding_specs:
            need = {32: 4, 16: 4, 8: 4, 4: 8, 2: 16}[b]
            assert d % need == 0, f"dim {d} must be a multiple of {need} for {b}-bit rows"
        self.max_D = max([d for _, d, _ in self.embedding_specs], default=4)
        self.weights_offsets: List[int] = []
        off = 0
        for r, d, b in self.embedding_specs:
            off = (off + 15) // 16 * 16  # tables start on 16-byte boundaries
            self.weights_offsets.append(off)
            off += r * row_bytes(d, b)
        self.total_bytes = off
        self.D_offsets = [0]
        for t in self.feature_table_map:
            self.D_offsets.append(self.D_offsets[-1] + self.embedding_specs[t][1])
        self.total_D = self.D_offsets[-1]
        # a collection that exposes per-table views of this buffer in its own state dict passes persistent_weights=False
        self.register_buffer("weights", torch.zeros(max(self.total_bytes, 16), dtype=torch.uint8, device=device), persistent=persistent_weights)
        self._meta: Optional[torch.Tensor] = None
        self._err: Optional[torch.Tensor] = None
        # all tables int8 or all int4 with one dim whose payload is 16 bytes x a power of two: the kernel shares a warp's lanes
        # out over several rows per load instruction
        self._uniform_bits = 0
        formats = {(d, b) for _, d, b in self.embedding_specs}
        if len(formats) == 1:
            d, b = next(iter(formats))
            lanes = d * b // 8 // 16
            if b in (8, 4) and (d * b // 8) % 16 == 0 and lanes in ((2, 4, 8, 16) if b == 8 else (1, 2, 4, 8)):
                self._uniform_bits = b

    def table_view(self, t: int) -> torch.Tensor:
        """uint8 ``[rows, row_bytes]`` view of table ``t`` inside the flat buffer."""
        r, d, b = self.embedding_specs[t]
        rb = row_bytes(d, b)
        return self.weights[self.weights_offsets[t]: self.weights_offsets[t] + r * rb].view(r, rb)

    def split_embedding_weights(self) -> List[torch.Tensor]:
        return [self.table_view(t) for t in range(len(self.embedding_specs))]

    def _meta_tensor(self, device: torch.device) -> torch.Tensor:
        if self._meta is None or self._meta.device != device:
            ftm = self.feature_table_map
            rows = [[self.weights_offsets[t] for t in ftm], [self.embedding_specs[t][0] for t in ftm], [self.embedding_specs[t][1] for t in ftm],
                    self.D_offsets[:-1], [self.embedding_specs[t][2] for t in ftm]]
            self._meta = torch.tensor(rows, dtype=torch.int64).reshape(5, len(ftm)).to(device)
            self._err = torch.zeros(1, dtype=torch.int32, device=device)
        return self._meta

    def forward(self, indices: torch.Tensor, offsets: torch.Tensor, per_sample_weights: Optional[torch.Tensor] = None) -> torch.Tensor:
        F = len(self.feature_table_map)
        B = (offsets.numel() - 1) // F if F else 0
        if self.weights.is_cuda:
            _ext.require_cuda_ext("qtbe_forward")
            meta = self._meta_tensor(self.weights.device)
            if indices.dtype != offsets.dtype:
                offsets = offsets.to(indices.dtype)
            psw = per_sample_weights.float() if per_sample_weights is not None else None
            return torch.ops.trb200.qtbe_forward(self.weights, meta, indices.contiguous(), offsets.contiguous(), psw, B, self.total_D, self.max_D,
                                                 int(self.pooling_mode), _OUT_CODE[self.output_dtype], self._err, self._uniform_bits)
        return self._forward_cpu(indices, offsets, per_sample_weights, B)

    def forward_into(self, indices: torch.Tensor, offsets: torch.Tensor, per_sample_weights: Optional[torch.Tensor], out: torch.Tensor,
                     cols: List[int]) -> None:
        """Pooled lookup stored into ``out[:, cols[f] : cols[f] + dim_f]`` for every feature ``f``.  ``out`` may sit on another CUDA
        device of this process (peer stores over NVLink); on CPU it is a plain slice assignment."""
        F = len(self.feature_table_map)
        assert len(cols) == F and self.pooling_mode != PoolingMode.NONE
        # the kernel stores four elements at a time: every destination column must keep those stores aligned
        if any(int(c) % 4 for c in cols) or out.stride(0) % 4:
            raise ValueError(f"output columns {list(cols)} and row stride {out.stride(0)} must be multiples of 4 elements")
        B = (offsets.numel() - 1) // F if F else 0
        if not self.weights.is_cuda:
            res = self._forward_cpu(indices, offsets, per_sample_weights, B)
            for f, c in enumerate(cols):
                out[:B, c: c + self.D_offsets[f + 1] - self.D_offsets[f]] = res[:, self.D_offsets[f]: self.D_offsets[f + 1]].to(out.dtype)
            return
        _ext.require_cuda_ext("qtbe_forward_into")
        key = tuple(int(c) for c in cols)
        cache = self.__dict__.setdefault("_meta_into", {})
        if key not in cache:
            m = self._meta_tensor(self.weights.device).clone()
            m[3] = torch.tensor(key, dtype=m.dtype, device=m.device)
            cache[key] = m
        if indices.dtype != offsets.dtype:
            offsets = offsets.to(indices.dtype)
        psw = per_sample_weights.float() if per_sample_weights is not None else None
        torch.ops.trb200.qtbe_forward_into(self.weights, cache[key], indices.contiguous(), offsets.contiguous(), psw, out, B, self.max_D,
                                           int(self.pooling_mode), self._err, self._uniform_bits)

    def _forward_cpu(self, indices, offsets, psw, B) -> torch.Tensor:
        off = offsets.to(torch.int64)
        idx = indices.to(torch.int64)
        F = len(self.feature_table_map)
        tables = [dequantize_rowwise_nbit(self.table_view(t), d, b) for t, (r, d, b) in enumerate(self.embedding_specs)]
        if self.pooling_mode == PoolingMode.NONE:
            outs = []
            for f in range(F):
                s, e = int(off[f * B]), int(off[(f + 1) * B])
                outs.append(tables[self.feature_table_map[f]].index_select(0, idx[s:e]))
            res = torch.cat(outs, 0) if outs else torch.zeros(0, self.max_D)
            return res.to(self.output_dtype)
        out = torch.zeros(B, self.total_D, dtype=torch.float32)
        for f in range(F):
            o = off[f * B: (f + 1) * B + 1]
            s, e = int(o[0]), int(o[-1])
            if e > s:
                res = torch.nn.functional.embedding_bag(idx[s:e], tables[self.feature_table_map[f]], o[:-1] - s, mode="sum",
                                                        per_sample_weights=None if psw is None else psw[s:e].float())
                if self.pooling_mode == PoolingMode.MEAN:
                    res = res / (o[1:] - o[:-1]).clamp(min=1).unsqueeze(1).float()
                out[:, self.D_offsets[f]: self.D_offsets[f + 1]] = res
        return out.to(self.output_dtype)

    def check_error(self) -> None:
        if self._err is not None and int(self._err.item()) != 0:
            self._err.zero_()
            raise IndexError("quantized embedding lookup received an id outside its table")
