"""Table-batched embedding (TBE) modules.

One module holds several embedding tables in ONE flat weight buffer and looks all of them
up with one kernel launch.  The backward pass never produces a weight gradient: it sorts
the ids, reduces the upstream gradient rows per table row and applies the optimizer in
place (``tbe_kernels.cu``).  The same class runs on CPU with plain torch math, which is
both the gloo path and the oracle for the kernels.

Role of ``SplitTableBatchedEmbeddingBagsCodegen`` / ``DenseTableBatchedEmbeddingBagsCodegen``
as used by the reference (``torchrec/distributed/batched_embedding_kernel.py:3168-3323``);
optimizer semantics follow ``torchrec/optim/rowwise_adagrad.py:196-232`` for row-wise Adagrad
and ``torch.optim`` for the others.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from torchrec_b200.modules.embedding_configs import PoolingMode
from . import _ext


class EmbOptimType(enum.Enum):
    SGD = "sgd"
    EXACT_SGD = "exact_sgd"
    LAMB = "lamb"
    ADAM = "adam"
    EXACT_ADAGRAD = "exact_adagrad"
    EXACT_ROWWISE_ADAGRAD = "exact_row_wise_adagrad"
    LARS_SGD = "lars_sgd"
    PARTIAL_ROWWISE_ADAM = "partial_row_wise_adam"
    PARTIAL_ROWWISE_LAMB = "partial_row_wise_lamb"
    NONE = "none"

    def __str__(self) -> str:
        return self.value


_OPT_CODE = {
    EmbOptimType.SGD: 0, EmbOptimType.EXACT_SGD: 0,
    EmbOptimType.EXACT_ROWWISE_ADAGRAD: 1,
    EmbOptimType.EXACT_ADAGRAD: 2,
    EmbOptimType.ADAM: 3,
    EmbOptimType.PARTIAL_ROWWISE_ADAM: 4,
    EmbOptimType.LARS_SGD: 5,
    EmbOptimType.LAMB: 6,
    EmbOptimType.PARTIAL_ROWWISE_LAMB: 7,
}
OPT_DENSE_GRAD = 100

_OUT_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

# which state tensors an optimizer keeps: (momentum1 kind, momentum2 kind); kind in {None,"row","elem"}
_STATE_KINDS = {
    EmbOptimType.SGD: (None, None), EmbOptimType.EXACT_SGD: (None, None), EmbOptimType.LARS_SGD: (None, None),
    EmbOptimType.EXACT_ROWWISE_ADAGRAD: ("row", None),
    EmbOptimType.EXACT_ADAGRAD: ("elem", None),
    EmbOptimType.ADAM: ("elem", "elem"), EmbOptimType.LAMB: ("elem", "elem"),
    EmbOptimType.PARTIAL_ROWWISE_ADAM: ("elem", "row"), EmbOptimType.PARTIAL_ROWWISE_LAMB: ("elem", "row"),
    EmbOptimType.NONE: (None, None),
}


@dataclass
class OptimizerArgs:
    optimizer: EmbOptimType = EmbOptimType.EXACT_SGD
    learning_rate: float = 0.01
    eps: float = 1.0e-8
    beta1: float = 0.9
    beta2: float = 0.999
    weight_decay: float = 0.0
    eta: float = 0.001  # LARS trust coefficient
    max_gradient: float = 0.0  # > 0 clamps the summed row gradient elementwise
    stochastic_rounding: bool = True  # fp16 / bf16 tables only: unbiased random rounding of the updated weights


class TBEPlan:
    """Sorted (row -> contributing bags) plan of one batch; built from ids only.  ``ready`` is set when the plan was built on a
    side stream: the consumer's stream waits for it before the backward kernels read the plan."""

    __slots__ = ("keys", "src", "w", "src_feature", "bag_scale", "n_valid", "ready")

    def __init__(self, tensors: List[torch.Tensor]) -> None:
        self.keys, self.src, self.w, self.src_feature, self.bag_scale = tensors[:5]
        # padded plans (ids in a fixed-capacity buffer): number of real entries, kept on the device
        self.n_valid: Optional[torch.Tensor] = tensors[5] if len(tensors) > 5 else None
        self.ready = None

    def wait(self) -> None:
        if self.ready is not None:
            torch.cuda.current_stream().wait_event(self.ready)
            self.ready = None


# The id sort of the backward depends on the ids only.  It is memory-bound while the dense towers that run between an embedding
# forward and its backward are tensor-core-bound, so it is issued on a side stream right after the forward lookup and overlaps them.
_PLAN_AHEAD = os.environ.get("TRB200_PLAN_AHEAD", "1") != "0"
# "kernel": the sm_100a kernels (the product).  "torch": the composite torch implementation on the device as well -- gather,
# ``embedding_bag``, ``unique`` + ``index_add`` and the optimizer written out in torch ops -- which is what a framework without
# its own embedding kernels runs; benchmarks use it as the plain-library baseline.
_TBE_BACKEND = os.environ.get("TRB200_TBE", "kernel")


def set_tbe_backend(name: str) -> None:
    global _TBE_BACKEND
    assert name in ("kernel", "torch")
    _TBE_BACKEND = name


def get_tbe_backend() -> str:
    return _TBE_BACKEND
_plan_streams: Dict[int, "torch.cuda.Stream"] = {}


def _plan_stream(device: torch.device) -> "torch.cuda.Stream":
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _plan_streams.get(idx)
    if s is None:
        s = _plan_streams[idx] = torch.cuda.Stream(device=device)
    return s


def _apply_rows_cpu(
    opt: OptimizerArgs, step: int, w_rows: torch.Tensor, g: torch.Tensor,
    m1: Optional[torch.Tensor], m2: Optional[torch.Tensor],
) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Reference optimizer math on the touched rows (fp32).  Returns new (w, m1, m2)."""
    o = opt.optimizer
    lr, eps, b1, b2, wd = opt.learning_rate, opt.eps, opt.beta1, opt.beta2, opt.weight_decay
    if opt.max_gradient > 0:
        g = g.clamp(-opt.max_gradient, opt.max_gradient)
    lamb = o in (EmbOptimType.LAMB, EmbOptimType.PARTIAL_ROWWISE_LAMB)
    if wd != 0 and not lamb:
        g = g + wd * w_rows
    if o in (EmbOptimType.SGD, EmbOptimType.EXACT_SGD):
        return w_rows - lr * g, m1, m2
    if o == EmbOptimType.LARS_SGD:
        wn, gn = w_rows.norm(dim=1, keepdim=True), g.norm(dim=1, keepdim=True)
        trust = torch.where((wn > 0) & (gn > 0), opt.eta * wn / gn.clamp(min=1e-30), torch.ones_like(wn))
        return w_rows - lr * trust * g, m1, m2
    if o == EmbOptimType.EXACT_ROWWISE_ADAGRAD:
        m1 = m1 + g.pow(2).mean(dim=1)
        return w_rows - lr * g / (m1.sqrt() + eps).unsqueeze(1), m1, m2
    if o == EmbOptimType.EXACT_ADAGRAD:
        m1 = m1 + g * g
        return w_rows - lr * g / (m1.sqrt() + eps), m1, m2
    bc1, bc2 = 1 - b1 ** max(step, 1), 1 - b2 ** max(step, 1)
    m1 = b1 * m1 + (1 - b1) * g
    if o in (EmbOptimType.PARTIAL_ROWWISE_ADAM, EmbOptimType.PARTIAL_ROWWISE_LAMB):
        m2 = b2 * m2 + (1 - b2) * g.pow(2).mean(dim=1)
        denom = (m2 / bc2).sqrt().unsqueeze(1) + eps
    else:
        m2 = b2 * m2 + (1 - b2) * g * g
        denom = (m2 / bc2).sqrt() + eps
    upd = (m1 / bc1) / denom
    if lamb:
        if wd != 0:
            upd = upd + wd * w_rows
        wn, un = w_rows.norm(dim=1, keepdim=True), upd.norm(dim=1, keepdim=True)
        trust = torch.where((wn > 0) & (un > 0), wn / un.clamp(min=1e-30), torch.ones_like(wn))
        return w_rows - lr * trust * upd, m1, m2
    return w_rows - lr * upd, m1, m2


class _TBEFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dummy, module, indices, offsets, psw, B, plan):
        out = module._forward_impl(indices, offsets, psw, B)
        if plan is None:
            plan = module.build_plan_ahead(indices, offsets, psw, B)
        ctx.module = module
        ctx.B = B
        ctx.plan = plan
        ctx.save_for_backward(indices, offsets, psw if psw is not None else torch.empty(0))
        ctx.has_psw = psw is not None
        return out

    @staticmethod
    def backward(ctx, grad_out):
        indices, offsets, psw = ctx.saved_tensors
        m = ctx.module
        # the gradient of the per-sample weights reads the rows as the forward saw them: before the fused update
        psw_grad = m._psw_grad(grad_out, indices, offsets, ctx.B) if ctx.has_psw and ctx.needs_input_grad[4] else None
        dense_grad = m._backward_impl(grad_out, indices, offsets, psw if ctx.has_psw else None, ctx.B, ctx.plan)
        return dense_grad, None, None, None, psw_grad, None, None


class TableBatchedEmbeddingBags(nn.Module):
    """Several tables, one flat buffer, one lookup kernel.

    Args:
        embedding_specs: ``(num_rows, dim)`` per table.
        feature_table_map: table index of every feature (default: one feature per table).
        pooling_mode: SUM / MEAN / NONE (unpooled, all dims must be equal).
        weights_precision: dtype of the table storage (fp32 / fp16 / bf16).
        output_dtype: dtype of the lookup result.
        optimizer_args: fused optimizer; ``fused=False`` makes ``weights`` an ordinary
            parameter whose dense gradient is returned to autograd (data-parallel tables).
    """

    def __init__(
        self,
        embedding_specs: List[Tuple[int, int]],
        feature_table_map: Optional[List[int]] = None,
        pooling_mode: PoolingMode = PoolingMode.SUM,
        weights_precision: torch.dtype = torch.float32,
        output_dtype: torch.dtype = torch.float32,
        optimizer_args: Optional[OptimizerArgs] = None,
        fused: bool = True,
        device: Optional[torch.device] = None,
    ) -> None:
        super().__init__()
        self.embedding_specs = [(int(r), int(d)) for r, d in embedding_specs]
        T = len(self.embedding_specs)
        self.feature_table_map = list(feature_table_map) if feature_table_map is not None else list(range(T))
        self.pooling_mode = PoolingMode(int(pooling_mode))
        self.output_dtype = output_dtype
        self.fused = fused
        self.optimizer_args = optimizer_args if optimizer_args is not None else OptimizerArgs()
        self.step = 0
        device = torch.device(device) if device is not None else torch.device("cpu")
        for _, d in self.embedding_specs:
            assert d % 4 == 0, "embedding dims must be multiples of 4"
        if self.pooling_mode == PoolingMode.NONE:
            assert len({d for _, d in self.embedding_specs}) <= 1, "unpooled lookups need equal dims"
        self.max_D = max([d for _, d in self.embedding_specs], default=4)
        w_off, h_off = [0], [0]
        for r, d in self.embedding_specs:
            w_off.append(w_off[-1] + r * d)
            h_off.append(h_off[-1] + r)
        self.weights_offsets = w_off
        self.hash_offsets = h_off
        self.total_rows = h_off[-1]
        d_off = [0]
        for t in self.feature_table_map:
            d_off.append(d_off[-1] + self.embedding_specs[t][1])
        self.D_offsets = d_off
        self.total_D = d_off[-1]
        w = torch.empty(w_off[-1], dtype=weights_precision, device=device)
        self.weights = nn.Parameter(w, requires_grad=True)
        kinds = _STATE_KINDS[self.optimizer_args.optimizer] if fused else (None, None)
        self._state_kinds = kinds
        self.register_buffer("momentum1", self._alloc_state(kinds[0], device), persistent=False)
        self.register_buffer("momentum2", self._alloc_state(kinds[1], device), persistent=False)
        self._meta: Optional[torch.Tensor] = None
        self._err: Optional[torch.Tensor] = None
        self._dummy = torch.zeros(1, requires_grad=True)  # lets autograd reach the fused backward

    # ---- construction helpers ---------------------------------------------------------
    def _alloc_state(self, kind: Optional[str], device: torch.device) -> torch.Tensor:
        if kind == "row":
            return torch.zeros(self.total_rows, dtype=torch.float32, device=device)
        if kind == "elem":
            return torch.zeros(self.weights_offsets[-1], dtype=torch.float32, device=device)
        return torch.zeros(0, dtype=torch.float32, device=device)

    def _meta_tensor(self, device: torch.device) -> torch.Tensor:
        if self._meta is None or self._meta.device != device:
            rows = []
            ftm = self.feature_table_map
            rows.append([self.weights_offsets[t] for t in ftm])
            rows.append([self.hash_offsets[t] for t in ftm])
            rows.append([self.embedding_specs[t][0] for t in ftm])
            rows.append([self.embedding_specs[t][1] for t in ftm])
            rows.append(self.D_offsets[:-1])
            self._meta = torch.tensor(rows, dtype=torch.int64).reshape(5, len(ftm)).to(device)
            self._err = torch.zeros(1, dtype=torch.int32, device=device)
        return self._meta

    def _sr_counter(self) -> Optional[torch.Tensor]:
        """Device-side call counter that salts stochastic rounding (16-bit tables with ``stochastic_rounding`` on), else None."""
        if not self.optimizer_args.stochastic_rounding or self.weights.dtype == torch.float32 or not self.weights.is_cuda:
            return None
        c = self.__dict__.get("_sr_count")
        if c is None or c.device != self.weights.device:
            c = self.__dict__["_sr_count"] = torch.zeros(1, dtype=torch.int64, device=self.weights.device)
        return c

    def split_embedding_weights(self) -> List[torch.Tensor]:
        """Per-table ``[rows, dim]`` views into the flat buffer."""
        return [
            self.weights.detach()[self.weights_offsets[t]: self.weights_offsets[t + 1]].view(r, d)
            for t, (r, d) in enumerate(self.embedding_specs)
        ]

    def split_optimizer_states(self) -> List[Dict[str, torch.Tensor]]:
        """Per-table views of the fused optimizer state (``momentum1`` / ``momentum2``)."""
        out: List[Dict[str, torch.Tensor]] = []
        for t, (r, d) in enumerate(self.embedding_specs):
            st: Dict[str, torch.Tensor] = {}
            for name, kind, buf in (("momentum1", self._state_kinds[0], self.momentum1), ("momentum2", self._state_kinds[1], self.momentum2)):
                if kind == "row":
                    st[name] = buf[self.hash_offsets[t]: self.hash_offsets[t + 1]]
                elif kind == "elem":
                    st[name] = buf[self.weights_offsets[t]: self.weights_offsets[t + 1]].view(r, d)
            out.append(st)
        return out

    def init_embedding_weights_uniform(self, min_val: float, max_val: float) -> None:
        with torch.no_grad():
            if self.weights.dtype == torch.float32:
                self.weights.uniform_(min_val, max_val)
            else:
                self.weights.copy_(torch.empty_like(self.weights, dtype=torch.float32).uniform_(min_val, max_val))

    def set_learning_rate(self, lr: float) -> None:
        self.optimizer_args.learning_rate = float(lr)

    # ---- forward ----------------------------------------------------------------------
    def forward(
        self,
        indices: torch.Tensor,
        offsets: torch.Tensor,
        per_sample_weights: Optional[torch.Tensor] = None,
        batch_size: Optional[int] = None,
        plan: Optional[TBEPlan] = None,
    ) -> torch.Tensor:
        """``indices [N]``, ``offsets [F*B+1]`` feature-major.  Returns ``[B, total_D]`` (pooled)
        or ``[N, D]`` (unpooled)."""
        F = len(self.feature_table_map)
        B = batch_size if batch_size is not None else ((offsets.numel() - 1) // F if F else 0)
        if per_sample_weights is not None and per_sample_weights.dtype != torch.float32:
            per_sample_weights = per_sample_weights.float()
        if torch.is_grad_enabled() and (self.fused or self.weights.requires_grad):
            if self.fused:
                if self._dummy.device != torch.device("cpu"):
                    self._dummy = torch.zeros(1, requires_grad=True)
                anchor = self._dummy
            else:
                anchor = self.weights
            return _TBEFunction.apply(anchor, self, indices, offsets, per_sample_weights, B, plan)
        return self._forward_impl(indices, offsets, per_sample_weights, B)

    def _forward_impl(self, indices, offsets, psw, B) -> torch.Tensor:
        w = self.weights.detach()
        if w.is_cuda and _TBE_BACKEND == "kernel":
            _ext.require_cuda_ext("tbe_forward")
            meta = self._meta_tensor(w.device)
            if indices.dtype != offsets.dtype:
                offsets = offsets.to(indices.dtype)
            return torch.ops.trb200.tbe_forward(
                w, meta, indices.contiguous(), offsets.contiguous(), psw, B, self.total_D, self.max_D,
                int(self.pooling_mode), _OUT_CODE[self.output_dtype], self._err,
            )
        return self._forward_cpu(w, indices, offsets, psw, B)

    def _forward_cpu(self, w, indices, offsets, psw, B) -> torch.Tensor:
        F = len(self.feature_table_map)
        off = offsets.to(torch.int64)
        idx = indices.to(torch.int64)
        tables = [w[self.weights_offsets[t]: self.weights_offsets[t + 1]].view(r, d).float() for t, (r, d) in enumerate(self.embedding_specs)]
        if self.pooling_mode == PoolingMode.NONE:
            outs = []
            for f in range(F):
                s, e = int(off[f * B]), int(off[(f + 1) * B])
                outs.append(tables[self.feature_table_map[f]].index_select(0, idx[s:e]))
            res = torch.cat(outs, 0) if outs else w.new_zeros((0, self.max_D), dtype=torch.float32)
            return res.to(self.output_dtype)
        out = torch.zeros(B, self.total_D, dtype=torch.float32, device=w.device)
        for f in range(F):
            tbl = tables[self.feature_table_map[f]]
            o = off[f * B: (f + 1) * B + 1]
            s, e = int(o[0]), int(o[-1])
            if e > s:
                res = torch.nn.functional.embedding_bag(
                    idx[s:e], tbl, o[:-1] - s, mode="sum",
                    per_sample_weights=None if psw is None else psw[s:e].float(), include_last_offset=False,
                )
                if self.pooling_mode == PoolingMode.MEAN:
                    res = res / (o[1:] - o[:-1]).clamp(min=1).unsqueeze(1).float()
                out[:, self.D_offsets[f]: self.D_offsets[f + 1]] = res
        return out.to(self.output_dtype)

    # ---- backward ---------------------------------------------------------------------
    def build_plan(self, indices: torch.Tensor, offsets: torch.Tensor, psw: Optional[torch.Tensor], B: int, padded: bool = False) -> Optional[TBEPlan]:
        """Sort the ids of a batch by table row.  Depends on the ids only, so it can run ahead of
        the backward pass (e.g. on a side stream during the dense forward).  ``padded``: ``indices`` is a buffer of
        fixed capacity and only positions ``[offsets[0], offsets[-1])`` hold ids of this module; the count of real
        entries stays on the device (``TBEPlan.n_valid``)."""
        if not self.weights.is_cuda or _TBE_BACKEND != "kernel":
            return None
        meta = self._meta_tensor(self.weights.device)
        if indices.dtype != offsets.dtype:
            offsets = offsets.to(indices.dtype)
        return TBEPlan(
            torch.ops.trb200.tbe_build_plan(
                meta, indices.contiguous(), offsets.contiguous(), psw, B, max(self.total_rows, 2),
                self.pooling_mode != PoolingMode.NONE, self.pooling_mode == PoolingMode.MEAN, padded, self._err,
            )
        )

    def build_plan_ahead(self, indices: torch.Tensor, offsets: torch.Tensor, psw: Optional[torch.Tensor], B: int, padded: bool = False) -> Optional[TBEPlan]:
        """:meth:`build_plan` issued on the side stream, ordered after everything already queued on the current stream.  The
        plan's tensors are marked as used by the current stream so that their memory is not recycled under the backward."""
        if not (_PLAN_AHEAD and self.weights.is_cuda and indices.numel() > 0 and _TBE_BACKEND == "kernel"):
            return None
        cur = torch.cuda.current_stream()
        side = _plan_stream(self.weights.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            plan = self.build_plan(indices, offsets, psw, B, padded)
            plan.ready = torch.cuda.Event()
            plan.ready.record(side)
        for t in (plan.keys, plan.src, plan.w, plan.src_feature, plan.bag_scale, plan.n_valid):
            if t is not None and t.numel() > 0:
                t.record_stream(cur)
        for t in (indices, offsets, psw):
            if t is not None and t.is_cuda:
                t.record_stream(side)
        return plan

    def _backward_impl(self, grad_out, indices, offsets, psw, B, plan) -> Optional[torch.Tensor]:
        w = self.weights.detach()
        if self.fused:
            self.step += 1
        if w.is_cuda and _TBE_BACKEND == "kernel":
            _ext.require_cuda_ext("tbe_backward")
            if plan is None:
                plan = self.build_plan(indices, offsets, psw, B)
            else:
                plan.wait()
            # the kernel reads gradient rows through a row stride: a column slice of a wider tensor (the gradient of a concat)
            # needs no copy as long as rows are dense and 16-byte aligned
            esz = grad_out.element_size()
            if grad_out.dim() != 2 or grad_out.stride(1) != 1 or grad_out.data_ptr() % 16 != 0 or (grad_out.stride(0) * esz) % 16 != 0:
                grad_out = grad_out.contiguous()
            o = self.optimizer_args
            dense_grad = None
            if not self.fused:
                dense_grad = torch.zeros(w.numel(), dtype=torch.float32, device=w.device)
            code = _OPT_CODE[o.optimizer] if self.fused else OPT_DENSE_GRAD
            eps = o.eta if o.optimizer == EmbOptimType.LARS_SGD else o.eps
            torch.ops.trb200.tbe_backward_apply(
                w, self.momentum1 if self.momentum1.numel() else None, self.momentum2 if self.momentum2.numel() else None,
                dense_grad, self._meta_tensor(w.device), plan.keys, plan.src, plan.w, plan.src_feature, plan.bag_scale,
                grad_out, grad_out.stride(0), B, self.max_D, self.pooling_mode != PoolingMode.NONE, code,
                o.learning_rate, eps, o.beta1, o.beta2, o.weight_decay, self.step, o.max_gradient, plan.n_valid, self._sr_counter(),
            )
            return None if self.fused else dense_grad.to(w.dtype)
        return self._backward_cpu(w, grad_out, indices, offsets, psw, B)

    # ---- fused lookup + exchange over peer-mapped buffers (one node, NVLink) ---------------------------
    def _meta_tensor_at(self, device: torch.device, col_base) -> torch.Tensor:
        """Metadata whose output column offsets start at ``col_base`` (this rank's block of the exchanged row), or, when
        ``col_base`` is a sequence, are exactly those per-feature columns (tables stored at their final place in the row)."""
        cache = self.__dict__.setdefault("_meta_at", {})
        absolute = not isinstance(col_base, int)
        key = (str(device), tuple(int(c) for c in col_base) if absolute else int(col_base))
        if key not in cache:
            m = self._meta_tensor(device).clone()
            if absolute:
                assert len(col_base) == m.shape[1], "one output column per feature"
                m[4] = torch.tensor([int(c) for c in col_base], dtype=m.dtype, device=m.device)
            else:
                m[4] += int(col_base)
            cache[key] = m
        return cache[key]

    def forward_push(self, indices: torch.Tensor, offsets: torch.Tensor, psw: Optional[torch.Tensor], B: int, B_local: int,
                     out_ptrs: List[int], out_stride: int, col_base, out_dtype: torch.dtype, pooling: Optional[int] = None) -> None:
        """Pooled lookup of the global batch (``B`` bags per feature) whose result rows are stored directly into the
        ``[B_local, out_stride]`` buffers of the ranks that own the samples (``out_ptrs[b // B_local]``), at column
        ``col_base`` + the table's offset.  No output tensor: the caller synchronises with a peer barrier."""
        _ext.require_cuda_ext("tbe_forward_dist")
        w = self.weights.detach()
        if indices.dtype != offsets.dtype:
            offsets = offsets.to(indices.dtype)
        torch.ops.trb200.tbe_forward_dist(
            w, self._meta_tensor_at(w.device, col_base), indices.contiguous(), offsets.contiguous(), psw, out_ptrs,
            _OUT_CODE[out_dtype], out_stride, B, B_local, self.max_D, int(self.pooling_mode) if pooling is None else pooling, False, False, self._err,
        )

    def backward_pull(self, grad_local: torch.Tensor, grad_ptrs: List[int], grad_stride: int, indices: torch.Tensor, offsets: torch.Tensor,
                      psw: Optional[torch.Tensor], B: int, B_local: int, col_base, grad_scale: float, plan: Optional[TBEPlan] = None,
                      padded: bool = False) -> None:
        """Backward + fused optimizer of ``forward_push``: the gradient row of bag ``b`` is read from
        ``grad_ptrs[b // B_local]`` (``grad_local`` is this rank's own buffer among them)."""
        assert self.fused, "the fused exchange is for tables with an in-backward optimizer"
        _ext.require_cuda_ext("tbe_backward_apply_dist")
        w = self.weights.detach()
        self.step += 1
        if plan is None:
            plan = self.build_plan(indices, offsets, psw, B, padded)
        else:
            plan.wait()
        o = self.optimizer_args
        eps = o.eta if o.optimizer == EmbOptimType.LARS_SGD else o.eps
        torch.ops.trb200.tbe_backward_apply_dist(
            w, self.momentum1 if self.momentum1.numel() else None, self.momentum2 if self.momentum2.numel() else None, None,
            self._meta_tensor_at(w.device, col_base), plan.keys, plan.src, plan.w, plan.src_feature, plan.bag_scale, grad_local,
            grad_stride, B, self.max_D, True, _OPT_CODE[o.optimizer], o.learning_rate, eps, o.beta1, o.beta2, o.weight_decay,
            self.step, o.max_gradient, grad_ptrs, B_local, grad_scale, plan.n_valid,
        )

    def seq_forward_push(self, indices: torch.Tensor, offsets: torch.Tensor, ret: torch.Tensor, B: int, out_ptrs: List[int], out_rows: int,
                         out_stride: int, cols, out_dtype: torch.dtype) -> None:
        """Unpooled lookup of ids that arrived with return addresses (``ret[k]`` = requesting rank << 32 | row): the row of id
        ``k`` is stored into row ``ret[k] & 0xffffffff`` of ``out_ptrs[ret[k] >> 32]`` (``[out_rows, out_stride]`` buffers), at the
        per-feature columns ``cols``.  ``indices`` / ``ret`` are fixed-capacity buffers delimited by ``offsets``."""
        _ext.require_cuda_ext("tbe_seq_forward_dist")
        assert self.pooling_mode == PoolingMode.NONE
        w = self.weights.detach()
        if indices.dtype != offsets.dtype:
            offsets = offsets.to(indices.dtype)
        torch.ops.trb200.tbe_seq_forward_dist(
            w, self._meta_tensor_at(w.device, cols), indices, offsets.contiguous(), ret, out_ptrs, out_rows, _OUT_CODE[out_dtype], out_stride, B,
            self.max_D, self._err,
        )

    def seq_backward_pull(self, grad_local: torch.Tensor, grad_ptrs: List[int], ret: torch.Tensor, indices: torch.Tensor, offsets: torch.Tensor,
                          B: int, cols, grad_scale: float, plan: Optional[TBEPlan] = None) -> None:
        """Backward + fused optimizer of :meth:`seq_forward_push`: the gradient row of id ``k`` is read from row
        ``ret[k] & 0xffffffff`` of ``grad_ptrs[ret[k] >> 32]`` at the per-feature columns ``cols``."""
        assert self.fused, "the fused exchange is for tables with an in-backward optimizer"
        _ext.require_cuda_ext("tbe_backward_apply_dist")
        w = self.weights.detach()
        self.step += 1
        if plan is None:
            plan = self.build_plan(indices, offsets, None, B, True)
        else:
            plan.wait()
        o = self.optimizer_args
        eps = o.eta if o.optimizer == EmbOptimType.LARS_SGD else o.eps
        torch.ops.trb200.tbe_backward_apply_dist(
            w, self.momentum1 if self.momentum1.numel() else None, self.momentum2 if self.momentum2.numel() else None, None,
            self._meta_tensor_at(w.device, cols), plan.keys, plan.src, plan.w, plan.src_feature, plan.bag_scale, grad_local,
            grad_local.stride(0), B, self.max_D, False, _OPT_CODE[o.optimizer], o.learning_rate, eps, o.beta1, o.beta2, o.weight_decay,
            self.step, o.max_gradient, grad_ptrs, 0, grad_scale, plan.n_valid, ret, self._sr_counter(),
        )

    def backward_local(self, grad: torch.Tensor, indices: torch.Tensor, offsets: torch.Tensor, psw: Optional[torch.Tensor], B: int, cols,
                       plan: Optional[TBEPlan] = None, padded: bool = False) -> None:
        """Backward + fused optimizer reading the pooled gradient of bag ``b`` from row ``b`` of ``grad`` (a local ``[B, stride]``
        slab), at the per-feature columns ``cols``."""
        assert self.fused, "the fused exchange is for tables with an in-backward optimizer"
        _ext.require_cuda_ext("tbe_backward_apply")
        w = self.weights.detach()
        self.step += 1
        if plan is None:
            plan = self.build_plan(indices, offsets, psw, B, padded)
        else:
            plan.wait()
        o = self.optimizer_args
        eps = o.eta if o.optimizer == EmbOptimType.LARS_SGD else o.eps
        torch.ops.trb200.tbe_backward_apply(
            w, self.momentum1 if self.momentum1.numel() else None, self.momentum2 if self.momentum2.numel() else None, None,
            self._meta_tensor_at(w.device, cols), plan.keys, plan.src, plan.w, plan.src_feature, plan.bag_scale, grad, grad.stride(0), B,
            self.max_D, True, _OPT_CODE[o.optimizer], o.learning_rate, eps, o.beta1, o.beta2, o.weight_decay, self.step, o.max_gradient,
            plan.n_valid, self._sr_counter(),
        )

    def _psw_grad(self, grad_out: torch.Tensor, indices: torch.Tensor, offsets: torch.Tensor, B: int) -> torch.Tensor:
        """``d loss / d per_sample_weights[i] = <grad of the bag of i, row of i>`` (learned position weights of feature
        processors); composite, one gather per feature."""
        w = self.weights.detach()
        F = len(self.feature_table_map)
        off = offsets.to(torch.int64)
        idx = indices.to(torch.int64)
        N = idx.numel()
        out = torch.zeros(N, dtype=torch.float32, device=w.device)
        if N == 0:
            return out
        bounds = off[:: max(B, 1)][: F + 1].tolist() if B > 0 else [0] * (F + 1)
        lens = off[1:] - off[:-1]
        bag = torch.repeat_interleave(torch.arange(F * B, device=w.device), lens, output_size=N)
        g_out = grad_out.float()
        for f in range(F):
            s, e = bounds[f], bounds[f + 1]
            if e == s:
                continue
            t = self.feature_table_map[f]
            r, d = self.embedding_specs[t]
            rows = w[self.weights_offsets[t]: self.weights_offsets[t + 1]].view(r, d).index_select(0, idx[s:e]).float()
            if self.pooling_mode == PoolingMode.NONE:
                g = g_out[s:e, :d]
            else:
                g = g_out[bag[s:e] - f * B, self.D_offsets[f]: self.D_offsets[f + 1]]
                if self.pooling_mode == PoolingMode.MEAN:
                    g = g / lens[bag[s:e]].clamp(min=1).unsqueeze(1).float()
            out[s:e] = (rows * g).sum(dim=1)
        return out

    def _backward_cpu(self, w, grad_out, indices, offsets, psw, B) -> Optional[torch.Tensor]:
        F = len(self.feature_table_map)
        off = offsets.to(torch.int64)
        idx = indices.to(torch.int64)
        g_out = grad_out.float()
        N = idx.numel()
        lens = off[1:] - off[:-1]
        bag = torch.repeat_interleave(torch.arange(F * B, device=w.device), lens, output_size=N)
        dense_grad = None if self.fused else torch.zeros(w.numel(), dtype=torch.float32, device=w.device)
        splits = self.split_optimizer_states() if self.fused else None
        # group features by table so that a row touched through two features is updated once
        by_table: Dict[int, List[int]] = {}
        for f, t in enumerate(self.feature_table_map):
            by_table.setdefault(t, []).append(f)
        for t, feats in by_table.items():
            r, d = self.embedding_specs[t]
            ids_l, grads_l = [], []
            for f in feats:
                s, e = int(off[f * B]), int(off[(f + 1) * B])
                if e == s:
                    continue
                ids = idx[s:e]
                if self.pooling_mode == PoolingMode.NONE:
                    g = g_out[s:e, :d]
                else:
                    b = bag[s:e] - f * B
                    g = g_out[b, self.D_offsets[f]: self.D_offsets[f + 1]]
                    if self.pooling_mode == PoolingMode.MEAN:
                        g = g / lens[bag[s:e]].clamp(min=1).unsqueeze(1).float()
                if psw is not None:
                    g = g * psw[s:e].float().unsqueeze(1)
                ids_l.append(ids)
                grads_l.append(g)
            if not ids_l:
                continue
            ids = torch.cat(ids_l)
            g = torch.cat(grads_l)
            uniq, inv = torch.unique(ids, return_inverse=True)
            gsum = torch.zeros(uniq.numel(), d, dtype=torch.float32, device=w.device).index_add_(0, inv, g)
            tbl = w[self.weights_offsets[t]: self.weights_offsets[t + 1]].view(r, d)
            if not self.fused:
                dense_grad[self.weights_offsets[t]: self.weights_offsets[t + 1]].view(r, d).index_add_(0, uniq, gsum)
                continue
            st = splits[t]
            m1 = st["momentum1"][uniq] if "momentum1" in st else None
            m2 = st["momentum2"][uniq] if "momentum2" in st else None
            new_w, m1, m2 = _apply_rows_cpu(self.optimizer_args, self.step, tbl[uniq].float(), gsum, m1, m2)
            tbl[uniq] = new_w.to(tbl.dtype)
            if m1 is not None:
                st["momentum1"][uniq] = m1
            if m2 is not None:
                st["momentum2"][uniq] = m2
        return None if self.fused else dense_grad.to(w.dtype)

    def check_error(self) -> None:
        """Raise if a kernel saw an out-of-range id since the last check (one host sync)."""
        if self._err is not None and int(self._err.item()) != 0:
            self._err.zero_()
            raise IndexError("TableBatchedEmbeddingBags: id out of range for its table")
