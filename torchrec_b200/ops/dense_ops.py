"""Dense-tower operators: fused linear+bias+activation, low-rank cross layer, dot interaction, BCE.

On CUDA the GEMMs run in bf16 with fp32 accumulation through the hand-written tcgen05 kernel
(``torchrec_b200/csrc/cuda/gemm_tcgen05.cu``); parameters stay fp32 ("master" weights) and a bf16
copy is refreshed once per optimizer step.  On CPU (or when the compute dtype is fp32) the same
functions fall back to plain torch math, which is also the oracle the kernels are tested against.

The reference runs these layers as ``nn.Linear`` / ``torch.bmm`` library calls
(``torchrec/modules/mlp.py:61-80``, ``torchrec/modules/crossnet.py:178-181``,
``torchrec/models/dlrm.py:216-219``).
"""
from __future__ import annotations

import os
import weakref
from typing import Optional, Tuple

import torch

from . import _ext

ACT_NONE = 0
ACT_RELU = 1
ACT_SIGMOID = 2

_COMPUTE_DTYPE: torch.dtype = torch.float32
_GEMM_BACKEND = os.environ.get("TRB200_GEMM", "tcgen05")  # "tcgen05" | "cublas"


def set_dense_compute_dtype(dtype: torch.dtype) -> None:
    """Select the dtype of dense-tower GEMM operands on CUDA (fp32 -> plain torch, bf16 -> fused kernels)."""
    global _COMPUTE_DTYPE
    assert dtype in (torch.float32, torch.bfloat16)
    _COMPUTE_DTYPE = dtype


def get_dense_compute_dtype() -> torch.dtype:
    return _COMPUTE_DTYPE


def set_gemm_backend(name: str) -> None:
    global _GEMM_BACKEND
    assert name in ("tcgen05", "cublas")
    _GEMM_BACKEND = name


def get_gemm_backend() -> str:
    return _GEMM_BACKEND


def fused_dense_enabled(x: torch.Tensor) -> bool:
    return x.is_cuda and _COMPUTE_DTYPE == torch.bfloat16


# --------------------------------------------------------------------------------------
# bf16 weight cache: one cast per parameter version, shared by forward and backward
# --------------------------------------------------------------------------------------
class _Bf16Cache:
    """bf16 (and transposed bf16) copies of fp32 parameters.

    Unmanaged parameters are re-cast when their version counter moves.  Parameters of a ``FlatParamBuffer``
    (``optim/fused_dense.py``) are *managed*: their copies live at fixed addresses and are rewritten by the optimizer
    kernel itself, so a forward pass launches no cast; a managed copy is only refreshed here when the parameter was
    changed behind the optimizer's back (a checkpoint load, an in-place init)."""

    def __init__(self) -> None:
        self._store = {}
        self._managed = {}

    def register(self, p: torch.Tensor, w16: torch.Tensor, wT16: Optional[torch.Tensor]) -> None:
        self._managed[id(p)] = [p._version, w16, wT16, p]

    def mark_fresh(self, p: torch.Tensor) -> None:
        ent = self._managed.get(id(p))
        if ent is not None:
            ent[0] = p._version

    def get(self, p: torch.Tensor, transposed: bool = False) -> torch.Tensor:
        m = self._managed.get(id(p))
        if m is not None and m[3] is p and (m[2] is not None or not transposed):
            if m[0] != p._version:
                with torch.no_grad():
                    m[1].copy_(p.detach())
                    if m[2] is not None:
                        m[2].copy_(p.detach().reshape(m[2].shape[1], m[2].shape[0]).t())
                m[0] = p._version
            return m[2] if transposed else m[1]
        key = (id(p), transposed)
        ent = self._store.get(key)
        ver = p._version
        if ent is not None and ent[0] == ver and ent[1].device == p.device and ent[2] is p:
            return ent[1]
        src = p.detach()
        t = (src.t().contiguous() if transposed else src).to(torch.bfloat16)
        self._store[key] = (ver, t, p)
        return t

    def clear(self) -> None:
        self._store.clear()
        self._managed.clear()


bf16_cache = _Bf16Cache()


def _grad_sink(p: torch.Tensor) -> Optional[torch.Tensor]:
    """Where the gradient of ``p`` may be accumulated directly: its view into a flat gradient buffer (``FlatParamBuffer``),
    provided that buffer was zeroed for this step.  The weight-gradient GEMM and the bias column sum then reduce straight into
    it, which removes an output allocation, a zero fill and an accumulation pass per parameter."""
    buf = getattr(p, "_trb_flat", None)
    if buf is None or not getattr(buf, "direct_grads", False):
        return None
    g = p.grad
    if g is None or g.dtype != torch.float32 or not g.is_cuda or not g.is_contiguous() or not _ext.has_cuda_ext():
        return None
    buf.note_direct_write()
    return g


# --------------------------------------------------------------------------------------
# GEMM primitive: C[M,N] = A[M,K] @ B[N,K]^T  (both operands K-major), bf16 in, fp32 accumulate
# --------------------------------------------------------------------------------------
def gemm_nt(
    a: torch.Tensor,
    b: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    act: int = ACT_NONE,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """``act(a @ b.T + bias)`` with ``a [M,K]``, ``b [N,K]`` bf16 row-major."""
    if a.is_cuda and _GEMM_BACKEND == "tcgen05" and _ext.has_cuda_ext() and _tcgen05_ok(a, b) and not (
        out_dtype == torch.float32 and (bias is not None or act != ACT_NONE)
    ):
        if bias is None and act != ACT_NONE:
            bias = torch.zeros(b.shape[0], dtype=torch.float32, device=a.device)  # the fused epilogues are bias+act
        return torch.ops.trb200.gemm_nt_bf16(a, b, bias, act, out_dtype == torch.float32)
    y = torch.matmul(a, b.t())
    if bias is not None:
        y = y + bias.to(y.dtype)
    if act == ACT_RELU:
        y = torch.relu(y)
    elif act == ACT_SIGMOID:
        y = torch.sigmoid(y)
    return y.to(out_dtype)


def _tcgen05_ok(a: torch.Tensor, b: torch.Tensor) -> bool:
    # TMA needs 16-byte aligned row pitches: K % 8 == 0 for bf16 operands, N % 8 == 0 for the output.
    return (
        a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_contiguous() and b.is_contiguous()
        and a.shape[1] % 8 == 0 and b.shape[0] % 8 == 0 and a.shape[0] > 0
    )


class _LinearAct(torch.autograd.Function):
    """y = act(x W^T + b) with bf16 GEMMs; saves bf16 activations only."""

    @staticmethod
    def forward(ctx, x, weight, bias, act: int):
        w16 = bf16_cache.get(weight)
        x16 = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        y = gemm_nt(x16, w16, bias, act, torch.bfloat16)
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.bias_ref = weakref.ref(bias) if bias is not None else None
        ctx.save_for_backward(x16, weight, y)
        ctx.x_dtype = x.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x16, weight, y = ctx.saved_tensors
        dy = dy.contiguous()
        if dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        if ctx.act == ACT_RELU:
            dz = act_backward(dy, y, ACT_RELU)
        elif ctx.act == ACT_SIGMOID:
            dz = act_backward(dy, y, ACT_SIGMOID)
        else:
            dz = dy
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            wT16 = bf16_cache.get(weight, transposed=True)  # [K, N]
            dx = gemm_nt(dz, wT16, None, ACT_NONE, torch.bfloat16).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            dw = gemm_tn(dz, x16, into=_grad_sink(weight))  # [N, K] fp32, or None when it went straight into weight.grad
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = colsum(dz, into=_grad_sink(ctx.bias_ref()) if ctx.bias_ref is not None else None)
        return dx, dw, db, None


def act_backward(dy: torch.Tensor, y: torch.Tensor, act: int) -> torch.Tensor:
    if dy.is_cuda and _ext.has_cuda_ext():
        return torch.ops.trb200.act_backward_bf16(dy, y, act)
    if act == ACT_RELU:
        return dy * (y > 0).to(dy.dtype)
    yf = y.float()
    return (dy.float() * yf * (1 - yf)).to(dy.dtype)


def gemm_tn(a: torch.Tensor, b: torch.Tensor, into: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``a.T @ b`` with ``a [M,N]``, ``b [M,K]`` bf16 -> ``[N,K]`` fp32 (weight gradient).  With ``into`` the product is added to
    that tensor and ``None`` is returned."""
    if a.is_cuda and _GEMM_BACKEND == "tcgen05" and _ext.has_cuda_ext() and _tcgen05_tn_ok(a, b):
        if into is not None:
            torch.ops.trb200.gemm_tn_bf16_acc(a, b, into.view(a.shape[1], b.shape[1]))
            return None
        return torch.ops.trb200.gemm_tn_bf16(a, b)
    out = torch.matmul(a.t(), b).float()
    if into is not None:
        into.add_(out.view_as(into))
        return None
    return out


def colsum(x: torch.Tensor, into: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Column sums of a bf16 matrix in fp32 (bias gradient); with ``into`` they are added to that tensor and ``None`` is returned."""
    if x.is_cuda and _ext.has_cuda_ext() and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] % 2 == 0:
        if into is not None:
            torch.ops.trb200.colsum_bf16_acc(x, into)
            return None
        return torch.ops.trb200.colsum_bf16(x)
    out = x.float().sum(0)
    if into is not None:
        into.add_(out)
        return None
    return out


def _tcgen05_tn_ok(a: torch.Tensor, b: torch.Tensor) -> bool:
    return (
        a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_contiguous() and b.is_contiguous()
        and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.shape[0] % 8 == 0 and a.shape[0] > 0
    )


class _LinearSmallK(torch.autograd.Function):
    """``act(x W^T + b)`` for a layer with a handful of input features (K <= 32, e.g. the 13 dense features of the Criteo models):
    CUDA-core kernels that keep the weight in shared memory; the weight gradient is accumulated in fp32."""

    @staticmethod
    def forward(ctx, x, weight, bias, act: int):
        x16 = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
        y = torch.ops.trb200.linear_small_k_fwd(x16, weight.detach().float().contiguous(), None if bias is None else bias.detach().float(), act)
        ctx.act = act
        ctx.bias_ref = weakref.ref(bias) if bias is not None else None
        ctx.save_for_backward(x16, weight, y)
        ctx.x_dtype = x.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x16, weight, y = ctx.saved_tensors
        dy = dy.contiguous()
        if dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        dz = act_backward(dy, y, ctx.act) if ctx.act in (ACT_RELU, ACT_SIGMOID) else dy
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.matmul(dz, weight.to(torch.bfloat16)).to(ctx.x_dtype)
        if ctx.needs_input_grad[1]:
            sink = _grad_sink(weight)
            target = sink if sink is not None else torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
            torch.ops.trb200.linear_small_k_wgrad_acc(dz, x16, target)
            dw = None if sink is not None else target.to(weight.dtype)
        if ctx.bias_ref is not None and ctx.needs_input_grad[2]:
            db = colsum(dz, into=_grad_sink(ctx.bias_ref()))
        return dx, dw, db, None


def _small_k_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    K, N = weight.shape[1], weight.shape[0]
    return x.is_cuda and _ext.has_cuda_ext() and K <= 32 and K % 8 != 0 and N % 8 == 0 and weight.dtype == torch.float32


def linear_act(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], act: int = ACT_NONE) -> torch.Tensor:
    """Fused ``act(x @ weight.T + bias)``; bf16 tensor-core path on CUDA, torch math elsewhere."""
    if fused_dense_enabled(x):
        lead = x.shape[:-1]
        fn = _LinearSmallK if _small_k_ok(x, weight) else _LinearAct
        y = fn.apply(x.reshape(-1, x.shape[-1]), weight, bias, act)
        return y.view(*lead, weight.shape[0])
    y = torch.nn.functional.linear(x, weight, bias)
    if act == ACT_RELU:
        return torch.relu(y)
    if act == ACT_SIGMOID:
        return torch.sigmoid(y)
    return y


# --------------------------------------------------------------------------------------
# dot interaction: strict upper triangle of X X^T per sample, concatenated after the dense vector
# --------------------------------------------------------------------------------------
class _DotInteraction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dense, sparse):
        # dense [B, D], sparse [B, F, D] -> [B, D + C(F+1, 2)]
        out = torch.ops.trb200.dot_interaction_fwd(dense, sparse)
        ctx.save_for_backward(dense, sparse)
        return out

    @staticmethod
    def backward(ctx, dout):
        dense, sparse = ctx.saved_tensors
        dd, ds = torch.ops.trb200.dot_interaction_bwd(dout.contiguous(), dense, sparse)
        return dd, ds


def dot_interaction(dense: torch.Tensor, sparse: torch.Tensor) -> torch.Tensor:
    """``cat([dense, triu(X X^T, 1)])`` with ``X = cat([dense[:,None], sparse], 1)``.

    Pair order follows ``torch.triu_indices(F+1, F+1, offset=1)`` (row-major over i<j).
    """
    if dense.is_cuda and _ext.has_cuda_ext() and dense.dtype in (torch.float32, torch.bfloat16) and os.environ.get("TRB200_DOT", "kernel") == "kernel":
        return _DotInteraction.apply(dense.contiguous(), sparse.contiguous().to(dense.dtype))
    B, D = dense.shape
    x = torch.cat((dense.unsqueeze(1), sparse.to(dense.dtype)), dim=1)
    z = torch.bmm(x, x.transpose(1, 2))
    n = x.shape[1]
    iu = torch.triu_indices(n, n, offset=1, device=dense.device)
    return torch.cat((dense, z[:, iu[0], iu[1]]), dim=1)


# --------------------------------------------------------------------------------------
# loss
# --------------------------------------------------------------------------------------
class _BCEWithLogits(torch.autograd.Function):
    """Mean binary cross entropy whose forward kernel also writes d(loss)/d(logit): backward is one scale."""

    @staticmethod
    def forward(ctx, logits, labels, weights):
        loss, grad = torch.ops.trb200.bce_with_logits_fwd_bwd(logits.contiguous(), labels.float().contiguous(), None if weights is None else weights.float().contiguous())
        ctx.save_for_backward(grad)
        ctx.in_dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        (grad,) = ctx.saved_tensors
        return (grad * g).to(ctx.in_dtype), None, None


def bce_with_logits_mean(logits: torch.Tensor, labels: torch.Tensor, weights: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``mean(w * BCE(sigmoid(logits), labels))``; on a CUDA device one fused kernel computes loss and gradient."""
    if logits.is_cuda and logits.dtype in (torch.float32, torch.float16, torch.bfloat16) and _ext.use_cuda_kernel(logits, "bce_with_logits"):
        return _BCEWithLogits.apply(logits, labels, weights)
    return torch.nn.functional.binary_cross_entropy_with_logits(logits.float(), labels.float(), weight=None if weights is None else weights.float())


# --------------------------------------------------------------------------------------
# DCN-v2 low-rank cross layer: y = x0 * (W (V x) + b) + x
# --------------------------------------------------------------------------------------
def gemm_nt_cross(v: torch.Tensor, w16: torch.Tensor, bias: torch.Tensor, x0: torch.Tensor, xl: torch.Tensor):
    """Second GEMM of the cross layer with its epilogue: returns ``(u, y)`` where
    ``u = v @ w16.T + bias`` and ``y = x0 * u + xl`` (both bf16)."""
    if v.is_cuda and _GEMM_BACKEND == "tcgen05" and _ext.has_cuda_ext() and _tcgen05_ok(v, w16):
        return torch.ops.trb200.gemm_nt_bf16_cross(v, w16, bias, x0, xl)
    u = (torch.matmul(v, w16.t()).float() + bias.float()).to(torch.bfloat16)
    y = (x0.float() * u.float() + xl.float()).to(torch.bfloat16)
    return u, y


class _LowRankCross(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x0, xl, V, W, bias):
        # x0, xl [B, N] bf16 ; V [r, N] ; W [N, r] ; bias [N]
        V16 = bf16_cache.get(V)
        W16 = bf16_cache.get(W)
        v = gemm_nt(xl, V16, None, ACT_NONE, torch.bfloat16)  # [B, r]
        u, y = gemm_nt_cross(v, W16, bias, x0, xl)
        ctx.save_for_backward(x0, xl, v, u, V, W)
        return y

    @staticmethod
    def backward(ctx, dy):
        x0, xl, v, u, V, W = ctx.saved_tensors
        dy = dy.contiguous()
        if dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        # du = dy * x0 ; dx0 = dy * u   (one fused elementwise pass on CUDA)
        if dy.is_cuda and _ext.has_cuda_ext():
            du, dx0 = torch.ops.trb200.cross_bwd_elementwise(dy, x0, u)
        else:
            du = (dy.float() * x0.float()).to(torch.bfloat16)
            dx0 = (dy.float() * u.float()).to(torch.bfloat16)
        WT16 = bf16_cache.get(W, transposed=True)  # [r, N]
        VT16 = bf16_cache.get(V, transposed=True)  # [N, r]
        dv = gemm_nt(du, WT16, None, ACT_NONE, torch.bfloat16)  # [B, r]
        dW = gemm_tn(du, v)  # [N, r]
        db = torch.ops.trb200.colsum_bf16(du) if (du.is_cuda and _ext.has_cuda_ext()) else du.float().sum(0)
        # dxl = dy + dv @ V   (residual add in the GEMM epilogue)
        dxl = gemm_nt_add(dv, VT16, dy)
        dV = gemm_tn(dv, xl)  # [r, N]
        return dx0, dxl, dV, dW, db


def gemm_nt_add(a: torch.Tensor, b: torch.Tensor, add: torch.Tensor) -> torch.Tensor:
    """``a @ b.T + add`` (bf16)."""
    if a.is_cuda and _GEMM_BACKEND == "tcgen05" and _ext.has_cuda_ext() and _tcgen05_ok(a, b):
        return torch.ops.trb200.gemm_nt_bf16_add(a, b, add)
    return (torch.matmul(a, b.t()).float() + add.float()).to(torch.bfloat16)


def lowrank_cross_layer(x0, xl, V, W, bias) -> torch.Tensor:
    return _LowRankCross.apply(x0, xl, V, W, bias)


def _cross_bwd_fused(dy, x0, u, dx0_acc, add_dy):
    """``du = dy*x0``, running ``dx0 (+)= dy*u (+ dy)``, ``db = colsum(du)`` in one pass."""
    if dy.is_cuda and _ext.has_cuda_ext():
        return torch.ops.trb200.cross_bwd_fused(dy, x0, u, dx0_acc, add_dy)
    du = (dy.float() * x0.float()).to(torch.bfloat16)
    g = dy.float() * u.float()
    if dx0_acc is not None:
        g = g + dx0_acc.float()
    if add_dy:
        g = g + dy.float()
    return du, g.to(torch.bfloat16), du.float().sum(0)


class _LowRankCrossStack(torch.autograd.Function):
    """All layers of a low-rank cross network ``x_{l+1} = x0 * (W_l (V_l x_l) + b_l) + x_l`` as one autograd node.

    Keeping the stack in one node lets the backward carry the gradient of ``x0`` (which every layer multiplies by)
    as a running sum inside the fused elementwise kernel instead of leaving one ``[B, N]`` addition per layer to
    autograd; the bias gradient comes out of the same pass.  Per layer the backward is then one elementwise pass
    and four GEMMs (two with fused epilogues)."""

    @staticmethod
    def forward(ctx, x0, num_layers, *params):
        Vs, Ws, bs = params[:num_layers], params[num_layers: 2 * num_layers], params[2 * num_layers:]
        saved = [x0]
        xl = x0
        for V, W, b in zip(Vs, Ws, bs):
            v = gemm_nt(xl, bf16_cache.get(V), None, ACT_NONE, torch.bfloat16)
            u, y = gemm_nt_cross(v, bf16_cache.get(W), b, x0, xl)
            saved += [xl, v, u]
            xl = y
        ctx.num_layers = num_layers
        ctx.save_for_backward(*saved, *Vs, *Ws)
        return xl

    @staticmethod
    def backward(ctx, dy):
        L = ctx.num_layers
        t = ctx.saved_tensors
        x0 = t[0]
        per_layer = t[1: 1 + 3 * L]
        Vs, Ws = t[1 + 3 * L: 1 + 4 * L], t[1 + 4 * L: 1 + 5 * L]
        dy = dy.contiguous()
        if dy.dtype != torch.bfloat16:
            dy = dy.to(torch.bfloat16)
        dVs, dWs, dbs = [None] * L, [None] * L, [None] * L
        dx0_acc = None
        dx0 = None
        for l in reversed(range(L)):
            xl, v, u = per_layer[3 * l: 3 * l + 3]
            last = l == 0
            du, dx0_acc, dbs[l] = _cross_bwd_fused(dy, x0, u, dx0_acc, last)
            dv = gemm_nt(du, bf16_cache.get(Ws[l], transposed=True), None, ACT_NONE, torch.bfloat16)  # [B, r]
            dWs[l] = gemm_tn(du, v, into=_grad_sink(Ws[l]))
            dVs[l] = gemm_tn(dv, xl, into=_grad_sink(Vs[l]))
            VT16 = bf16_cache.get(Vs[l], transposed=True)
            if last:
                dx0 = gemm_nt_add(dv, VT16, dx0_acc)  # x_0 is also the x input of layer 0
            else:
                dy = gemm_nt_add(dv, VT16, dy)
        return (dx0, None, *dVs, *dWs, *dbs)


def lowrank_cross_stack(x0, Vs, Ws, biases) -> torch.Tensor:
    """Run a whole low-rank cross network (lists of per-layer ``V [r, N]``, ``W [N, r]``, ``bias [N]``)."""
    return _LowRankCrossStack.apply(x0, len(Vs), *Vs, *Ws, *biases)


class _LinearOut1(torch.autograd.Function):
    """Logit layer ``x [M, K] bf16 -> [M, 1] fp32``: one warp per row forward; the backward writes ``dx`` and reduces the weight and
    bias gradients in one pass over ``x``."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        y = torch.ops.trb200.linear_out1_fwd(x, weight.detach().reshape(-1), None if bias is None else bias.detach())
        ctx.bias_ref = weakref.ref(bias) if bias is not None else None
        ctx.save_for_backward(x, weight)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        bias = ctx.bias_ref() if ctx.bias_ref is not None else None
        w_sink = _grad_sink(weight) if ctx.needs_input_grad[1] else None
        b_sink = _grad_sink(bias) if bias is not None and ctx.needs_input_grad[2] else None
        dw = w_sink if w_sink is not None else torch.zeros(weight.shape, dtype=torch.float32, device=x.device)
        db = None
        if bias is not None:
            db = b_sink if b_sink is not None else torch.zeros(1, dtype=torch.float32, device=x.device)
        dx = torch.ops.trb200.linear_out1_bwd(dy.contiguous().float().reshape(-1), x, weight.detach().reshape(-1), dw.view(-1), db, ctx.needs_input_grad[0])
        return (dx if ctx.needs_input_grad[0] else None, None if w_sink is not None or not ctx.needs_input_grad[1] else dw,
                None if bias is None or b_sink is not None or not ctx.needs_input_grad[2] else db)


def linear_small_out(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """Final logits layer in fp32 (``out_features`` tiny, e.g. 1): a CUDA-core dot-product kernel is a better fit than a
    tensor-core tile; other shapes go through ``F.linear`` in fp32."""
    if (x.is_cuda and _ext.has_cuda_ext() and x.dim() == 2 and x.dtype == torch.bfloat16 and x.is_contiguous() and weight.shape[0] == 1
            and weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[1] % 8 == 0 and weight.shape[1] <= 1024
            and (bias is None or bias.dtype == torch.float32)):
        return _LinearOut1.apply(x, weight, bias)
    return torch.nn.functional.linear(x.float(), weight, bias)
