"""One-launch optimizer for the dense (replicated) parameters of a recommender model.

``FlatParamBuffer`` moves a list of parameters into ONE flat fp32 master buffer (each parameter becomes a view), with a
flat gradient buffer of the same layout, and keeps two bf16 copies current for the tensor-core GEMMs: the weights as
they are and, for matrices, their transposes (what input-gradient GEMMs read).  ``FusedDenseOptimizer`` updates all of
it with one kernel launch per step (Adagrad / SGD / Adam) that also rewrites the bf16 copies, instead of a multi-tensor
update followed by some forty cast and transpose launches.  Because every address is fixed and no host value changes
from step to step (Adam's step counter lives on the device), the step can be captured in a CUDA graph.

On CPU the same classes run plain torch math, which is the oracle of the kernel test.

The reference uses ``torch.optim`` through ``KeyedOptimizerWrapper`` (``torchrec/optim/keyed.py:425-453``).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

import torch

_ALIGN = 64  # elements: every parameter starts on a 128-byte boundary of the bf16 copies (TMA needs 16)
_OPT_CODE = {"adagrad": 0, "sgd": 1, "adam": 2}


class FlatParamBuffer:
    """Flat master / gradient / bf16 storage for ``params`` (all on one device, fp32)."""

    def __init__(self, params: Sequence[torch.nn.Parameter], grad_alloc: Optional[Callable[[int], torch.Tensor]] = None) -> None:
        self.params: List[torch.nn.Parameter] = list(params)
        assert self.params, "no parameters"
        dev = self.params[0].device
        assert all(p.device == dev and p.dtype == torch.float32 for p in self.params), "fp32 parameters on one device expected"
        self.device = dev
        if dev.type == "cuda":
            from torchrec_b200.ops import _ext

            _ext.require_cuda_ext("fused dense optimizer")  # its one-launch step is a kernel of the CUDA library
        self.offsets: List[int] = []
        total = 0
        for p in self.params:
            self.offsets.append(total)
            total += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.total = max(total, _ALIGN)
        self.master = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.grad = grad_alloc(self.total) if grad_alloc is not None else torch.zeros(self.total, dtype=torch.float32, device=dev)
        assert self.grad.numel() >= self.total and self.grad.dtype == torch.float32
        self.w16 = torch.zeros(self.total, dtype=torch.bfloat16, device=dev)
        self.wT16 = torch.zeros(self.total, dtype=torch.bfloat16, device=dev)
        rows_cols = []
        tile0 = 0
        desc = []
        for p, off in zip(self.params, self.offsets):
            n = p.numel()
            rows, cols = (p.shape[0], n // max(p.shape[0], 1)) if p.dim() >= 2 else (1, n)
            with torch.no_grad():
                self.master[off: off + n].copy_(p.detach().reshape(-1))
            p.data = self.master[off: off + n].view(p.shape)
            p.grad = self.grad[off: off + n].view(p.shape)
            p._trb_flat = self  # type: ignore[attr-defined]
            desc.append([off, rows, cols, tile0, 1 if p.dim() >= 2 else 0])
            tile0 += ((rows + 31) // 32) * ((cols + 31) // 32)
            rows_cols.append((rows, cols))
        self.rows_cols = rows_cols
        self.total_tiles = tile0
        # direct gradient accumulation (ops/dense_ops.py::_grad_sink): valid while every p.grad is its view of the zeroed flat buffer
        self.direct_grads = False
        self.on_direct_write: Optional[Callable[[], None]] = None
        self.desc = torch.tensor(desc, dtype=torch.int64, device=dev).reshape(-1, 5)
        self._register_bf16()
        self.refresh_bf16()

    # ---- views ------------------------------------------------------------------------------------------------------
    def w16_view(self, i: int) -> torch.Tensor:
        p, off = self.params[i], self.offsets[i]
        return self.w16[off: off + p.numel()].view(p.shape)

    def wT16_view(self, i: int) -> Optional[torch.Tensor]:
        p, off = self.params[i], self.offsets[i]
        if p.dim() < 2:
            return None
        rows, cols = self.rows_cols[i]
        return self.wT16[off: off + p.numel()].view(cols, rows)

    def _register_bf16(self) -> None:
        from torchrec_b200.ops.dense_ops import bf16_cache

        for i, p in enumerate(self.params):
            bf16_cache.register(p, self.w16_view(i), self.wT16_view(i))

    def refresh_bf16(self) -> None:
        """Recompute both bf16 copies from the master weights (after a load or an external in-place change)."""
        from torchrec_b200.ops.dense_ops import bf16_cache

        with torch.no_grad():
            self.w16.copy_(self.master)
            for i, p in enumerate(self.params):
                t = self.wT16_view(i)
                if t is not None:
                    rows, cols = self.rows_cols[i]
                    t.copy_(p.detach().reshape(rows, cols).t())
                bf16_cache.mark_fresh(p)

    def attach_grads(self) -> None:
        """Make every ``p.grad`` the view into the flat gradient again (a ``zero_grad(set_to_none=True)`` elsewhere, or a
        first backward that stored its own tensor, detaches it); gradients found elsewhere are copied in."""
        for p, off in zip(self.params, self.offsets):
            view = self.grad[off: off + p.numel()].view(p.shape)
            g = p.grad
            if g is None:
                view.zero_()
                p.grad = view
            elif g.data_ptr() != view.data_ptr():
                view.copy_(g)
                p.grad = view

    def note_direct_write(self) -> None:
        if self.on_direct_write is not None:
            self.on_direct_write()

    def zero_grad(self) -> None:
        self.grad.zero_()
        for p, off in zip(self.params, self.offsets):
            if p.grad is None or p.grad.data_ptr() != self.grad.data_ptr() + 4 * off:
                p.grad = self.grad[off: off + p.numel()].view(p.shape)
        self.direct_grads = True  # from here to the optimizer step, gradient kernels may reduce straight into the flat buffer


def flat_buffer_of(params: Sequence[torch.nn.Parameter]) -> Optional[FlatParamBuffer]:
    """The ``FlatParamBuffer`` that holds exactly ``params`` (in any order), if there is one."""
    bufs = {id(getattr(p, "_trb_flat", None)) for p in params}
    if len(bufs) != 1:
        return None
    buf = getattr(params[0], "_trb_flat", None)
    if buf is None or {id(p) for p in buf.params} != {id(p) for p in params}:
        return None
    return buf


class FusedDenseOptimizer(torch.optim.Optimizer):
    """Adagrad / SGD / Adam over a ``FlatParamBuffer`` in one launch.

    ``params`` that are not yet flat are moved into a new buffer.  State: ``sum`` (Adagrad) or ``exp_avg`` /
    ``exp_avg_sq`` / ``step`` (Adam), exposed per parameter as views so that ``state_dict`` looks like ``torch.optim``'s.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], optimizer: str = "adagrad", lr: float = 0.01, eps: float = 1e-10,
                 betas=(0.9, 0.999), weight_decay: float = 0.0, initial_accumulator_value: float = 0.0) -> None:
        plist = [p for p in params if p.requires_grad]
        assert optimizer in _OPT_CODE, f"unsupported optimizer {optimizer}"
        super().__init__(plist, dict(lr=lr, eps=eps, betas=betas, weight_decay=weight_decay, optimizer=optimizer))
        self.buffer = flat_buffer_of(plist) or FlatParamBuffer(plist)
        b = self.buffer
        self._kind = optimizer
        self.s1 = torch.full((b.total,), float(initial_accumulator_value), dtype=torch.float32, device=b.device) if optimizer != "sgd" else None
        self.s2 = torch.zeros(b.total, dtype=torch.float32, device=b.device) if optimizer == "adam" else None
        self.step_count = torch.zeros(1, dtype=torch.int64, device=b.device)
        names = {"adagrad": ("sum", None), "adam": ("exp_avg", "exp_avg_sq"), "sgd": (None, None)}[optimizer]
        for p, off in zip(b.params, b.offsets):
            st: Dict[str, Any] = {}
            if names[0] is not None:
                st[names[0]] = self.s1[off: off + p.numel()].view(p.shape)
            if names[1] is not None:
                st[names[1]] = self.s2[off: off + p.numel()].view(p.shape)
            if optimizer == "adam":
                st["step"] = self.step_count
            self.state[p] = st

    def zero_grad(self, set_to_none: bool = False) -> None:  # gradients always stay views of the flat buffer
        self.buffer.zero_grad()

    @torch.no_grad()
    def step(self, closure: Any = None) -> None:
        b = self.buffer
        g = self.param_groups[0]
        lr, eps, wd = float(g["lr"]), float(g["eps"]), float(g["weight_decay"])
        b1, b2 = g["betas"]
        if not torch.cuda.is_current_stream_capturing() if b.device.type == "cuda" else True:
            b.attach_grads()
        self.step_count.add_(1)
        b.direct_grads = False
        if b.device.type == "cuda":
            torch.ops.trb200.dense_optimizer_step(b.master, b.grad, self.s1, self.s2, b.w16, b.wT16, b.desc, b.total_tiles, _OPT_CODE[self._kind],
                                                  lr, eps, float(b1), float(b2), wd, self.step_count if self._kind == "adam" else None)
            from torchrec_b200.ops.dense_ops import bf16_cache

            for p in b.params:
                bf16_cache.mark_fresh(p)
            return
        w, gr = b.master, b.grad[: b.total]
        if wd != 0:
            gr = gr + wd * w
        if self._kind == "adagrad":
            self.s1.addcmul_(gr, gr)
            w.addcdiv_(gr, self.s1.sqrt().add_(eps), value=-lr)
        elif self._kind == "sgd":
            w.add_(gr, alpha=-lr)
        else:
            t = float(self.step_count.item())
            self.s1.mul_(b1).add_(gr, alpha=1 - b1)
            self.s2.mul_(b2).addcmul_(gr, gr, value=1 - b2)
            w.addcdiv_(self.s1 / (1 - b1 ** t), (self.s2 / (1 - b2 ** t)).sqrt().add_(eps), value=-lr)
        b.refresh_bf16()
