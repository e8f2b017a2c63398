"""Perceptron / MLP (counterpart of ``torchrec/modules/mlp.py:18-190``).

Parameter names match the reference (``_mlp.<i>._linear.{weight,bias}``).  On CUDA with the
bf16 dense compute mode a ``Perceptron`` whose activation is ReLU, sigmoid or identity runs as
one fused GEMM+bias+activation tcgen05 kernel (``torchrec_b200.ops.dense_ops.linear_act``).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Union

import torch
from torch import nn

from torchrec_b200.modules.activation import SwishLayerNorm
from torchrec_b200.ops import dense_ops


def extract_module_or_tensor_callable(
    module_or_callable: Union[Callable[[], nn.Module], nn.Module, Callable[[torch.Tensor], torch.Tensor]],
) -> Union[nn.Module, Callable[[torch.Tensor], torch.Tensor]]:
    """A zero-argument factory is called to make a fresh module; modules and tensor functions pass through."""
    try:
        module = module_or_callable()  # type: ignore[call-arg]
        if isinstance(module, nn.Module):
            return module
        raise ValueError("Expected callable that takes no input to return a torch.nn.Module")
    except TypeError as e:
        if "required positional argument" in str(e) or "missing" in str(e) or "takes" in str(e):
            return module_or_callable  # type: ignore[return-value]
        raise


def _act_code(fn) -> Optional[int]:
    if fn is torch.relu or isinstance(fn, nn.ReLU) or fn is torch.nn.functional.relu:
        return dense_ops.ACT_RELU
    if fn is torch.sigmoid or isinstance(fn, nn.Sigmoid):
        return dense_ops.ACT_SIGMOID
    if isinstance(fn, nn.Identity):
        return dense_ops.ACT_NONE
    return None


class Perceptron(nn.Module):
    """Linear transformation followed by an activation."""

    def __init__(
        self,
        in_size: int,
        out_size: int,
        bias: bool = True,
        activation: Union[nn.Module, Callable[[torch.Tensor], torch.Tensor]] = torch.relu,
        device: Optional[torch.device] = None,
        dtype: torch.dtype = torch.float32,
    ) -> None:
        super().__init__()
        self._out_size = out_size
        self._in_size = in_size
        self._linear: nn.Linear = nn.Linear(in_size, out_size, bias=bias, device=device, dtype=dtype)
        self._activation_fn: Callable[[torch.Tensor], torch.Tensor] = activation
        self._act_code = _act_code(activation)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self._act_code is not None and dense_ops.fused_dense_enabled(input):
            return dense_ops.linear_act(input, self._linear.weight, self._linear.bias, self._act_code)
        if dense_ops.fused_dense_enabled(input):
            return self._activation_fn(dense_ops.linear_act(input, self._linear.weight, self._linear.bias, dense_ops.ACT_NONE))
        return self._activation_fn(self._linear(input))


class MLP(nn.Module):
    """A stack of ``Perceptron`` layers."""

    def __init__(
        self,
        in_size: int,
        layer_sizes: List[int],
        bias: bool = True,
        activation: Union[str, Callable[[], nn.Module], nn.Module, Callable[[torch.Tensor], torch.Tensor]] = torch.relu,
        device: Optional[torch.device] = None,
        dtype: torch.dtype = torch.float32,
        activation_on_last: bool = True,
    ) -> None:
        super().__init__()
        if activation == "relu":
            activation = torch.relu
        elif activation == "sigmoid":
            activation = torch.sigmoid
        if not isinstance(activation, str):
            self._mlp: nn.Module = nn.Sequential(
                *[
                    Perceptron(
                        layer_sizes[i - 1] if i > 0 else in_size,
                        layer_sizes[i],
                        bias=bias,
                        activation=(
                            nn.Identity()
                            if not activation_on_last and i == len(layer_sizes) - 1
                            else extract_module_or_tensor_callable(activation)
                        ),
                        device=device,
                        dtype=dtype,
                    )
                    for i in range(len(layer_sizes))
                ]
            )
        elif activation == "swish_layernorm":
            self._mlp = nn.Sequential(
                *[
                    Perceptron(
                        layer_sizes[i - 1] if i > 0 else in_size,
                        layer_sizes[i],
                        bias=bias,
                        activation=(
                            nn.Identity()
                            if not activation_on_last and i == len(layer_sizes) - 1
                            else SwishLayerNorm(layer_sizes[i], device=device)
                        ),
                        device=device,
                    )
                    for i in range(len(layer_sizes))
                ]
            )
        else:
            raise ValueError("MLP supports the activation strings relu, sigmoid and swish_layernorm")

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return self._mlp(input)
