"""Cross networks (counterpart of ``torchrec/modules/crossnet.py:21-440``).

``LowRankCrossNet`` is the DCN-v2 layer used by ``DLRM_DCN``:
``x_{l+1} = x_0 * (W_l (V_l x_l) + b_l) + x_l``.  On CUDA in bf16 mode each layer is two tcgen05
GEMMs, the second of which applies ``x_0 * (acc + b) + x_l`` in its epilogue
(``torchrec_b200.ops.dense_ops.lowrank_cross_layer``).
"""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch

from torchrec_b200.ops import dense_ops


def _xavier(count: int, *shape: int) -> torch.nn.ParameterList:
    """``count`` Xavier-normal parameters of ``shape`` (one per layer)."""
    return torch.nn.ParameterList([torch.nn.Parameter(torch.nn.init.xavier_normal_(torch.empty(*shape))) for _ in range(count)])


def _zeros(count: int, *shape: int) -> torch.nn.ParameterList:
    return torch.nn.ParameterList([torch.nn.Parameter(torch.zeros(*shape)) for _ in range(count)])


class CrossNet(torch.nn.Module):
    """Full-rank cross network: ``x_{l+1} = x_0 * (W_l x_l + b_l) + x_l`` with ``W_l [N, N]``."""

    def __init__(self, in_features: int, num_layers: int) -> None:
        super().__init__()
        self._num_layers = num_layers
        self.kernels = _xavier(num_layers, in_features, in_features)
        self.bias = _zeros(num_layers, in_features, 1)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x = input
        for w, b in zip(self.kernels, self.bias):  # rows of the batch are independent: plain [B, N] algebra
            x = torch.addcmul(x, input, torch.nn.functional.linear(x, w, b.view(-1)))
        return x


class LowRankCrossNet(torch.nn.Module):
    """Cross network with ``W_l`` factored as ``W_l [N, r] @ V_l [r, N]``."""

    def __init__(self, in_features: int, num_layers: int, low_rank: int = 1) -> None:
        super().__init__()
        assert low_rank >= 1, "Low rank must be larger or equal to 1"
        self._num_layers, self._low_rank = num_layers, low_rank
        self.W_kernels = _xavier(num_layers, in_features, low_rank)
        self.V_kernels = _xavier(num_layers, low_rank, in_features)
        self.bias = _zeros(num_layers, in_features)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        tensor_core_shapes = input.shape[1] % 8 == 0 and self._low_rank % 8 == 0
        if tensor_core_shapes and dense_ops.fused_dense_enabled(input):
            x0 = input if input.dtype == torch.bfloat16 else input.to(torch.bfloat16)
            return dense_ops.lowrank_cross_stack(x0, list(self.V_kernels), list(self.W_kernels), list(self.bias))
        x = input
        for v, w, b in zip(self.V_kernels, self.W_kernels, self.bias):
            projected = torch.nn.functional.linear(torch.nn.functional.linear(x, v), w, b)
            x = torch.addcmul(x, input, projected)
        return x


class VectorCrossNet(torch.nn.Module):
    """DCN-v1 cross network: ``x_{l+1} = x_0 * <w_l, x_l> + b_l + x_l`` with a vector ``w_l``."""

    def __init__(self, in_features: int, num_layers: int) -> None:
        super().__init__()
        self._num_layers = num_layers
        self.kernels = _xavier(num_layers, in_features, 1)
        self.bias = _zeros(num_layers, in_features, 1)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x = input
        for w, b in zip(self.kernels, self.bias):
            x = input * (x @ w) + b.view(-1) + x  # (x @ w) is one scalar per sample
        return x


class LowRankMixtureCrossNet(torch.nn.Module):
    """Mixture of low-rank experts per layer with a softmax gate over experts."""

    def __init__(
        self,
        in_features: int,
        num_layers: int,
        num_experts: int = 1,
        low_rank: int = 1,
        activation: Union[torch.nn.Module, Callable[[torch.Tensor], torch.Tensor]] = torch.relu,
    ) -> None:
        super().__init__()
        assert num_experts >= 1, "num_experts must be larger or equal to 1"
        assert low_rank >= 1, "Low rank must be larger or equal to 1"
        self._num_layers, self._num_experts, self._low_rank, self._in_features = num_layers, num_experts, low_rank, in_features
        self._activation = activation
        self.U_kernels = _xavier(num_layers, num_experts, in_features, low_rank)
        self.V_kernels = _xavier(num_layers, num_experts, low_rank, in_features)
        self.bias = _zeros(num_layers, in_features, 1)
        self.gates: Optional[torch.nn.Module] = None
        if num_experts > 1:
            self.gates = torch.nn.ModuleList([torch.nn.Linear(in_features, 1, bias=False) for _ in range(num_experts)])
        self.C_kernels = _xavier(num_layers, num_experts, low_rank, low_rank)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        act = self._activation
        x = input
        for u, c, v, b in zip(self.U_kernels, self.C_kernels, self.V_kernels, self.bias):
            # all experts at once: [B, N] -> [B, E, r] -> [B, E, r] -> [B, E, N]
            h = act(torch.einsum("ern,bn->ber", v, x))
            h = act(torch.einsum("ers,bes->ber", c, h))
            experts = input.unsqueeze(1) * (torch.einsum("enr,ber->ben", u, h) + b.view(1, 1, -1))
            if self.gates is None:
                x = experts.squeeze(1) + x
            else:
                scores = torch.cat([gate(x) for gate in self.gates], dim=1)  # [B, E]
                x = torch.einsum("ben,be->bn", experts, torch.softmax(scores, dim=1)) + x
        return x
