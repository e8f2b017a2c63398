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


class CrossNet(torch.nn.Module):
    """Full-rank cross network: ``x_{l+1} = x_0 * (W_l x_l + b_l) + x_l`` with ``W_l [N, N]``."""

    def __init__(self, in_features: int, num_layers: int) -> None:
        super().__init__()
        self._num_layers = num_layers
        self.kernels: torch.nn.ParameterList = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.xavier_normal_(torch.empty(in_features, in_features))) for _ in range(num_layers)]
        )
        self.bias: torch.nn.ParameterList = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.zeros_(torch.empty(in_features, 1))) for _ in range(num_layers)]
        )

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x_0 = input.unsqueeze(2)  # (B, N, 1)
        x_l = x_0
        for layer in range(self._num_layers):
            xl_w = torch.matmul(self.kernels[layer], x_l)
            x_l = x_0 * (xl_w + self.bias[layer]) + x_l
        return torch.squeeze(x_l, dim=2)


class LowRankCrossNet(torch.nn.Module):
    """Cross network with ``W_l`` factored as ``W_l [N, r] @ V_l [r, N]``."""

    def __init__(self, in_features: int, num_layers: int, low_rank: int = 1) -> None:
        super().__init__()
        assert low_rank >= 1, "Low rank must be larger or equal to 1"
        self._num_layers = num_layers
        self._low_rank = low_rank
        self.W_kernels: torch.nn.ParameterList = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.xavier_normal_(torch.empty(in_features, low_rank))) for _ in range(num_layers)]
        )
        self.V_kernels: torch.nn.ParameterList = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.xavier_normal_(torch.empty(low_rank, in_features))) for _ in range(num_layers)]
        )
        self.bias: torch.nn.ParameterList = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.zeros_(torch.empty(in_features))) for _ in range(num_layers)]
        )

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x_0 = input
        x_l = x_0
        if dense_ops.fused_dense_enabled(input) and input.shape[1] % 8 == 0 and self._low_rank % 8 == 0:
            x_0 = x_0 if x_0.dtype == torch.bfloat16 else x_0.to(torch.bfloat16)
            return dense_ops.lowrank_cross_stack(x_0, list(self.V_kernels), list(self.W_kernels), list(self.bias))
        for layer in range(self._num_layers):
            x_l_v = torch.nn.functional.linear(x_l, self.V_kernels[layer])
            x_l_w = torch.nn.functional.linear(x_l_v, self.W_kernels[layer])
            x_l = x_0 * (x_l_w + self.bias[layer]) + x_l
        return x_l


class VectorCrossNet(torch.nn.Module):
    """DCN-v1 cross network: ``x_{l+1} = x_0 * <w_l, x_l> + b_l + x_l`` with a vector ``w_l``."""

    def __init__(self, in_features: int, num_layers: int) -> None:
        super().__init__()
        self._num_layers = num_layers
        self.kernels: torch.nn.ParameterList = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.xavier_normal_(torch.empty(in_features, 1))) for _ in range(num_layers)]
        )
        self.bias: torch.nn.ParameterList = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.zeros_(torch.empty(in_features, 1))) for _ in range(num_layers)]
        )

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x_0 = input.unsqueeze(2)
        x_l = x_0
        for layer in range(self._num_layers):
            xl_w = torch.tensordot(x_l, self.kernels[layer], dims=([1], [0]))
            x_l = torch.matmul(x_0, xl_w) + self.bias[layer] + x_l
        return torch.squeeze(x_l, dim=2)


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
        self._num_layers = num_layers
        self._num_experts = num_experts
        self._low_rank = low_rank
        self._in_features = in_features
        mk = lambda *s: torch.nn.Parameter(torch.nn.init.xavier_normal_(torch.empty(*s)))  # noqa: E731
        self.U_kernels = torch.nn.ParameterList([mk(num_experts, in_features, low_rank) for _ in range(num_layers)])
        self.V_kernels = torch.nn.ParameterList([mk(num_experts, low_rank, in_features) for _ in range(num_layers)])
        self.bias = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.nn.init.zeros_(torch.empty(in_features, 1))) for _ in range(num_layers)]
        )
        self.gates: Optional[torch.nn.Module] = (
            torch.nn.ModuleList([torch.nn.Linear(in_features, 1, bias=False) for _ in range(num_experts)])
            if num_experts > 1 else None
        )
        self._activation = activation
        self.C_kernels = torch.nn.ParameterList([mk(num_experts, low_rank, low_rank) for _ in range(num_layers)])

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        x_0 = input.unsqueeze(2)
        x_l = x_0
        for layer in range(self._num_layers):
            gating = None
            if self._num_experts > 1:
                gating = torch.stack([self.gates[i](x_l.squeeze(2)) for i in range(self._num_experts)], 1)
            experts = []
            for i in range(self._num_experts):
                e = torch.matmul(self.V_kernels[layer][i], x_l)
                e = torch.matmul(self.C_kernels[layer][i], self._activation(e))
                e = torch.matmul(self.U_kernels[layer][i], self._activation(e))
                e = x_0 * (e + self.bias[layer])
                experts.append(e.squeeze(2))
            experts = torch.stack(experts, 2)
            if gating is not None:
                x_l = torch.matmul(experts, torch.nn.functional.softmax(gating, 1)) + x_l
            else:
                x_l = experts + x_l
        return torch.squeeze(x_l, dim=2)
