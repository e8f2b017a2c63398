"""Semi-synchronous (local-SGD style) training: a *local* optimizer steps every iteration on this rank's replica; every
``num_local_steps`` iterations the replicas are averaged across ranks and a *global* optimizer consumes the averaged
drift as its gradient (DiLoCo style).  Counterpart of ``torchrec/optim/semi_sync.py`` (``SemisyncOptimizer``)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from torchrec_b200.optim.keyed import KeyedOptimizer

SEMI_SYNC_GLOBAL_OPTIM_KEY: str = "semi_sync_global_"
SEMI_SYNC_LOCAL_OPTIM_KEY: str = "semi_sync_local_"
SEMI_SYNC_GLOBAL_STATE_KEY: str = "semi_sync_global_"
SEMI_SYNC_LOCAL_STATE_KEY: str = "semi_sync_local_"


class SemisyncOptimizer(KeyedOptimizer):
    def __init__(self, global_params: Any, optimizer: KeyedOptimizer, local_optimizer: KeyedOptimizer, num_local_steps: int = 16,
                 semi_sync_worker_shift: int = 0, offsync_steps: Optional[int] = None, non_global_params: Optional[Any] = None,
                 process_group: Optional[dist.ProcessGroup] = None) -> None:
        self._optimizer = optimizer
        self._local_optimizer = local_optimizer
        self._num_local_steps = num_local_steps
        self._pg = process_group
        self._local_step_counter = torch.tensor(0, dtype=torch.int64)
        self._global_step_counter = torch.tensor(0, dtype=torch.int64)
        self._global_params: List[torch.Tensor] = list(global_params)
        self._anchor: List[torch.Tensor] = [p.detach().clone() for p in self._global_params]  # values at the last sync
        params = {**{SEMI_SYNC_GLOBAL_OPTIM_KEY + k: v for k, v in optimizer.params.items()}, **{SEMI_SYNC_LOCAL_OPTIM_KEY + k: v for k, v in local_optimizer.params.items()}}
        state = {**dict(optimizer.state), **dict(local_optimizer.state)}
        param_groups = list(optimizer.param_groups) + list(local_optimizer.param_groups)
        super().__init__(params, state, param_groups)
        self.defaults["_save_param_groups"] = False

    @property
    def param_groups(self):
        return list(self._optimizer.param_groups) + list(self._local_optimizer.param_groups)

    @param_groups.setter
    def param_groups(self, v) -> None:
        pass

    def zero_grad(self, set_to_none: bool = False) -> None:
        self._local_optimizer.zero_grad(set_to_none=set_to_none)
        self._optimizer.zero_grad(set_to_none=set_to_none)

    def step(self, closure: Any = None) -> None:
        self._local_optimizer.step(closure)
        self._local_step_counter += 1
        if int(self._local_step_counter) % self._num_local_steps == 0:
            self._global_step()

    @torch.no_grad()
    def _global_step(self) -> None:
        world = dist.get_world_size(self._pg) if dist.is_available() and dist.is_initialized() else 1
        for p, a in zip(self._global_params, self._anchor):
            avg = p.detach().clone()
            if world > 1:
                dist.all_reduce(avg, group=self._pg)
                avg /= world
            # pseudo-gradient: how far the averaged replicas moved away from the anchor
            p.grad = (a - avg).to(p.dtype)
            p.copy_(a)
        self._optimizer.step()
        for p, a in zip(self._global_params, self._anchor):
            a.copy_(p.detach())
            p.grad = None
        self._global_step_counter += 1

    def state_dict(self) -> Dict[str, Any]:
        return {"global": self._optimizer.state_dict(), "local": self._local_optimizer.state_dict(),
                "local_step_counter": self._local_step_counter.clone(), "global_step_counter": self._global_step_counter.clone(),
                "anchor": [a.clone() for a in self._anchor]}

    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        self._optimizer.load_state_dict(state_dict["global"])
        self._local_optimizer.load_state_dict(state_dict["local"])
        self._local_step_counter.copy_(state_dict["local_step_counter"])
        self._global_step_counter.copy_(state_dict["global_step_counter"])
        for a, s in zip(self._anchor, state_dict["anchor"]):
            a.copy_(s)

    def post_load_state_dict(self) -> None:
        self._optimizer.post_load_state_dict()
        self._local_optimizer.post_load_state_dict()

    def save_param_groups(self, save: bool) -> None:
        self._optimizer.save_param_groups(save)
        self._local_optimizer.save_param_groups(save)
