"""Sharded embedding towers, in two forms chosen by the plan.

*One owner* (all tables table-wise on one rank): the ids of the tower's features travel to the owning rank (the table-wise input
distribution of the embedding module), the owner looks the rows up for the *global* batch and runs the interaction on them, and
only the interaction's output -- usually much narrower than the concatenated embeddings -- is sent back through the pooled
all-to-all.  The interaction's parameters are trained on the owning rank only and are excluded from the data-parallel wrapper.

*Spread* (row-wise, table-row-wise, column-wise or table-wise over several ranks): the tables are sharded like any embedding
collection -- on GPUs through the fused engine over peer memory -- every rank receives the pooled rows of its own samples, and the
interaction runs data-parallel on them with replicated parameters (the data-parallel wrapper averages their gradients).  On one
node this is what the reference's table-row-wise tower computes (``torchrec/distributed/embedding_tower_sharding.py:95-440``,
collection ``:442``); over several nodes the reference additionally confines a tower to one node, which this form does not do.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Type

import torch
import torch.distributed as dist
from torch import nn

from torchrec_b200.distributed.comm_ops import alltoall_pooled
from torchrec_b200.distributed.embedding_types import BaseEmbeddingSharder, KJTList, ShardedEmbeddingModule
from torchrec_b200.distributed.embeddingbag import EmbeddingBagCollectionSharder, ShardedEmbeddingBagCollection
from torchrec_b200.distributed.types import Awaitable, LazyAwaitable, NoWait, ParameterSharding, QuantizedCommCodecs, ShardingEnv, ShardingType
from torchrec_b200.modules.embedding_modules import EmbeddingBagCollection
from torchrec_b200.modules.embedding_tower import EmbeddingTower, EmbeddingTowerCollection
from torchrec_b200.sparse.jagged_tensor import KeyedJaggedTensor, KeyedTensor
from torchrec_b200.streamable import Multistreamable


class _TowerOutput(LazyAwaitable[torch.Tensor]):
    def __init__(self, awaitable: Awaitable[torch.Tensor]) -> None:
        super().__init__()
        self._awaitable = awaitable

    def _wait_impl(self) -> torch.Tensor:
        return self._awaitable.wait()


class ShardedEmbeddingTower(ShardedEmbeddingModule):
    def __init__(self, module: EmbeddingTower, table_name_to_parameter_sharding: Dict[str, ParameterSharding], embedding_sharder: EmbeddingBagCollectionSharder,
                 env: ShardingEnv, device: torch.device, module_fqn: Optional[str] = None) -> None:
        super().__init__()
        assert isinstance(module.embedding, EmbeddingBagCollection), "a sharded tower holds an EmbeddingBagCollection"
        kinds = {ps.sharding_type for ps in table_name_to_parameter_sharding.values()}
        owners = {r for ps in table_name_to_parameter_sharding.values() for r in (ps.ranks or [])}
        assert ShardingType.DATA_PARALLEL.value not in kinds, "tower tables are model-parallel"
        self._spread = not (kinds == {ShardingType.TABLE_WISE.value} and len(owners) == 1)
        self._owner = -1 if self._spread else owners.pop()
        self._env, self._device = env, device
        self._rank, self._world = env.rank, env.world_size
        self._pg = env.process_group
        self._active = self._spread or self._rank == self._owner
        self.embedding: ShardedEmbeddingBagCollection = embedding_sharder.shard(module.embedding, table_name_to_parameter_sharding, env=env, device=device,
                                                                              module_fqn=(module_fqn + ".embedding") if module_fqn else None)
        if not self._spread and hasattr(self.embedding, "disable_fused_engine"):
            self.embedding.disable_fused_engine()  # the tower consumes the owner-side lookup before any exchange
        self._lookups = self.embedding._lookups
        self.interaction = module.interaction.to(device) if device.type != "meta" else module.interaction
        self._out_dim: Optional[int] = None

    # ---- stages ------------------------------------------------------------------------------------------------
    def input_dist(self, ctx, features: KeyedJaggedTensor) -> Awaitable[Awaitable[KJTList]]:
        ctx.local_batch = features.stride()
        return self.embedding.input_dist(ctx, features)

    def compute(self, ctx, dist_input: KJTList) -> torch.Tensor:
        embs = self.embedding.compute(ctx, dist_input)
        if self._spread:
            return embs
        assert len(embs) == 1
        pooled = embs[0]
        if self._active:
            sharding = self.embedding._embedding_shardings[0]
            kt = KeyedTensor(keys=sharding.embedding_names(), length_per_key=sharding.embedding_dims(), values=pooled)
            out = self.interaction(kt)
            assert out.dim() == 2 and out.shape[0] == pooled.shape[0], "the interaction must return [batch, features]"
            return out
        # ranks that do not own the tower still take part in the exchange with a zero-width slice
        return torch.empty((dist_input[0].stride(), 0), device=self._device, requires_grad=True)

    def _output_dim(self, out: torch.Tensor) -> int:
        if self._out_dim is None:
            t = torch.tensor([out.shape[1] if self._active else 0], device=self._device if self._device.type == "cuda" else torch.device("cpu"))
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._pg)
            self._out_dim = int(t.item())
        return self._out_dim

    def output_dist(self, ctx, output: torch.Tensor) -> LazyAwaitable[torch.Tensor]:
        if self._spread:
            return _InteractionOnArrival(self.embedding.output_dist(ctx, output), self.interaction)
        O = self._output_dim(output)
        dims = [O if r == self._owner else 0 for r in range(self._world)]
        B = ctx.local_batch
        return _TowerOutput(alltoall_pooled(output.contiguous(), batch_size_per_rank=[B] * self._world, dim_sum_per_rank=dims, group=self._pg))

    def compute_and_output_dist(self, ctx, input: KJTList) -> LazyAwaitable[torch.Tensor]:
        if self._spread:  # the embedding module's own fused lookup + exchange (the engine's path on GPUs)
            return _InteractionOnArrival(self.embedding.compute_and_output_dist(ctx, input), self.interaction)
        return self.output_dist(ctx, self.compute(ctx, input))

    def create_context(self):
        ctx = self.embedding.create_context()
        ctx.local_batch = 0
        return ctx

    # ---- parameters: everything here is owned by one rank ------------------------------------------------------------
    def sharded_parameter_names(self, prefix: str = "") -> Iterator[str]:
        p = prefix + "." if prefix else ""
        yield from self.embedding.sharded_parameter_names(p + "embedding")
        if not self._spread:  # a spread tower's interaction is replicated: the data-parallel wrapper owns its gradients
            for name, _ in self.interaction.named_parameters():
                yield f"{p}interaction.{name}"

    @property
    def owner_rank(self) -> int:
        """The rank that holds a one-owner tower; -1 for a spread tower."""
        return self._owner

    @property
    def unsharded_module_type(self) -> Type[EmbeddingTower]:
        return EmbeddingTower


class _InteractionOnArrival(LazyAwaitable[torch.Tensor]):
    """The spread form's output: the interaction runs on this rank's pooled rows once the embedding exchange has delivered them."""

    def __init__(self, pooled: Awaitable[KeyedTensor], interaction: nn.Module) -> None:
        super().__init__()
        self._pooled, self._interaction = pooled, interaction

    def _wait_impl(self) -> torch.Tensor:
        kt = self._pooled.wait()
        out = self._interaction(kt)
        assert out.dim() == 2 and out.shape[0] == kt.values().shape[0], "the interaction must return [batch, features]"
        return out


class EmbeddingTowerSharder(BaseEmbeddingSharder[EmbeddingTower]):
    def __init__(self, embedding_sharder: Optional[EmbeddingBagCollectionSharder] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._embedding_sharder = embedding_sharder or EmbeddingBagCollectionSharder(qcomm_codecs_registry=self.qcomm_codecs_registry)

    def shard(self, module: EmbeddingTower, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedEmbeddingTower:
        device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        return ShardedEmbeddingTower(module, params, self._embedding_sharder, env, device, module_fqn)

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._embedding_sharder.fused_params

    def shardable_parameters(self, module: EmbeddingTower) -> Dict[str, nn.Parameter]:
        return self._embedding_sharder.shardable_parameters(module.embedding)

    @property
    def module_type(self) -> Type[EmbeddingTower]:
        return EmbeddingTower

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return [ShardingType.TABLE_WISE.value, ShardingType.ROW_WISE.value, ShardingType.TABLE_ROW_WISE.value, ShardingType.COLUMN_WISE.value]


@dataclass
class EmbeddingTowerCollectionContext(Multistreamable):
    """The contexts of the towers of one step of a sharded tower collection, in tower order."""

    embedding_contexts: List[Any] = field(default_factory=list)

    def record_stream(self, stream: torch.Stream) -> None:
        for ctx in self.embedding_contexts:
            ctx.record_stream(stream)


class ShardedEmbeddingTowerCollection(nn.Module):
    """Every tower sharded on its own; ``forward`` concatenates the tower outputs like the unsharded collection."""

    def __init__(self, module: EmbeddingTowerCollection, tower_to_params: List[Dict[str, ParameterSharding]], tower_sharder: EmbeddingTowerSharder, env: ShardingEnv,
                 device: torch.device) -> None:
        super().__init__()
        self.towers = nn.ModuleList([tower_sharder.shard(t, p, env, device, module_fqn=f"towers.{i}") for i, (t, p) in enumerate(zip(module.towers, tower_to_params))])
        self._input_params = module._input_params

    def create_context(self) -> EmbeddingTowerCollectionContext:
        return EmbeddingTowerCollectionContext(embedding_contexts=[tower.create_context() for tower in self.towers])

    def forward(self, features: Optional[KeyedJaggedTensor] = None, weighted_features: Optional[KeyedJaggedTensor] = None) -> torch.Tensor:
        pending = []
        for tower, (has_f, has_w) in zip(self.towers, self._input_params):
            pending.append(tower(features if has_f else weighted_features))
        return torch.cat([p.wait() for p in pending], dim=1)


class EmbeddingTowerCollectionSharder(BaseEmbeddingSharder[EmbeddingTowerCollection]):
    """Shards a whole ``EmbeddingTowerCollection``: the plan names every table of every tower (table names are unique across the
    towers), each tower is sharded on its own with the tower sharder."""

    def __init__(self, tower_sharder: Optional[EmbeddingTowerSharder] = None, qcomm_codecs_registry: Optional[Dict[str, QuantizedCommCodecs]] = None) -> None:
        super().__init__(qcomm_codecs_registry=qcomm_codecs_registry)
        self._tower_sharder = tower_sharder or EmbeddingTowerSharder(qcomm_codecs_registry=self.qcomm_codecs_registry)

    def shard(self, module: EmbeddingTowerCollection, params: Dict[str, ParameterSharding], env: ShardingEnv, device: Optional[torch.device] = None,
              module_fqn: Optional[str] = None) -> ShardedEmbeddingTowerCollection:
        device = device if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        per_tower = []
        for tower in module.towers:
            names = [cfg.name for cfg in tower.embedding.embedding_bag_configs()]
            missing = [n for n in names if n not in params]
            assert not missing, f"the plan has no entry for the tower tables {missing}"
            per_tower.append({n: params[n] for n in names})
        return ShardedEmbeddingTowerCollection(module, per_tower, self._tower_sharder, env, device)

    @property
    def fused_params(self) -> Optional[Dict[str, Any]]:
        return self._tower_sharder.fused_params

    def shardable_parameters(self, module: EmbeddingTowerCollection) -> Dict[str, nn.Parameter]:
        found: Dict[str, nn.Parameter] = {}
        for tower in module.towers:
            for name, p in self._tower_sharder.shardable_parameters(tower).items():
                assert name not in found, f"table {name} appears in more than one tower"
                found[name] = p
        return found

    @property
    def module_type(self) -> Type[EmbeddingTowerCollection]:
        return EmbeddingTowerCollection

    def sharding_types(self, compute_device_type: str) -> List[str]:
        return self._tower_sharder.sharding_types(compute_device_type)


TowerLazyAwaitable = _TowerOutput  # the output of a one-owner tower, under the reference's name
