"""Sharding planner (cf. ``torchrec/distributed/planner/__init__.py``)."""
from torchrec_b200.distributed.planner.planners import EmbeddingShardingPlanner, HeteroEmbeddingShardingPlanner  # noqa: F401
from torchrec_b200.distributed.planner.types import ParameterConstraints, Topology  # noqa: F401
from torchrec_b200.distributed.planner.utils import bytes_to_gb, sharder_name  # noqa: F401
