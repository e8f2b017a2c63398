"""Tracking of the embedding rows a model touched (delta checkpoints / online publishing)."""
from torchrec_b200.distributed.model_tracker.delta_store import DeltaStore  # noqa: F401
from torchrec_b200.distributed.model_tracker.model_delta_tracker import ModelDeltaTracker  # noqa: F401
from torchrec_b200.distributed.model_tracker.types import DeltaRows, EmbdUpdateMode, IndexedLookup, ModelTrackerConfig, TrackingMode  # noqa: F401
