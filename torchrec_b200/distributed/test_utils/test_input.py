"""Synthetic model inputs (``torchrec/distributed/test_utils/test_input.py``): ``ModelInput`` lives with the test model; ``TdModelInput``
carries the sparse features as a ``TensorDict`` of jagged tensors instead of a KJT."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from torchrec_b200.distributed.test_utils.test_model import ModelInput  # noqa: F401
from torchrec_b200.sparse.tensor_dict import maybe_td_to_kjt


@dataclass
class TdModelInput(ModelInput):
    """``idlist_features`` is a dictionary-of-jagged-tensors container; ``to_kjt()`` converts for modules that want a KJT."""

    @staticmethod
    def generate(*args, **kwargs) -> Tuple["TdModelInput", List["TdModelInput"]]:  # type: ignore[override]
        whole, parts = ModelInput.generate(*args, **kwargs)

        def conv(m: ModelInput) -> "TdModelInput":
            td = m.idlist_features.to_dict() if m.idlist_features is not None else None
            return TdModelInput(m.float_features, td, m.idscore_features, m.label)  # type: ignore[arg-type]

        return conv(whole), [conv(p) for p in parts]

    def to_kjt(self, keys: Optional[List[str]] = None):
        return maybe_td_to_kjt(self.idlist_features, keys)
