"""Reserved keys of the ``fused_params`` dictionary.

``fused_params`` travels from a sharder to the table-batched kernels.  Keys that start with ``__register`` are directives for the
sharded *module* (what to expose in ``named_modules``, how the quantized state dict is laid out, row alignment, ...) and must be
stripped before the dictionary reaches a kernel constructor: ``tbe_fused_params`` does that.
Counterpart of ``torchrec/distributed/fused_params.py:20-128``."""
from __future__ import annotations

from typing import Any, Dict, Iterable, Optional

import torch

from torchrec_b200.distributed.types import BoundsCheckMode

FUSED_PARAM_REGISTER_TBE_BOOL: str = "__register_tbes_in_named_modules"
FUSED_PARAM_QUANT_STATE_DICT_SPLIT_SCALE_BIAS: str = "__register_quant_state_dict_split_scale_bias"
FUSED_PARAM_TBE_ROW_ALIGNMENT: str = "__register_tbe_row_alignment"
FUSED_PARAM_BOUNDS_CHECK_MODE: str = "__register_tbe_bounds_check_mode"
# turn lengths into offsets once, ahead of the lookup kernels
FUSED_PARAM_LENGTHS_TO_OFFSETS_LOOKUP: str = "__register_lengths_to_offsets_lookup"
# tables kept on the key-value store behind the embedding cache instead of HBM
FUSED_PARAM_SSD_TABLE_LIST: str = "__register_ssd_table_list"
FUSED_PARAM_IS_SSD_TABLE: str = "__register_is_ssd_table"

_MODULE_LEVEL_KEYS = (
    FUSED_PARAM_REGISTER_TBE_BOOL,
    FUSED_PARAM_QUANT_STATE_DICT_SPLIT_SCALE_BIAS,
    FUSED_PARAM_TBE_ROW_ALIGNMENT,
    FUSED_PARAM_BOUNDS_CHECK_MODE,
    FUSED_PARAM_LENGTHS_TO_OFFSETS_LOOKUP,
    FUSED_PARAM_SSD_TABLE_LIST,
)


class TBEToRegisterMixIn:
    """A lookup that can list its table-batched kernels with the grouped config each one serves."""

    def get_tbes_to_register(self) -> Dict[torch.nn.Module, Any]:
        raise NotImplementedError


def get_tbes_to_register_from_iterable(iterable: Iterable[torch.nn.Module]) -> Dict[torch.nn.Module, Any]:
    found: Dict[torch.nn.Module, Any] = {}
    for m in iterable:
        if isinstance(m, TBEToRegisterMixIn):
            found.update(m.get_tbes_to_register())
    return found


def _flag(fused_params: Optional[Dict[str, Any]], key: str) -> bool:
    return bool(fused_params) and bool(fused_params.get(key, False))


def _value(fused_params: Optional[Dict[str, Any]], key: str, default: Any = None) -> Any:
    return default if not fused_params else fused_params.get(key, default)


def is_fused_param_register_tbe(fused_params: Optional[Dict[str, Any]]) -> bool:
    return _flag(fused_params, FUSED_PARAM_REGISTER_TBE_BOOL)


def is_fused_param_quant_state_dict_split_scale_bias(fused_params: Optional[Dict[str, Any]]) -> bool:
    return _flag(fused_params, FUSED_PARAM_QUANT_STATE_DICT_SPLIT_SCALE_BIAS)


def get_fused_param_tbe_row_alignment(fused_params: Optional[Dict[str, Any]]) -> Optional[int]:
    return _value(fused_params, FUSED_PARAM_TBE_ROW_ALIGNMENT)


def fused_param_bounds_check_mode(fused_params: Optional[Dict[str, Any]]) -> Optional[BoundsCheckMode]:
    return _value(fused_params, FUSED_PARAM_BOUNDS_CHECK_MODE)


def fused_param_lengths_to_offsets_lookup(fused_params: Optional[Dict[str, Any]]) -> bool:
    return bool(_value(fused_params, FUSED_PARAM_LENGTHS_TO_OFFSETS_LOOKUP, False))


def tbe_fused_params(fused_params: Optional[Dict[str, Any]]) -> Optional[Dict[str, Any]]:
    """The subset of ``fused_params`` meant for the kernels (``None`` when empty)."""
    if not fused_params:
        return None
    return {k: v for k, v in fused_params.items() if k not in _MODULE_LEVEL_KEYS}
