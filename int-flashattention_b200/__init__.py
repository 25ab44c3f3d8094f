"""B200-native (sm_100a) INT8 FlashAttention forward.

The directory name contains a hyphen, so import it with
    importlib.import_module("int-flashattention_b200")
from the repository root (or use the drop-in modules under dropin/, which carry the
reference's module names).
"""
from .ops import (attention_full_int8, attention_int8, int_flash_attention, quant_pertoken,
                  quant_pertensor, quant_perchannel, quant_qkv, check_status, default_G)
from . import shard
from .host import HostPipeline
from ._lib import IntfaError, LIB_PATH

__all__ = ["HostPipeline", "attention_full_int8", "attention_int8", "int_flash_attention", "quant_pertoken",
           "quant_pertensor", "quant_perchannel", "quant_qkv", "check_status", "default_G", "shard",
           "IntfaError", "LIB_PATH"]
