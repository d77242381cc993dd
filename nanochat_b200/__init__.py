"""B200-native (sm_100a) decode hot path of the nanochat fork: fp8 (e4m3) KV-cache append/quantise and
single-token attention over that cache, behind a ctypes C ABI (include/nanochat_b200.h)."""

from .attention import (decode_attention, decode_attention_partial, decode_step_attention, kv_append, merge_partials, rotary_table,
                        workspace_bytes)
from .kv_cache import Fp8KVCache
from .native import NativeError, build_library, cuda_library
from .step import DecodeStep

__all__ = ["DecodeStep", "Fp8KVCache", "NativeError", "build_library", "cuda_library", "decode_attention",
           "decode_attention_partial", "decode_step_attention", "kv_append", "merge_partials", "rotary_table", "workspace_bytes"]
