"""B200-native generation-phase attention over the paged KV cache (drop-in for the decode branch
of TensorRT-LLM's GPT attention plugin).

The directory name contains a hyphen, so import it through ``__graft_entry__.load_package()``
(registers it as ``tensorrt_llm_b200``) or put an importlib spec on it yourself.
"""
from .plugin import (DX_OK, DecodeAttnError, GPTAttentionPlugin, PositionEmbeddingType, QuantMode,  # noqa: F401
                     RotaryScalingType, gpt_attention, library_path, load_library)
from . import kv_cache_manager  # noqa: F401
from .kv_cache_manager import GenerationSequence, KVCacheManager  # noqa: F401

__all__ = ["GPTAttentionPlugin", "QuantMode", "gpt_attention", "DecodeAttnError", "load_library", "library_path",
           "DX_OK"]
