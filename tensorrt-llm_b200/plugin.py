"""Host-side mirror of the reference operator for the generation phase, over the C ABI.

``GPTAttentionPlugin`` keeps the static attributes of the reference plugin
(cpp/tensorrt_llm/plugins/gptAttentionCommon/gptAttentionCommon.cpp:1558-1596) and its
``enqueue_generation`` takes the per-step tensors of ``tensorrt_llm.functional.gpt_attention``
(tensorrt_llm/functional.py:3487-3906: qkv, sequence_length, host_past_key_value_lengths,
kv_cache_block_pointers, kv_orig_quant_scale, kv_quant_orig_scale ...) with the same names and
meaning.  torch is used only for device memory and streams; all compute happens in
libdecode_attn.so, which must be present - there is no fallback path.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

DX_OK, DX_ERR_BAD_ARG, DX_ERR_UNSUPPORTED, DX_ERR_WORKSPACE, DX_ERR_CUDA, DX_ERR_TIMEOUT, DX_ERR_BOUNDS = range(7)
DX_DTYPE_FP16, DX_DTYPE_BF16 = 0, 1

_LIB: Optional[ctypes.CDLL] = None


class PositionEmbeddingType:
    """Values of tensorrt_llm::kernels::PositionEmbeddingType (cpp/tensorrt_llm/kernels/gptKernels.h:41-51)."""
    learned_absolute = 0
    rope_gptj = 1
    rope_gpt_neox = 2
    alibi = 3
    alibi_with_scale = 4
    relative = 5


class RotaryScalingType:
    """Values of tensorrt_llm::kernels::RotaryScalingType (cpp/tensorrt_llm/kernels/gptKernels.h:53-58)."""
    none = 0
    linear = 1
    dynamic = 2


class QuantMode:
    """Bit values of tensorrt_llm.quantization.mode.QuantMode that concern the KV cache
    (tensorrt_llm/quantization/mode.py:47-49)."""
    NONE = 0
    INT8_KV_CACHE = 1 << 6
    FP8_KV_CACHE = 1 << 7


class DecodeAttnError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {_strerror(status)} (status {status})")


class _Config(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("layer_idx", ctypes.c_int32), ("num_heads", ctypes.c_int32),
                ("num_kv_heads", ctypes.c_int32), ("head_size", ctypes.c_int32), ("q_scaling", ctypes.c_float),
                ("tp_size", ctypes.c_int32), ("tp_rank", ctypes.c_int32), ("multi_block_mode", ctypes.c_int32),
                ("enable_xqa", ctypes.c_int32), ("kv_cache_quant_mode", ctypes.c_int32),
                ("paged_kv_cache", ctypes.c_int32), ("tokens_per_block", ctypes.c_int32),
                ("type_id", ctypes.c_int32), ("device", ctypes.c_int32),
                ("position_embedding_type", ctypes.c_int32), ("rotary_embedding_dim", ctypes.c_int32),
                ("rotary_embedding_base", ctypes.c_float), ("rotary_embedding_scale_type", ctypes.c_int32),
                ("rotary_embedding_scale", ctypes.c_float), ("rotary_embedding_max_positions", ctypes.c_int32),
                ("qkv_bias_enabled", ctypes.c_int32)]


class _GenParams(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("attention_input", ctypes.c_void_p),
                ("sequence_lengths", ctypes.c_void_p), ("host_past_key_value_lengths", ctypes.c_void_p),
                ("past_kv_length", ctypes.c_int32), ("beam_width", ctypes.c_int32),
                ("num_requests", ctypes.c_int32), ("max_blocks_per_sequence", ctypes.c_int32),
                ("max_attention_window", ctypes.c_int32), ("cyclic_attention_window_size", ctypes.c_int32),
                ("sink_token_length", ctypes.c_int32), ("block_pointers", ctypes.c_void_p),
                ("host_block_pointers", ctypes.c_void_p), ("kv_scale_orig_quant", ctypes.c_void_p),
                ("kv_scale_quant_orig", ctypes.c_void_p), ("context_buf", ctypes.c_void_p),
                ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
                ("cache_indir", ctypes.c_void_p), ("qkv_bias", ctypes.c_void_p),
                ("context_lengths", ctypes.c_void_p), ("alibi_slopes", ctypes.c_void_p),
                ("input_seq_length", ctypes.c_int32), ("reserved0", ctypes.c_int32),
                ("medusa_packed_mask", ctypes.c_void_p), ("medusa_position_offsets", ctypes.c_void_p),
                ("relative_attention_bias", ctypes.c_void_p), ("relative_attention_bias_stride", ctypes.c_int32),
                ("max_distance", ctypes.c_int32)]


EXPORTED_SYMBOLS = [
    "dx_abi_version", "dx_strerror", "dx_attn_create", "dx_attn_destroy", "dx_attn_workspace_size",
    "dx_attn_enqueue_generation", "dx_attn_enqueue_generation_host", "dx_attn_host_sync", "dx_kv_cache_step", "dx_attn_validate", "dx_attn_plan", "dx_attn_plan_lengths",
    "dx_attn_device_status", "dx_attn_last_cuda_error", "dx_attn_launch_count",
    "dx_attn_enqueue_generation_static_scratch", "dx_attn_static_scratch_bytes", "dx_attn_append_context",
    "dx_attn_append_context_cyclic", "dx_build_has_bounds_check", "dx_attn_set_pool_range",
    "dx_attn_selftest_wait_timeout",
]


def library_path() -> Path:
    override = os.environ.get("DX_DECODE_ATTN_LIB")  # alternative build of the same library (tuning)
    return Path(override) if override else Path(__file__).resolve().parent / "libdecode_attn.so"


def load_library() -> ctypes.CDLL:
    """Loads libdecode_attn.so; raises if it has not been built (no fallback exists)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        raise RuntimeError(f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`; "
                           "this package has no non-CUDA path")
    lib = ctypes.CDLL(str(path))
    lib.dx_abi_version.restype = ctypes.c_int
    lib.dx_strerror.restype = ctypes.c_char_p
    lib.dx_strerror.argtypes = [ctypes.c_int]
    lib.dx_attn_create.restype = ctypes.c_int
    lib.dx_attn_create.argtypes = [ctypes.POINTER(_Config), ctypes.POINTER(ctypes.c_void_p)]
    lib.dx_attn_destroy.restype = None
    lib.dx_attn_destroy.argtypes = [ctypes.c_void_p]
    lib.dx_attn_workspace_size.restype = ctypes.c_size_t
    lib.dx_attn_workspace_size.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32]
    lib.dx_attn_enqueue_generation.restype = ctypes.c_int
    lib.dx_attn_enqueue_generation.argtypes = [ctypes.c_void_p, ctypes.POINTER(_GenParams), ctypes.c_void_p]
    lib.dx_attn_enqueue_generation_host.restype = ctypes.c_int
    lib.dx_attn_enqueue_generation_host.argtypes = [ctypes.c_void_p, ctypes.POINTER(_GenParams), ctypes.c_void_p,
                                                    ctypes.c_int32]
    lib.dx_kv_cache_step.restype = ctypes.c_int
    lib.dx_kv_cache_step.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                     ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.dx_attn_host_sync.restype = ctypes.c_int
    lib.dx_attn_host_sync.argtypes = [ctypes.c_void_p]
    lib.dx_attn_enqueue_generation_static_scratch.restype = ctypes.c_int
    lib.dx_attn_enqueue_generation_static_scratch.argtypes = [ctypes.c_void_p, ctypes.POINTER(_GenParams),
                                                              ctypes.c_void_p]
    lib.dx_attn_static_scratch_bytes.restype = ctypes.c_size_t
    lib.dx_attn_append_context.restype = ctypes.c_int
    lib.dx_attn_append_context.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                                           ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.dx_attn_append_context_cyclic.restype = ctypes.c_int
    lib.dx_attn_append_context_cyclic.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                  ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                                  ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    lib.dx_build_has_bounds_check.restype = ctypes.c_int
    lib.dx_attn_set_pool_range.restype = ctypes.c_int
    lib.dx_attn_set_pool_range.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    lib.dx_attn_validate.restype = ctypes.c_int
    lib.dx_attn_validate.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                     ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t]
    lib.dx_attn_plan_lengths.restype = ctypes.c_int
    lib.dx_attn_plan_lengths.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                         ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32),
                                         ctypes.POINTER(ctypes.c_int32)]
    lib.dx_attn_plan.restype = ctypes.c_int
    lib.dx_attn_plan.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.POINTER(ctypes.c_int32),
                                 ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
    lib.dx_attn_selftest_wait_timeout.restype = ctypes.c_int
    lib.dx_attn_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
    lib.dx_attn_device_status.restype = ctypes.c_int
    lib.dx_attn_device_status.argtypes = [ctypes.c_void_p]
    lib.dx_attn_last_cuda_error.restype = ctypes.c_int
    lib.dx_attn_last_cuda_error.argtypes = [ctypes.c_void_p]
    lib.dx_attn_launch_count.restype = ctypes.c_int64
    lib.dx_attn_launch_count.argtypes = [ctypes.c_void_p]
    if lib.dx_abi_version() != 1:
        raise RuntimeError("libdecode_attn.so has an unexpected ABI version")
    _LIB = lib
    return lib


def _strerror(status: int) -> str:
    return load_library().dx_strerror(status).decode()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class GPTAttentionPlugin:
    """One instance per (GPU, layer configuration), like one plugin object per engine layer."""

    def __init__(self, *, num_heads: int, num_kv_heads: int, head_size: int, q_scaling: float = 1.0,
                 tp_size: int = 1, tp_rank: int = 0, multi_block_mode: bool = False, enable_xqa: bool = True,
                 kv_cache_quant_mode: int = QuantMode.NONE, paged_kv_cache: bool = True, tokens_per_block: int = 64,
                 type_id: torch.dtype = torch.float16, layer_idx: int = 0, device: int = 0,
                 position_embedding_type: int = PositionEmbeddingType.learned_absolute,
                 rotary_embedding_dim: int = 0, rotary_embedding_base: float = 10000.0,
                 rotary_embedding_scale_type: int = RotaryScalingType.none, rotary_embedding_scale: float = 1.0,
                 rotary_embedding_max_positions: int = 1024, qkv_bias: bool = False):
        if type_id not in (torch.float16, torch.bfloat16):
            raise DecodeAttnError(DX_ERR_UNSUPPORTED, "type_id")
        self.lib = load_library()
        self.dtype = type_id
        self.num_heads, self.num_kv_heads, self.head_size = num_heads, num_kv_heads, head_size
        self.tokens_per_block = tokens_per_block
        self.kv_cache_quant_mode = kv_cache_quant_mode
        self.device = device
        cfg = _Config(ctypes.sizeof(_Config), layer_idx, num_heads, num_kv_heads, head_size, q_scaling, tp_size,
                      tp_rank, int(multi_block_mode), int(enable_xqa), kv_cache_quant_mode, int(paged_kv_cache),
                      tokens_per_block, DX_DTYPE_FP16 if type_id == torch.float16 else DX_DTYPE_BF16, device,
                      position_embedding_type, rotary_embedding_dim, rotary_embedding_base,
                      rotary_embedding_scale_type, rotary_embedding_scale, rotary_embedding_max_positions,
                      int(qkv_bias))
        handle = ctypes.c_void_p()
        st = self.lib.dx_attn_create(ctypes.byref(cfg), ctypes.byref(handle))
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_attn_create")
        self._h = handle
        self._workspace: Optional[torch.Tensor] = None

    def close(self) -> None:
        if getattr(self, "_h", None):
            self.lib.dx_attn_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # --- reference: getWorkspaceSizeForGeneration ---
    def get_workspace_size(self, batch: int, max_past_len: int) -> int:
        return int(self.lib.dx_attn_workspace_size(self._h, batch, max_past_len))

    def plan(self, batch: int, max_past_len: int, host_past_key_value_lengths: Optional[torch.Tensor] = None):
        """Split-K plan of the next enqueue: for the given host lengths when passed (what the enqueue itself
        plans), else for a batch in which every sequence has max_past_len tokens."""
        n, c, k = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        if host_past_key_value_lengths is not None:
            hp = host_past_key_value_lengths.to(torch.int32).contiguous().cpu()
            st = self.lib.dx_attn_plan_lengths(self._h, ctypes.c_void_p(hp.data_ptr()), hp.numel(), ctypes.byref(n),
                                               ctypes.byref(c), ctypes.byref(k))
        else:
            st = self.lib.dx_attn_plan(self._h, batch, max_past_len, ctypes.byref(n), ctypes.byref(c), ctypes.byref(k))
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_attn_plan")
        kernel = {0: "mha_cuda_core", 1: "gqa_tensor_core", 2: "wide_group_tcgen05",
                  3: "token_major_tcgen05", 4: "token_major_tcgen05_persistent", 5: "general_cuda_core"}.get(k.value, "?")
        if n.value < 0:  # stream-K launch: equal token ranges per CTA
            return {"num_partitions": 0, "tokens_per_partition": c.value, "kernel": kernel,
                    "stream_k_ctas": -n.value}
        return {"num_partitions": n.value, "tokens_per_partition": c.value, "kernel": kernel}

    def set_pool_range(self, pool: Optional[torch.Tensor]) -> None:
        """Bounds-checked build: the only memory cache blocks may lie in (None: no range)."""
        st = self.lib.dx_attn_set_pool_range(self._h, _ptr(pool), 0 if pool is None else pool.numel() * pool.element_size())
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_attn_set_pool_range")

    def launch_count(self) -> int:
        return int(self.lib.dx_attn_launch_count(self._h))

    def device_status(self) -> int:
        return int(self.lib.dx_attn_device_status(self._h))

    def validate(self, host_kv_cache_block_pointers: torch.Tensor, host_past_key_value_lengths: torch.Tensor,
                 pool_base: int, pool_bytes: int) -> int:
        t = host_kv_cache_block_pointers.contiguous()
        l = host_past_key_value_lengths.to(torch.int32).contiguous()
        return int(self.lib.dx_attn_validate(self._h, t.data_ptr(), l.data_ptr(), l.numel(), t.shape[-1],
                                             pool_base, pool_bytes))

    def _params(self, qkv, sequence_length, host_past_key_value_lengths, kv_cache_block_pointers,
                kv_orig_quant_scale, kv_quant_orig_scale, out, workspace, max_attention_window,
                host_kv_cache_block_pointers=None, cache_indirection=None, beam_width=1, sink_token_length=0,
                qkv_bias=None, cyclic_attention_window_size=None, context_lengths=None, alibi_slopes=None,
                input_seq_length=1, medusa_packed_mask=None, medusa_position_offsets=None,
                relative_attention_bias=None, max_distance=0):
        B = qkv.shape[0] // max(1, input_seq_length)
        M = kv_cache_block_pointers.shape[-1]
        hp = host_past_key_value_lengths
        max_past = int(hp.max()) if hp is not None and hp.numel() else 0
        window = max_attention_window if max_attention_window is not None else M * self.tokens_per_block
        p = _GenParams()
        p.struct_size = ctypes.sizeof(_GenParams)
        p.attention_input = _ptr(qkv)
        p.sequence_lengths = _ptr(sequence_length)
        p.host_past_key_value_lengths = _ptr(hp)
        p.past_kv_length = max_past
        p.beam_width = beam_width
        p.num_requests = B // max(1, beam_width)
        p.max_blocks_per_sequence = M
        p.max_attention_window = window
        p.cyclic_attention_window_size = window if cyclic_attention_window_size is None else cyclic_attention_window_size
        p.sink_token_length = sink_token_length
        p.block_pointers = _ptr(kv_cache_block_pointers)
        p.host_block_pointers = _ptr(host_kv_cache_block_pointers)
        p.kv_scale_orig_quant = _ptr(kv_orig_quant_scale)
        p.kv_scale_quant_orig = _ptr(kv_quant_orig_scale)
        p.context_buf = _ptr(out)
        p.workspace = _ptr(workspace)
        p.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
        p.cache_indir = _ptr(cache_indirection)
        p.qkv_bias = _ptr(qkv_bias)
        p.context_lengths = _ptr(context_lengths)
        p.alibi_slopes = _ptr(alibi_slopes)
        p.input_seq_length = input_seq_length
        p.medusa_packed_mask = _ptr(medusa_packed_mask)
        p.medusa_position_offsets = _ptr(medusa_position_offsets)
        p.relative_attention_bias = _ptr(relative_attention_bias)
        p.relative_attention_bias_stride = 0 if relative_attention_bias is None else int(relative_attention_bias.shape[1])
        p.max_distance = max_distance
        return p, max_past

    def _ensure_workspace(self, batch: int, max_past: int, device) -> Optional[torch.Tensor]:
        need = self.get_workspace_size(batch, max_past)
        if need == 0:
            return None
        if self._workspace is None or self._workspace.numel() < need or self._workspace.device != device:
            self._workspace = torch.empty(need, dtype=torch.uint8, device=device)
        return self._workspace

    # --- reference: enqueueGeneration ---
    def enqueue_generation(self, qkv: torch.Tensor, sequence_length: torch.Tensor,
                           host_past_key_value_lengths: torch.Tensor, kv_cache_block_pointers: torch.Tensor,
                           kv_orig_quant_scale: Optional[torch.Tensor] = None,
                           kv_quant_orig_scale: Optional[torch.Tensor] = None, *, out: Optional[torch.Tensor] = None,
                           workspace: Optional[torch.Tensor] = None, max_attention_window: Optional[int] = None,
                           host_kv_cache_block_pointers: Optional[torch.Tensor] = None,
                           cache_indirection: Optional[torch.Tensor] = None, beam_width: int = 1,
                           sink_token_length: int = 0, qkv_bias: Optional[torch.Tensor] = None,
                           cyclic_attention_window_size: Optional[int] = None,
                           context_lengths: Optional[torch.Tensor] = None,
                           alibi_slopes: Optional[torch.Tensor] = None,
                           medusa_packed_mask: Optional[torch.Tensor] = None,
                           medusa_position_offsets: Optional[torch.Tensor] = None,
                           relative_attention_bias: Optional[torch.Tensor] = None, max_distance: int = 0,
                           stream: Optional[torch.cuda.Stream] = None, static_scratch: bool = False) -> torch.Tensor:
        """qkv: T [B, (H+2Hkv)*Dh] (device); sequence_length: int32 [B] (device, includes the new token);
        host_past_key_value_lengths: int32 [B] (host); kv_cache_block_pointers: int64 [B, 2, M] (device).
        Appends the new token to the cache and returns the attention output T [B, H*Dh].  Asynchronous.
        Beam search: B = batch * beam_width, cache_indirection int32 [B, max_attention_window] and
        context_lengths int32 [B] on the device.  Sliding window: cyclic_attention_window_size (and
        sink_token_length).  ALiBi: alibi_slopes T [H] on the device (plugin built with an ALiBi type).
        Several new tokens per sequence (the reference's Medusa mode): medusa_packed_mask int32
        [B, Q, ceil(Q / 32)] on the device (and optionally medusa_position_offsets int32 [B, Q]); qkv and the
        result then have B * Q rows and sequence_length includes all Q new tokens.
        Relative attention bias (plugin built with position_embedding_type 5): relative_attention_bias T
        [H, max_seq_len, max_seq_len] on the device, or with max_distance > 0 the bucket table T [H, buckets].
        static_scratch: no workspace is allocated or passed; the step runs through
        dx_attn_enqueue_generation_static_scratch on the fixed scratch array inside the library."""
        if not qkv.is_cuda:
            raise DecodeAttnError(DX_ERR_BAD_ARG, "enqueue_generation needs device tensors (no CPU path exists)")
        if qkv.dtype != self.dtype:
            raise DecodeAttnError(DX_ERR_BAD_ARG, "qkv dtype")
        B = qkv.shape[0]  # rows: sequences x new tokens per sequence
        q_len = 1 if medusa_packed_mask is None else int(medusa_packed_mask.shape[-2])
        if out is None:
            out = torch.empty(B, self.num_heads * self.head_size, dtype=self.dtype, device=qkv.device)
        hp = host_past_key_value_lengths.to(torch.int32).contiguous()
        max_past = int(hp.max()) if hp.numel() else 0
        if workspace is None and not static_scratch:
            workspace = self._ensure_workspace(B, max_past, qkv.device)
        p, _ = self._params(qkv, sequence_length, hp, kv_cache_block_pointers, kv_orig_quant_scale,
                            kv_quant_orig_scale, out, workspace, max_attention_window,
                            host_kv_cache_block_pointers, cache_indirection, beam_width, sink_token_length, qkv_bias,
                            cyclic_attention_window_size, context_lengths, alibi_slopes, q_len,
                            None if medusa_packed_mask is None else medusa_packed_mask.contiguous(),
                            None if medusa_position_offsets is None else medusa_position_offsets.contiguous(),
                            None if relative_attention_bias is None else relative_attention_bias.contiguous(),
                            max_distance)
        s = stream if stream is not None else torch.cuda.current_stream(qkv.device)
        enqueue = (self.lib.dx_attn_enqueue_generation_static_scratch if static_scratch
                   else self.lib.dx_attn_enqueue_generation)
        st = enqueue(self._h, ctypes.byref(p), ctypes.c_void_p(s.cuda_stream))
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_attn_enqueue_generation")
        return out

    # --- reference: invokeTranspose4dBatchMajor (context-phase KV write) ---
    def append_context(self, k: torch.Tensor, v: torch.Tensor, sequence_length: torch.Tensor,
                       kv_cache_block_pointers: torch.Tensor, kv_orig_quant_scale: Optional[torch.Tensor] = None,
                       *, attention_window_size: Optional[int] = None, sink_token_length: int = 0,
                       stream: Optional[torch.cuda.Stream] = None) -> None:
        """k, v: T [B, Hkv, seq_len, Dh] (device, contiguous); stores tokens < sequence_length[b] of every
        sequence into the paged cache, quantising on write.  attention_window_size shorter than a sequence: the
        cache is cyclic and keeps the last attention_window_size tokens (sink tokens keep their slots).
        Asynchronous."""
        if not (k.is_cuda and v.is_cuda and k.is_contiguous() and v.is_contiguous()):
            raise DecodeAttnError(DX_ERR_BAD_ARG, "append_context needs contiguous device tensors")
        B, Hkv, L, Dh = k.shape
        if Hkv != self.num_kv_heads or Dh != self.head_size or k.dtype != self.dtype or v.shape != k.shape:
            raise DecodeAttnError(DX_ERR_BAD_ARG, "append_context shapes")
        M = kv_cache_block_pointers.shape[-1]
        window = attention_window_size if attention_window_size is not None else M * self.tokens_per_block
        s = stream if stream is not None else torch.cuda.current_stream(k.device)
        st = self.lib.dx_attn_append_context_cyclic(self._h, k.data_ptr(), v.data_ptr(), sequence_length.data_ptr(),
                                                    B, L, window, sink_token_length,
                                                    kv_cache_block_pointers.data_ptr(), M,
                                                    _ptr(kv_orig_quant_scale), ctypes.c_void_p(s.cuda_stream))
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_attn_append_context_cyclic")

    def bind_generation(self, qkv: torch.Tensor, sequence_length: torch.Tensor,
                        host_past_key_value_lengths: torch.Tensor, kv_cache_block_pointers: torch.Tensor,
                        kv_orig_quant_scale: Optional[torch.Tensor] = None,
                        kv_quant_orig_scale: Optional[torch.Tensor] = None, *, out: torch.Tensor,
                        workspace: Optional[torch.Tensor] = None, max_attention_window: Optional[int] = None,
                        stream: Optional[torch.cuda.Stream] = None, host: bool = False, sync: bool = True):
        """Pre-marshals one step's arguments and returns a zero-argument callable that only makes the C
        call (a C++ caller has no marshalling cost; this keeps Python's out of timed loops).  The tensors
        must stay alive and unchanged in place while the callable is used.  host=True binds the
        host-buffer entry point instead."""
        hp = host_past_key_value_lengths.to(torch.int32).contiguous()
        max_past = int(hp.max()) if hp.numel() else 0
        dev = torch.device("cuda", self.device)
        if workspace is None:
            workspace = self._ensure_workspace(qkv.shape[0], max_past, dev)
        p, _ = self._params(qkv, sequence_length, hp, kv_cache_block_pointers, kv_orig_quant_scale,
                            kv_quant_orig_scale, out, workspace, max_attention_window)
        s = stream if stream is not None else torch.cuda.current_stream(dev)
        sp = ctypes.c_void_p(s.cuda_stream)
        pref = ctypes.byref(p)
        keep = (p, hp, workspace, qkv, sequence_length, kv_cache_block_pointers, out)
        h = self._h
        if host:
            fn, flag = self.lib.dx_attn_enqueue_generation_host, int(sync)

            def call(_keep=keep):
                st = fn(h, pref, sp, flag)
                if st != DX_OK:
                    raise DecodeAttnError(st, "dx_attn_enqueue_generation_host")
        else:
            fn = self.lib.dx_attn_enqueue_generation

            def call(_keep=keep):
                st = fn(h, pref, sp)
                if st != DX_OK:
                    raise DecodeAttnError(st, "dx_attn_enqueue_generation")
        return call

    def kv_cache_step(self, sequence_length: torch.Tensor, kv_cache_block_pointers: torch.Tensor,
                      free_blocks: torch.Tensor, free_cursor: torch.Tensor,
                      stream: Optional[torch.cuda.Stream] = None) -> None:
        """Device-resident KVCacheManager.step: sequence_length (int32 [B], device) += 1 in place; sequences whose
        new token starts a block take the next (K pointer, V pointer) row of free_blocks (int64 [n, 2], device)
        into kv_cache_block_pointers (int64 [B, 2, M], device) in place; free_cursor (int32 [1], device)
        advances.  Asynchronous; capturable in a CUDA graph."""
        for t in (sequence_length, kv_cache_block_pointers, free_blocks, free_cursor):
            if not t.is_cuda or not t.is_contiguous():
                raise DecodeAttnError(DX_ERR_BAD_ARG, "kv_cache_step needs contiguous device tensors")
        s = stream if stream is not None else torch.cuda.current_stream(sequence_length.device)
        st = self.lib.dx_kv_cache_step(self._h, sequence_length.data_ptr(), kv_cache_block_pointers.data_ptr(),
                                       sequence_length.numel(), kv_cache_block_pointers.shape[-1],
                                       free_blocks.data_ptr(), free_blocks.shape[0], free_cursor.data_ptr(),
                                       ctypes.c_void_p(s.cuda_stream))
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_kv_cache_step")

    def host_sync(self) -> None:
        """Waits until the outputs of all host-buffer calls made so far are in host memory."""
        st = self.lib.dx_attn_host_sync(self._h)
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_attn_host_sync")

    def enqueue_generation_host(self, qkv: torch.Tensor, sequence_length: torch.Tensor,
                                host_past_key_value_lengths: torch.Tensor, kv_cache_block_pointers: torch.Tensor,
                                kv_orig_quant_scale: Optional[torch.Tensor], kv_quant_orig_scale: Optional[torch.Tensor],
                                out: torch.Tensor, *, workspace: Optional[torch.Tensor] = None,
                                max_attention_window: Optional[int] = None, sync: bool = True,
                                stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """Same step with the step inputs (qkv, sequence_length, block pointers) and the output in HOST
        memory; scales, KV pool and workspace are device resident."""
        for t in (qkv, sequence_length, kv_cache_block_pointers, out):
            if t.is_cuda:
                raise DecodeAttnError(DX_ERR_BAD_ARG, "enqueue_generation_host takes host tensors")
        hp = host_past_key_value_lengths.to(torch.int32).contiguous()
        max_past = int(hp.max()) if hp.numel() else 0
        dev = torch.device("cuda", self.device)
        if workspace is None:
            workspace = self._ensure_workspace(qkv.shape[0], max_past, dev)
        p, _ = self._params(qkv, sequence_length, hp, kv_cache_block_pointers, kv_orig_quant_scale,
                            kv_quant_orig_scale, out, workspace, max_attention_window)
        s = stream if stream is not None else torch.cuda.current_stream(dev)
        st = self.lib.dx_attn_enqueue_generation_host(self._h, ctypes.byref(p), ctypes.c_void_p(s.cuda_stream),
                                                      int(sync))
        if st != DX_OK:
            raise DecodeAttnError(st, "dx_attn_enqueue_generation_host")
        return out


def gpt_attention(*, qkv: torch.Tensor, sequence_length: torch.Tensor, host_past_key_value_lengths: torch.Tensor,
                  kv_cache_block_pointers: torch.Tensor, num_heads: int, num_kv_heads: int,
                  hidden_size_per_head: int, q_scaling: float = 1.0, kv_orig_quant_scale=None,
                  kv_quant_orig_scale=None, kv_cache_quant_mode: int = QuantMode.NONE, tokens_per_block: int = 64,
                  multi_block_mode: bool = False, max_attention_window: Optional[int] = None,
                  plugin: Optional[GPTAttentionPlugin] = None) -> torch.Tensor:
    """Functional form with the argument names of tensorrt_llm.functional.gpt_attention
    (tensorrt_llm/functional.py:3487) restricted to the generation phase with a paged cache."""
    own = plugin is None
    if own:
        plugin = GPTAttentionPlugin(num_heads=num_heads, num_kv_heads=num_kv_heads, head_size=hidden_size_per_head,
                                    q_scaling=q_scaling, multi_block_mode=multi_block_mode,
                                    kv_cache_quant_mode=kv_cache_quant_mode, tokens_per_block=tokens_per_block,
                                    type_id=qkv.dtype, device=qkv.device.index or 0)
    try:
        out = plugin.enqueue_generation(qkv, sequence_length, host_past_key_value_lengths, kv_cache_block_pointers,
                                        kv_orig_quant_scale, kv_quant_orig_scale,
                                        max_attention_window=max_attention_window)
        if own:
            torch.cuda.synchronize(qkv.device)
    finally:
        if own:
            plugin.close()
    return out
