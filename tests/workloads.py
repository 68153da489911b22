"""Seeded synthetic decode-attention workloads with the shapes of the five benchmark configs.

No dataset is involved: the configs name model *shapes* only.  Q/K/V ~ N(0,1), past lengths
uniform in a range, per-tensor KV scale amax/127 (INT8) or amax/448 (FP8), paged pool with a
shuffled free list so that page tables are non-trivial (like the reference's known-answer test,
cpp/tests/runtime/transposeKVKernelTest.cpp:190-206).  Pool layout follows the reference's
Python block manager (tensorrt_llm/runtime/kv_cache_manager.py:97-109): all K blocks, then all V
blocks; block = [num_kv_heads, tokens_per_block, head_size] cache elements.
"""
from __future__ import annotations

import dataclasses
import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import sys
from pathlib import Path

import torch

_ROOT = Path(__file__).resolve().parent.parent
if str(_ROOT) not in sys.path:
    sys.path.insert(0, str(_ROOT))
import __graft_entry__ as _entry  # noqa: E402

_pkg = _entry.load_package()
QuantMode = _pkg.QuantMode


@dataclass(frozen=True)
class DecodeConfig:
    name: str
    batch: int
    num_heads: int
    num_kv_heads: int
    head_size: int
    dtype: torch.dtype
    cache: str  # "none" | "int8" | "fp8"
    tokens_per_block: int
    len_lo: int
    len_hi: int
    multi_block_mode: bool
    seed: int
    note: str = ""

    @property
    def quant_mode(self) -> int:
        return {"none": QuantMode.NONE, "int8": QuantMode.INT8_KV_CACHE, "fp8": QuantMode.FP8_KV_CACHE}[self.cache]

    @property
    def elem_bytes(self) -> int:
        return 2 if self.cache == "none" else 1

    @property
    def block_bytes(self) -> int:
        return self.num_kv_heads * self.tokens_per_block * self.head_size * self.elem_bytes


CONFIGS: Dict[str, DecodeConfig] = {
    "c1": DecodeConfig("c1_gpt2_small_mha", 4, 12, 12, 64, torch.float16, "none", 64, 1, 512, False, 1001,
                       "GPT-2-small-shaped MHA, fp16 paged cache, no quantisation"),
    "c2": DecodeConfig("c2_llama2_7b_mha_int8", 64, 32, 32, 128, torch.bfloat16, "int8", 64, 1024, 2048, False, 1002,
                       "Llama-2-7B-shaped MHA, INT8 paged cache, multi_block off"),
    "c3": DecodeConfig("c3_falcon_7b_mqa_fp8", 128, 71, 1, 64, torch.float16, "fp8", 64, 256, 2048, True, 1003,
                       "Falcon-7B-shaped MQA (71:1), FP8 paged cache"),
    "c4": DecodeConfig("c4_llama2_70b_gqa_fp8", 128, 64, 8, 128, torch.bfloat16, "fp8", 64, 2048, 4096, True, 1004,
                       "Llama-2-70B-shaped GQA (group 8), FP8 paged cache, ragged"),
    "c5": DecodeConfig("c5_mixtral_long_gqa_int8", 8, 32, 8, 128, torch.bfloat16, "int8", 128, 16384, 32768, True, 1005,
                       "Mixtral-8x7B-shaped long-context GQA (group 4), INT8 paged cache, split-K"),
    # not one of the reference's benchmark configurations: c4's shape with an unquantised cache (half the batch,
    # the same KV bytes), the case the 16-bit grouped-head kernel exists for
    "c4kv16": DecodeConfig("c4kv16_llama2_70b_gqa_bf16_cache", 64, 64, 8, 128, torch.bfloat16, "none", 64, 2048, 4096,
                           True, 1006, "Llama-2-70B-shaped GQA (group 8), bf16 paged cache, ragged"),
}


def shard_config(cfg: DecodeConfig, tp_size: int) -> DecodeConfig:
    """Local shapes of one tensor-parallel rank: q heads / tp, kv heads ceil(/tp) - the counts the
    reference builds each rank's plugin with (tensorrt_llm/layers/attention.py:462-468, :851-852)."""
    if tp_size == 1:
        return cfg
    assert cfg.num_heads % tp_size == 0
    return dataclasses.replace(cfg, num_heads=cfg.num_heads // tp_size,
                               num_kv_heads=(cfg.num_kv_heads + tp_size - 1) // tp_size,
                               name=f"{cfg.name}_tp{tp_size}")


def scaled_config(cfg: DecodeConfig, *, batch: Optional[int] = None, len_div: int = 1) -> DecodeConfig:
    """Smaller instance of the same shape family (for parity tests and CPU samples)."""
    return dataclasses.replace(cfg, batch=batch or cfg.batch, len_lo=max(1, cfg.len_lo // len_div),
                               len_hi=max(1, cfg.len_hi // len_div))


def quantize_for_cache(x: torch.Tensor, scale_orig_quant: float, cache: str) -> torch.Tensor:
    """Bytes a cache of the given mode holds for activations x (fp16/bf16).  Used to fill the
    synthetic past KV; the kernels quantise the new token themselves."""
    if cache == "none":
        return x.contiguous().view(torch.uint8)
    s = torch.tensor(scale_orig_quant, dtype=torch.float32, device=x.device)
    if cache == "int8":
        return torch.round(x.float() * s).clamp_(-128, 127).to(torch.int8).view(torch.uint8)
    prod = (x * s.to(x.dtype)).float().clamp_(-448.0, 448.0)
    return prod.to(torch.float8_e4m3fn).view(torch.uint8)


@dataclass
class DecodeWorkload:
    cfg: DecodeConfig
    qkv: torch.Tensor                       # T [B, (H + 2 Hkv) Dh]
    sequence_length: torch.Tensor           # int32 [B], includes the new token
    host_past_key_value_lengths: torch.Tensor  # int32 [B] on the host
    pool: torch.Tensor                      # uint8 [2 * blocks * block_bytes]
    offset_table: torch.Tensor              # int64 [B, 2, M] byte offsets from the pool base (host, -1 unused)
    kv_cache_block_pointers: torch.Tensor   # int64 [B, 2, M] absolute device pointers (0 unused)
    host_kv_cache_block_pointers: torch.Tensor
    kv_orig_quant_scale: Optional[torch.Tensor]  # float32 [1] on the device, or None
    kv_quant_orig_scale: Optional[torch.Tensor]
    scale_orig_quant: float
    scale_quant_orig: float
    blocks: int
    max_blocks_per_seq: int

    @property
    def kv_bytes(self) -> int:
        """Algorithmic bytes of one step: every past K and V byte once."""
        c = self.cfg
        return int(self.host_past_key_value_lengths.sum().item()) * c.num_kv_heads * c.head_size * 2 * c.elem_bytes

    @property
    def flops(self) -> int:
        c = self.cfg
        return int((self.host_past_key_value_lengths + 1).sum().item()) * 4 * c.num_heads * c.head_size


def draw_lengths(cfg: DecodeConfig) -> torch.Tensor:
    g = torch.Generator().manual_seed(cfg.seed)
    return torch.randint(cfg.len_lo, cfg.len_hi + 1, (cfg.batch,), generator=g, dtype=torch.int64).to(torch.int32)


def build_workload(cfg: DecodeConfig, device: torch.device | str = "cpu", *, lengths: Optional[torch.Tensor] = None,
                   shuffle_pages: bool = True, spare_blocks: int = 3, seed_offset: int = 0) -> DecodeWorkload:
    device = torch.device(device)
    B, H, Hkv, Dh, tpb = cfg.batch, cfg.num_heads, cfg.num_kv_heads, cfg.head_size, cfg.tokens_per_block
    past = draw_lengths(cfg) if lengths is None else lengths.to(torch.int32).cpu()
    assert past.numel() == B
    need = [(int(l) + 1 + tpb - 1) // tpb for l in past]
    blocks = sum(need) + spare_blocks
    M = max(need)
    gcpu = torch.Generator().manual_seed(cfg.seed * 7919 + 17 + seed_offset)
    order = torch.randperm(blocks, generator=gcpu).tolist() if shuffle_pages else list(range(blocks))
    blk = cfg.block_bytes
    offs = torch.full((B, 2, M), -1, dtype=torch.int64)
    it = iter(order)
    for b in range(B):
        for i in range(need[b]):
            idx = next(it)
            offs[b, 0, i] = idx * blk
            offs[b, 1, i] = idx * blk + blocks * blk

    # ---- past K/V: the whole pool is filled with quantised N(0,1) values, chunk by chunk ----
    gdev = torch.Generator(device=device).manual_seed(cfg.seed * 104729 + 5 + seed_offset)
    qkv = torch.randn(B, (H + 2 * Hkv) * Dh, generator=gdev, device=device, dtype=torch.float32).to(cfg.dtype)
    elems_per_block = Hkv * tpb * Dh
    chunk_blocks = max(1, (1 << 26) // elems_per_block)
    chunk_seeds: List[int] = []
    amax = 0.0
    for c0 in range(0, 2 * blocks, chunk_blocks):
        chunk_seeds.append(cfg.seed * 15485863 + c0 + seed_offset)
    # pass 1: amax of the values (in T) that will be stored
    for ci, c0 in enumerate(range(0, 2 * blocks, chunk_blocks)):
        n = min(chunk_blocks, 2 * blocks - c0)
        g = torch.Generator(device=device).manual_seed(chunk_seeds[ci])
        x = torch.randn(n * elems_per_block, generator=g, device=device, dtype=torch.float32).to(cfg.dtype)
        amax = max(amax, float(x.abs().max()))
    if cfg.cache == "int8":
        s_qo = amax / 127.0
    elif cfg.cache == "fp8":
        s_qo = amax / 448.0
    else:
        s_qo = 1.0
    s_qo = float(torch.tensor(s_qo, dtype=torch.float32))
    s_oq = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(s_qo, dtype=torch.float32))
    pool = torch.empty(2 * blocks * blk, dtype=torch.uint8, device=device)
    for ci, c0 in enumerate(range(0, 2 * blocks, chunk_blocks)):
        n = min(chunk_blocks, 2 * blocks - c0)
        g = torch.Generator(device=device).manual_seed(chunk_seeds[ci])
        x = torch.randn(n * elems_per_block, generator=g, device=device, dtype=torch.float32).to(cfg.dtype)
        pool[c0 * blk:(c0 + n) * blk] = quantize_for_cache(x, s_oq, cfg.cache).reshape(-1)
        del x

    base = pool.data_ptr()
    ptrs = torch.where(offs >= 0, offs + base, torch.zeros_like(offs))
    quant = cfg.cache != "none"
    return DecodeWorkload(
        cfg=cfg, qkv=qkv, sequence_length=(past + 1).to(torch.int32).to(device),
        host_past_key_value_lengths=past.clone(), pool=pool, offset_table=offs,
        kv_cache_block_pointers=ptrs.to(device), host_kv_cache_block_pointers=ptrs.clone(),
        kv_orig_quant_scale=torch.tensor([s_oq], dtype=torch.float32, device=device) if quant else None,
        kv_quant_orig_scale=torch.tensor([s_qo], dtype=torch.float32, device=device) if quant else None,
        scale_orig_quant=s_oq, scale_quant_orig=s_qo, blocks=blocks, max_blocks_per_seq=M)


def to_device(w: DecodeWorkload, device: torch.device | str) -> DecodeWorkload:
    """Copies a (CPU-built) workload to a device and rebases the pointer table on the new pool."""
    device = torch.device(device)
    pool = w.pool.to(device)
    base = pool.data_ptr()
    ptrs = torch.where(w.offset_table >= 0, w.offset_table + base, torch.zeros_like(w.offset_table))
    return dataclasses.replace(
        w, qkv=w.qkv.to(device), sequence_length=w.sequence_length.to(device), pool=pool,
        kv_cache_block_pointers=ptrs.to(device), host_kv_cache_block_pointers=ptrs.clone(),
        kv_orig_quant_scale=None if w.kv_orig_quant_scale is None else w.kv_orig_quant_scale.to(device),
        kv_quant_orig_scale=None if w.kv_quant_orig_scale is None else w.kv_quant_orig_scale.to(device))


def shard_workload(w: DecodeWorkload, tp_size: int, tp_rank: int) -> DecodeWorkload:
    """The slice of a full workload that tensor-parallel rank tp_rank owns: its q heads, its kv
    heads and only those heads of every cache block (block = [Hkv_local, tokens, Dh]).  Same
    lengths and page table on every rank; no data is shared between ranks."""
    c = w.cfg
    assert c.num_heads % tp_size == 0 and c.num_kv_heads % tp_size == 0
    lc = shard_config(c, tp_size)
    H, Hkv, Dh = c.num_heads, c.num_kv_heads, c.head_size
    h0, k0 = tp_rank * lc.num_heads, tp_rank * lc.num_kv_heads
    q = w.qkv[:, h0 * Dh:(h0 + lc.num_heads) * Dh]
    k = w.qkv[:, (H + k0) * Dh:(H + k0 + lc.num_kv_heads) * Dh]
    v = w.qkv[:, (H + Hkv + k0) * Dh:(H + Hkv + k0 + lc.num_kv_heads) * Dh]
    qkv = torch.cat([q, k, v], dim=1).contiguous()
    row = c.tokens_per_block * Dh * c.elem_bytes
    pool = w.pool.view(2 * w.blocks, Hkv, row)[:, k0:k0 + lc.num_kv_heads].contiguous().view(-1)
    offs = torch.where(w.offset_table >= 0, w.offset_table // c.block_bytes * lc.block_bytes, w.offset_table)
    base = pool.data_ptr()
    ptrs = torch.where(offs >= 0, offs + base, torch.zeros_like(offs))
    return dataclasses.replace(w, cfg=lc, qkv=qkv, pool=pool, offset_table=offs,
                               kv_cache_block_pointers=ptrs.to(pool.device), host_kv_cache_block_pointers=ptrs.clone())


def make_plugin(cfg: DecodeConfig, device_index: int = 0, *, tp_size: int = 1, tp_rank: int = 0,
                multi_block_mode: Optional[bool] = None):
    return _pkg.GPTAttentionPlugin(num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads, head_size=cfg.head_size,
                              q_scaling=1.0, tp_size=tp_size, tp_rank=tp_rank,
                              multi_block_mode=cfg.multi_block_mode if multi_block_mode is None else multi_block_mode,
                              kv_cache_quant_mode=cfg.quant_mode, tokens_per_block=cfg.tokens_per_block,
                              type_id=cfg.dtype, device=device_index)


def run_step(plugin, w: DecodeWorkload, out: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None):
    return plugin.enqueue_generation(w.qkv, w.sequence_length, w.host_past_key_value_lengths,
                                     w.kv_cache_block_pointers, w.kv_orig_quant_scale, w.kv_quant_orig_scale,
                                     out=out, workspace=workspace,
                                     max_attention_window=w.max_blocks_per_seq * w.cfg.tokens_per_block)
