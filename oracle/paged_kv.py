"""TEST INFRASTRUCTURE ONLY - paged KV cache index math, restated from the reference.

Follows
  cpp/tensorrt_llm/kernels/kvCacheUtils.h:101-107  (getRowPtr: data + b*M*2 + kv*M)
  cpp/tensorrt_llm/kernels/kvCacheUtils.h:119-122  (getBlockPtr: row[token >> log2(tpb)])
  cpp/tensorrt_llm/kernels/kvCacheUtils.h:144-152  (getKVLocalIdx: h*tpb*Dh + (token & (tpb-1))*Dh + c)
and the pool / pointer-table construction of
  tensorrt_llm/runtime/kv_cache_manager.py:97-109, 189-225
  (K block i at pool + i*blockBytes, V block i at + blocks*blockBytes; table [B, beam, 2, M]).
"""
from __future__ import annotations

from typing import List, Sequence

import torch


def block_bytes(num_kv_heads: int, tokens_per_block: int, head_size: int, elem_bytes: int) -> int:
    return num_kv_heads * tokens_per_block * head_size * elem_bytes


def kv_token_block(token_idx: int, tokens_per_block: int) -> int:
    """Index into a sequence's pointer row (kvCacheUtils.h:119-122)."""
    log2 = tokens_per_block.bit_length() - 1
    assert 1 << log2 == tokens_per_block, "tokens_per_block must be a power of two"
    return token_idx >> log2


def kv_local_index(token_idx: int, head_idx: int, dims_per_head: int, channel: int, tokens_per_block: int) -> int:
    """Element index inside a block (kvCacheUtils.h:144-152)."""
    return head_idx * tokens_per_block * dims_per_head + (token_idx & (tokens_per_block - 1)) * dims_per_head + channel


class PagedPoolModel:
    """Host model of the block pool and the per-sequence pointer table.

    Offsets are relative to the pool base, so the same table addresses a CPU copy of the pool
    (oracle) and the device pool (kernels: base + offset).
    """

    def __init__(self, blocks: int, blk_bytes: int, max_blocks_per_seq: int, free_order: Sequence[int] | None = None):
        self.blocks = blocks
        self.blk_bytes = blk_bytes
        self.max_blocks_per_seq = max_blocks_per_seq
        self.free: List[int] = list(free_order) if free_order is not None else list(range(blocks))
        assert sorted(self.free) == list(range(blocks))
        self.seq_blocks: List[List[int]] = []
        self.lens: List[int] = []

    @property
    def pool_bytes(self) -> int:
        return 2 * self.blocks * self.blk_bytes

    def add_sequence(self, tokens: int, tokens_per_block: int) -> int:
        need = (tokens + tokens_per_block - 1) // tokens_per_block
        assert need <= self.max_blocks_per_seq and need <= len(self.free)
        self.seq_blocks.append([self.free.pop(0) for _ in range(need)])
        self.lens.append(tokens)
        return len(self.seq_blocks) - 1

    def step(self, tokens_per_block: int) -> None:
        """One generation step for every sequence: a sequence whose next token starts a new block
        gets one more block first (kv_cache_manager.py:305-345, no cyclic cache, beam width 1)."""
        for b in range(len(self.seq_blocks)):
            if self.lens[b] % tokens_per_block == 0:
                self.seq_blocks[b].append(self.free.pop(0))
            self.lens[b] += 1

    def k_offset(self, block_idx: int) -> int:
        return block_idx * self.blk_bytes

    def v_offset(self, block_idx: int) -> int:
        return block_idx * self.blk_bytes + self.blocks * self.blk_bytes

    def offset_table(self) -> torch.Tensor:
        """int64 [B, 2, M] of byte offsets from the pool base; unused slots hold -1."""
        B, M = len(self.seq_blocks), self.max_blocks_per_seq
        t = torch.full((B, 2, M), -1, dtype=torch.int64)
        for b, blks in enumerate(self.seq_blocks):
            for i, blk in enumerate(blks):
                t[b, 0, i] = self.k_offset(blk)
                t[b, 1, i] = self.v_offset(blk)
        return t

    def pointer_table(self, base_ptr: int) -> torch.Tensor:
        """int64 [B, 2, M] of absolute pointers; unused slots hold 0 (kv_cache_manager.py:204-212)."""
        off = self.offset_table()
        return torch.where(off >= 0, off + base_ptr, torch.zeros_like(off))
