"""Host-side paged-KV block manager producing the pointer table the decode step consumes.

Same bookkeeping and table format as the reference's Python runtime manager
(tensorrt_llm/runtime/kv_cache_manager.py:74-387): blocks are handed out from a free list in order,
K block i lives at pool + i * block_bytes and V block i at + blocks * block_bytes, a sequence gets a new
block when its next token starts one, and get_block_pointers() returns int64 [B, 2, M] (beam width 1;
unused slots 0).  Sliding-window / sink / beam sharing are not implemented (the kernels do not support
them either).  Host logic only; the table is uploaded by the caller (or bound once and updated in place).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


class GenerationSequence:
    def __init__(self, seq_idx: int, batch_idx: int):
        self.seq_idx, self.batch_idx = seq_idx, batch_idx

    def get_batch_idx(self) -> int:
        return self.batch_idx

    def get_seq_idx(self) -> int:
        return self.seq_idx

    def __eq__(self, other):
        return isinstance(other, GenerationSequence) and (self.seq_idx, self.batch_idx) == (other.seq_idx, other.batch_idx)

    def __hash__(self):
        return self.seq_idx


class KVCacheManager:
    def __init__(self, pool: torch.Tensor, blocks: int, tokens_per_block: int, max_blocks_per_seq: int,
                 free_order: Optional[Sequence[int]] = None):
        """pool: uint8 tensor of 2 * blocks * block_bytes bytes (device or host)."""
        assert pool.dtype == torch.uint8 and pool.numel() % (2 * blocks) == 0
        if tokens_per_block & (tokens_per_block - 1):
            raise ValueError("tokens_per_block must be a power of two")
        self.pool, self.blocks = pool, blocks
        self.block_bytes = pool.numel() // (2 * blocks)
        self.tokens_per_block, self.max_blocks_per_seq = tokens_per_block, max_blocks_per_seq
        self.free_blocks: List[int] = list(free_order) if free_order is not None else list(range(blocks))
        self.sequences: List[GenerationSequence] = []
        self.lens: List[int] = []
        self.allocated: Dict[int, List[int]] = {}

    def has_free_block(self) -> bool:
        return bool(self.free_blocks)

    def _allocate(self, seq: GenerationSequence) -> None:
        if not self.free_blocks:
            raise RuntimeError("Can't allocate new block for KV cache")
        blks = self.allocated.setdefault(seq.seq_idx, [])
        if len(blks) >= self.max_blocks_per_seq:
            raise RuntimeError("sequence exceeds max_blocks_per_seq")
        blks.append(self.free_blocks.pop(0))

    def add_sequence(self, sequence: GenerationSequence, context_len: int) -> None:
        self.sequences.append(sequence)
        self.lens.append(context_len)
        for _ in range((context_len + self.tokens_per_block - 1) // self.tokens_per_block):
            self._allocate(sequence)

    def step(self, finished: Sequence[bool]) -> None:
        """One generation step: sequences whose next token starts a new block get one; finished ones are freed."""
        for seq in self.sequences:
            b = seq.get_batch_idx()
            if not finished[b] and self.lens[b] % self.tokens_per_block == 0:
                self._allocate(seq)
            self.lens[b] += 1
        keep = []
        for seq, fin in zip(self.sequences, finished):
            if fin:
                self.free_blocks.extend(self.allocated.pop(seq.seq_idx, []))
            else:
                keep.append(seq)
        self.lens = [l for l, f in zip(self.lens, finished) if not f]
        for i, seq in enumerate(keep):
            seq.batch_idx = i
        self.sequences = keep

    def get_block_pointers(self) -> torch.Tensor:
        """int64 [B, 2, M] host tensor of absolute pointers into the pool (0 = unused)."""
        base = self.pool.data_ptr()
        t = torch.zeros(len(self.sequences), 2, self.max_blocks_per_seq, dtype=torch.int64)
        for seq in self.sequences:
            b = seq.get_batch_idx()
            for i, blk in enumerate(self.allocated.get(seq.seq_idx, [])):
                t[b, 0, i] = base + blk * self.block_bytes
                t[b, 1, i] = base + (blk + self.blocks) * self.block_bytes
        return t

    def host_past_key_value_lengths(self) -> torch.Tensor:
        return torch.tensor(self.lens, dtype=torch.int32)
