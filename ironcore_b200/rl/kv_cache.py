"""Block (paged) KV cache: fixed-size pages, a host-side free list, per-sequence block tables.

Per layer the cache holds ``k`` and ``v`` pools of shape ``[num_blocks, block_size, kv_heads, head_dim]``.
A sequence owns a list of physical blocks; ``block_table[seq, i]`` is the block of its i-th page and
``seq_lens[seq]`` its current length. The tables live on the device (updated in place, so a captured
CUDA graph of the decode step keeps reading the current state)."""

from __future__ import annotations

from typing import List

import torch


class BlockKVCache:
    def __init__(self, num_layers: int, kv_heads: int, head_dim: int, num_blocks: int, block_size: int = 16,
                 max_seqs: int = 128, max_seq_len: int = 1024, dtype=torch.bfloat16, device="cuda"):
        if block_size % 16:
            raise ValueError("block_size must be a multiple of 16")
        self.num_layers, self.kv_heads, self.head_dim = num_layers, kv_heads, head_dim
        self.num_blocks, self.block_size = num_blocks, block_size
        self.max_seqs = max_seqs
        self.max_blocks_per_seq = (max_seq_len + block_size - 1) // block_size
        self.dtype, self.device = dtype, torch.device(device)
        shape = (num_blocks, block_size, kv_heads, head_dim)
        self.k = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(num_layers)]
        self.v = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(num_layers)]
        self.block_table = torch.zeros((max_seqs, self.max_blocks_per_seq), dtype=torch.int32, device=self.device)
        self.seq_lens = torch.zeros(max_seqs, dtype=torch.int32, device=self.device)
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))
        self._owned: List[List[int]] = [[] for _ in range(max_seqs)]
        self._host_lens = [0] * max_seqs

    # ---- allocation (host side) ----
    @property
    def free_blocks(self) -> int:
        return len(self._free)

    def reset(self):
        self._free = list(range(self.num_blocks - 1, -1, -1))
        self._owned = [[] for _ in range(self.max_seqs)]
        self._host_lens = [0] * self.max_seqs
        self.seq_lens.zero_()

    def reserve(self, seq: int, new_len: int):
        """Make sure sequence ``seq`` owns enough pages for ``new_len`` tokens."""
        need = (new_len + self.block_size - 1) // self.block_size
        owned = self._owned[seq]
        if need > self.max_blocks_per_seq:
            raise RuntimeError(f"sequence {seq} exceeds the cache's max_seq_len")
        if need > len(owned):
            add = need - len(owned)
            if add > len(self._free):
                raise RuntimeError("KV cache is out of blocks")
            new = [self._free.pop() for _ in range(add)]
            start = len(owned)
            owned.extend(new)
            self.block_table[seq, start:start + add] = torch.tensor(new, dtype=torch.int32, device=self.device)

    def reserve_all(self, num_seqs: int, new_len: int):
        """Batched form of :meth:`reserve` for sequences 0..num_seqs-1 of equal length: one table write."""
        need = (new_len + self.block_size - 1) // self.block_size
        if need > self.max_blocks_per_seq:
            raise RuntimeError("sequences exceed the cache's max_seq_len")
        have = len(self._owned[0]) if num_seqs else 0
        if any(len(self._owned[s]) != have for s in range(num_seqs)):
            for s in range(num_seqs):
                self.reserve(s, new_len)
            return
        add = need - have
        if add <= 0:
            return
        if add * num_seqs > len(self._free):
            raise RuntimeError("KV cache is out of blocks")
        rows = []
        for s in range(num_seqs):
            new = [self._free.pop() for _ in range(add)]
            self._owned[s].extend(new)
            rows.append(new)
        self.block_table[:num_seqs, have:have + add] = torch.tensor(rows, dtype=torch.int32, device=self.device)

    def free(self, seq: int):
        self._free.extend(reversed(self._owned[seq]))
        self._owned[seq] = []
        self._host_lens[seq] = 0
        self.seq_lens[seq] = 0

    # ---- slot mapping ----
    def slots_for(self, seq_ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Flat cache slots (block * block_size + offset) for tokens at ``positions`` of ``seq_ids``."""
        page = (positions // self.block_size).long()
        blk = self.block_table[seq_ids.long(), page].long()
        return blk * self.block_size + (positions % self.block_size).long()

    def bytes_per_token(self) -> int:
        return 2 * self.num_layers * self.kv_heads * self.head_dim * torch.empty((), dtype=self.dtype).element_size()
