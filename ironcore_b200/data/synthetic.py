"""Synthetic uniform-random token stream (benchmarks, parity runs, tests): every batch is
``micro_batch x (seq + 1)`` ids drawn uniformly from ``[0, vocab)`` with a seeded generator,
built in pinned host memory so the trainer's host-to-device copy is asynchronous."""

from __future__ import annotations

from typing import Dict, Iterator, Optional

import torch


class SyntheticTokenStream:
    def __init__(self, vocab_size: int, seq_len: int, micro_batch: int, seed: int = 1234, dp_rank: int = 0,
                 pin: Optional[bool] = None, num_batches: Optional[int] = None):
        self.vocab_size, self.seq_len, self.micro_batch = vocab_size, seq_len, micro_batch
        self.gen = torch.Generator(device="cpu")
        self.gen.manual_seed(int(seed) + 7919 * int(dp_rank))
        self.pin = torch.cuda.is_available() if pin is None else pin
        self.num_batches = num_batches
        self._count = 0
        # rotating pool of pinned staging buffers: a buffer is reused only after `depth` later
        # batches were produced, by which time its asynchronous copy has long been consumed
        self._pool = []
        self._depth = 256

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        return self

    def __next__(self) -> Dict[str, torch.Tensor]:
        if self.num_batches is not None and self._count >= self.num_batches:
            raise StopIteration
        self._count += 1
        if self.pin:
            slot = (self._count - 1) % self._depth
            if slot >= len(self._pool):
                self._pool.append(torch.empty((self.micro_batch, self.seq_len + 1), dtype=torch.int64).pin_memory())
            tokens = self._pool[slot]
            torch.randint(0, self.vocab_size, tokens.shape, generator=self.gen, dtype=torch.int64, out=tokens)
        else:
            tokens = torch.randint(0, self.vocab_size, (self.micro_batch, self.seq_len + 1), generator=self.gen,
                                   dtype=torch.int64)
        return {"input_ids": tokens[:, :-1], "labels": tokens[:, 1:]}
