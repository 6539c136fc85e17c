"""Synthetic data: uniform-random token ids, generated per step from ``(seed, step)`` on the host.

The *global* batch is a pure function of ``(seed, step)``; each rank slices its rows (data
parallel) and its sequence chunk (context parallel), so a run is comparable across parallel layouts.
Batches are produced in pinned host memory; the trainer copies them to the device every step.
"""
from __future__ import annotations

import torch


class SyntheticData:
    def __init__(self, vocab_size: int, seq_length: int, global_batch_size: int, micro_batch_size: int,
                 dp_rank: int, dp_size: int, cp_rank: int = 0, cp_size: int = 1, seed: int = 0,
                 pin: bool = False):
        self.vocab, self.seq, self.gbs, self.mbs = vocab_size, seq_length, global_batch_size, micro_batch_size
        self.dp_rank, self.dp_size, self.cp_rank, self.cp_size = dp_rank, dp_size, cp_rank, cp_size
        self.seed = seed
        self.pin = pin and torch.cuda.is_available()
        if global_batch_size % (micro_batch_size * dp_size):
            raise ValueError("global_batch_size must be a multiple of micro_batch_size * dp")
        self.num_microbatches = global_batch_size // (micro_batch_size * dp_size)
        self.cursor = 0                       # next step to be served (checkpointed)

    def global_batch(self, step: int) -> torch.Tensor:
        g = torch.Generator()
        g.manual_seed((self.seed * 1_000_003 + step) & 0x7FFFFFFFFFFFFFFF)
        return torch.randint(0, self.vocab, (self.gbs, self.seq + 1), generator=g, dtype=torch.int64)

    def microbatches(self, step: int) -> list[tuple[torch.Tensor, torch.Tensor]]:
        """List of ``(tokens [mbs, S/cp], targets [mbs, S/cp])`` host tensors for this rank."""
        full = self.global_batch(step)
        per_rank = self.gbs // self.dp_size
        mine = full[self.dp_rank * per_rank:(self.dp_rank + 1) * per_rank]
        chunk = self.seq // self.cp_size
        lo = self.cp_rank * chunk
        out = []
        for i in range(self.num_microbatches):
            rows = mine[i * self.mbs:(i + 1) * self.mbs]
            tok = rows[:, lo:lo + chunk].contiguous()
            tgt = rows[:, lo + 1:lo + chunk + 1].contiguous()
            if self.pin:
                tok, tgt = tok.pin_memory(), tgt.pin_memory()
            out.append((tok, tgt))
        self.cursor = step + 1
        return out
