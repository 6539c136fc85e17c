"""Training data: synthetic uniform-random token ids, or a flat file of token ids.

Either way the *global* batch is a pure function of ``(seed, step)``; each rank slices its rows (data
parallel) and its sequence chunk (context parallel), so a run is comparable across parallel layouts and a
resumed run continues with the batches it would have seen.  Batches are produced in pinned host memory; the
trainer copies them to the device every step.

``TokenFileData`` reads a binary file of token ids (``.bin``/``.u16`` = uint16, ``.u32`` = uint32, ``.i32`` =
int32, or ``.npy``) through a memory map: a step's rows are ``global_batch_size`` windows of ``seq_length + 1``
tokens at offsets drawn from ``(seed, step)``.  The reference's runs read Megatron-style pre-tokenised files
(``notes/2026-04/2026-04-19_gptoss_01_mlperf_best_e2e_run.md:60-110``); the on-disk format here is the plain
token stream those are built from.
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


_SUFFIX_DTYPE = {".bin": "uint16", ".u16": "uint16", ".u32": "uint32", ".i32": "int32"}


def write_token_file(path, tokens) -> None:
    """Write a 1-D sequence of token ids in the format ``TokenFileData`` reads (dtype from the suffix)."""
    import numpy as np
    from pathlib import Path
    p = Path(path)
    arr = np.asarray(tokens)
    if p.suffix == ".npy":
        np.save(p, arr.astype(np.int32))
    else:
        arr.astype(_SUFFIX_DTYPE[p.suffix]).tofile(p)


class TokenFileData(SyntheticData):
    """Same batch contract as ``SyntheticData`` with rows cut from a token file."""

    def __init__(self, path: str, vocab_size: int, seq_length: int, global_batch_size: int, micro_batch_size: int,
                 dp_rank: int, dp_size: int, cp_rank: int = 0, cp_size: int = 1, seed: int = 0, pin: bool = False):
        super().__init__(vocab_size, seq_length, global_batch_size, micro_batch_size, dp_rank, dp_size, cp_rank,
                         cp_size, seed, pin)
        import numpy as np
        from pathlib import Path
        p = Path(path)
        if not p.exists():
            raise FileNotFoundError(f"token file {path} does not exist")
        if p.suffix == ".npy":
            self.tokens = np.load(p, mmap_mode="r")
        elif p.suffix in _SUFFIX_DTYPE:
            self.tokens = np.memmap(p, dtype=_SUFFIX_DTYPE[p.suffix], mode="r")
        else:
            raise ValueError(f"unknown token file suffix {p.suffix!r}; use one of {sorted(_SUFFIX_DTYPE)} or .npy")
        self.n_windows = len(self.tokens) - (seq_length + 1)
        if self.n_windows < 1:
            raise ValueError(f"{path}: {len(self.tokens)} tokens are fewer than one sequence of {seq_length + 1}")

    def global_batch(self, step: int) -> torch.Tensor:
        import numpy as np
        g = torch.Generator()
        g.manual_seed((self.seed * 1_000_003 + step) & 0x7FFFFFFFFFFFFFFF)
        starts = torch.randint(0, self.n_windows, (self.gbs,), generator=g).tolist()
        rows = np.stack([np.asarray(self.tokens[s:s + self.seq + 1]) for s in starts]).astype(np.int64)
        out = torch.from_numpy(rows)
        if int(out.max()) >= self.vocab:
            raise ValueError(f"token id {int(out.max())} in the file exceeds vocab_size {self.vocab}")
        return out


def make_data(spec: str, **kw):
    """``"synthetic"`` or a token file path."""
    if spec in ("", "synthetic"):
        return SyntheticData(**kw)
    return TokenFileData(spec, **kw)
