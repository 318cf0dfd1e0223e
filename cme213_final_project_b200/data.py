"""Character tokenizer, sequential batcher and seeded synthetic token streams.

Semantics follow the reference (``FINAL_CLEAN_CODE_/src/data/dataset.cpp:19-79``,
``FINAL_CLEAN_CODE_/include/data.h:16-33``):

* vocabulary = sorted set of the bytes that occur in the corpus; encoding skips unknown characters;
* a batch is ``B`` chunks of ``T+1`` consecutive tokens, ``input = chunk[0:T]``, ``target = chunk[1:T+1]``;
  the cursor advances by ``B*(T+1)`` and ``num_batches = (N-1) // (B*(T+1))``;
* under data parallelism rank ``r`` trains on batch ``step*world + r`` and the remainder is dropped
  (``FINAL_CLEAN_CODE_/src/main.cu:252-253,325``).

All batches are materialised once as ``int32`` tensors so the training loop does no per-step host work
(the reference preloads every batch to the device, ``main.cu:273-292``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


def read_file(path: str) -> bytes:
    with open(path, "rb") as f:
        return f.read()


class CharTokenizer:
    """Byte-level tokenizer over the sorted set of bytes present in the training text."""

    def __init__(self) -> None:
        self.id_to_char: List[int] = []
        self.char_to_id: Dict[int, int] = {}

    @property
    def vocab_size(self) -> int:
        return len(self.id_to_char)

    def build(self, text: bytes) -> "CharTokenizer":
        if isinstance(text, str):
            text = text.encode("utf-8")
        # the reference sorts signed ``char``; bytes >= 0x80 would sort first there
        present = np.unique(np.frombuffer(text, dtype=np.uint8))
        self.id_to_char = sorted(present.tolist(), key=lambda b: b - 256 if b >= 128 else b)
        self.char_to_id = {c: i for i, c in enumerate(self.id_to_char)}
        return self

    def encode(self, text: bytes) -> np.ndarray:
        if isinstance(text, str):
            text = text.encode("utf-8")
        table = np.full(256, -1, dtype=np.int32)
        for c, i in self.char_to_id.items():
            table[c] = i
        ids = table[np.frombuffer(text, dtype=np.uint8)]
        return ids[ids >= 0]

    def decode(self, ids) -> bytes:
        return bytes(self.id_to_char[i] for i in ids if 0 <= int(i) < self.vocab_size)


class Dataset:
    """Sequential batcher over one token stream."""

    def __init__(self, tokens: np.ndarray, seq_len: int, batch_size: int) -> None:
        self.tokens = np.asarray(tokens, dtype=np.int32)
        self.seq_len = seq_len
        self.batch_size = batch_size
        self.cursor = 0

    @classmethod
    def load(cls, path: str, tok: CharTokenizer, seq_len: int, batch_size: int, verbose: bool = False) -> "Dataset":
        ds = cls(tok.encode(read_file(path)), seq_len, batch_size)
        if verbose:
            print(f"Dataset: {len(ds.tokens)} tokens, vocab_size={tok.vocab_size}, "
                  f"seq_len={seq_len}, batch_size={batch_size}")
        return ds

    def reset(self) -> None:
        self.cursor = 0

    def num_batches(self) -> int:
        per_batch = self.batch_size * (self.seq_len + 1)
        return (len(self.tokens) - 1) // per_batch if per_batch > 0 else 0

    def next_batch(self) -> Optional[Tuple[np.ndarray, np.ndarray]]:
        chunk = self.seq_len + 1
        need = self.batch_size * chunk
        if self.cursor + need > len(self.tokens):
            return None
        block = self.tokens[self.cursor:self.cursor + need].reshape(self.batch_size, chunk)
        self.cursor += need
        return block[:, :-1].reshape(-1).copy(), block[:, 1:].reshape(-1).copy()

    def all_batches(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Every batch at once: two ``[num_batches, B*T]`` int32 tensors."""
        n = self.num_batches()
        chunk = self.seq_len + 1
        need = self.batch_size * chunk
        block = self.tokens[: n * need].reshape(n, self.batch_size, chunk)
        x = np.ascontiguousarray(block[:, :, :-1]).reshape(n, -1)
        y = np.ascontiguousarray(block[:, :, 1:]).reshape(n, -1)
        return torch.from_numpy(x), torch.from_numpy(y)


def synthetic_tokens(vocab_size: int, count: int, seed: int = 0) -> np.ndarray:
    """``count`` token ids i.i.d. uniform in ``[0, vocab_size)`` from ``seed``."""
    rng = np.random.default_rng(seed)
    return rng.integers(0, vocab_size, size=count, dtype=np.int32)


def synthetic_batches(vocab_size: int, seq_len: int, batch_size: int, num_batches: int,
                      seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Synthetic stream cut into batches with the same chunking as :class:`Dataset`."""
    need = batch_size * (seq_len + 1) * num_batches + 1
    ds = Dataset(synthetic_tokens(vocab_size, need, seed), seq_len, batch_size)
    return ds.all_batches()


@dataclass
class ShardPlan:
    """Rank-strided assignment of batches to ranks."""

    num_batches: int
    world_size: int

    @property
    def local_batches(self) -> int:
        return self.num_batches // self.world_size

    @property
    def dropped(self) -> int:
        return self.num_batches - self.local_batches * self.world_size

    def batch_index(self, step: int, rank: int) -> int:
        return step * self.world_size + rank


def reference_corpus_path() -> str:
    """Where the reference's tiny-Shakespeare corpus (``FINAL_CLEAN_CODE_/inp.txt``) is expected:
    ``$CME213_REFERENCE_DIR`` if set, else a ``reference`` checkout next to this repository.  The file may not
    exist; callers fall back to synthetic tokens."""
    import os
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    root = os.environ.get("CME213_REFERENCE_DIR") or os.path.join(os.path.dirname(here), "reference")
    return os.path.join(root, "FINAL_CLEAN_CODE_", "inp.txt")
