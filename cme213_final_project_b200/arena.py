"""Flat parameter / gradient / optimizer-state arenas laid out in backward-production order.

The reference keeps parameters, gradients and both Adam moments in one contiguous buffer each and
orders the 15 tensors so that gradients become final in address order during backward
(``FINAL_CLEAN_CODE_/src/model/transformer.cu:166-235``, order at ``:171-188``):

    Wout[D,V], W2[FF,D], b2[D], W1[D,FF], b1[FF], ln2_g[D], ln2_b[D], Wo[D,D],
    Wq[D,D], Wk[D,D], Wv[D,D], ln1_g[D], ln1_b[D], tok_embed[V,D], pos_embed[T,D]

so every gradient bucket is a contiguous range.  This module generalises that order to ``N`` blocks
(last block first; GPT mode stores one fused ``Wqkv[D,3D]`` per block), an optional final LayerNorm (right after the output head) and tied embeddings
(no ``Wout``; the shared table is the last range because the embedding scatter is the last gradient
to be produced).  With one block, untied, no final LN, the layout is exactly the reference's.

Weights are stored ``[in, out]`` (row-major) like the reference, so ``y = x @ W``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from .config import ModelConfig


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    offset: int          # element offset inside the arena
    kind: str            # "weight" | "bias" | "ln_gamma" | "ln_beta" | "embed"
    init_seed: int       # xorshift seed offset (reference: transformer.cu:237-252); -1 = constant init
    bucket: int          # index of the natural bucket this tensor belongs to

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass(frozen=True)
class Bucket:
    """A contiguous gradient range ``[start, end)`` that becomes final at one point of backward."""
    index: int
    start: int
    end: int
    names: Tuple[str, ...]

    @property
    def numel(self) -> int:
        return self.end - self.start


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class ArenaLayout:
    """Names, shapes, offsets and natural buckets for one model configuration.

    ``align`` (elements) rounds every tensor offset up so that each tensor starts on a 16-byte
    boundary for any element type used on the device (TMA and 128-bit vector loads need that).
    Padding elements are zero and stay zero under Adam/AdamW.  For the reference shapes (all dims
    multiples of 8) there is no padding and offsets equal the reference's running offsets.
    """

    def __init__(self, cfg: ModelConfig, align: int = 8, shard_multiple: int = 1) -> None:
        self.cfg = cfg
        self.align = align
        D, FF, V, T = cfg.hidden, cfg.ff, cfg.vocab_size, cfg.seq_len
        specs: List[ParamSpec] = []
        buckets: List[List[str]] = []
        off = 0

        def add(name, shape, kind, seed, bucket_names):
            nonlocal off
            off = _round_up(off, align)
            specs.append(ParamSpec(name, tuple(shape), off, kind, seed, len(buckets)))
            bucket_names.append(name)
            n = 1
            for s in shape:
                n *= s
            off += n

        def close(bucket_names):
            if bucket_names:
                buckets.append(list(bucket_names))
                bucket_names.clear()

        cur: List[str] = []
        if not cfg.tied_embeddings:
            add("Wout", (D, V), "weight", 2, cur)
            close(cur)
        if cfg.final_layernorm:
            add("lnf_gamma", (D,), "ln_gamma", -1, cur)
            add("lnf_beta", (D,), "ln_beta", -1, cur)
            close(cur)
        for l in reversed(range(cfg.layers)):
            p = f"h{l}." if (cfg.layers > 1 or cfg.mode == "gpt") else ""
            s = 100 * l   # distinct streams per block; block 0 keeps the reference seeds 10..21
            add(p + "W2", (FF, D), "weight", s + 21, cur)
            add(p + "b2", (D,), "bias", -1, cur)
            close(cur)
            add(p + "W1", (D, FF), "weight", s + 20, cur)
            add(p + "b1", (FF,), "bias", -1, cur)
            close(cur)
            add(p + "ln2_gamma", (D,), "ln_gamma", -1, cur)
            add(p + "ln2_beta", (D,), "ln_beta", -1, cur)
            close(cur)
            add(p + "Wo", (D, D), "weight", s + 13, cur)
            close(cur)
            if cfg.mode == "gpt":
                # one fused [D, 3D] projection: columns [0,D) = Q, [D,2D) = K, [2D,3D) = V
                add(p + "Wqkv", (D, 3 * D), "weight", s + 10, cur)
            else:
                add(p + "Wq", (D, D), "weight", s + 10, cur)
                add(p + "Wk", (D, D), "weight", s + 11, cur)
                add(p + "Wv", (D, D), "weight", s + 12, cur)
            close(cur)
            add(p + "ln1_gamma", (D,), "ln_gamma", -1, cur)
            add(p + "ln1_beta", (D,), "ln_beta", -1, cur)
            close(cur)
        add("tok_embed", (V, D), "embed", 0, cur)
        add("pos_embed", (T, D), "embed", 1, cur)
        close(cur)

        self.specs: List[ParamSpec] = specs
        self.by_name: Dict[str, ParamSpec] = {s.name: s for s in specs}
        self.used = off
        # total is padded so that it splits evenly into `shard_multiple` 16-byte aligned shards
        self.total = _round_up(off, max(align, 1) * max(shard_multiple, 1))
        self.natural_buckets: List[Bucket] = []
        for i, names in enumerate(buckets):
            start = self.by_name[names[0]].offset
            last = self.by_name[names[-1]]
            end = last.offset + last.numel
            self.natural_buckets.append(Bucket(i, start, end, tuple(names)))
        # make buckets tile the arena exactly (absorb alignment gaps and the tail pad)
        fixed = []
        for i, b in enumerate(self.natural_buckets):
            end = self.natural_buckets[i + 1].start if i + 1 < len(self.natural_buckets) else self.total
            fixed.append(Bucket(b.index, b.start, end, b.names))
        self.natural_buckets = fixed

    # ---------------------------------------------------------------------------------------------
    def num_params(self) -> int:
        return sum(s.numel for s in self.specs)

    def views(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Named views into a flat arena tensor."""
        assert flat.numel() >= self.total, (flat.numel(), self.total)
        return {s.name: flat[s.offset:s.offset + s.numel].view(*s.shape) for s in self.specs}

    def coalesced_buckets(self, min_elems: int, merge_tail: bool = False) -> List[Bucket]:
        """Merge adjacent natural buckets, in emission order, until each has at least ``min_elems``
        elements (the reference's ``--bucket-kb`` rule, ``transformer.cu:428-457``).  A trailing
        remainder smaller than the floor is still emitted (flush at the end of backward).

        ``merge_tail`` (models with several blocks): the gradients that only become final in the last stretch of
        backward -- block 0 and the embeddings -- form one bucket, and the buckets before it are cut so that the
        last of them completes when block 1 does (a remainder below the floor joins its predecessor).  A bucket
        that ends inside block 0 would be launched at the very end of backward and delay the embedding bucket
        behind it; this way one kernel handles everything that cannot overlap, and nothing else is left."""
        if min_elems <= 0:
            return list(self.natural_buckets)
        nat = self.natural_buckets
        tail_at = len(nat)
        if merge_tail and self.cfg.layers > 1 and "h0.W2" in self.by_name:
            tail_at = self.by_name["h0.W2"].bucket
        out: List[Bucket] = []
        start: Optional[int] = None
        names: List[str] = []
        for b in nat[:tail_at]:
            if start is None:
                start = b.start
            names += list(b.names)
            if b.end - start >= min_elems:
                out.append(Bucket(len(out), start, b.end, tuple(names)))
                start, names = None, []
        if start is not None:
            end = nat[tail_at - 1].end
            if tail_at < len(nat) and out:      # remainder before the tail group: joins the bucket before it
                prev = out.pop()
                out.append(Bucket(len(out), prev.start, end, prev.names + tuple(names)))
            else:
                out.append(Bucket(len(out), start, end, tuple(names)))
        if tail_at < len(nat):
            tnames = tuple(n for b in nat[tail_at:] for n in b.names)
            out.append(Bucket(len(out), nat[tail_at].start, nat[-1].end, tnames))
        return out

    def bucket_ready_after(self, buckets: Sequence[Bucket]) -> Dict[int, int]:
        """For each coalesced bucket, the index of the natural bucket whose completion makes it ready."""
        ready = {}
        for b in buckets:
            last = max(nb.index for nb in self.natural_buckets if nb.start >= b.start and nb.end <= b.end)
            ready[b.index] = last
        return ready


# --------------------------------------------------------------------------------------------------
# Initialisation
# --------------------------------------------------------------------------------------------------

def xorshift_uniform(n: int, seed: int, scale: float = 0.02) -> torch.Tensor:
    """The reference's per-element initialiser (``transformer.cu:5-13``): one xorshift round of
    ``seed + i`` mapped to a uniform value in ``[-scale, scale]``, evaluated in float32."""
    import numpy as np
    s = (np.arange(n, dtype=np.uint64) + np.uint64(seed & 0xFFFFFFFF)) & np.uint64(0xFFFFFFFF)
    s = s.astype(np.uint32)
    s ^= (s << np.uint32(13))
    s ^= (s >> np.uint32(17))
    s ^= (s << np.uint32(5))
    u = (s & np.uint32(0x7FFFFFFF)).astype(np.float32) / np.float32(0x7FFFFFFF)
    return torch.from_numpy((u * np.float32(2.0) - np.float32(1.0)) * np.float32(scale))


def init_flat(layout: ArenaLayout, seed: int = 42, dtype=torch.float32) -> torch.Tensor:
    """Initial flat parameter vector.

    ``init="xorshift"``: weights/embeddings uniform in +-0.02 from seeds ``seed + {0,1,2,10,...}``,
    LayerNorm gamma 1, beta 0, biases 0 (``transformer.cu:237-252``).
    ``init="normal"``: weights/embeddings ``N(0, 0.02)`` from a ``torch.Generator`` seeded per tensor.
    """
    flat = torch.zeros(layout.total, dtype=torch.float32)
    for s in layout.specs:
        dst = flat[s.offset:s.offset + s.numel]
        if s.kind == "ln_gamma":
            dst.fill_(1.0)
        elif s.kind in ("ln_beta", "bias"):
            dst.zero_()
        elif layout.cfg.init == "xorshift":
            dst.copy_(xorshift_uniform(s.numel, seed + s.init_seed))
        else:
            g = torch.Generator().manual_seed(seed * 1000003 + s.init_seed)
            dst.copy_(torch.randn(s.numel, generator=g) * 0.02)
    return flat.to(dtype)
