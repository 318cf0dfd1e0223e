"""Flat checkpoint dump / load, parameter statistics and the trajectory hash.

The reference has no file output; what it has is (a) the flat in-memory order of parameters and Adam
moments (``FINAL_CLEAN_CODE_/include/model.h:115-123``) and (b) ``--trace-trajectory``, which copies
the whole parameter buffer to the host every step and prints its sum, sum of squares, max |x| and an
FNV-1a hash of the raw float bits (``FINAL_CLEAN_CODE_/src/main.cu:40-65,397-418``).  The dump format
defined here stores exactly that state, in that order, and the loader re-computes the four statistics
to verify integrity.

File layout (little-endian):

    magic    8 bytes  b"CME213CK"
    version  u32      1
    header   u32 len + UTF-8 JSON: model config, optimizer step, tensor table (name, shape, offset),
                      statistics of the parameter section
    params   f32[num_params]   tensors packed tightly in arena order (no alignment padding)
    adam_m   f32[num_params]
    adam_v   f32[num_params]
"""
from __future__ import annotations

import dataclasses
import json
import struct
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from .arena import ArenaLayout
from .config import ModelConfig

MAGIC = b"CME213CK"
VERSION = 1
FNV_OFFSET = 1469598103934665603
FNV_PRIME = 1099511628211
_MASK = (1 << 64) - 1


@dataclass
class ParamStats:
    sum: float = 0.0
    sumsq: float = 0.0
    max_abs: float = 0.0
    hash: int = FNV_OFFSET

    def hex_hash(self) -> str:
        return f"{self.hash:016x}"


def fnv1a_words(bits: np.ndarray, h: int = FNV_OFFSET) -> int:
    """FNV-1a over 32-bit words: ``h ^= word; h *= prime`` (64-bit wrap), one round per float —
    the reference hashes whole float bit patterns, not bytes (``main.cu:57-62``)."""
    from .ops import host_lib
    lib = host_lib()
    bits = np.ascontiguousarray(bits, dtype=np.uint32)
    if lib is not None:
        return int(lib.fnv1a_u32(bits.ctypes.data, bits.size, h))
    for w in bits.tolist():
        h = ((h ^ w) * FNV_PRIME) & _MASK
    return h


def param_stats(flat: torch.Tensor) -> ParamStats:
    """Sum, sum of squares and max |x| in float64 plus the bit hash of a float32 vector."""
    a = flat.detach().to(torch.float32).cpu().contiguous().numpy()
    d = a.astype(np.float64)
    return ParamStats(float(d.sum()), float((d * d).sum()), float(np.abs(d).max()) if d.size else 0.0,
                      fnv1a_words(a.view(np.uint32)))


def _pack(layout: ArenaLayout, flat: torch.Tensor) -> np.ndarray:
    a = flat.detach().to(torch.float32).cpu().numpy()
    return np.concatenate([a[s.offset:s.offset + s.numel] for s in layout.specs]) if layout.specs else a[:0]


def _unpack(layout: ArenaLayout, packed: np.ndarray) -> torch.Tensor:
    out = np.zeros(layout.total, dtype=np.float32)
    pos = 0
    for s in layout.specs:
        out[s.offset:s.offset + s.numel] = packed[pos:pos + s.numel]
        pos += s.numel
    return torch.from_numpy(out)


def save_checkpoint(path: str, layout: ArenaLayout, params: torch.Tensor, adam_m: torch.Tensor,
                    adam_v: torch.Tensor, step: int, extra: Optional[Dict] = None) -> ParamStats:
    p = _pack(layout, params)
    stats = ParamStats(float(p.astype(np.float64).sum()), float((p.astype(np.float64) ** 2).sum()),
                       float(np.abs(p).max()) if p.size else 0.0, fnv1a_words(p.view(np.uint32)))
    header = {
        "model": dataclasses.asdict(layout.cfg),
        "step": int(step),
        "num_params": int(p.size),
        "dtype": "float32",
        "tensors": [{"name": s.name, "shape": list(s.shape)} for s in layout.specs],
        "stats": {"sum": stats.sum, "sumsq": stats.sumsq, "max_abs": stats.max_abs, "hash": stats.hex_hash()},
        "extra": extra or {},
    }
    hb = json.dumps(header).encode("utf-8")
    with open(path, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<II", VERSION, len(hb)))
        f.write(hb)
        f.write(p.astype("<f4").tobytes())
        f.write(_pack(layout, adam_m).astype("<f4").tobytes())
        f.write(_pack(layout, adam_v).astype("<f4").tobytes())
    return stats


def load_checkpoint(path: str, layout: Optional[ArenaLayout] = None, verify: bool = True
                    ) -> Tuple[ArenaLayout, torch.Tensor, torch.Tensor, torch.Tensor, int, Dict]:
    with open(path, "rb") as f:
        if f.read(8) != MAGIC:
            raise ValueError(f"{path}: not a CME213 checkpoint")
        version, hlen = struct.unpack("<II", f.read(8))
        if version != VERSION:
            raise ValueError(f"{path}: unsupported checkpoint version {version}")
        header = json.loads(f.read(hlen).decode("utf-8"))
        n = header["num_params"]
        body = np.frombuffer(f.read(3 * 4 * n), dtype="<f4")
    if body.size != 3 * n:
        raise ValueError(f"{path}: truncated checkpoint ({body.size} of {3 * n} floats)")
    cfg = ModelConfig(**header["model"])
    if layout is None:
        layout = ArenaLayout(cfg)
    names = [(s.name, list(s.shape)) for s in layout.specs]
    if names != [(t["name"], t["shape"]) for t in header["tensors"]]:
        raise ValueError(f"{path}: tensor table does not match the model configuration")
    p, m, v = body[:n].copy(), body[n:2 * n].copy(), body[2 * n:].copy()
    if verify:
        st = header["stats"]
        got = fnv1a_words(p.view(np.uint32))
        if f"{got:016x}" != st["hash"]:
            raise ValueError(f"{path}: parameter hash mismatch ({got:016x} != {st['hash']})")
        if not np.isclose(p.astype(np.float64).sum(), st["sum"], rtol=1e-12, atol=1e-12):
            raise ValueError(f"{path}: parameter sum mismatch")
    return layout, _unpack(layout, p), _unpack(layout, m), _unpack(layout, v), int(header["step"]), header


def trajectory_line(epoch: int, step: int, loss: float, stats: ParamStats, spans: Tuple[float, float, float]) -> str:
    """The ``TRAJECTORY`` line, field for field as the reference prints it (``main.cu:408-416``)."""
    return ("TRAJECTORY epoch=%d step=%d loss=%.9g param_sum=%.17g param_sumsq=%.17g "
            "param_maxabs=%.9g param_hash=%016x sum_span=%.3e sumsq_span=%.3e maxabs_span=%.3e"
            % (epoch, step, loss, stats.sum, stats.sumsq, stats.max_abs, stats.hash,
               spans[0], spans[1], spans[2]))
