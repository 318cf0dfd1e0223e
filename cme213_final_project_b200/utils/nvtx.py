"""NVTX ranges, emitted only when profiling is requested.

Role of the reference's ``NvtxRange`` RAII helper (``FINAL_CLEAN_CODE_/include/profiling.h:8-22``), which
is compiled in with ``USE_NVTX=1``; here it is a run-time switch (``--profile``)."""
from __future__ import annotations

import contextlib

import torch


@contextlib.contextmanager
def nvtx_range(name: str, enabled: bool = False):
    on = enabled and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
