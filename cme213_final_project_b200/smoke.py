"""One tiny training step of the flagship (GPT-mode) model on a GPU through the native engine."""
from __future__ import annotations

import torch

from .config import ModelConfig, OptimConfig, RunConfig
from .data import synthetic_batches


def run_smoke(device: torch.device) -> float:
    from .models.engine import NativeEngine
    torch.cuda.set_device(device)
    cfg = ModelConfig(mode="gpt", vocab_size=512, seq_len=128, hidden=128, heads=2, ff=512, layers=2, batch_size=4,
                      activation="gelu", causal=True, head_layout="split", tied_embeddings=True, final_layernorm=True,
                      init="normal")
    opt = OptimConfig(lr=1e-3, beta2=0.95, weight_decay=0.1, clip_norm=0.0)
    eng = NativeEngine(cfg, opt, RunConfig(), device=device)
    x, y = synthetic_batches(cfg.vocab_size, cfg.seq_len, cfg.batch_size, 4, seed=0)
    x, y = x.to(device), y.to(device)
    first = None
    for i in range(4):
        eng.train_step([x[0]], [y[0]])
        eng.update()
        loss = eng.read_loss()
        first = loss if first is None else first
    assert ops_ok(), "a bounded device wait ran out"
    assert loss == loss and loss < first, (first, loss)
    print(f"smoke: loss {first:.4f} -> {loss:.4f}")
    return loss


def ops_ok() -> bool:
    from . import ops
    return ops.gemm_check_status() == 0
