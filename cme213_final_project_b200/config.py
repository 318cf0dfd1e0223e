"""Run-time configuration: model shape, optimizer, synchronisation policy, presets and validation.

The reference fixes the model shape at compile time (``-DHIDDEN_DIM`` ... in
``FINAL_CLEAN_CODE_/include/common.h:32-62``), parses run flags by hand
(``FINAL_CLEAN_CODE_/src/main.cu:148-184``) and toggles features with ``CME213_*`` environment
variables checked by ``validate_cme213_config`` (``main.cu:91-132``).  Here everything is one run-time
configuration.  The reference's flag names and the ``--validate-config`` contract (exit status 0 and the
line ``Configuration validation: PASS``, or exit status 2 and ``Invalid CME213 configuration: ...`` on
stderr) are kept; the environment toggles are still honoured so existing job scripts keep working.
"""
from __future__ import annotations

import argparse
import dataclasses
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple


@dataclass
class ModelConfig:
    """Shape and functional variant of the transformer.

    ``mode="parity"`` is the reference's exact function (``FINAL_CLEAN_CODE_/src/model/transformer.cu:337-408``):
    one block, ReLU, non-causal attention, heads as a flat reinterpretation of ``[B*T, D]`` as
    ``[B*H, T, HD]``, untied input/output embeddings, no final LayerNorm.
    ``mode="gpt"`` is a standard pre-LN GPT decoder: N blocks, GELU (tanh form), causal attention,
    the usual head split, tied embeddings and a final LayerNorm.
    """

    mode: str = "parity"
    vocab_size: int = 65
    seq_len: int = 64
    hidden: int = 128
    heads: int = 4
    ff: int = 512
    layers: int = 1
    batch_size: int = 32           # sequences per rank per micro-step
    activation: str = "relu"       # "relu" | "gelu"
    causal: bool = False
    head_layout: str = "flat"      # "flat" (reference view) | "split" (standard [B,H,T,HD])
    tied_embeddings: bool = False
    final_layernorm: bool = False
    ln_eps: float = 1e-5
    init: str = "xorshift"         # "xorshift" (reference) | "normal" (N(0, 0.02))

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def tokens_per_step(self) -> int:
        return self.batch_size * self.seq_len

    def validate(self) -> List[str]:
        errs = []
        if self.mode not in ("parity", "gpt"):
            errs.append(f"unknown model mode '{self.mode}'")
        if self.hidden % self.heads:
            errs.append("hidden must be divisible by heads")
        if self.activation not in ("relu", "gelu"):
            errs.append(f"unknown activation '{self.activation}'")
        if self.head_layout not in ("flat", "split"):
            errs.append(f"unknown head layout '{self.head_layout}'")
        if self.head_layout == "flat" and self.seq_len % self.heads:
            errs.append("flat head layout needs seq_len divisible by heads")
        if self.mode == "parity" and (self.layers != 1 or self.tied_embeddings or self.final_layernorm
                                      or self.causal or self.activation != "relu" or self.head_layout != "flat"):
            errs.append("parity mode is the reference function: 1 layer, relu, non-causal, flat heads, untied, no final LN")
        return errs


@dataclass
class OptimConfig:
    """Adam (reference: betas 0.9/0.999, eps 1e-8, global-norm clip 1.0 inside the update,
    ``transformer.cu:598-636``) or AdamW (GPT mode: betas 0.9/0.95, weight decay 0.1, no clip)."""

    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0
    clip_norm: float = 1.0         # <= 0 disables clipping


@dataclass
class RunConfig:
    """Flags of the training driver (names follow ``main.cu:148-184``)."""

    data_path: str = "inp.txt"
    epochs: int = 10
    max_steps: int = -1
    sync_mode: str = "blocking"    # blocking | overlap | auto
    bucket_kb: int = 0
    auto_overlap_max_mb: float = 8.0
    validate_config: bool = False
    trace_trajectory: bool = False
    # additions
    comm_backend: str = "auto"     # auto | fused | nccl | gloo | host
    comm_algo: str = "auto"        # fused path, per bucket: auto (measured table) | one_shot | two_shot | nvls
    comm_table: Optional[str] = None   # JSON written by benchmarks/bench_allreduce.py --table (default: the shipped one)
    defer_grad_avg: bool = False
    comm_thread: bool = False
    cuda_graph: bool = False
    grad_accum: int = 1
    gemm_backend: str = "auto"     # auto | tcgen05 | simt
    compute_dtype: str = "bf16"    # bf16 | tf32 (fp32 storage, tf32 tensor-core products) | fp32 (strict: SIMT)
    synthetic: bool = False
    seed: int = 42
    save_checkpoint: Optional[str] = None
    load_checkpoint: Optional[str] = None
    profile: bool = False
    device: str = "auto"           # auto | cuda | cpu
    engine: str = "auto"           # auto | native | torch
    log_every: int = 100
    step_timeout_s: float = 0.0    # > 0: end the process if no step completes for this long (host watchdog)
    epilogue_fusion: bool = True   # False: bias / activation / residual as separate kernels (ablation)
    ffn_precision: str = "full"    # fp32 storage only: full | store (feed-forward activation kept at bf16 precision)
                                   # | bf16 (feed-forward products on bf16 copies of their operands, fp32 results)


# --------------------------------------------------------------------------------------------------
# Presets: the reference's three logged shapes and the five target configurations.
# --------------------------------------------------------------------------------------------------

def _parity(hidden: int) -> Tuple[ModelConfig, OptimConfig]:
    return (ModelConfig(mode="parity", hidden=hidden, ff=4 * hidden, heads=4, seq_len=64, vocab_size=65,
                        batch_size=32, layers=1),
            OptimConfig(lr={128: 3e-4, 256: 1e-4, 512: 5e-5}.get(hidden, 1e-4)))


def _gpt(vocab, ctx, d, heads, layers, ff, batch) -> Tuple[ModelConfig, OptimConfig]:
    return (ModelConfig(mode="gpt", vocab_size=vocab, seq_len=ctx, hidden=d, heads=heads, layers=layers, ff=ff,
                        batch_size=batch, activation="gelu", causal=True, head_layout="split",
                        tied_embeddings=True, final_layernorm=True, init="normal"),
            OptimConfig(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, clip_norm=0.0))


PRESETS: Dict[str, Tuple[ModelConfig, OptimConfig]] = {
    "parity-h128": _parity(128),
    "parity-h256": _parity(256),
    "parity-h512": _parity(512),
    "tiny-gpt": _gpt(65, 64, 128, 4, 2, 512, 8),
    "char-gpt": _gpt(65, 256, 384, 6, 6, 1536, 64),
    "gpt2-small": _gpt(50304, 1024, 768, 12, 12, 3072, 16),
    "gpt2-medium": _gpt(50304, 1024, 1024, 16, 24, 4096, 8),
}


def preset(name: str) -> Tuple[ModelConfig, OptimConfig]:
    if name not in PRESETS:
        raise KeyError(f"unknown preset '{name}' (have: {', '.join(sorted(PRESETS))})")
    m, o = PRESETS[name]
    return dataclasses.replace(m), dataclasses.replace(o)


# --------------------------------------------------------------------------------------------------
# Environment toggles (the reference's CME213_* variables, FINAL_CLEAN_CODE_/scripts/common_env.sh:6-20)
# --------------------------------------------------------------------------------------------------

ENV_TOGGLES = (
    "CME213_GEMM_BACKEND", "CME213_LT_FUSION", "CME213_USE_CUDA_GRAPH", "CME213_USE_NCCL",
    "CME213_ALLOW_UNVALIDATED_NCCL", "CME213_COMM_THREAD", "CME213_DEFER_GRAD_AVG_TO_ADAM",
    "CME213_ASYNC_DEVICE_MPI", "CME213_CUDA_AWARE_MPI", "CME213_STRICT_FP32", "CME213_MIXED_PRECISION",
    "CME213_FP16_STORAGE_ONLY", "CME213_FFN_FP16",
)


# The reference selects among its own kernels and two library paths (``gemm.cu:16-106``).  This framework has two
# GEMM implementations, both its own: the tcgen05 tensor-core kernel and the SIMT kernel.  The reference's names
# are accepted and mapped onto them: its hand-written kernels to the SIMT kernel, its library paths (which exist
# to reach the tensor cores) to the tensor-core kernel.
GEMM_BACKEND_MAP = {"auto": "tcgen05", "custom": "simt", "cublas": "tcgen05", "cublas_tc": "tcgen05",
                    "tcgen05": "tcgen05", "simt": "simt"}


def env_enabled(name: str, env: Optional[Dict[str, str]] = None) -> bool:
    """A toggle is on when set to anything but the empty string or "0" (``main.cu:69-72``)."""
    v = (os.environ if env is None else env).get(name)
    return v is not None and v != "" and v != "0"


def environment_report(env: Optional[Dict[str, str]] = None, gemm_requested: str = "auto") -> List[str]:
    """The ``CME213 environment:`` banner (``main.cu:74-89``)."""
    env = os.environ if env is None else env
    lines = ["CME213 environment:"]
    found = [f"  {k}={v}" for k, v in env.items() if k.startswith("CME213_")]
    lines += found if found else ["  (none set)"]
    lines.append(f"  GEMM requested={gemm_requested} effective={GEMM_BACKEND_MAP.get(gemm_requested, gemm_requested)} "
                 f"auto_policy=tcgen05")
    return lines


def validate_environment(world_size: int, env: Optional[Dict[str, str]] = None) -> Tuple[List[str], List[str]]:
    """Return ``(errors, warnings)`` for the toggle combination, with the reference's rules
    (``main.cu:91-132``) re-expressed for this framework.

    * the fp16 experiments must not be combined with epilogue fusion and exclude one another;
    * ``CME213_MIXED_PRECISION`` names a mode this framework provides as ``--compute-dtype bf16``;
      the variable itself stays rejected so that a script relying on the reference's refusal still sees it;
    * the fp16 experiments are single-GPU only; ``CME213_FFN_FP16`` is not combined with graphs.
    """
    errs: List[str] = []
    warns: List[str] = []
    on = lambda n: env_enabled(n, env)
    mixed, fp16s, ffn16 = on("CME213_MIXED_PRECISION"), on("CME213_FP16_STORAGE_ONLY"), on("CME213_FFN_FP16")
    if (mixed or fp16s or ffn16) and on("CME213_LT_FUSION"):
        errs.append("FP16 modes must not be combined with CME213_LT_FUSION=1")
    if mixed:
        errs.append("CME213_MIXED_PRECISION is planned but not implemented in this build")
    if (mixed and fp16s) or (mixed and ffn16) or (fp16s and ffn16):
        errs.append("CME213_MIXED_PRECISION, CME213_FP16_STORAGE_ONLY, and CME213_FFN_FP16 are mutually exclusive")
    if (fp16s or ffn16) and world_size > 1:
        errs.append("FP16 experimental paths are currently validated only for single-GPU runs")
    if ffn16 and on("CME213_USE_CUDA_GRAPH"):
        errs.append("CME213_FFN_FP16 is not yet validated with CME213_USE_CUDA_GRAPH=1")
    if on("CME213_USE_NCCL") and not on("CME213_ALLOW_UNVALIDATED_NCCL"):
        warns.append("Warning: CME213_USE_NCCL=1 requested without CME213_ALLOW_UNVALIDATED_NCCL=1; "
                     "the fused peer-memory path stays the default")
    backend = (os.environ if env is None else env).get("CME213_GEMM_BACKEND")
    if backend not in (None, "") and backend not in GEMM_BACKEND_MAP:
        errs.append(f"unknown CME213_GEMM_BACKEND '{backend}'")
    return errs, warns


def validate_run(model: ModelConfig, run: RunConfig, world_size: int) -> List[str]:
    errs = list(model.validate())
    if run.sync_mode not in ("blocking", "overlap", "auto"):
        errs.append(f"Unknown sync mode '{run.sync_mode}'")
    if run.comm_backend not in ("auto", "fused", "nccl", "gloo", "host"):
        errs.append(f"unknown comm backend '{run.comm_backend}'")
    if run.grad_accum < 1:
        errs.append("--grad-accum must be >= 1")
    if run.bucket_kb < 0:
        errs.append("--bucket-kb must be >= 0")
    if run.compute_dtype not in ("bf16", "tf32", "fp32"):
        errs.append(f"unknown compute dtype '{run.compute_dtype}'")
    if run.ffn_precision not in ("full", "store", "bf16"):
        errs.append(f"unknown feed-forward precision '{run.ffn_precision}'")
    elif run.ffn_precision != "full" and run.compute_dtype == "bf16":
        errs.append("--ffn-precision store|bf16 applies to fp32 storage (--compute-dtype tf32 or fp32); "
                    "bf16 storage already runs the feed-forward products in bf16")
    if run.gemm_backend not in ("auto", "tcgen05", "simt"):
        errs.append(f"unknown gemm backend '{run.gemm_backend}'")
    if run.comm_algo not in ("auto", "one_shot", "two_shot", "nvls"):
        errs.append(f"unknown comm algorithm '{run.comm_algo}'")
    if run.comm_thread and run.comm_backend == "fused":
        errs.append("--comm-thread drives host-issued collectives; it is not combined with the fused device path")
    return errs


def apply_environment(run: RunConfig, env: Optional[Dict[str, str]] = None) -> RunConfig:
    """Fold the reference's environment toggles into the run configuration."""
    e = os.environ if env is None else env
    run = dataclasses.replace(run)
    if env_enabled("CME213_USE_CUDA_GRAPH", e):
        run.cuda_graph = True
    if env_enabled("CME213_DEFER_GRAD_AVG_TO_ADAM", e):
        run.defer_grad_avg = True
    if env_enabled("CME213_COMM_THREAD", e):
        run.comm_thread = True
    if env_enabled("CME213_USE_NCCL", e) and env_enabled("CME213_ALLOW_UNVALIDATED_NCCL", e):
        run.comm_backend = "nccl"
    if e.get("CME213_LT_FUSION") == "0":          # the reference's epilogue-fusion switch, here on by default
        run.epilogue_fusion = False
    if env_enabled("CME213_STRICT_FP32", e):
        run.compute_dtype = "fp32"
    # the reference's reduced-precision feed-forward experiments act on its fp32 storage
    # (FINAL_CLEAN_CODE_/src/model/transformer.cu:37-45); here they select fp32 storage with tf32 products unless
    # strict fp32 was asked for, and 16-bit means bf16
    for name, mode in (("CME213_FP16_STORAGE_ONLY", "store"), ("CME213_FFN_FP16", "bf16")):
        if env_enabled(name, e):
            run.ffn_precision = mode
            if run.compute_dtype == "bf16":
                run.compute_dtype = "tf32"
    b = e.get("CME213_GEMM_BACKEND")
    if b:
        run.gemm_backend = GEMM_BACKEND_MAP.get(b, b) if b != "auto" else "auto"
    return run


# --------------------------------------------------------------------------------------------------
# Command line
# --------------------------------------------------------------------------------------------------

def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="train", description="B200-native data-parallel transformer trainer")
    p.add_argument("data", nargs="?", default="inp.txt", help="text file (character-level corpus)")
    p.add_argument("--epochs", type=int, default=10)
    p.add_argument("--max-steps", type=int, default=-1)
    p.add_argument("--lr", type=float, default=None)
    p.add_argument("--overlap", action="store_true", help="same as --sync-mode overlap")
    p.add_argument("--auto-sync", action="store_true", help="same as --sync-mode auto")
    p.add_argument("--sync-mode", default=None)
    p.add_argument("--bucket-kb", type=int, default=0)
    p.add_argument("--auto-overlap-max-mb", type=float, default=8.0)
    p.add_argument("--validate-config", action="store_true")
    p.add_argument("--trace-trajectory", action="store_true")
    # model shape (compile-time macros in the reference)
    p.add_argument("--preset", default="parity-h128", choices=sorted(PRESETS))
    p.add_argument("--hidden", type=int)
    p.add_argument("--ff", type=int)
    p.add_argument("--heads", type=int)
    p.add_argument("--layers", type=int)
    p.add_argument("--seq-len", type=int)
    p.add_argument("--batch-size", type=int)
    p.add_argument("--vocab-size", type=int)
    # run options
    p.add_argument("--comm-backend", default="auto")
    p.add_argument("--comm-algo", default="auto", help="fused path: auto (measured table) | one_shot | two_shot | nvls")
    p.add_argument("--comm-table", default=None, help="algorithm table written by benchmarks/bench_allreduce.py")
    p.add_argument("--defer-grad-avg", action="store_true")
    p.add_argument("--comm-thread", action="store_true")
    p.add_argument("--cuda-graph", action="store_true")
    p.add_argument("--grad-accum", type=int, default=1)
    p.add_argument("--gemm-backend", default="auto")
    p.add_argument("--compute-dtype", default="bf16")
    p.add_argument("--synthetic", action="store_true", help="uniform random token ids instead of a text file")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--save-checkpoint")
    p.add_argument("--load-checkpoint")
    p.add_argument("--profile", action="store_true", help="emit NVTX ranges")
    p.add_argument("--device", default="auto")
    p.add_argument("--engine", default="auto")
    p.add_argument("--log-every", type=int, default=100)
    p.add_argument("--step-timeout", type=float, default=0.0,
                   help="seconds without a completed step after which the process ends itself (0 = off)")
    p.add_argument("--ffn-precision", default="full",
                   help="fp32 storage: full | store (activation kept at bf16 precision) | bf16 (bf16 operand copies)")
    p.add_argument("--no-epilogue-fusion", action="store_true",
                   help="run bias / activation / residual / activation-derivative as separate kernels (ablation)")
    return p


def parse_args(argv: Optional[Sequence[str]] = None) -> Tuple[ModelConfig, OptimConfig, RunConfig]:
    a = build_parser().parse_args(argv)
    model, optim = preset(a.preset)
    for name, attr in (("hidden", "hidden"), ("ff", "ff"), ("heads", "heads"), ("layers", "layers"),
                       ("seq_len", "seq_len"), ("batch_size", "batch_size"), ("vocab_size", "vocab_size")):
        v = getattr(a, name)
        if v is not None:
            setattr(model, attr, v)
    if a.hidden is not None and a.ff is None:
        model.ff = 4 * model.hidden
    if a.lr is not None:
        optim.lr = a.lr
    sync = a.sync_mode or ("overlap" if a.overlap else "auto" if a.auto_sync else "blocking")
    run = RunConfig(data_path=a.data, epochs=a.epochs, max_steps=a.max_steps, sync_mode=sync,
                    bucket_kb=a.bucket_kb, auto_overlap_max_mb=a.auto_overlap_max_mb,
                    validate_config=a.validate_config, trace_trajectory=a.trace_trajectory,
                    comm_backend=a.comm_backend, comm_algo=a.comm_algo, comm_table=a.comm_table,
                    defer_grad_avg=a.defer_grad_avg, comm_thread=a.comm_thread,
                    cuda_graph=a.cuda_graph, grad_accum=a.grad_accum, gemm_backend=a.gemm_backend,
                    compute_dtype=a.compute_dtype, synthetic=a.synthetic, seed=a.seed,
                    save_checkpoint=a.save_checkpoint, load_checkpoint=a.load_checkpoint, profile=a.profile,
                    device=a.device, engine=a.engine, log_every=a.log_every,
                    epilogue_fusion=not a.no_epilogue_fusion, step_timeout_s=a.step_timeout,
                    ffn_precision=a.ffn_precision)
    return model, optim, apply_environment(run)


def effective_overlap(run: RunConfig, grad_mb: float, world_size: int) -> bool:
    """``--sync-mode auto`` overlaps iff the gradient volume is at most ``--auto-overlap-max-mb``
    (``main.cu:219-227``); a single rank never synchronises."""
    if world_size <= 1:
        return False
    return run.sync_mode == "overlap" or (run.sync_mode == "auto" and grad_mb <= run.auto_overlap_max_mb)


def min_bucket_elems(bucket_kb: int, elem_bytes: int = 4) -> int:
    """``--bucket-kb K`` -> smallest bucket in elements (``main.cu:196-200``)."""
    return (bucket_kb * 1024 + elem_bytes - 1) // elem_bytes if bucket_kb > 0 else 0
