"""The native sm_100a engine behind the flat-arena model interface.

Python owns memory (arenas and the activation workspace are ``torch`` tensors), policy (bucket
coalescing, which synchronisation path runs, CUDA-graph capture) and the optimizer launch; the C++
executor (``ops/csrc/engine.cu``) owns the op sequence of forward and backward.  Interface and role
match the reference's ``TransformerModel`` (``FINAL_CLEAN_CODE_/include/model.h:93-145``): public flat
buffers, ``zero_grad / forward / backward / update / read_loss``.

Arenas: ``params`` (compute dtype: bf16, or fp32 in strict mode), ``master`` (fp32; aliases ``params`` in
strict mode), ``grads`` (compute dtype), ``adam_m`` / ``adam_v`` (fp32).
"""
from __future__ import annotations

import ctypes
from typing import Callable, List, Optional, Sequence

import torch

from .. import ops
from ..arena import ArenaLayout, Bucket, init_flat
from ..config import ModelConfig, OptimConfig, RunConfig


class _EngineDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("V", "T", "D", "H", "FF", "L", "B", "act", "causal", "head_flat", "tied",
                                             "final_ln", "fused_qkv", "allow_tf32", "fuse_epilogues", "ffn_lowp")] + \
               [("ln_eps", ctypes.c_float), ("prob_eps", ctypes.c_float)] + \
               [(n, ctypes.c_int) for n in ("dtype", "gemm_backend", "attn_backend")]


class _LayerSlots(ctypes.Structure):
    _fields_ = [(n, ctypes.c_longlong) for n in ("W2", "b2", "W1", "b1", "ln2g", "ln2b", "Wo", "Wq", "Wk", "Wv",
                                                  "Wqkv", "ln1g", "ln1b")]


class _GlobalSlots(ctypes.Structure):
    _fields_ = [(n, ctypes.c_longlong) for n in ("Wout", "lnfg", "lnfb", "tok", "pos")]


_BUCKET_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int)


class NativeEngine:
    handles_sync = False

    def __init__(self, cfg: ModelConfig, optim: OptimConfig, run: Optional[RunConfig] = None, dist_ctx=None,
                 seed: int = 42, device=None, shard_multiple: int = 1, align: int = 64) -> None:
        run = run or RunConfig()
        self.cfg, self.optim, self.run = cfg, optim, run
        self.device = torch.device(device) if device is not None else (
            dist_ctx.device if dist_ctx is not None else torch.device("cuda", torch.cuda.current_device()))
        if self.device.type != "cuda":
            raise ops.NativeError("the native engine needs a CUDA device")
        self.lib = ops.lib()
        with torch.cuda.device(self.device):
            ops._check(self.lib.cme_init_device())               # status words exist before any stream capture
        # "fp32": fp32 storage and exact fp32 products on the SIMT kernels (the reference's CME213_STRICT_FP32);
        # "tf32": fp32 storage, products on the tensor cores with tf32 inputs and fp32 accumulation, element-wise work
        # in separate fp32 kernels (the reference's default: fp32 storage with tensor-core math through cuBLAS,
        # FINAL_CLEAN_CODE_/src/kernels/gemm.cu:274-289); "bf16": bf16 storage with fp32 master weights.
        self.tf32 = run.compute_dtype == "tf32"
        self.strict = run.compute_dtype in ("fp32", "tf32")          # fp32 storage: params are the master copy
        self.dtype = torch.float32 if self.strict else torch.bfloat16
        # `align` (elements) is 64 unless the arena has to split into per-rank slices for a world size whose
        # 8 * world does not divide 64 (parallel.fused_sync.shard_align)
        self.layout = ArenaLayout(cfg, align=align, shard_multiple=shard_multiple)
        n = self.layout.total
        with torch.cuda.device(self.device):
            flat = init_flat(self.layout, seed).to(self.device)
            self.master = flat                                    # fp32
            self.params = flat if self.strict else flat.to(torch.bfloat16)
            self.grads = torch.zeros(n, dtype=self.dtype, device=self.device)
            self.adam_m = torch.zeros(n, dtype=torch.float32, device=self.device)
            self.adam_v = torch.zeros(n, dtype=torch.float32, device=self.device)
            self.step_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.lr_dev = torch.full((1,), optim.lr, dtype=torch.float32, device=self.device)
            self.loss_dev = torch.zeros(1, dtype=torch.float32, device=self.device)
            self.normsq = torch.zeros(1, dtype=torch.float32, device=self.device)
            # early loss read-back: after the forward of every step the loss and a sequence number are copied to
            # pinned host memory, so a caller can read the step's loss while backward is still running
            self.seq_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
            self.seq_host = torch.zeros(1, dtype=torch.int32).pin_memory()
            self._norm_partial = torch.empty(1024, dtype=torch.float32, device=self.device)
        self.seq_expected = 0          # steps handed to the device so far (the trainer counts graph replays too)
        self._loss_host_dev, self._seq_host_dev = ctypes.c_void_p(), ctypes.c_void_p()
        ops._check(self.lib.cme_host_device_ptr(ctypes.c_void_p(self.loss_host.data_ptr()),
                                                ctypes.byref(self._loss_host_dev)))
        ops._check(self.lib.cme_host_device_ptr(ctypes.c_void_p(self.seq_host.data_ptr()),
                                                ctypes.byref(self._seq_host_dev)))
        nd = [(s.offset, s.offset + s.numel) for s in self.layout.specs if s.kind not in ("weight", "embed")]
        self.nodecay = torch.tensor(nd, dtype=torch.int64, device=self.device).reshape(-1, 2)
        self.step_count = 0

        gemm_backend = {"auto": 0, "tcgen05": 0, "simt": 2}[run.gemm_backend]
        d = _EngineDesc(V=cfg.vocab_size, T=cfg.seq_len, D=cfg.hidden, H=cfg.heads, FF=cfg.ff, L=cfg.layers,
                        B=cfg.batch_size, act=ops.ACT[cfg.activation], causal=int(cfg.causal),
                        head_flat=int(cfg.head_layout == "flat"), tied=int(cfg.tied_embeddings),
                        final_ln=int(cfg.final_layernorm), fused_qkv=int(cfg.mode == "gpt"),
                        allow_tf32=int(self.tf32), fuse_epilogues=int(run.epilogue_fusion and not self.tf32),
                        ffn_lowp={"full": 0, "store": 1, "bf16": 2}[run.ffn_precision] if self.strict else 0,
                        ln_eps=cfg.ln_eps,
                        prob_eps=1e-9 if cfg.mode == "parity" else 0.0, dtype=ops.F32 if self.strict else ops.BF16,
                        gemm_backend=gemm_backend if (self.tf32 or not self.strict) else 2,
                        attn_backend=2 if self.strict else 0)
        off = lambda name: self.layout.by_name[name].offset if name in self.layout.by_name else -1
        layers = (_LayerSlots * cfg.layers)()
        for l in range(cfg.layers):
            p = f"h{l}." if (cfg.layers > 1 or cfg.mode == "gpt") else ""
            layers[l] = _LayerSlots(off(p + "W2"), off(p + "b2"), off(p + "W1"), off(p + "b1"), off(p + "ln2_gamma"),
                                    off(p + "ln2_beta"), off(p + "Wo"), off(p + "Wq"), off(p + "Wk"), off(p + "Wv"),
                                    off(p + "Wqkv"), off(p + "ln1_gamma"), off(p + "ln1_beta"))
        g = _GlobalSlots(off("Wout"), off("lnf_gamma"), off("lnf_beta"), off("tok_embed"), off("pos_embed"))
        self._h = ctypes.c_void_p()
        self.lib.cme_engine_workspace_bytes.restype = ctypes.c_longlong
        self.lib.cme_engine_logits.restype = ctypes.c_void_p
        ops._check(self.lib.cme_engine_create(ctypes.byref(d), layers, ctypes.byref(g), ctypes.byref(self._h)))
        nbytes = int(self.lib.cme_engine_workspace_bytes(self._h))
        self.workspace = torch.empty(nbytes + 256, dtype=torch.uint8, device=self.device)
        base = (self.workspace.data_ptr() + 255) // 256 * 256
        ops._check(self.lib.cme_engine_bind(self._h, ctypes.c_void_p(self.params.data_ptr()),
                                            ctypes.c_void_p(self.grads.data_ptr()), ctypes.c_void_p(base),
                                            ctypes.c_longlong(nbytes)))
        self._ws_base, self._ws_bytes = base, nbytes
        # weight-gradient products on a second stream beside the input-gradient chain (CME213_WGRAD_STREAM=0: off)
        import os
        self.overlap_wgrad = False
        self.set_overlap(os.environ.get("CME213_WGRAD_STREAM", "1") != "0")
        self._tokens: Optional[torch.Tensor] = None
        self._cb_keepalive = None
        self.fused = None                 # set by parallel.fused_sync.attach_fused_sync
        self.handles_sync = False

    def set_overlap(self, on: bool) -> None:
        """Run the weight-gradient products of backward on the engine's second stream (outside stream capture)."""
        with torch.cuda.device(self.device):
            ops._check(self.lib.cme_engine_set_overlap(self._h, int(bool(on))))
        self.overlap_wgrad = bool(on)

    def fence(self, target: "torch.cuda.Stream") -> None:
        """Make ``target`` wait for everything backward has enqueued so far, on the current stream and on the
        engine's second stream: call it from a bucket callback before reading the bucket on ``target``."""
        ops._check(self.lib.cme_engine_fence(self._h, ops._stream(), ctypes.c_void_p(target.cuda_stream)))

    def rebind(self, params: torch.Tensor, grads: torch.Tensor) -> None:
        """Point the executor at other parameter / gradient arenas (e.g. symmetric, peer-mapped buffers)."""
        assert params.numel() >= self.layout.total and grads.numel() >= self.layout.total
        assert params.dtype == self.dtype and grads.dtype == self.dtype
        self.params, self.grads = params, grads
        if self.strict:
            self.master = params
        ops._check(self.lib.cme_engine_bind(self._h, ctypes.c_void_p(params.data_ptr()),
                                            ctypes.c_void_p(grads.data_ptr()), ctypes.c_void_p(self._ws_base),
                                            ctypes.c_longlong(self._ws_bytes)))

    # ---------------------------------------------------------------------------------------------
    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self.lib.cme_engine_destroy(self._h)
                self._h = None
        except Exception:
            pass

    @property
    def total_param_count(self) -> int:
        return self.layout.total

    def master_params(self) -> torch.Tensor:
        """fp32 view of the parameters for checksums and trajectory statistics.  Under the fused path each rank
        keeps fp32 master values only for the slices it owns, so the (rank-identical) bf16 parameters are used."""
        if self.fused is not None and self.fused.world > 1:
            return self.params.float()
        return self.master

    def state(self):
        if self.fused is not None and self.fused.world > 1:
            return self.fused.gather_state()
        return self.master, self.adam_m, self.adam_v, int(self.step_dev.item())

    def load_state(self, p, m, v, step: int) -> None:
        self.master.copy_(p.to(self.device))
        if not self.strict:
            self.params.copy_(self.master)
        self.adam_m.copy_(m.to(self.device))
        self.adam_v.copy_(v.to(self.device))
        self.step_count = step
        self.step_dev.fill_(step)

    def set_params(self, flat_fp32: torch.Tensor) -> None:
        self.master.copy_(flat_fp32.to(self.device, torch.float32))
        if not self.strict:
            self.params.copy_(self.master)

    def zero_grad(self) -> None:
        """Kept for interface parity: backward overwrites gradients, so nothing needs clearing."""
        self._micro = 0

    def set_lr(self, lr: float) -> None:
        self.lr_dev.fill_(lr)

    # ---------------------------------------------------------------------------------------------
    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor], loss_weight: float = 1.0,
                accumulate_loss: bool = False, grad_scale: Optional[float] = None) -> torch.Tensor:
        """Enqueue the forward pass; the mean loss lands in ``self.loss_dev`` (no host sync)."""
        self._tokens = tokens
        gs = (1.0 / self.cfg.tokens_per_step) if grad_scale is None else grad_scale
        with torch.cuda.device(self.device):
            ops._check(self.lib.cme_engine_forward(
                self._h, ops._p(tokens), ops._p(targets), ops._p(self.loss_dev), ctypes.c_float(loss_weight),
                int(accumulate_loss), ctypes.c_float(gs), ops._stream()))
        return self.loss_dev

    def backward(self, bucket_callback: Optional[Callable[[Bucket], None]] = None,
                 buckets: Optional[Sequence[Bucket]] = None, scale: float = 1.0, accumulate: bool = False) -> None:
        """Enqueue the backward pass.  ``bucket_callback(bucket)`` runs on the host as soon as the launches that
        complete a (coalesced) bucket have been enqueued.  ``scale`` must already have been applied through
        ``forward(grad_scale=...)``; it is accepted for interface parity with the oracle model."""
        cb = _BUCKET_FN(0)
        if bucket_callback is not None:
            ready = {}
            for b in buckets:
                last = max(nb.index for nb in self.layout.natural_buckets if b.start <= nb.start and nb.end <= b.end)
                ready[last] = b

            def _cb(_user, idx):
                b = ready.get(idx)
                if b is not None:
                    bucket_callback(b)

            cb = _BUCKET_FN(_cb)
        self._cb_keepalive = cb
        with torch.cuda.device(self.device):
            ops._check(self.lib.cme_engine_backward(self._h, ops._p(self._tokens), int(accumulate), cb, None,
                                                    ops._stream()))

    def logits(self) -> torch.Tensor:
        """A copy of the logits buffer (after ``forward`` with targets it holds d(logits))."""
        self.lib.cme_engine_logits_ld.restype = ctypes.c_longlong
        ld = int(self.lib.cme_engine_logits_ld(self._h))        # rows are padded to a multiple of 8 elements
        n = self.cfg.tokens_per_step * ld
        ptr = self.lib.cme_engine_logits(self._h)
        out = torch.empty(n, dtype=self.dtype, device=self.device)
        ops._check(self.lib.cme_copy_d2d(ops._p(out), ctypes.c_void_p(ptr), ctypes.c_longlong(n * out.element_size()),
                                         ops._stream()))
        return out.view(self.cfg.tokens_per_step, ld)[:, :self.cfg.vocab_size].contiguous()

    def update(self, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        """Unfused optimizer path: global norm (if clipping) then Adam / AdamW over the whole arena.
        With the fused synchronisation path attached the update already happened inside the bucket kernels."""
        if self.handles_sync:
            return
        o = self.optim
        if lr is not None:
            self.set_lr(lr)
        self.step_count += 1
        with torch.cuda.device(self.device):
            ops._check(self.lib.cme_step_inc(ops._p(self.step_dev), ops._stream()))
            normsq = None
            if o.clip_norm > 0:
                ops._check(self.lib.cme_grad_normsq(ops._dt(self.grads), ops._p(self.grads),
                                                    ctypes.c_longlong(self.grads.numel()), ops._p(self._norm_partial),
                                                    ops._p(self.normsq), ops._stream()))
                normsq = self.normsq
            ops.adam_step(self.master, self.grads, self.adam_m, self.adam_v, self.step_dev, self.lr_dev,
                          compute=None if self.strict else self.params, normsq=normsq, beta1=o.beta1, beta2=o.beta2,
                          eps=o.eps, weight_decay=o.weight_decay, grad_scale=grad_scale, clip_norm=o.clip_norm,
                          nodecay=self.nodecay if o.weight_decay > 0 else None)

    def train_step(self, tokens: Sequence[torch.Tensor], targets: Sequence[torch.Tensor],
                   bucket_callback=None, buckets=None) -> None:
        """zero_grad + forward/backward over the micro-batches (gradients accumulate, the loss is their mean).
        With the fused path attached this is the whole optimizer step: buckets are reduced, applied and
        redistributed by device kernels while backward runs."""
        if self.fused is not None:
            self.fused.train_step(tokens, targets)
        else:
            self.train_step_raw(tokens, targets, bucket_callback, buckets)

    def train_step_raw(self, tokens: Sequence[torch.Tensor], targets: Sequence[torch.Tensor],
                       bucket_callback=None, buckets=None) -> None:
        accum = len(tokens)
        gs = 1.0 / (self.cfg.tokens_per_step * accum)
        for i, (x, y) in enumerate(zip(tokens, targets)):
            self.forward(x, y, loss_weight=1.0 / accum, accumulate_loss=i > 0, grad_scale=gs)
            last = i == accum - 1
            if last:
                self._publish_loss()
            self.backward(bucket_callback if last else None, buckets if last else None, accumulate=i > 0)

    def _publish_loss(self) -> None:
        """Enqueue (capturable) one single-thread kernel that bumps the sequence number and writes the loss, then the
        sequence number, into pinned host memory: the host sees the new number only after the loss has landed."""
        with torch.cuda.device(self.device):
            ops._check(self.lib.cme_publish_loss(ops._p(self.loss_dev), ops._p(self.seq_dev), self._loss_host_dev,
                                                 self._seq_host_dev, ops._stream()))

    def read_loss(self) -> float:
        return float(self.loss_dev.item())

    def wait_loss(self, timeout_s: float = 30.0) -> float:
        """Loss of the most recently enqueued step, as soon as its forward pass has finished: polls the pinned
        sequence number instead of synchronising the stream, so backward and the optimizer keep running and the
        caller can already enqueue the next step.  Falls back to a full synchronisation after ``timeout_s``."""
        import time
        want = self.seq_expected
        t0 = time.perf_counter()
        spins = 0
        while int(self.seq_host.item()) < want:
            spins += 1
            if (spins & 1023) == 0 and time.perf_counter() - t0 > timeout_s:
                torch.cuda.synchronize(self.device)
                return float(self.loss_dev.item())
        return float(self.loss_host.item())
