"""Pure-PyTorch oracle model over the flat arena (CPU or GPU, any float dtype, autograd backward).

This is the numerical oracle for the native engine and the model used by the CPU/gloo plumbing
configuration.  In parity mode it computes exactly the function of the reference's fp64 CPU model
(``FINAL_CLEAN_CODE_/tests/test_model_reference.cu:104-202``): ``LN1 -> QKV -> attention -> Wo ->
(+embedded) -> LN2 -> FFN(ReLU) -> (+residual1) -> Wout`` with non-causal attention over the flat
``[B*T, D] -> [B*H, T, HD]`` reinterpretation, and the loss ``-log(softmax + 1e-9)`` averaged over tokens
(``FINAL_CLEAN_CODE_/src/kernels/activations.cu:463-470``).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from ..arena import ArenaLayout, init_flat
from ..config import ModelConfig, OptimConfig


def layer_norm(x: torch.Tensor, g: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(var + eps) * g + b


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cfg: ModelConfig, B: int) -> torch.Tensor:
    """q, k, v: ``[B*T, D]``.  Returns ``[B*T, D]``."""
    T, H, HD, D = cfg.seq_len, cfg.heads, cfg.head_dim, cfg.hidden
    if cfg.head_layout == "flat":
        # the reference views the row-major [B*T, D] buffer as [B*H, T, HD] with no transpose
        qh, kh, vh = (t.reshape(B * H, T, HD) for t in (q, k, v))
    else:
        qh, kh, vh = (t.reshape(B, T, H, HD).permute(0, 2, 1, 3).reshape(B * H, T, HD) for t in (q, k, v))
    s = torch.matmul(qh, kh.transpose(1, 2)) * (1.0 / math.sqrt(HD))
    if cfg.causal:
        mask = torch.ones(T, T, dtype=torch.bool, device=s.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.matmul(p, vh)
    if cfg.head_layout == "flat":
        return o.reshape(B * T, D)
    return o.reshape(B, H, T, HD).permute(0, 2, 1, 3).reshape(B * T, D)


def forward(P: Dict[str, torch.Tensor], cfg: ModelConfig, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None
            ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """``tokens``/``targets``: flat ``[B*T]`` integer tensors.  Returns ``(mean loss, logits [B*T, V])``."""
    T, D = cfg.seq_len, cfg.hidden
    BT = tokens.numel()
    B = BT // T
    tok = tokens.long()
    pos = torch.arange(BT, device=tok.device) % T
    x = P["tok_embed"][tok] + P["pos_embed"][pos]
    for l in range(cfg.layers):
        p = f"h{l}." if (cfg.layers > 1 or cfg.mode == "gpt") else ""
        h = layer_norm(x, P[p + "ln1_gamma"], P[p + "ln1_beta"], cfg.ln_eps)
        if cfg.mode == "gpt":
            q, k, v = (h @ P[p + "Wqkv"]).split(D, dim=-1)
        else:
            q, k, v = h @ P[p + "Wq"], h @ P[p + "Wk"], h @ P[p + "Wv"]
        a = attention(q, k, v, cfg, B)
        x = x + a @ P[p + "Wo"]
        h = layer_norm(x, P[p + "ln2_gamma"], P[p + "ln2_beta"], cfg.ln_eps)
        f = h @ P[p + "W1"] + P[p + "b1"]
        f = torch.relu(f) if cfg.activation == "relu" else gelu_tanh(f)
        x = x + f @ P[p + "W2"] + P[p + "b2"]
    if cfg.final_layernorm:
        x = layer_norm(x, P["lnf_gamma"], P["lnf_beta"], cfg.ln_eps)
    logits = x @ (P["tok_embed"].t() if cfg.tied_embeddings else P["Wout"])
    if targets is None:
        return None, logits
    if cfg.mode == "parity":
        m = logits.max(-1, keepdim=True).values
        e = torch.exp(logits - m)
        prob = e.gather(1, targets.long()[:, None]).squeeze(1) / e.sum(-1)
        loss = -(torch.log(prob + 1e-9)).mean()
    else:
        loss = F.cross_entropy(logits.float() if logits.dtype in (torch.bfloat16, torch.float16) else logits,
                               targets.long())
    return loss, logits


class ReferenceModel:
    """Flat-arena model with explicit ``zero_grad / forward / backward / update`` like the
    reference's ``TransformerModel`` (``FINAL_CLEAN_CODE_/include/model.h:93-145``), on autograd."""

    def __init__(self, cfg: ModelConfig, optim: OptimConfig, device="cpu", dtype=torch.float32, seed: int = 42,
                 layout: Optional[ArenaLayout] = None) -> None:
        self.cfg, self.optim = cfg, optim
        self.layout = layout or ArenaLayout(cfg)
        self.params = init_flat(self.layout, seed).to(device=device, dtype=dtype).requires_grad_(True)
        self.grads = torch.zeros_like(self.params)
        self.adam_m = torch.zeros_like(self.params)
        self.adam_v = torch.zeros_like(self.params)
        self.step_count = 0
        self.loss: Optional[torch.Tensor] = None
        self.logits: Optional[torch.Tensor] = None
        self._hooks = []

    @property
    def total_param_count(self) -> int:
        return self.layout.total

    def views(self) -> Dict[str, torch.Tensor]:
        return self.layout.views(self.params)

    def zero_grad(self) -> None:
        self.grads.zero_()

    def forward(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self._views = self.views()
        self.loss, self.logits = forward(self._views, self.cfg, tokens.to(self.params.device),
                                         targets.to(self.params.device))
        return self.loss

    def backward(self, bucket_callback=None, buckets=None, scale: float = 1.0) -> None:
        """Accumulate d(loss*scale)/d(params) into ``self.grads``.

        With ``bucket_callback`` and ``buckets`` (a list of :class:`~..arena.Bucket`), the callback is
        invoked as ``callback(bucket)`` as soon as every tensor of the bucket has its gradient, in the
        order autograd produces them, i.e. while backward is still running — the role of
        ``backward_bucketed`` in the reference (``transformer.cu:417-590``)."""
        views = self._views          # the view tensors the forward graph was built on
        names = list(views)
        tensors = [views[n] for n in names]
        if bucket_callback is None:
            gs = torch.autograd.grad(self.loss * scale, tensors, allow_unused=True)
            gv = self.layout.views(self.grads)
            for n, g in zip(names, gs):
                if g is not None:
                    gv[n].add_(g)
            return
        gv = self.layout.views(self.grads)
        pending = {b.index: set(b.names) for b in buckets}
        owner = {n: b for b in buckets for n in b.names}
        emitted = []

        def make_hook(name):
            def hook(g):
                gv[name].add_(g)
                b = owner[name]
                pending[b.index].discard(name)
                if not pending[b.index]:
                    emitted.append(b.index)
                    bucket_callback(b)
                return g
            return hook

        handles = [t.register_hook(make_hook(n)) for n, t in zip(names, tensors)]
        try:
            torch.autograd.backward(self.loss * scale)
        finally:
            for h in handles:
                h.remove()
            self.params.grad = None
        for b in buckets:                      # tensors that received no gradient
            if b.index not in emitted:
                bucket_callback(b)

    @torch.no_grad()
    def grad_norm(self, grad_scale: float = 1.0) -> float:
        return float(self.grads.double().pow(2).sum().sqrt()) * grad_scale

    @torch.no_grad()
    def update(self, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        """Adam / AdamW on the flat arena with global-norm clipping inside the update
        (``transformer.cu:598-636``): ``g = grad * grad_scale * clip`` where
        ``clip = min(1, clip_norm / ||grad * grad_scale||)``; bias-corrected moments; decoupled weight decay."""
        o = self.optim
        lr = o.lr if lr is None else lr
        self.step_count += 1
        t = self.step_count
        clip = 1.0
        if o.clip_norm > 0:
            norm = float(self.grads.double().pow(2).sum().sqrt()) * grad_scale
            clip = min(1.0, o.clip_norm / norm) if norm > 0 else 1.0
        g = self.grads * (grad_scale * clip)
        self.adam_m.mul_(o.beta1).add_(g, alpha=1 - o.beta1)
        self.adam_v.mul_(o.beta2).addcmul_(g, g, value=1 - o.beta2)
        mhat = self.adam_m / (1 - o.beta1 ** t)
        vhat = self.adam_v / (1 - o.beta2 ** t)
        p = self.params.data
        if o.weight_decay > 0:
            decay = torch.zeros_like(p)
            for s in self.layout.specs:
                if s.kind in ("weight", "embed"):
                    decay[s.offset:s.offset + s.numel] = 1.0
            p.mul_(1 - lr * o.weight_decay * decay)
        p.sub_(lr * mhat / (vhat.sqrt() + o.eps))

    def read_loss(self) -> float:
        return float(self.loss.detach())
