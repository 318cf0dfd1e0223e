"""Python face of the native sm_100a library (``libcme213_b200.so``, built in-tree by :mod:`.build`).

The library has a plain C ABI (pointers, sizes, a stream handle) and is loaded with ``ctypes``; every
wrapper here takes ``torch`` tensors, checks them, passes ``data_ptr()`` and the current CUDA stream, and
raises :class:`NativeError` with the library's message when a call fails.  There is no PyTorch fallback
behind these functions: on a GPU machine a missing library is an error, not a silent slow path.

The op list mirrors the reference's kernel header (``FINAL_CLEAN_CODE_/include/kernels.h:6-138``).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "libcme213_b200.so"
_lib: Optional[ctypes.CDLL] = None
_tried = False

F32, BF16 = 0, 1
ACT = {"none": 0, None: 0, "relu": 1, "gelu": 2}


class NativeError(RuntimeError):
    pass


class CmeGemm(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("batch", ctypes.c_int),
        ("A", ctypes.c_void_p), ("lda", ctypes.c_longlong), ("strideA", ctypes.c_longlong), ("a_trans", ctypes.c_int),
        ("B", ctypes.c_void_p), ("ldb", ctypes.c_longlong), ("strideB", ctypes.c_longlong), ("b_trans", ctypes.c_int),
        ("C", ctypes.c_void_p), ("ldc", ctypes.c_longlong), ("strideC", ctypes.c_longlong), ("c_dtype", ctypes.c_int),
        ("ab_dtype", ctypes.c_int),
        ("bias", ctypes.c_void_p),
        ("residual", ctypes.c_void_p), ("ldres", ctypes.c_longlong),
        ("aux_out", ctypes.c_void_p), ("aux_in", ctypes.c_void_p), ("ldaux", ctypes.c_longlong),
        ("act", ctypes.c_int), ("dact", ctypes.c_int), ("accumulate", ctypes.c_int),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_longlong),
        ("force_bn", ctypes.c_int), ("force_splits", ctypes.c_int),
        ("aux_deriv", ctypes.c_int),
        ("colsum", ctypes.c_void_p), ("colsum_slabs", ctypes.POINTER(ctypes.c_int)),
        ("allow_tf32", ctypes.c_int),
    ]


def _load() -> Optional[ctypes.CDLL]:
    global _lib, _tried
    if _lib is not None or _tried:
        return _lib
    _tried = True
    if not LIB_PATH.exists():
        return None
    try:
        lib = ctypes.CDLL(str(LIB_PATH))
    except OSError:
        return None
    lib.cme_last_error.restype = ctypes.c_char_p
    lib.fnv1a_u32.restype = ctypes.c_ulonglong
    lib.fnv1a_u32.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_ulonglong]
    _lib = lib
    return lib


def host_lib() -> Optional[ctypes.CDLL]:
    """The library if it has been built, else ``None`` (host-only helpers have Python fallbacks)."""
    return _load()


def lib() -> ctypes.CDLL:
    l = _load()
    if l is None:
        raise NativeError(f"native library not found at {LIB_PATH}; run `python -m cme213_final_project_b200.ops.build`")
    return l


def available() -> bool:
    return _load() is not None and torch.cuda.is_available()


def _check(rc: int) -> None:
    if rc != 0:
        raise NativeError(f"native call failed (status {rc}): {lib().cme_last_error().decode()}")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise NativeError(f"unsupported dtype {t.dtype}")


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _cuda(*ts) -> None:
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise NativeError("native ops need contiguous CUDA tensors")


_workspaces = {}


def workspace(nbytes: int = 64 << 20) -> torch.Tensor:
    """Per-device fp32 scratch shared by split-K GEMMs launched through the Python wrappers."""
    dev = torch.cuda.current_device()
    w = _workspaces.get(dev)
    if w is None or w.numel() * 4 < nbytes:
        w = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
        _workspaces[dev] = w
    return w


# --------------------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_trans: bool = False, b_trans: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         bias: Optional[torch.Tensor] = None, act: Optional[str] = None, aux_out: Optional[torch.Tensor] = None,
         dact: Optional[str] = None, aux_in: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
         accumulate: bool = False, backend: str = "auto", force_bn: int = 0, force_splits: int = 0,
         aux_deriv: bool = False, dbias: Optional[torch.Tensor] = None, allow_tf32: bool = True) -> torch.Tensor:
    """``out (+)= epilogue(op(a) @ op(b))`` for 2-D or batched 3-D row-major operands.

    ``a``: ``[M, K]`` (or ``[K, M]`` with ``a_trans``); ``b``: ``[K, N]`` (or ``[N, K]`` with ``b_trans``);
    a leading batch dimension on either operand makes the product batched (a 2-D operand is shared).
    Epilogue order: ``+bias`` -> store pre-activation to ``aux_out`` -> ``act`` -> ``* act'(aux_in)`` (``dact``)
    -> ``+residual`` -> ``+out`` (``accumulate``).  ``backend``: ``auto`` | ``tcgen05`` | ``simt``.
    ``aux_deriv``: the auxiliary tensor holds ``act'(pre-activation)`` instead of the pre-activation (forward
    stores it, backward multiplies by it).  ``dbias`` (a ``[N]`` tensor): receives the column sums of ``out`` --
    from the GEMM's own epilogue when the kernel that runs can produce them, else from a separate pass.
    fp32 operands: ``backend="simt"`` multiplies them exactly; the tcgen05 kernel takes them as tf32 (plain products
    with fp32 output only) unless ``allow_tf32=False``.
    """
    _cuda(a, b, out, bias, aux_out, aux_in, residual)
    batch = 1
    if a.dim() == 3:
        batch = a.shape[0]
    if b.dim() == 3:
        batch = max(batch, b.shape[0])
    a2, b2 = a.shape[-2:], b.shape[-2:]
    M, K = (a2[1], a2[0]) if a_trans else (a2[0], a2[1])
    Kb, N = (b2[1], b2[0]) if b_trans else (b2[0], b2[1])
    if K != Kb:
        raise NativeError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    odt = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is None:
        shape = (batch, M, N) if (a.dim() == 3 or b.dim() == 3) else (M, N)
        out = torch.empty(shape, dtype=odt, device=a.device)
    ws = workspace()
    g = CmeGemm()
    g.M, g.N, g.K, g.batch = M, N, K, batch
    g.A, g.lda, g.strideA, g.a_trans = a.data_ptr(), a2[1], (a2[0] * a2[1] if a.dim() == 3 else 0), int(a_trans)
    g.B, g.ldb, g.strideB, g.b_trans = b.data_ptr(), b2[1], (b2[0] * b2[1] if b.dim() == 3 else 0), int(b_trans)
    g.C, g.ldc, g.strideC, g.c_dtype = out.data_ptr(), N, M * N, _dt(out)
    g.ab_dtype = _dt(a)
    g.bias = 0 if bias is None else bias.data_ptr()
    g.residual, g.ldres = (0 if residual is None else residual.data_ptr()), N
    g.aux_out = 0 if aux_out is None else aux_out.data_ptr()
    g.aux_in = 0 if aux_in is None else aux_in.data_ptr()
    g.ldaux = N
    g.act, g.dact, g.accumulate = ACT[act], ACT[dact], int(accumulate)
    g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel() * 4
    g.force_bn, g.force_splits = force_bn, force_splits
    g.aux_deriv = int(aux_deriv)
    g.allow_tf32 = int(allow_tf32)
    slabs = ctypes.c_int(0)
    if dbias is not None:
        part = torch.empty((M + 31) // 32 * N, dtype=torch.float32, device=a.device)
        g.colsum, g.colsum_slabs = part.data_ptr(), ctypes.pointer(slabs)
    _check(lib().cme_gemm(ctypes.byref(g), {"auto": 0, "tcgen05": 1, "simt": 2}[backend], _stream()))
    if dbias is not None:
        gemm.last_colsum_slabs = slabs.value          # 0: the epilogue did not sum (tests look at this)
        if slabs.value:
            _check(lib().cme_colsum_slabs_finalize(_dt(dbias), _p(part), slabs.value, N, _p(dbias), 0, _stream()))
        else:
            dact_colsum(out.reshape(-1, N), want_g=False, dbias=dbias)
    return out


def gemm_check_status() -> int:
    """Read and clear the device status word of the tcgen05 GEMM (non-zero: a bounded wait ran out)."""
    v = ctypes.c_int(0)
    _check(lib().cme_gemm_check_status(ctypes.byref(v)))
    return v.value


# --------------------------------------------------------------------------------------------------
# LayerNorm
# --------------------------------------------------------------------------------------------------
def layernorm_fwd(x, gamma, beta, eps: float = 1e-5, residual=None, save_sum: bool = False):
    """``y = LN(x [+ residual])``.  Returns ``(y, mean, rstd, summed)`` where ``summed`` is
    ``x + residual`` when ``save_sum`` (the fused residual + LayerNorm forward) else ``None``."""
    _cuda(x, gamma, beta, residual)
    rows, D = x.numel() // x.shape[-1], x.shape[-1]
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty_like(mean)
    r = torch.empty_like(x) if (save_sum and residual is not None) else None
    _check(lib().cme_layernorm_fwd(_dt(x), _p(x), _p(residual), _p(r), _p(gamma), _p(beta), _p(y), _p(mean), _p(rstd),
                                   rows, D, ctypes.c_float(eps), _stream()))
    return y, mean, rstd, r


def layernorm_bwd(dy, x, gamma, mean, rstd, dres=None, dgamma=None, dbeta=None, accumulate: bool = False):
    """Returns ``(dx, dgamma, dbeta)``; ``dx`` includes ``+ dres`` when given (fused residual-gradient add)."""
    _cuda(dy, x, gamma, mean, rstd, dres, dgamma, dbeta)
    rows, D = x.numel() // x.shape[-1], x.shape[-1]
    dx = torch.empty_like(x)
    if dgamma is None:
        dgamma, dbeta, accumulate = torch.empty_like(gamma), torch.empty_like(gamma), False
    nb = lib().cme_layernorm_bwd_blocks(rows)
    scratch = torch.empty(nb * 2 * D, dtype=torch.float32, device=x.device)
    _check(lib().cme_layernorm_bwd(_dt(x), _p(dy), _p(x), _p(gamma), _p(mean), _p(rstd), _p(dres), _p(dx), _p(dgamma),
                                   _p(dbeta), _p(scratch), rows, D, int(accumulate), _stream()))
    return dx, dgamma, dbeta


# --------------------------------------------------------------------------------------------------
# Bias / activation / residual, column sums
# --------------------------------------------------------------------------------------------------
def bias_act_residual(x, bias=None, act=None, residual=None, save_pre: bool = False):
    """``out = act(x + bias) + residual``; returns ``(out, pre)`` with ``pre = x + bias`` if ``save_pre``."""
    _cuda(x, bias, residual)
    cols = x.shape[-1]
    rows = x.numel() // cols
    out = torch.empty_like(x)
    pre = torch.empty_like(x) if save_pre else None
    _check(lib().cme_bias_act_residual(_dt(x), _p(x), _p(bias), _p(residual), _p(pre), _p(out),
                                       ctypes.c_longlong(rows), cols, ACT[act], _stream()))
    return out, pre


def dact_colsum(dout, pre=None, act=None, want_g: bool = True, dbias=None, accumulate: bool = False):
    """``g = dout * act'(pre)`` and ``dbias (+)= g.sum(0)`` — the fused activation-backward + bias-backward."""
    _cuda(dout, pre, dbias)
    cols = dout.shape[-1]
    rows = dout.numel() // cols
    g = torch.empty_like(dout) if (want_g and pre is not None) else None
    if dbias is None:
        dbias, accumulate = torch.empty(cols, dtype=dout.dtype, device=dout.device), False
    scratch = torch.empty(lib().cme_colsum_splits(rows, cols) * cols, dtype=torch.float32, device=dout.device)
    _check(lib().cme_dact_colsum(_dt(dout), _p(dout), _p(pre), _p(g), _p(dbias), _p(scratch), rows, cols, ACT[act],
                                 int(accumulate), _stream()))
    return g, dbias


def scale_(x, s: float):
    _cuda(x)
    _check(lib().cme_scale(_dt(x), _p(x), ctypes.c_longlong(x.numel()), ctypes.c_float(s), _stream()))
    return x


def cast(x, dtype):
    _cuda(x)
    y = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(lib().cme_cast(_dt(x), _p(x), _dt(y), _p(y), ctypes.c_longlong(x.numel()), _stream()))
    return y


def add(a, b):
    _cuda(a, b)
    out = torch.empty_like(a)
    _check(lib().cme_add(_dt(a), _p(a), _p(b), _p(out), ctypes.c_longlong(a.numel()), _stream()))
    return out


def relu_bwd(x, dy):
    _cuda(x, dy)
    dx = torch.empty_like(dy)
    _check(lib().cme_relu_bwd(_dt(x), _p(x), _p(dy), _p(dx), ctypes.c_longlong(x.numel()), _stream()))
    return dx


def init_uniform_(out, scale: float, seed: int):
    _cuda(out)
    _check(lib().cme_init_uniform(_dt(out), _p(out), ctypes.c_longlong(out.numel()), ctypes.c_float(scale),
                                  ctypes.c_uint(seed & 0xFFFFFFFF), _stream()))
    return out


# --------------------------------------------------------------------------------------------------
# Embedding
# --------------------------------------------------------------------------------------------------
def embedding_fwd(tokens, tok, pos):
    _cuda(tokens, tok, pos)
    BT, (V, D), T = tokens.numel(), tok.shape, pos.shape[0]
    out = torch.empty(BT, D, dtype=tok.dtype, device=tok.device)
    _check(lib().cme_embedding_fwd(_dt(tok), _p(tokens), _p(tok), _p(pos), _p(out), BT, T, D, V, _stream()))
    return out


def embedding_bwd(tokens, dout, V: int, T: int, dtok=None, dpos=None, accumulate: bool = False):
    _cuda(tokens, dout, dtok, dpos)
    BT, D = dout.shape
    if dtok is None:
        dtok, dpos, accumulate = (torch.empty(V, D, dtype=dout.dtype, device=dout.device),
                                  torch.empty(T, D, dtype=dout.dtype, device=dout.device), False)
    _check(lib().cme_embedding_bwd(_dt(dout), _p(tokens), _p(dout), _p(dtok), _p(dpos), BT, T, D, V, int(accumulate),
                                   _stream()))
    return dtok, dpos


# --------------------------------------------------------------------------------------------------
# Loss and optimizer
# --------------------------------------------------------------------------------------------------
def cross_entropy(logits, targets, grad_scale: Optional[float] = None, prob_eps: float = 0.0, inplace: bool = False):
    """Returns ``(mean loss [1] fp32, dlogits, per-row losses)``; ``dlogits = (softmax - onehot) * grad_scale``
    (default ``1/rows``).  ``prob_eps = 1e-9`` reproduces the reference's ``-log(p + 1e-9)`` form."""
    _cuda(logits, targets)
    rows, V = logits.shape
    dl = logits if inplace else torch.empty_like(logits)
    losses = torch.empty(rows, dtype=torch.float32, device=logits.device)
    loss = torch.zeros(1, dtype=torch.float32, device=logits.device)
    gs = 1.0 / rows if grad_scale is None else grad_scale
    _check(lib().cme_cross_entropy(_dt(logits), _p(logits), _p(targets), _p(dl), _p(losses), _p(loss), rows, V,
                                   ctypes.c_longlong(V), ctypes.c_float(gs), ctypes.c_float(prob_eps),
                                   ctypes.c_float(1.0), 0, _stream()))
    return loss, dl, losses


def grad_normsq(g):
    _cuda(g)
    partial = torch.empty(1024, dtype=torch.float32, device=g.device)
    out = torch.empty(1, dtype=torch.float32, device=g.device)
    _check(lib().cme_grad_normsq(_dt(g), _p(g), ctypes.c_longlong(g.numel()), _p(partial), _p(out), _stream()))
    return out


def adam_step(master, grads, m, v, step_dev, lr_dev, *, compute=None, normsq=None, beta1=0.9, beta2=0.999, eps=1e-8,
              weight_decay=0.0, grad_scale=1.0, clip_norm=0.0, nodecay=None):
    """One Adam / AdamW update over a flat range.  ``step_dev`` (int32 [1], already incremented) and
    ``lr_dev`` (fp32 [1]) live on the device; ``nodecay`` is an int64 ``[k, 2]`` tensor of sorted ranges."""
    _cuda(master, grads, m, v, step_dev, lr_dev, compute, normsq, nodecay)
    nn = 0 if nodecay is None else nodecay.shape[0]
    _check(lib().cme_adam(_dt(grads), _p(master), _p(compute), _p(grads), _p(m), _p(v),
                          ctypes.c_longlong(master.numel()), _p(step_dev), _p(lr_dev), _p(normsq),
                          ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                          ctypes.c_float(weight_decay), ctypes.c_float(grad_scale), ctypes.c_float(clip_norm),
                          _p(nodecay), nn, _stream()))


# --------------------------------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------------------------------
class CmeAttn(ctypes.Structure):
    _fields_ = [
        ("nb", ctypes.c_int), ("nh", ctypes.c_int), ("T", ctypes.c_int), ("HD", ctypes.c_int),
        ("sb", ctypes.c_longlong), ("sh", ctypes.c_longlong), ("st", ctypes.c_longlong),
        ("osb", ctypes.c_longlong), ("osh", ctypes.c_longlong), ("ost", ctypes.c_longlong),
        ("causal", ctypes.c_int), ("scale", ctypes.c_float), ("dtype", ctypes.c_int),
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("o", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("d_o", ctypes.c_void_p), ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
        ("delta", ctypes.c_void_p), ("dq_accum", ctypes.c_void_p),
        ("ws", ctypes.c_void_p), ("ws_bytes", ctypes.c_longlong),
        ("dq_sem", ctypes.c_void_p), ("dq_mode", ctypes.c_int), ("dq_accum_clean", ctypes.c_int),
    ]


_BACKENDS = {"auto": 0, "tc": 1, "simt": 2, "gemm": 3}


def _attn_desc(q, B, H, T, layout, causal):
    D = q.shape[-1]
    HD = D // H
    a = CmeAttn()
    a.T, a.HD, a.causal, a.scale, a.dtype = T, HD, int(causal), 1.0 / (HD ** 0.5), _dt(q)
    if layout == "flat":
        a.nb, a.nh, a.sb, a.sh, a.st = B * H, 1, T * HD, 0, HD
    else:
        a.nb, a.nh, a.sb, a.sh, a.st = B, H, T * D, HD, D
    a.osb, a.osh, a.ost = a.sb, a.sh, a.st
    if layout == "flat" and T <= 512 and q.dtype == torch.bfloat16:      # scratch of the batched-GEMM path
        l = lib()
        l.cme_attention_gemm_ws_bytes.restype = ctypes.c_longlong
        nbytes = int(l.cme_attention_gemm_ws_bytes(B * H, T))
        ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=q.device)
        a._ws_keepalive = ws
        a.ws = (ws.data_ptr() + 255) // 256 * 256
        a.ws_bytes = nbytes
    return a


def attention_fwd(q, k, v, B: int, H: int, T: int, layout: str = "split", causal: bool = False,
                  backend: str = "auto"):
    """``q, k, v``: ``[B*T, D]``.  ``layout="flat"`` views each as ``[B*H, T, HD]`` without a transpose (the
    reference's head layout); ``"split"`` is the standard ``[B, T, H, HD]`` split.  Returns ``(out, lse)``."""
    _cuda(q, k, v)
    a = _attn_desc(q, B, H, T, layout, causal)
    out = torch.empty_like(q)
    lse = torch.empty(B * H * T, dtype=torch.float32, device=q.device)
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    _check(lib().cme_attention_fwd(ctypes.byref(a), _BACKENDS[backend], _stream()))
    return out, lse


def attention_bwd(q, k, v, out, lse, dout, B: int, H: int, T: int, layout: str = "split", causal: bool = False,
                  backend: str = "auto", ordered_dq: bool = False, dq_mode: Optional[int] = None,
                  scratch=None):
    """Returns ``(dq, dk, dv)``.  How the tensor-core kernel completes dQ from the key blocks' parts (``dq_mode``):
    0 (default) clears an fp32 scratch, adds the parts in arrival order and converts the sums with a second kernel;
    1 (``ordered_dq``) adds them in a fixed order (bit-reproducible, slower); 2 (up to 64 query blocks) adds them in
    arrival order and lets the CTA whose part comes last scale and cast the sums (two launches fewer, slower at
    large shapes).  ``scratch`` = (fp32 tensor of ``q.numel()``
    zeros, int32 tensor of ``B * H * ceil(T / 128)`` zeros) lets calls share the buffers; modes 1 and 2 leave both
    zero again."""
    _cuda(q, k, v, out, lse, dout)
    a = _attn_desc(q, B, H, T, layout, causal)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    delta = torch.empty_like(lse)
    if dq_mode is None:
        dq_mode = 1 if ordered_dq else 0
    if scratch is not None:
        acc, sem = scratch
    else:
        acc = torch.zeros(q.numel(), dtype=torch.float32, device=q.device)
        sem = torch.zeros(B * H * ((T + 127) // 128), dtype=torch.int32, device=q.device)
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.d_o, a.dq, a.dk, a.dv = dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.delta, a.dq_accum = delta.data_ptr(), acc.data_ptr()
    a.dq_sem, a.dq_mode = sem.data_ptr(), int(dq_mode)
    _check(lib().cme_attention_bwd(ctypes.byref(a), _BACKENDS[backend], _stream()))
    return dq, dk, dv


def launch_count() -> int:
    """Kernels launched (or captured) by the native library so far in this process."""
    l = lib()
    l.cme_launch_count.restype = ctypes.c_longlong
    return int(l.cme_launch_count())


def attention_check_status() -> int:
    """Read and clear the status word of the tensor-core attention kernels (non-zero: a wait ran out)."""
    v = ctypes.c_int(0)
    _check(lib().cme_attention_check_status(ctypes.byref(v)))
    return v.value
