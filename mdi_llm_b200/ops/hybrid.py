"""Operations of the hybrid (attention + recurrent) model family over packed variable-length batches.

Every function has two bodies.  On a CUDA tensor it launches the sm_100a kernel of ``csrc/hybrid_mixers.cu``
(library ``_mdi_hybrid.so``, built on first use; a missing or unbuildable library raises — a CUDA tensor never
takes the PyTorch body).  On a CPU tensor it runs the same arithmetic with plain PyTorch operations, which is how
the models are brought up and tested on a machine without a GPU.

A *plan* (:class:`BatchPlan`) describes the step: for each sequence its first row in the packed token matrix, its
token count, its state slot and the position of its first token.  Prompts and one-token decoding differ only in
the plan.  Row-wise inputs may be column slices of a wider matrix (one fused projection feeds several
consumers): the functions pass the row stride down, the last dimension must be dense.

What is always computed in fp32, whatever the activation type: normalisation statistics, softmax, decays and
their logarithms, gates of the recurrences, unit norms, the recurrent state itself and the residual stream.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from . import build as _build

__all__ = ["BatchPlan", "HybridOpsError", "lib", "embed_rows", "cast_into", "norm_rows", "norm_accumulate", "gelu_",
           "headmajor_gate", "softcap", "glu", "latent_append", "latent_attn", "causal_softmax", "matmul_f32", "conv_silu", "gated_recurrence", "linear",
           "rotary_inv_freq", "scaled_inv_freq", "linear_f32", "grouped_linear", "window_append", "window_attn", "head_gate", "relu2_",
           "token_side_gate", "router_topk", "moe_gemv", "gather_scale_rows", "combine_rows", "act_mul", "scaled_branches",
           "full_norm_append", "lightning_recurrence", "norm_gate_rows", "gated_sum_norm_accumulate"]


class HybridOpsError(RuntimeError):
    pass


_lib: Optional[ctypes.CDLL] = None


class _RecArgs(ctypes.Structure):
    _fields_ = ([(n, c_void_p) for n in ("q", "k", "v", "z", "g", "beta", "zb", "a_log", "w", "out", "state", "meta")]
                + [(n, c_longlong) for n in ("q_stride", "k_stride", "v_stride", "z_stride", "g_stride", "beta_stride",
                                             "out_stride")]
                + [(n, c_int) for n in ("H", "G", "D", "V", "mode")] + [("tau", c_float), ("eps", c_float)])


def lib() -> ctypes.CDLL:
    """Load ``_mdi_hybrid.so``, compiling it first when it is missing or older than its source."""
    global _lib
    if _lib is not None:
        return _lib
    if not _build.hybrid_is_fresh():
        if _build.nvcc_path() is None:
            raise HybridOpsError("the hybrid kernel library is not built and nvcc is not available")
        _build.build_hybrid()
    h = ctypes.CDLL(str(_build.HYBRID_LIB))
    vp, i32, i64, f32 = c_void_p, c_int, c_longlong, c_float
    h.hyb_error_string.restype = ctypes.c_char_p
    h.hyb_error_string.argtypes = [i32]
    h.hyb_embed_rows.argtypes = [vp, vp, vp, i32, i32, vp, vp, vp, f32, i32, vp]
    h.hyb_cast_rows.argtypes = [vp, i64, i32, vp, i64, i32, i32, i32, vp]
    h.hyb_norm_rows.argtypes = [vp, i64, i32, vp, vp, i32, vp, i64, i32, i32, i32, f32, i32, i32, f32, f32, vp, vp]
    h.hyb_gelu_rows.argtypes = [vp, i64, i32, i32, vp]
    h.hyb_window_append.argtypes = [vp, i64, vp, i64, vp, i64, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp, vp, i64, vp, i32, vp]
    h.hyb_window_attn.argtypes = [vp, i64, vp, i64, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, i32, vp, vp, i32, i32, i32, f32, vp, i32, vp]
    h.hyb_head_gate.argtypes = [vp, vp, i64, vp, i32, i32, i32, i32, vp]
    h.hyb_token_side_gate.argtypes = [vp, i64, vp, i64, i32, vp, vp, i32, i32, i32, vp]
    h.hyb_router_topk.argtypes = [vp, vp, vp, i32, i32, i32, i32, vp, vp]
    h.hyb_moe_up.argtypes = [vp, i64, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32, vp]
    h.hyb_moe_down.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, i64, i32, vp]
    h.hyb_gather_scale_rows.argtypes = [vp, i64, vp, vp, vp, i32, i32, i32, vp]
    h.hyb_combine_rows.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp, i32, vp, i64, i32, vp]
    h.hyb_act_mul_rows.argtypes = [vp, i64, vp, i64, i32, i32, f32, i32, vp]
    h.hyb_scaled_branches.argtypes = [vp, i64, vp, i64, vp, vp, i64, vp, i64, vp, i32, i32, i32, vp]
    h.hyb_headmajor_gate.argtypes = [vp, vp, i64, vp, i32, i32, i32, i32, vp]
    h.hyb_softcap.argtypes = [vp, vp, i64, f32, i32, vp]
    h.hyb_latent_append.argtypes = [vp, i64, vp, i64, vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32, vp]
    h.hyb_latent_attn.argtypes = [vp, vp, i64, vp, i64, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, vp, vp, i32, vp]
    h.hyb_causal_softmax.argtypes = [vp, vp, i64, i32, i32, i32, f32, i32, i32, i32, i32, f32, vp, i32, i32, vp]
    h.hyb_full_norm_append.argtypes = [vp, i64, vp, i64, vp, i64, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp, i32, vp]
    h.hyb_lightning.argtypes = [vp, i64, vp, i64, vp, i64, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, i32, vp, i32, vp]
    h.hyb_norm_gate_rows.argtypes = [vp, vp, vp, i64, vp, i32, i32, f32, i32, vp]
    h.hyb_gated_sum_norm.argtypes = [vp, i64, vp, i64, vp, i64, vp, vp, i64, i32, i32, f32, i32, vp, i32, vp]
    h.hyb_conv_silu.argtypes = [vp, i64, vp, vp, vp, i64, vp, vp, i32, i32, i32, i32, i32, vp]
    h.hyb_gated_recurrence.argtypes = [ctypes.POINTER(_RecArgs), i32, i32, i32, i32, vp, vp, vp, vp]
    _lib = h
    return h


def _check(code: int, what: str) -> None:
    if code != 0:
        msg = {-2: "invalid shape/alignment", -3: "unsupported configuration"}.get(code) or lib().hyb_error_string(code).decode()
        raise HybridOpsError(f"{what} failed: {msg} ({code})")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise HybridOpsError(f"unsupported dtype {t.dtype}")


def _st() -> int:
    return torch.cuda.current_stream().cuda_stream


def _rows(t: torch.Tensor) -> Tuple[int, int]:
    """(row stride, width) of a 2-D tensor or column slice whose last dimension is dense."""
    if t.dim() != 2 or (t.size(1) > 1 and t.stride(1) != 1):
        raise HybridOpsError(f"expected rows with a dense last dimension, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0), t.size(1)


@dataclass
class BatchPlan:
    """One step's packed batch: ``seqs[i] = (first row, tokens, slot, position of the first token)``.

    ``shared`` is the step's scratch between layers: what one layer computes for this step's tokens and a later layer
    reads (the values of the first value-mixing attention layer).  The model clears it when a step starts."""

    seqs: List[Tuple[int, int, int, int]]
    n_tokens: int
    meta: torch.Tensor      # int32 [n_seq, 4] on the compute device
    tok_seq: torch.Tensor   # int32 [n_tokens]: sequence index of every row
    positions: torch.Tensor  # int64 [n_tokens]
    shared: Dict[str, torch.Tensor] = field(default_factory=dict)

    @classmethod
    def make(cls, lengths: Sequence[int], slots: Sequence[int], starts: Sequence[int], device: torch.device) -> "BatchPlan":
        seqs, row = [], 0
        for n, s, p in zip(lengths, slots, starts):
            seqs.append((row, int(n), int(s), int(p)))
            row += int(n)
        meta = torch.tensor(seqs, dtype=torch.int32).view(-1, 4)
        tok_seq = torch.repeat_interleave(torch.arange(len(seqs), dtype=torch.int32), meta[:, 1].long())
        pos = torch.cat([torch.arange(p, p + n) for _, n, _, p in seqs]) if seqs else torch.zeros(0, dtype=torch.long)
        return cls(seqs, row, meta.to(device), tok_seq.to(device), pos.to(device))

    @property
    def last_rows(self) -> List[int]:
        return [r + n - 1 for r, n, _, _ in self.seqs]


def rotary_inv_freq(dims: int, base: float, device: torch.device) -> torch.Tensor:
    """``base^(-2i/dims)`` for ``i < dims/2``, evaluated in float64 and rounded once to fp32."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return (float(base) ** (-2.0 * i / dims)).to(torch.float32).to(device)


# ---------------------------------------------------------------------------------------------------------
# matrix products (vendor GEMM on both devices; fp32 means fp32: TF32 is switched off for the call)
# ---------------------------------------------------------------------------------------------------------
def scaled_inv_freq(dims: int, base: float, scaling: Optional[dict], device: torch.device) -> torch.Tensor:
    """Rotary frequencies with the wavelength-dependent stretch used for context extension: with ``l = 2 pi / f``,
    ``f`` is kept for ``l < original/high``, divided by ``factor`` for ``l > original/low``, and blended linearly in
    ``s = (original/l - low) / (high - low)`` between the two.  float64, rounded once to fp32."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    if scaling:
        factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
        orig = float(scaling["original"])
        wl = 2.0 * math.pi / f
        s = (orig / wl - low) / (high - low) if high != low else torch.ones_like(f)
        mid = (1.0 - s) * f / factor + s * f
        f = torch.where(wl < orig / high, f, torch.where(wl > orig / low, f / factor, mid))
    return f.to(torch.float32).to(device)


def linear_f32(x: torch.Tensor, w32: torch.Tensor, b32: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w32.T (+ b32)`` in fp32 (routers): the input may be the activation type, the product and the result are fp32."""
    if x.is_cuda and torch.backends.cuda.matmul.allow_tf32:
        raise HybridOpsError("TF32 matrix products are on; router logits are fp32")
    return F.linear(x.float(), w32, b32)


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
    """Rows of ``x [M, K]`` sorted by group, ``counts [E]`` rows per group (on the device): row ``i`` of group ``e`` times
    ``w[e].T`` (``w [E, out, K]``).  bf16 on CUDA is one vendor grouped matrix product with no host synchronisation;
    anything else (fp32 must stay true fp32, CPU) is one product per non-empty group."""
    aligned = x.size(1) % 8 == 0 and w.size(1) % 8 == 0 and x.is_contiguous() and w.is_contiguous()  # 16-byte rows
    if x.is_cuda and x.dtype == torch.bfloat16 and aligned and hasattr(F, "grouped_mm"):
        return F.grouped_mm(x, w.transpose(1, 2), offs=counts.cumsum(0).to(torch.int32))
    out = torch.empty(x.size(0), w.size(1), device=x.device, dtype=x.dtype)
    r = 0
    for e, c in enumerate(counts.tolist()):
        if c:
            out[r:r + c] = linear(x[r:r + c], w[e])
            r += c
    return out


def linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ b)`` in the activation type with fp32 accumulation."""
    if x.is_cuda and x.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
        raise HybridOpsError("TF32 matrix products are on; fp32 mode needs torch.backends.cuda.matmul.allow_tf32 = False")
    return F.linear(x, w, b)


# ---------------------------------------------------------------------------------------------------------
# rows
# ---------------------------------------------------------------------------------------------------------
def embed_rows(table: torch.Tensor, tokens: torch.Tensor, pos_table: Optional[torch.Tensor] = None,
               plan: Optional["BatchPlan"] = None, scale: float = 1.0) -> torch.Tensor:
    """fp32 rows of ``table`` for int32 ``tokens [N]``, times ``scale``; with ``pos_table [positions, width]`` the learned
    vector of each token's position in its sequence (from ``plan``) is added, unscaled, in fp32."""
    if not table.is_cuda:
        x = table[tokens.long()].float()
        if scale != 1.0:
            x = x * float(scale)
        return x if pos_table is None else x + pos_table[plan.positions].float()
    x = torch.empty(tokens.numel(), table.size(1), device=table.device, dtype=torch.float32)
    if pos_table is not None and (pos_table.dtype != table.dtype or pos_table.size(1) != table.size(1) or not pos_table.is_contiguous()):
        raise HybridOpsError("the position table has the embedding table's type and width")
    _check(lib().hyb_embed_rows(table.data_ptr(), tokens.data_ptr(), x.data_ptr(), tokens.numel(), table.size(1),
                                None if pos_table is None else pos_table.data_ptr(),
                                None if pos_table is None else plan.meta.data_ptr(),
                                None if pos_table is None else plan.tok_seq.data_ptr(), float(scale), _dt(table), _st()), "embed_rows")
    return x


def cast_into(src: torch.Tensor, dst: torch.Tensor) -> None:
    """``dst[:] = src`` with a type change; both may be column slices."""
    if not src.is_cuda:
        dst.copy_(src)
        return
    ss, n = _rows(src)
    ds, n2 = _rows(dst)
    assert n == n2 and src.size(0) == dst.size(0)
    _check(lib().hyb_cast_rows(src.data_ptr(), ss, _dt(src), dst.data_ptr(), ds, _dt(dst), src.size(0), n, _st()), "cast_rows")


def _norm_torch(x: torch.Tensor, w: Optional[torch.Tensor], b: Optional[torch.Tensor], eps: float, kind: str,
                w_offset: float = 0.0) -> torch.Tensor:
    xf = x.float()
    if kind == "none":
        return xf
    if kind == "layer":
        xf = xf - xf.mean(-1, keepdim=True)
    y = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * (w.float() + w_offset if w_offset else w.float())
    if b is not None:
        y = y + b.float()
    return y


def norm_rows(x: torch.Tensor, w: Optional[torch.Tensor], b: Optional[torch.Tensor], eps: float, kind: str,
              out_dtype: torch.dtype, w_offset: float = 0.0) -> torch.Tensor:
    """Layer norm (``kind="layer"``: weight and bias) or RMS norm (``kind="rms"``) of every row, statistics in fp32.
    The weight applied is ``w_offset + w`` (``w_offset = 1``: a weight stored as its deviation from one), summed in fp32."""
    if not x.is_cuda:
        return _norm_torch(x, w, b, eps, kind, w_offset).to(out_dtype)
    xs, n = _rows(x)
    out = torch.empty(x.size(0), n, device=x.device, dtype=out_dtype)
    ref = w if w is not None else x
    _check(lib().hyb_norm_rows(x.data_ptr(), xs, _dt(x), None if w is None else w.data_ptr(),
                               None if b is None else b.data_ptr(), _dt(ref), out.data_ptr(), n, _dt(out), x.size(0), n,
                               eps, _NORM_KINDS[kind], 0, 1.0, float(w_offset), None, _st()), "norm_rows")
    return out


_NORM_KINDS = {"layer": 0, "rms": 1, "none": 2}


def norm_accumulate(resid: torch.Tensor, y: torch.Tensor, w: Optional[torch.Tensor], b: Optional[torch.Tensor], eps: float,
                    kind: str = "layer", scale: float = 1.0, copy: Optional[torch.Tensor] = None) -> None:
    """``resid += scale * norm(y)`` in one pass over the fp32 residual: the post-norm and residual sum of a sandwich
    block (``kind`` "layer" or "rms"), or the scaled residual sum of a pre-norm block (``kind="none"``: no norm).
    ``copy`` (dense, the weight's type, with a norm): also receives the updated residual, rounded — what the next
    sublayer of a post-norm block reads."""
    if resid.dtype != torch.float32:
        raise HybridOpsError("the residual stream is fp32")
    if not y.is_cuda:
        resid.add_(_norm_torch(y, w, b, eps, kind), alpha=float(scale))
        if copy is not None:
            copy.copy_(resid)
        return
    if copy is not None and (w is None or copy.dtype != w.dtype or not copy.is_contiguous() or copy.shape != resid.shape):
        raise HybridOpsError("the residual's copy is dense and has the norm weight's type")
    ys, n = _rows(y)
    ref = w if w is not None else y
    _check(lib().hyb_norm_rows(y.data_ptr(), ys, _dt(y), None if w is None else w.data_ptr(),
                               None if b is None else b.data_ptr(), _dt(ref), resid.data_ptr(), resid.stride(0), 1,
                               y.size(0), n, eps, _NORM_KINDS[kind], 1, float(scale), 0.0,
                               None if copy is None else copy.data_ptr(), _st()), "norm_accumulate")


def gelu_(x: torch.Tensor) -> torch.Tensor:
    """Exact (erf) GELU in place on a dense tensor."""
    if not x.is_cuda:
        return x.copy_(F.gelu(x.float()).to(x.dtype))
    assert x.is_contiguous()
    _check(lib().hyb_gelu_rows(x.data_ptr(), x.numel(), _dt(x), 0, _st()), "gelu")
    return x


def relu2_(x: torch.Tensor) -> torch.Tensor:
    """``max(x, 0)^2`` in place on a dense tensor."""
    if not x.is_cuda:
        return x.copy_(torch.relu(x.float()).square().to(x.dtype))
    assert x.is_contiguous()
    _check(lib().hyb_gelu_rows(x.data_ptr(), x.numel(), _dt(x), 1, _st()), "relu2")
    return x


def head_gate(a: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """``a [heads, rows, hv]`` (head-major) times ``sigmoid(g [rows, heads])``, one gate per head -> ``[rows, heads*hv]``."""
    H, N, hv = a.shape
    if not a.is_cuda:
        return (a.permute(1, 0, 2).float() * torch.sigmoid(g.float())[:, :, None]).reshape(N, H * hv).to(a.dtype)
    assert a.is_contiguous()
    gs, _ = _rows(g)
    out = torch.empty(N, H * hv, device=a.device, dtype=a.dtype)
    _check(lib().hyb_head_gate(a.data_ptr(), g.data_ptr(), gs, out.data_ptr(), N, H, hv, _dt(a), _st()), "head_gate")
    return out


def token_side_gate(z: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, col0: int) -> torch.Tensor:
    """``gelu_tanh(z [N, d]) * table[tokens, col0:col0+d]``: the gate of a per-layer token embedding."""
    N, d = z.shape
    if not z.is_cuda:
        e = table[tokens.long(), col0:col0 + d].float()
        return (F.gelu(z.float(), approximate="tanh") * e).to(z.dtype)
    zs, _ = _rows(z)
    out = torch.empty(N, d, device=z.device, dtype=z.dtype)
    _check(lib().hyb_token_side_gate(z.data_ptr(), zs, table.data_ptr(), table.stride(0), int(col0), tokens.data_ptr(),
                                     out.data_ptr(), N, d, _dt(z), _st()), "token_side_gate")
    return out


def headmajor_gate(a: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """``a [heads, rows, hv]`` (head-major) times ``sigmoid(g [rows, heads*hv])`` -> ``[rows, heads*hv]``."""
    H, N, hv = a.shape
    if not a.is_cuda:
        return (a.permute(1, 0, 2).reshape(N, H * hv).float() * torch.sigmoid(g.float())).to(a.dtype)
    assert a.is_contiguous()
    gs, _ = _rows(g)
    out = torch.empty(N, H * hv, device=a.device, dtype=a.dtype)
    _check(lib().hyb_headmajor_gate(a.data_ptr(), g.data_ptr(), gs, out.data_ptr(), N, H, hv, _dt(a), _st()), "headmajor_gate")
    return out


def softcap(logits: torch.Tensor, cap: float) -> torch.Tensor:
    """fp32 ``cap * tanh(logits / cap)`` (``cap <= 0``: a plain conversion to fp32)."""
    if not logits.is_cuda:
        lf = logits.float()
        return cap * torch.tanh(lf / cap) if cap > 0 else lf
    assert logits.is_contiguous()
    out = torch.empty(logits.shape, device=logits.device, dtype=torch.float32)
    _check(lib().hyb_softcap(logits.data_ptr(), out.data_ptr(), logits.numel(), float(cap), _dt(logits), _st()), "softcap")
    return out


# ---------------------------------------------------------------------------------------------------------
# latent attention
# ---------------------------------------------------------------------------------------------------------
def latent_append(ckv: torch.Tensor, q: torch.Tensor, w: torch.Tensor, inv_freq: torch.Tensor, cache: torch.Tensor,
                  plan: BatchPlan, H: int, D: int, R: int, L: int, nrot: int, eps: float) -> None:
    """Per token: RMS-norm the latent (first ``L`` of the ``ckv`` row), rotate the shared key part (last ``R``) and
    write both to ``cache[slot, pos]``; rotate the last ``R`` values of each of the ``H`` query heads of ``q`` in
    place.  Rotation pairs entry ``i`` with ``i + nrot/2`` for the first ``nrot`` entries, angle ``pos * inv_freq[i]``."""
    if not ckv.is_cuda:
        N = ckv.size(0)
        pos = plan.positions.float()
        ang = pos[:, None] * inv_freq[None, :]
        cs, sn = torch.cos(ang), torch.sin(ang)
        half = nrot // 2

        def rot(x: torch.Tensor) -> torch.Tensor:  # [..., R] with a leading token axis
            xf = x.float()
            u, v = xf[..., :half], xf[..., half:nrot]
            c, s = (cs, sn) if xf.dim() == 2 else (cs[:, None, :], sn[:, None, :])
            return torch.cat((u * c - v * s, v * c + u * s, xf[..., nrot:]), -1).to(x.dtype)

        lat = _norm_torch(ckv[:, :L], w, None, eps, "rms").to(cache.dtype)
        kr = rot(ckv[:, L:])
        qv = q.view(N, H, D + R)
        qv[..., D:] = rot(qv[..., D:])
        for r0, n, slot, p0 in plan.seqs:
            cache[slot, p0:p0 + n, :L] = lat[r0:r0 + n]
            cache[slot, p0:p0 + n, L:] = kr[r0:r0 + n]
        return
    cs_, _ = _rows(ckv)
    qs, _ = _rows(q)
    _check(lib().hyb_latent_append(ckv.data_ptr(), cs_, q.data_ptr(), qs, w.data_ptr(), inv_freq.data_ptr(), cache.data_ptr(),
                                   cache.stride(0), plan.meta.data_ptr(), plan.tok_seq.data_ptr(), ckv.size(0), H, D, R, L,
                                   nrot, eps, _dt(ckv), _st()), "latent_append")


_SM_TARGET = 148  # one block per SM of a B200


def latent_attn(qlat: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, plan: BatchPlan, H: int, D: int, R: int, L: int,
                scale: float, split: int = 0) -> torch.Tensor:
    """Causal softmax attention of ``H`` heads over the cached rows ``[L latent | R rotated key]`` of each token's slot.
    The query of head ``h`` is ``[qlat[h, tok] | q[tok, h, D:]]``, the value of a row is its latent part.
    Returns the attended latents ``[H, N, L]``.  ``split`` (CUDA): key shares per query, 0 = chosen from the batch shape."""
    N = q.size(0)
    if not q.is_cuda:
        out = torch.empty(H, N, L, dtype=q.dtype)
        qr = q.view(N, H, D + R)[..., D:].permute(1, 0, 2)
        qq = torch.cat((qlat, qr), -1).float() * scale  # [H, N, L+R]
        for r0, n, slot, p0 in plan.seqs:
            rows = cache[slot, :p0 + n].float()
            s = qq[:, r0:r0 + n] @ rows.T  # [H, n, keys]
            keys = torch.arange(p0 + n)
            s = s.masked_fill(keys[None, None, :] > (p0 + torch.arange(n))[None, :, None], float("-inf"))
            out[:, r0:r0 + n] = (torch.softmax(s, -1) @ rows[:, :L]).to(q.dtype)
        return out
    assert qlat.is_contiguous()
    qs, _ = _rows(q)
    out = torch.empty(H, N, L, device=q.device, dtype=q.dtype)
    # few query tokens (decoding) cannot fill the GPU with one block per token and 8 heads: split the keys of each
    # query over several blocks and merge the partial softmaxes.  The split count depends only on the batch shape,
    # so a captured step stays valid while contexts grow.
    blocks = N * ((H + 7) // 8)
    nsplit = 1 if blocks >= 2 * _SM_TARGET or split == 1 else (split or max(1, min(32, (2 * _SM_TARGET) // blocks)))
    pa = pm = None
    if nsplit > 1:
        pa = torch.empty(nsplit, H, N, L, device=q.device, dtype=torch.float32)
        pm = torch.empty(nsplit, H, N, 2, device=q.device, dtype=torch.float32)
    _check(lib().hyb_latent_attn(qlat.data_ptr(), q.data_ptr(), qs, cache.data_ptr(), cache.stride(0), plan.meta.data_ptr(),
                                 plan.tok_seq.data_ptr(), out.data_ptr(), N, H, D, R, L, float(scale), nsplit,
                                 None if pa is None else pa.data_ptr(), None if pm is None else pm.data_ptr(), _dt(q), _st()),
           "latent_attn")
    return out


def causal_softmax(scores: torch.Tensor, first_pos: int, scale: float, out_dtype: torch.dtype, window: int = 0,
                   key0: int = 0, sink: bool = False, split: bool = False, cap: float = 0.0,
                   sink_vals: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(scale * scores)`` over the visible keys of fp32 ``scores [heads, rows, keys]``: row ``i`` is position
    ``first_pos + i``, column ``j`` is position ``key0 + j``; a key is visible when it is not later than the row and,
    with ``window > 0``, fewer than ``window`` positions back.  Hidden keys get probability 0.  Result in ``out_dtype``.
    ``sink``: the denominator gains one slot of score zero that has no value, ``p_j = e^{s_j} / (1 + sum_k e^{s_k})``.
    ``split``: the result is ``[heads, rows, 2 * keys]``: the weights rounded to ``out_dtype`` and, behind them, what the
    rounding dropped (``p - round(p)``, rounded again).  A product with the values stacked twice then sums the weights to
    twice the mantissa of ``out_dtype`` on the tensor cores.
    ``cap > 0``: a scaled score ``s`` becomes ``cap * tanh(s / cap)``.  ``sink_vals`` (fp32 ``[heads]``, with ``sink``): the
    sink's score is a learned number per head instead of zero (neither scaled nor capped); the leading axis of
    ``scores`` runs over (anything, head) with the head innermost."""
    Hh, n, keys = scores.shape
    if not scores.is_cuda:
        j = key0 + torch.arange(keys)
        pi = (first_pos + torch.arange(n))[None, :, None]
        hidden = j[None, None, :] > pi
        if window > 0:
            hidden = hidden | (pi - j[None, None, :] >= window)
        sc = scores.float() * scale
        if cap > 0:
            sc = cap * torch.tanh(sc / cap)
        sc = sc.masked_fill(hidden, float("-inf"))
        if sink:
            col = sc.new_zeros(Hh, n, 1)
            if sink_vals is not None:
                col = col + sink_vals.float().repeat(Hh // sink_vals.numel())[:, None, None]
            sc = torch.cat((sc, col), -1)
        pr = torch.softmax(sc, -1)[..., :keys]
        if split:
            hi = pr.to(out_dtype)
            return torch.cat((hi, (pr - hi.float()).to(out_dtype)), -1)
        return pr.to(out_dtype)
    if scores.dtype != torch.float32 or not scores.is_contiguous():
        raise HybridOpsError("scores are dense fp32")
    if sink_vals is not None and (sink_vals.dtype != torch.float32 or not sink_vals.is_contiguous() or Hh % sink_vals.numel()):
        raise HybridOpsError("sink scores are dense fp32, one per head")
    p = torch.empty(Hh, n, 2 * keys if split else keys, device=scores.device, dtype=out_dtype)
    _check(lib().hyb_causal_softmax(scores.data_ptr(), p.data_ptr(), Hh * n, n, keys, int(first_pos), float(scale),
                                    int(window), int(key0), int(bool(sink)), int(bool(split)), float(cap),
                                    None if sink_vals is None else sink_vals.data_ptr(),
                                    0 if sink_vals is None else sink_vals.numel(), _dt(p), _st()), "causal_softmax")
    return p


# ---------------------------------------------------------------------------------------------------------
# windowed grouped-query attention with a per-slot key/value cache
# ---------------------------------------------------------------------------------------------------------
def window_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, inv_freq: Optional[torch.Tensor], cache: torch.Tensor,
                  plan: BatchPlan, H: int, G: int, D: int, V: int, nrot: int, eps: float,
                  qw: Optional[torch.Tensor] = None, kw: Optional[torch.Tensor] = None,
                  v_first: Optional[torch.Tensor] = None, lam: Optional[torch.Tensor] = None) -> None:
    """Per token: rotate the first ``nrot`` entries of every query and key head (entry ``2i`` paired with ``2i+1``,
    angle ``pos * inv_freq[i]``), divide each head by its root mean square over ``D`` (``eps`` inside the root), keep
    the queries in place and write ``[keys | values]`` to ``cache[slot, pos]`` (row = ``G*D`` keys then ``G*V`` values).
    ``qw`` / ``kw`` (``[D]``, shared by the heads) multiply the normalised queries / keys.  With ``lam`` (a one-element
    tensor) the values written are ``(1 - lam) v + lam v_first``, evaluated in fp32 (``v_first [N, G*V]``: the values
    another layer computed for the same tokens)."""
    if not q.is_cuda:
        N = q.size(0)

        def prep(x: torch.Tensor, heads: int, w: Optional[torch.Tensor]) -> torch.Tensor:
            xf = x.float().reshape(N, heads, D).clone()
            if nrot:
                ang = plan.positions.float()[:, None] * inv_freq[None, :]
                c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                u, w_ = xf[..., 0:nrot:2].clone(), xf[..., 1:nrot:2].clone()
                xf[..., 0:nrot:2] = u * c - w_ * s_
                xf[..., 1:nrot:2] = w_ * c + u * s_
            xf = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + eps)
            if w is not None:
                xf = xf * w.float()
            return xf.reshape(N, heads * D).to(x.dtype)

        q.copy_(prep(q, H, qw))
        kk = prep(k, G, kw)
        vv = v if lam is None else ((1.0 - lam.float()) * v.float() + lam.float() * v_first.float()).to(v.dtype)
        for r0, n, slot, p0 in plan.seqs:
            cache[slot, p0:p0 + n, :G * D] = kk[r0:r0 + n]
            cache[slot, p0:p0 + n, G * D:] = vv[r0:r0 + n]
        return
    for w in (qw, kw, lam):
        if w is not None and (w.dtype != q.dtype or not w.is_contiguous()):
            raise HybridOpsError("norm weights and the mixing factor have the activation type")
    _check(lib().hyb_window_append(q.data_ptr(), _rows(q)[0], k.data_ptr(), _rows(k)[0], v.data_ptr(), _rows(v)[0],
                                   None if inv_freq is None else inv_freq.data_ptr(), cache.data_ptr(), cache.stride(0),
                                   plan.meta.data_ptr(), plan.tok_seq.data_ptr(), q.size(0), H, G, D, V, int(nrot),
                                   float(eps), None if qw is None else qw.data_ptr(), None if kw is None else kw.data_ptr(),
                                   None if lam is None else v_first.data_ptr(), 0 if lam is None else _rows(v_first)[0],
                                   None if lam is None else lam.data_ptr(), _dt(q), _st()), "window_append")


_MASK_KINDS = {"window": 0, "chunk": 1}


def visible_from(pos: torch.Tensor, window: int, mask: str) -> torch.Tensor:
    """First visible position for queries at ``pos``: ``window`` positions back (``mask="window"``; 0 = unlimited), or
    the start of the query's own block of ``window`` positions counted from 0 (``mask="chunk"``)."""
    if window <= 0:
        return torch.zeros_like(pos)
    if mask == "chunk":
        return torch.div(pos, window, rounding_mode="floor") * window
    return torch.clamp(pos - window + 1, min=0)


def window_attn(q: torch.Tensor, g: Optional[torch.Tensor], cache: torch.Tensor, plan: BatchPlan, H: int, G: int, D: int,
                V: int, scale: float, window: int, split: int = 0, mask: str = "window", sink: bool = False,
                cap: float = 0.0, sink_vals: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Softmax attention of every token over the cached keys of its slot that are not later than it and (``window > 0``)
    fewer than ``window`` positions back; query head ``h`` reads key/value head ``h // (H/G)``.  Each head's output is
    multiplied by ``sigmoid(g[token, h])`` when ``g [N, H]`` is given, or channel by channel by ``sigmoid(g)`` for
    ``g [N, H*V]``.  ``mask="chunk"``: a token sees the earlier keys of its own block of ``window`` positions (blocks
    numbered from the first position of the sequence) instead of the last ``window``.  ``sink``: the softmax denominator gains
    one slot of score zero (or of the learned score ``sink_vals[h]``, fp32) without a value.  ``cap > 0``: a scaled score
    ``s`` becomes ``cap * tanh(s / cap)``.  Returns ``[N, H*V]``.  The form for one-token steps and
    short portions: one block per token and key/value head, the cache tile shared by the group's query heads.
    ``split`` (CUDA): key shares per token, 0 = chosen from the batch shape and the window alone, so that a captured
    step stays valid while contexts grow."""
    N = q.size(0)
    if not q.is_cuda:
        out = torch.empty(N, H * V, dtype=q.dtype)
        rep = H // G
        for r0, n, slot, p0 in plan.seqs:
            rows = cache[slot, :p0 + n].float()
            kk = rows[:, :G * D].reshape(-1, G, D).repeat_interleave(rep, 1)  # [keys, H, D]
            vv = rows[:, G * D:].reshape(-1, G, V).repeat_interleave(rep, 1)
            qq = q[r0:r0 + n].float().reshape(n, H, D)
            s = torch.einsum("nhd,khd->hnk", qq, kk) * scale
            if cap > 0:
                s = cap * torch.tanh(s / cap)
            pi = (p0 + torch.arange(n))[None, :, None]
            j = torch.arange(p0 + n)[None, None, :]
            hid = (j > pi) | (j < visible_from(pi, window, mask))
            s = s.masked_fill(hid, float("-inf"))
            if sink:
                col = s.new_zeros(H, n, 1) if sink_vals is None else sink_vals.float()[:, None, None].expand(H, n, 1)
                s = torch.cat((s, col), -1)
            o = torch.einsum("hnk,khv->nhv", torch.softmax(s, -1)[..., :p0 + n], vv)
            if g is not None and g.size(1) == H * V and V != 1:
                o = o * torch.sigmoid(g[r0:r0 + n].float()).view(n, H, V)
            elif g is not None:
                o = o * torch.sigmoid(g[r0:r0 + n].float())[:, :, None]
            out[r0:r0 + n] = o.reshape(n, H * V).to(q.dtype)
        return out
    if g is not None and g.size(1) not in (H, H * V):
        raise HybridOpsError("the gate has one column per head or per output channel")
    if sink_vals is not None and (sink_vals.dtype != torch.float32 or sink_vals.numel() != H or not sink_vals.is_contiguous()):
        raise HybridOpsError("sink scores are dense fp32, one per head")
    gate_mode = 0 if g is None else (1 if g.size(1) == H else 2)
    out = torch.empty(N, H * V, device=q.device, dtype=q.dtype)
    blocks = N * G
    tiles = (window + 31) // 32 if window > 0 else 16
    nsplit = min(32, split) or (1 if blocks >= 4 * _SM_TARGET else max(1, min(32, tiles, (4 * _SM_TARGET + blocks - 1) // blocks)))
    pa = pm = None
    if nsplit > 1:
        pa = torch.empty(nsplit, N, H, V, device=q.device, dtype=torch.float32)
        pm = torch.empty(nsplit, N, H, 2, device=q.device, dtype=torch.float32)
    _check(lib().hyb_window_attn(q.data_ptr(), _rows(q)[0], None if g is None else g.data_ptr(),
                                 0 if g is None else _rows(g)[0], cache.data_ptr(), cache.stride(0), plan.meta.data_ptr(),
                                 plan.tok_seq.data_ptr(), out.data_ptr(), N, H, G, D, V, float(scale), int(window), nsplit,
                                 None if pa is None else pa.data_ptr(), None if pm is None else pm.data_ptr(),
                                 _MASK_KINDS[mask if window > 0 else "window"], int(bool(sink)), gate_mode, float(cap),
                                 None if sink_vals is None else sink_vals.data_ptr(), _dt(q), _st()),
           "window_attn")  # no mask size: every earlier position, whichever kind
    return out


# ---------------------------------------------------------------------------------------------------------
# mixture of experts: sigmoid router, top-k choice, experts applied to the weighted input
# ---------------------------------------------------------------------------------------------------------
_ROUTER_MODES = {"sigmoid": 0, "softmax": 1, "softmax_all": 2}


def router_topk(z: torch.Tensor, top: int, mode: str = "sigmoid",
                correction: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """From fp32 router logits ``z [N, E]``: the ``top`` experts with the largest logits per token (ties go to the lower
    index) as int32 ``[N, top]`` and their scores as fp32 ``[N, top]``: ``sigmoid(z)`` of each, not renormalised
    (``mode="sigmoid"``), or the softmax restricted to the selected logits (``mode="softmax"``).
    ``mode="softmax_all"``: scores ``s`` are the softmax over ALL logits; the ``top`` largest ``s + correction`` are chosen
    (``correction`` fp32 ``[E]``, optional) and the result is the chosen ``s`` divided by their sum ``+ 1e-20``."""
    N, E = z.shape
    if not z.is_cuda:
        if mode == "softmax_all":
            s = torch.softmax(z.float(), -1)
            choice = s if correction is None else s + correction.float()
            idx = torch.argsort(-choice, dim=-1, stable=True)[:, :top]
            w = torch.gather(s, 1, idx)
            return idx.to(torch.int32), w / (w.sum(-1, keepdim=True) + 1e-20)
        if mode == "softmax":
            idx = torch.argsort(-z.float(), dim=-1, stable=True)[:, :top]
            return idx.to(torch.int32), torch.softmax(torch.gather(z.float(), 1, idx), -1)
        s = torch.sigmoid(z.float())
        idx = torch.argsort(-s, dim=-1, stable=True)[:, :top]
        return idx.to(torch.int32), torch.gather(s, 1, idx)
    if z.dtype != torch.float32 or not z.is_contiguous():
        raise HybridOpsError("router logits are dense fp32")
    idx = torch.empty(N, top, device=z.device, dtype=torch.int32)
    wt = torch.empty(N, top, device=z.device, dtype=torch.float32)
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E or not correction.is_contiguous()):
        raise HybridOpsError("the router's correction is dense fp32, one number per output")
    _check(lib().hyb_router_topk(z.data_ptr(), idx.data_ptr(), wt.data_ptr(), N, E, int(top), _ROUTER_MODES[mode],
                                 None if correction is None else correction.data_ptr(), _st()), "router_topk")
    return idx, wt


def glu(g: torch.Tensor, u: torch.Tensor, act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """The product of a gated feed-forward from its fp32 gate and up pre-activations: ``silu(g) u``, ``gelu_tanh(g) u``, or
    ``act="clamped"``: ``g' sigmoid(1.702 g') (u' + 1)`` with ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``."""
    if act == "clamped":
        g = torch.clamp(g, max=limit)
        return g * torch.sigmoid(1.702 * g) * (torch.clamp(u, -limit, limit) + 1.0)
    return (F.silu(g) if act == "silu" else F.gelu(g, approximate="tanh")) * u


def moe_gemv(h: torch.Tensor, idx: torch.Tensor, wt: torch.Tensor, up: torch.Tensor, down: torch.Tensor,
             gated: bool = False, act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """Experts read by index, per token.  ``gated=False``: ``sum_k down[e_k] relu(up[e_k] (w_k h))^2`` (``up [E, ff, C]``:
    the score scales the expert's input).  ``gated=True``: ``sum_k w_k down[e_k] (silu(G h) * (U h))`` with
    ``up [E, 2 ff, C]`` holding an expert's gate rows ``G`` and then its up rows ``U`` (the score weighs the expert's
    output; ``act`` / ``limit`` pick the gated product, see :func:`glu`).  A choice whose index is ``E`` or more is an
    identity expert: it has no tensors and contributes ``w_k h``.  ``down [E, C, ff]``.  The form for few tokens: weight-streaming kernels in which one block serves every
    token that chose its expert (an expert's weights are read once per step), no sorting and no host synchronisation."""
    N, C = h.shape
    E, ff, _ = up.shape
    if gated:
        ff //= 2
    top = idx.size(1)
    if not h.is_cuda:
        out = torch.zeros(N, C)
        for t in range(N):
            for k in range(top):
                e = int(idx[t, k])
                if e >= E:
                    out[t] += wt[t, k] * h[t].float()
                    continue
                if gated:
                    gu = F.linear(h[t], up[e]).float()
                    out[t] += wt[t, k] * F.linear(glu(gu[:ff], gu[ff:], act, limit).to(h.dtype), down[e]).float()
                    continue
                xin = (wt[t, k] * h[t].float()).to(h.dtype)
                a = torch.relu(F.linear(xin, up[e]).float()).square().to(h.dtype)
                out[t] += F.linear(a, down[e]).float()
        return out.to(h.dtype)
    assert up.is_contiguous() and down.is_contiguous() and idx.is_contiguous() and wt.is_contiguous()
    if act not in ("silu", "clamped"):
        raise HybridOpsError(f"experts by index know the gated products 'silu' and 'clamped', not {act!r}")
    act_ = torch.empty(N, top, ff, device=h.device, dtype=torch.float32)
    ypair = torch.empty(N, top, C, device=h.device, dtype=torch.float32)
    out = torch.empty(N, C, device=h.device, dtype=h.dtype)
    _check(lib().hyb_moe_up(h.data_ptr(), _rows(h)[0], idx.data_ptr(), wt.data_ptr(), up.data_ptr(), act_.data_ptr(), N, top,
                            C, ff, E, (2 if act == "clamped" else 1) if gated else 0, float(limit), _dt(h), _st()), "moe_up")
    _check(lib().hyb_moe_down(act_.data_ptr(), idx.data_ptr(), wt.data_ptr() if gated else None, down.data_ptr(),
                              ypair.data_ptr(), out.data_ptr(), N, top, C, ff, E, h.data_ptr(), _rows(h)[0], _dt(h), _st()),
           "moe_down")
    return out


def gather_scale_rows(h: torch.Tensor, rows: torch.Tensor, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[i] = scale[i] * h[rows[i]]`` (int32 ``rows``, fp32 ``scale``), rounded to the activation type; without
    ``scale`` a plain gather."""
    if not h.is_cuda:
        if scale is None:
            return h[rows.long()]
        return (h[rows.long()].float() * scale.float()[:, None]).to(h.dtype)
    M = rows.numel()
    out = torch.empty(M, h.size(1), device=h.device, dtype=h.dtype)
    _check(lib().hyb_gather_scale_rows(h.data_ptr(), _rows(h)[0], rows.data_ptr(), None if scale is None else scale.data_ptr(), out.data_ptr(), M,
                                       h.size(1), _dt(h), _st()), "gather_scale_rows")
    return out


def combine_rows(y: torch.Tensor, where: torch.Tensor, n: int, top: int, wt: Optional[torch.Tensor] = None,
                 idx: Optional[torch.Tensor] = None, n_experts: int = 0, h: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = sum_k wt[t, k] * y[where[t*top + k]]`` summed in fp32 in the order of ``k`` (int32 ``where``, fp32
    ``wt [n, top]``; without it a plain sum).  With ``idx [n, top]`` (int32), a choice whose index is ``n_experts`` or more
    is an identity expert: its term is ``wt[t, k] * h[t]`` and its row of ``y`` is not read."""
    if not y.is_cuda:
        g = y[where.long()].float().view(n, top, -1)
        if idx is not None:
            g = torch.where((idx.view(n, top, 1) >= n_experts), h.float().view(n, 1, -1), g)
        if wt is not None:
            g = g * wt.float().view(n, top, 1)
        return g.sum(1).to(y.dtype)
    assert y.is_contiguous() and (wt is None or (wt.is_contiguous() and wt.dtype == torch.float32))
    out = torch.empty(n, y.size(1), device=y.device, dtype=y.dtype)
    _check(lib().hyb_combine_rows(y.data_ptr(), where.data_ptr(), None if wt is None else wt.data_ptr(), out.data_ptr(), n,
                                  top, y.size(1), None if idx is None else idx.data_ptr(), int(n_experts),
                                  None if idx is None else h.data_ptr(), 0 if idx is None else _rows(h)[0], _dt(y), _st()),
           "combine_rows")
    return out


_ACTS = {"silu": 0, "gelu_tanh": 1, "clamped": 2}


def act_mul(gu: torch.Tensor, act: str = "silu", limit: float = 0.0) -> torch.Tensor:
    """``act(gu[:, :F]) * gu[:, F:]`` for rows ``gu [M, 2F]`` (a gated feed-forward whose gate and up projections are
    one matrix product), evaluated in fp32, result in the activation type; ``act="clamped"`` is the clamped product of
    :func:`glu` with ``limit``."""
    M, F2 = gu.shape
    Fh = F2 // 2
    if not gu.is_cuda:
        return glu(gu[:, :Fh].float(), gu[:, Fh:].float(), act, limit).to(gu.dtype)
    out = torch.empty(M, Fh, device=gu.device, dtype=gu.dtype)
    _check(lib().hyb_act_mul_rows(gu.data_ptr(), _rows(gu)[0], out.data_ptr(), M, Fh, _ACTS[act], float(limit), _dt(gu), _st()),
           "act_mul")
    return out


def scaled_branches(resid: torch.Tensor, a: torch.Tensor, ls1: Optional[torch.Tensor], b: Optional[torch.Tensor] = None,
                    b2: Optional[torch.Tensor] = None, ls2: Optional[torch.Tensor] = None) -> None:
    """``resid += ls1 * a + ls2 * (b + b2)`` in one pass over the fp32 residual: the update of a block whose mixer
    (``a``) and feed-forward (``b``, plus ``b2`` when it has an always-on part) read the same normed input, each
    branch with a learned scale per channel (absent: 1).  All sums are fp32."""
    if resid.dtype != torch.float32:
        raise HybridOpsError("the residual stream is fp32")
    if not a.is_cuda:
        y = a.float() * (ls1.float() if ls1 is not None else 1.0)
        if b is not None:
            f = b.float() + (b2.float() if b2 is not None else 0.0)
            y = y + f * (ls2.float() if ls2 is not None else 1.0)
        resid.add_(y)
        return
    N, C = a.shape
    for t in (ls1, ls2):
        if t is not None and (t.dtype != a.dtype or not t.is_contiguous()):
            raise HybridOpsError("branch scales have the activation type")
    _check(lib().hyb_scaled_branches(resid.data_ptr(), resid.stride(0), a.data_ptr(), _rows(a)[0],
                                     None if ls1 is None else ls1.data_ptr(), None if b is None else b.data_ptr(),
                                     0 if b is None else _rows(b)[0], None if b2 is None else b2.data_ptr(),
                                     0 if b2 is None else _rows(b2)[0], None if ls2 is None else ls2.data_ptr(), N, C,
                                     _dt(a), _st()), "scaled_branches")


def matmul_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Batched ``a @ b`` with an fp32 result whatever the operand type (scores that feed a softmax)."""
    if a.dtype == torch.float32:
        return torch.bmm(a, b)
    try:
        return torch.bmm(a, b, out_dtype=torch.float32)
    except (TypeError, RuntimeError):
        return torch.bmm(a.float(), b.float())


# ---------------------------------------------------------------------------------------------------------
# short convolution and the gated recurrences
# ---------------------------------------------------------------------------------------------------------
def conv_silu(x: torch.Tensor, w: torch.Tensor, state: torch.Tensor, plan: BatchPlan) -> torch.Tensor:
    """Causal per-channel convolution over time (``w [C, taps]``, last column = current token) then SiLU.
    ``state [slots, taps-1, C]`` supplies the inputs before this step and is updated to the step's last ones."""
    C, taps = w.shape
    if not x.is_cuda:
        y = torch.empty(x.size(0), C, dtype=x.dtype)
        for r0, n, slot, _ in plan.seqs:
            full = torch.cat((state[slot], x[r0:r0 + n]), 0).float()  # [taps-1+n, C]
            acc = torch.zeros(n, C)
            for j in range(taps):
                acc += full[j:j + n] * w[:, j].float()
            y[r0:r0 + n] = F.silu(acc).to(x.dtype)
            if taps > 1:
                state[slot] = full[-(taps - 1):].to(state.dtype)
        return y
    xs, _ = _rows(x)
    y = torch.empty(x.size(0), C, device=x.device, dtype=x.dtype)
    _check(lib().hyb_conv_silu(x.data_ptr(), xs, w.data_ptr(), state.data_ptr(), y.data_ptr(), C, plan.meta.data_ptr(),
                               plan.tok_seq.data_ptr(), x.size(0), len(plan.seqs), C, taps, _dt(x), _st()), "conv_silu")
    return y


def gated_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor, g: torch.Tensor,
                     w: torch.Tensor, state: torch.Tensor, plan: BatchPlan, *, heads: int, kv_heads: int, dim: int,
                     vdim: int, mode: str, eps: float, zb: Optional[torch.Tensor] = None, tau: float = 1.0,
                     beta: Optional[torch.Tensor] = None, a_log: Optional[torch.Tensor] = None, variant: int = 0) -> torch.Tensor:
    """A linear recurrence with a ``[dim, vdim]`` fp32 state per head and slot, read out, normed and gated.

    ``mode="gla"``:   ``a = sigmoid(z + zb)^(1/tau)``; ``S = diag(a) S + k v^T``; ``o = S^T q / sqrt(dim)``; gate SiLU.
    ``mode="delta"``: ``a = exp(-exp(a_log) softplus(z + zb))``; q, k made unit vectors (eps 1e-6);
    ``S = diag(a) S``; ``u = sigmoid(beta) (v - S^T k)``; ``S += k u^T``; ``o = S^T q / sqrt(dim)``; gate sigmoid.
    Output per head: ``o / rms(o) * w * gate(g)``, rows ``[N, heads * vdim]``.  ``state [slots, heads, dim, vdim]``
    is read at the start of the step and written back at its end.  ``variant`` (CUDA only): 0 chooses — steps that
    bring more tokens than sequences (prompts) run as prepare / scan / finish kernels (3) when ``dim <= 256``,
    one-token steps as the fused kernel with the state in registers (2) when the shape fits it, anything else as the
    fused kernel with the state in shared memory (1); 1, 2, 3 force one.
    """
    N = v.size(0)
    H, G, D, V = heads, kv_heads, dim, vdim
    if not q.is_cuda:
        out = torch.empty(N, H * V, dtype=v.dtype)
        rep = H // G
        zf = z.float().view(N, H, D) + (zb.float().view(H, D) if zb is not None else 0.0)
        if mode == "delta":
            a = torch.exp(-torch.exp(a_log.float())[None, :, None] * F.softplus(zf))
            bt = torch.sigmoid(beta.float())
        else:
            a = torch.exp(F.logsigmoid(zf) / tau)
        qf = q.float().reshape(N, G, D).repeat_interleave(rep, 1)
        kf = k.float().reshape(N, G, D).repeat_interleave(rep, 1)
        if mode == "delta":
            qf = qf / torch.sqrt((qf * qf).sum(-1, keepdim=True) + 1e-6)
            kf = kf / torch.sqrt((kf * kf).sum(-1, keepdim=True) + 1e-6)
        qf = qf * D ** -0.5
        vf = v.float().reshape(N, H, V)
        gf = g.float().reshape(N, H, V)
        gate = torch.sigmoid(gf) if mode == "delta" else F.silu(gf)
        for r0, n, slot, _ in plan.seqs:
            S = state[slot].clone()  # [H, D, V]
            for t in range(r0, r0 + n):
                S = a[t][:, :, None] * S
                u = vf[t]
                if mode == "delta":
                    u = bt[t][:, None] * (u - torch.einsum("hdv,hd->hv", S, kf[t]))
                S = S + kf[t][:, :, None] * u[:, None, :]
                o = torch.einsum("hdv,hd->hv", S, qf[t])
                o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * w.float()
                out[t] = (o * gate[t]).reshape(-1).to(v.dtype)
            state[slot] = S
        return out
    if state.dtype != torch.float32:
        raise HybridOpsError("recurrent state is fp32")
    out = torch.empty(N, H * V, device=v.device, dtype=v.dtype)
    a = _RecArgs()
    a.q, a.k, a.v, a.z, a.g = q.data_ptr(), k.data_ptr(), v.data_ptr(), z.data_ptr(), g.data_ptr()
    a.beta = None if beta is None else beta.data_ptr()
    a.zb = None if zb is None else zb.data_ptr()
    a.a_log = None if a_log is None else a_log.data_ptr()
    a.w, a.out, a.state, a.meta = w.data_ptr(), out.data_ptr(), state.data_ptr(), plan.meta.data_ptr()
    a.q_stride, a.k_stride, a.v_stride = _rows(q)[0], _rows(k)[0], _rows(v)[0]
    a.z_stride, a.g_stride = _rows(z)[0], _rows(g)[0]
    a.beta_stride = 0 if beta is None else _rows(beta)[0]
    a.out_stride = H * V
    a.H, a.G, a.D, a.V, a.mode = H, G, D, V, 1 if mode == "delta" else 0
    a.tau, a.eps = float(tau), float(eps)
    prep = bsig = oraw = None
    if variant in (0, 3) and D <= 256 and (variant == 3 or N > len(plan.seqs)):
        prep = torch.empty(N, H, D, 4, device=v.device, dtype=torch.float32)
        bsig = torch.empty(N, H, device=v.device, dtype=torch.float32)
        oraw = torch.empty(N, H * V, device=v.device, dtype=torch.float32)
    _check(lib().hyb_gated_recurrence(ctypes.byref(a), len(plan.seqs), N, _dt(v), int(variant),
                                      None if prep is None else prep.data_ptr(), None if bsig is None else bsig.data_ptr(),
                                      None if oraw is None else oraw.data_ptr(), _st()), "gated_recurrence")
    return out


# ---------------------------------------------------------------------------------------------------------
# post-norm blocks: norm over a whole projection, the fixed-decay recurrence, the norm of a gated sum
# ---------------------------------------------------------------------------------------------------------
def full_norm_append(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor],
                     cache: Optional[torch.Tensor], plan: BatchPlan, H: int, G: int, D: int, V: int, nrot: int, eps: float,
                     qw: torch.Tensor, kw: Optional[torch.Tensor]) -> None:
    """Per token: the query row (all ``H*D`` values at once) is divided by its root mean square (``eps`` inside the
    root) and multiplied by ``qw [H*D]``, then the first ``nrot`` entries of every head are rotated (entry ``2i`` with
    ``2i+1``, angle ``pos * inv_freq[i]``) and the row is kept in place; the key row (``G*D`` values, ``kw``) is treated
    the same way and written with the values behind it to ``cache[slot, pos]``.  ``k is None``: a layer that reads
    another layer's keys and values prepares its queries only.  fp32 arithmetic, one rounding at the end."""
    if not q.is_cuda:
        N = q.size(0)

        def prep(x: torch.Tensor, heads: int, w: torch.Tensor) -> torch.Tensor:
            xf = _norm_torch(x, w, None, eps, "rms").reshape(N, heads, D).clone()
            if nrot:
                ang = plan.positions.float()[:, None] * inv_freq[None, :]
                c, s_ = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                u, w_ = xf[..., 0:nrot:2].clone(), xf[..., 1:nrot:2].clone()
                xf[..., 0:nrot:2] = u * c - w_ * s_
                xf[..., 1:nrot:2] = w_ * c + u * s_
            return xf.reshape(N, heads * D).to(x.dtype)

        q.copy_(prep(q, H, qw))
        if k is not None:
            kk = prep(k, G, kw)
            for r0, n, slot, p0 in plan.seqs:
                cache[slot, p0:p0 + n, :G * D] = kk[r0:r0 + n]
                cache[slot, p0:p0 + n, G * D:] = v[r0:r0 + n]
        return
    for w in (qw, kw):
        if w is not None and (w.dtype != q.dtype or not w.is_contiguous()):
            raise HybridOpsError("norm weights have the activation type")
    _check(lib().hyb_full_norm_append(q.data_ptr(), _rows(q)[0], None if k is None else k.data_ptr(),
                                      0 if k is None else _rows(k)[0], None if k is None else v.data_ptr(),
                                      0 if k is None else _rows(v)[0], None if inv_freq is None else inv_freq.data_ptr(),
                                      None if k is None else cache.data_ptr(), 0 if k is None else cache.stride(0),
                                      plan.meta.data_ptr(), plan.tok_seq.data_ptr(), q.size(0), H, G, D, V, int(nrot),
                                      float(eps), qw.data_ptr(), None if kw is None else kw.data_ptr(), _dt(q), _st()),
           "full_norm_append")


lightning_chunk_from = 16  # a step whose longest sequence brings at least this many tokens takes the chunked kernel


def lightning_recurrence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                         plan: BatchPlan, heads: int, dim: int, vdim: int, variant: int = 0, act: bool = False) -> torch.Tensor:
    """``S <- decay_h S + k v^T``, ``o = S^T q`` per head and token, ``S [dim, vdim]`` fp32 in ``state[slot, head]``
    (read at the start of the step, written back at its end); no scale.  ``decay`` fp32 ``[heads]``.  Returns the raw
    read-outs as fp32 ``[N, heads * vdim]``.  ``act``: q, k, v are pre-activations, their SiLU is taken in fp32 as they
    are read.  ``variant`` (CUDA): 1 the token scan; 2 chunks of 64 tokens, all chunks of the step in parallel (a chunk
    is four small matrix products, only ``S' = decay^len S + U`` chains the chunks of a sequence, only non-negative powers
    of the decay occur); 0 chooses by the longest sequence."""
    N = v.size(0)
    H, D, V = heads, dim, vdim
    if state.dtype != torch.float32 or decay.dtype != torch.float32:
        raise HybridOpsError("recurrent state and decays are fp32")
    if not q.is_cuda:
        out = torch.empty(N, H * V, dtype=torch.float32)
        qf, kf, vf = q.float().reshape(N, H, D), k.float().reshape(N, H, D), v.float().reshape(N, H, V)
        if act:
            qf, kf, vf = F.silu(qf), F.silu(kf), F.silu(vf)
        lam = decay.float()[:, None, None]
        for r0, n, slot, _ in plan.seqs:
            S = state[slot].clone()
            for t in range(r0, r0 + n):
                S = lam * S + kf[t][:, :, None] * vf[t][:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, qf[t]).reshape(-1)
            state[slot] = S
        return out
    if not variant:
        variant = 2 if max(n for _, n, _, _ in plan.seqs) >= lightning_chunk_from else 1
    out = torch.empty(N, H * V, device=v.device, dtype=torch.float32)
    ctab = stab = scratch = None
    nchunks = 0
    if variant == 2:
        tabs = plan.shared.get("lightning_chunks")  # the same for every such layer of the step
        if tabs is None:
            chunks, per_seq = [], []
            for i, (r0, n, _, _) in enumerate(plan.seqs):
                per_seq.append((len(chunks), (n + 63) // 64))
                chunks += [(r0 + c, min(64, n - c), i, 0) for c in range(0, n, 64)]
            tabs = (torch.tensor(chunks, dtype=torch.int32).to(v.device), torch.tensor(per_seq, dtype=torch.int32).to(v.device), len(chunks))
            plan.shared["lightning_chunks"] = tabs
        ctab, stab, nchunks = tabs
        scratch = torch.empty(nchunks, H, D, V, device=v.device, dtype=torch.float32)
    _check(lib().hyb_lightning(q.data_ptr(), _rows(q)[0], k.data_ptr(), _rows(k)[0], v.data_ptr(), _rows(v)[0],
                               decay.data_ptr(), state.data_ptr(), plan.meta.data_ptr(), out.data_ptr(), len(plan.seqs),
                               H, D, V, int(variant), int(bool(act)), None if ctab is None else ctab.data_ptr(),
                               None if stab is None else stab.data_ptr(), nchunks,
                               None if scratch is None else scratch.data_ptr(), _dt(v), _st()), "lightning_recurrence")
    return out


def norm_gate_rows(o: torch.Tensor, w: torch.Tensor, g: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """``o / rms(o) * w * sigmoid(g)`` over whole rows of fp32 ``o [N, n]`` (``eps`` inside the root), in ``out_dtype``."""
    if not o.is_cuda:
        return (_norm_torch(o, w, None, eps, "rms") * torch.sigmoid(g.float())).to(out_dtype)
    if o.dtype != torch.float32 or not o.is_contiguous() or w.dtype != out_dtype or g.dtype != out_dtype:
        raise HybridOpsError("read-outs are dense fp32; weight and gate have the activation type")
    out = torch.empty(o.shape, device=o.device, dtype=out_dtype)
    _check(lib().hyb_norm_gate_rows(o.data_ptr(), w.data_ptr(), g.data_ptr(), _rows(g)[0], out.data_ptr(), o.size(0), o.size(1),
                                    float(eps), _dt(out), _st()), "norm_gate_rows")
    return out


def gated_sum_norm_accumulate(resid: torch.Tensor, a: torch.Tensor, b: Optional[torch.Tensor], sg: Optional[torch.Tensor],
                              w: torch.Tensor, eps: float, kind: str = "rms", copy: Optional[torch.Tensor] = None) -> None:
    """``resid += norm(a + sigmoid(sg) * b) * w`` in one pass over the fp32 residual: ``a`` and ``b`` are two branches
    of a feed-forward, ``sg [N, 1]`` one gate logit per token for ``b`` (absent: 1).  All sums are fp32.  ``copy``: as in
    :func:`norm_accumulate`."""
    if resid.dtype != torch.float32:
        raise HybridOpsError("the residual stream is fp32")
    if b is None:
        return norm_accumulate(resid, a, w, None, eps, kind, copy=copy)
    if not a.is_cuda:
        y = a.float() + (torch.sigmoid(sg.float()) if sg is not None else 1.0) * b.float()
        resid.add_(_norm_torch(y, w, None, eps, kind))
        if copy is not None:
            copy.copy_(resid)
        return
    if copy is not None and (copy.dtype != a.dtype or not copy.is_contiguous() or copy.shape != resid.shape):
        raise HybridOpsError("the residual's copy is dense and has the activation type")
    _check(lib().hyb_gated_sum_norm(a.data_ptr(), _rows(a)[0], b.data_ptr(), _rows(b)[0],
                                    None if sg is None else sg.data_ptr(), 0 if sg is None else sg.stride(0), w.data_ptr(),
                                    resid.data_ptr(), resid.stride(0), a.size(0), a.size(1), float(eps),
                                    _NORM_KINDS[kind], None if copy is None else copy.data_ptr(), _dt(a), _st()), "gated_sum_norm")
