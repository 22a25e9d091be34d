"""A plain float64 restatement of the Labepel design, one function per mechanism, for whole sequences only.

It shares nothing with the product path: no cache, no batches, no kernels.  ``T`` maps tensor names to tensors,
``cfg`` is the parsed ``config.json``.  Notation: ``C`` width, ``H``/``G`` query and key/value heads, ``D``/``V`` key
and value size per head, ``n`` tokens of one sequence.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the deviation from one."""
    return rms_unit(x, eps) * (1.0 + w.to(F64))


def norm_plain(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w.to(F64)


def lin(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ w.to(F64).T
    return y if b is None else y + b.to(F64)


def same_chunk_mask(n: int, size: int) -> torch.Tensor:
    """``m[i, j]`` true when position ``i`` may read position ``j``: not later, and in the same block of ``size``
    positions counted from the sequence's start (``size <= 0``: every earlier position)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if size > 0:
        ok = ok & (torch.div(i, size, rounding_mode="floor") == torch.div(j, size, rounding_mode="floor"))
    return ok


def softmax_with_sink(s: torch.Tensor, ok: torch.Tensor) -> torch.Tensor:
    """``p_j = e^{s_j} / (1 + sum_visible e^{s_k})``: an extra slot of score zero that carries no value."""
    s = s.masked_fill(~ok, float("-inf"))
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def attention(h: torch.Tensor, T: Dict[str, torch.Tensor], pre: str, m: dict, eps: float,
              v_first: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns the mixer output ``[n, C]`` and the values this layer used ``[n, G*V]`` (after mixing)."""
    n = h.size(0)
    Hh, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(h, T[pre + "q"], T[pre + "q.b"]).view(n, Hh, D)
    k = lin(h, T[pre + "k"], T[pre + "k.b"]).view(n, G, D)
    v = lin(h, T[pre + "v"], T[pre + "v.b"])
    q = norm_plain(q, T[pre + "q.norm"], eps)
    k = norm_plain(k, T[pre + "k.norm"], eps)
    if m.get("v_mix") and v_first is not None:
        lam = T[pre + "vmix"].to(F64)
        v = (1.0 - lam) * v + lam * v_first
    vv = v.view(n, G, V)
    ok = same_chunk_mask(n, int((m.get("mask") or {}).get("size", 0) or 0))
    out = torch.empty(n, Hh, V, dtype=F64)
    for hd in range(Hh):
        g = hd // (Hh // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        out[:, hd] = softmax_with_sink(s, ok) @ vv[:, g]
    gate = torch.sigmoid(lin(h, T[pre + "g"]))
    return lin(out.reshape(n, Hh * V) * gate, T[pre + "o"]), v


def gated_expert(h: torch.Tensor, T: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    a = lin(h, T[pre + "gate"])
    return lin(a * torch.sigmoid(a) * lin(h, T[pre + "up"]), T[pre + "down"])


def route(z: torch.Tensor, top: int) -> Tuple[List[int], torch.Tensor]:
    """The ``top`` largest logits of one token and the softmax over just those."""
    order = sorted(range(z.numel()), key=lambda e: (-float(z[e]), e))[:top]
    zs = torch.stack([z[e] for e in order])
    return order, torch.softmax(zs, 0)


def mixture(h: torch.Tensor, T: Dict[str, torch.Tensor], pre: str, mlp: dict) -> torch.Tensor:
    n = h.size(0)
    z = lin(h, T[pre + "router"], T[pre + "router.b"])
    out = torch.zeros(n, h.size(1), dtype=F64)
    for t in range(n):
        chosen, wts = route(z[t], int(mlp["router"]["top"]))
        for e, w in zip(chosen, wts):
            out[t] += w * gated_expert(h[t:t + 1], T, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out += gated_expert(h, T, pre + "shared.")
    return out


def forward(T: Dict[str, torch.Tensor], cfg: dict, tokens: List[int]) -> Tuple[torch.Tensor, List[torch.Tensor]]:
    """Logits ``[n, vocab]`` and the residual stream after every layer for one sequence from position 0."""
    eps = float(cfg["norm"]["eps"])
    n = len(tokens)
    x = T["embed"].to(F64)[torch.tensor(tokens)] + T["pos"].to(F64)[:n]
    v_first = None
    trace = []
    for i, spec in enumerate(cfg["layers"]):
        h = norm_one_plus(x, T[f"l{i}.norm1"], eps)
        y, v = attention(h, T, f"l{i}.mix.", spec["mixer"], eps, v_first)
        if spec["mixer"].get("v_mix") and v_first is None:
            v_first = v
        y = y * T[f"l{i}.ls1"].to(F64)
        if spec.get("mlp"):
            y = y + mixture(h, T, f"l{i}.mlp.", spec["mlp"]) * T[f"l{i}.ls2"].to(F64)
        x = x + y
        trace.append(x.clone())
    hN = norm_one_plus(x, T["final.norm"], eps)
    return lin(hN, T["embed"]), trace


def random_tensors(cfg: dict, seed: int = 0, dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights for a configuration, rounded to ``dtype`` (so that every precision reads the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    C = int(cfg["width"])

    def mat(o: int, i: int, s: float = 1.0) -> torch.Tensor:
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(nn: int, s: float, mean: float = 0.0) -> torch.Tensor:
        return (mean + torch.randn(nn, generator=g) * s).to(dtype)

    T = {"embed": (torch.randn(cfg["vocab"], C, generator=g)).to(dtype),
         "pos": (torch.randn(cfg["max_positions"], C, generator=g) * 0.5).to(dtype), "final.norm": vec(C, 0.1)}
    for i, spec in enumerate(cfg["layers"]):
        m = spec["mixer"]
        Hh, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        p = f"l{i}.mix."
        T[f"l{i}.norm1"] = vec(C, 0.1)
        T[p + "q"], T[p + "q.b"] = mat(Hh * D, C), vec(Hh * D, 0.2)
        T[p + "k"], T[p + "k.b"] = mat(G * D, C), vec(G * D, 0.2)
        T[p + "v"], T[p + "v.b"] = mat(G * V, C), vec(G * V, 0.2)
        T[p + "q.norm"], T[p + "k.norm"] = vec(D, 0.2, 1.5), vec(D, 0.2, 1.5)
        if m.get("v_mix"):
            T[p + "vmix"] = (torch.rand((), generator=g) * 0.6 + 0.2).to(dtype)
        T[p + "g"], T[p + "o"] = mat(Hh * V, C), mat(C, Hh * V)
        T[f"l{i}.ls1"] = vec(C, 0.2, 1.0)
        mlp = spec.get("mlp")
        if mlp:
            T[f"l{i}.ls2"] = vec(C, 0.2, 1.0)
            q = f"l{i}.mlp."
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                T[f"{q}e{e}.gate"], T[f"{q}e{e}.up"], T[f"{q}e{e}.down"] = mat(ff, C), mat(ff, C), mat(C, ff)
            T[q + "router"], T[q + "router.b"] = mat(E, C, 2.0), vec(E, 0.5)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                T[q + "shared.gate"], T[q + "shared.up"], T[q + "shared.down"] = mat(sf, C), mat(sf, C), mat(C, sf)
    return T
