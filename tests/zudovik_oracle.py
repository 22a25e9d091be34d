"""A plain, slow restatement of the Zudovik design: one function per mechanism, python loops over tokens and heads,
float64 by default.  It shares no code with ``mdi_llm_b200``; the tests compare the framework with it.

Notation: ``x`` a residual row, ``h`` what a sublayer reads (``x`` itself: the design norms sublayer *outputs*),
``t`` a position counted from 0 in its own sequence.  ``W["name"]`` are tensors by checkpoint name.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

DT = torch.float64


def rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * w over the whole vector."""
    return x / torch.sqrt((x * x).mean() + eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def rotate_pairs(head: torch.Tensor, t: int, ndims: int, base: float) -> torch.Tensor:
    """Neighbours (2i, 2i+1) of the first ``ndims`` entries turn by the angle t * base^(-2i/ndims)."""
    out = head.clone()
    for i in range(ndims // 2):
        a = t * base ** (-2.0 * i / ndims)
        u, v = head[2 * i], head[2 * i + 1]
        out[2 * i] = u * math.cos(a) - v * math.sin(a)
        out[2 * i + 1] = v * math.cos(a) + u * math.sin(a)
    return out


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """Weights over the keys; the denominator holds one more term, exp(sink), that has no value."""
    m = max(float(scores.max()), float(sink))
    e = torch.exp(scores - m)
    return e / (e.sum() + math.exp(float(sink) - m))


def attention_queries(W: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor, t: int, eps: float) -> torch.Tensor:
    q = W[pre + "q"] @ h + W[pre + "q.b"]
    q = rms(q, W[pre + "q.norm"], eps).view(m["heads"], m["dim"])
    return torch.stack([rotate_pairs(q[a], t, m["rot"]["dims"], m["rot"]["base"]) for a in range(m["heads"])])


def attention_keys_values(W: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor, t: int, eps: float):
    k = W[pre + "k"] @ h + W[pre + "k.b"]
    k = rms(k, W[pre + "k.norm"], eps).view(m["kv_heads"], m["dim"])
    k = torch.stack([rotate_pairs(k[g], t, m["rot"]["dims"], m["rot"]["base"]) for g in range(m["kv_heads"])])
    v = (W[pre + "v"] @ h + W[pre + "v.b"]).view(m["kv_heads"], m["vdim"])
    return k, v


def attention_mixer(W: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor, t: int, eps: float,
                    keys: List[torch.Tensor], values: List[torch.Tensor]) -> torch.Tensor:
    """``keys`` / ``values`` already hold positions 0..t (this layer's own, or those of the layer it borrows from)."""
    H, G = m["heads"], m["kv_heads"]
    q = attention_queries(W, pre, m, h, t, eps)
    gate = sigmoid(W[pre + "g"] @ h)
    K, Vv = torch.stack(keys[:t + 1]), torch.stack(values[:t + 1])  # [t+1, G, .]
    outs = []
    for a in range(H):
        g = a // (H // G)
        s = (K[:, g] @ q[a]) * m["scale"]  # one score per position j <= t
        cap = m.get("softcap", 0.0)
        if cap:
            s = cap * torch.tanh(s / cap)
        p = sink_softmax(s, W[pre + "sink"][a])
        outs.append((p @ Vv[:, g]) * gate[a])
    return W[pre + "o"] @ torch.cat(outs)


def lightning_mixer(W: Dict[str, torch.Tensor], pre: str, m: Dict[str, Any], h: torch.Tensor, eps: float,
                    state: List[torch.Tensor]) -> torch.Tensor:
    """state[a] is head a's [dim, vdim] matrix; it is advanced in place."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(W[pre + "q"] @ h).view(H, D)
    k = silu(W[pre + "k"] @ h).view(H, D)
    v = silu(W[pre + "v"] @ h).view(H, V)
    outs = []
    for a in range(H):
        state[a] = m["decay"][a] * state[a] + torch.outer(k[a], v[a])
        outs.append(state[a].T @ q[a])
    o = rms(torch.cat(outs), W[pre + "norm"], eps) * sigmoid(W[pre + "g"] @ h)
    return W[pre + "o"] @ o


def dense_ff(W: Dict[str, torch.Tensor], pre: str, h: torch.Tensor) -> torch.Tensor:
    return W[pre + "down"] @ torch.relu(W[pre + "up"] @ h) ** 2


def clamped_expert(W: Dict[str, torch.Tensor], pre: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(W[pre + "gate"] @ h, max=limit)
    u = torch.clamp(W[pre + "up"] @ h, -limit, limit)
    return W[pre + "down"] @ (g * sigmoid(1.702 * g) * (u + 1.0))


def route(W: Dict[str, torch.Tensor], pre: str, h: torch.Tensor, top: int):
    """Chosen router outputs (largest softmax score + correction first) and their weights (scores without it)."""
    z = W[pre + "router"] @ h
    s = torch.exp(z - z.max())
    s = s / s.sum()
    choice = s + W[pre + "correction"]
    chosen = sorted(range(len(z)), key=lambda e: (-float(choice[e]), e))[:top]
    tot = sum(s[e] for e in chosen) + 1e-20
    return chosen, [s[e] / tot for e in chosen]


def moe_ff(W: Dict[str, torch.Tensor], pre: str, mlp: Dict[str, Any], h: torch.Tensor) -> torch.Tensor:
    E = mlp["router"]["experts"]
    chosen, weights = route(W, pre, h, mlp["router"]["top"])
    y = torch.zeros_like(h)
    for e, w in zip(chosen, weights):
        y = y + w * (clamped_expert(W, f"{pre}e{e}.", h, mlp["expert"]["limit"]) if e < E else h)
    if mlp.get("shared"):
        y = y + sigmoid(W[pre + "shared.sg"] @ h)[0] * clamped_expert(W, pre + "shared.", h, mlp["shared"]["limit"])
    return y


def forward(cfg: Dict[str, Any], W: Dict[str, torch.Tensor], tokens: List[int], dtype: torch.dtype = DT,
            layers_out: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits ``[len(tokens), vocab]`` of one sequence, token by token.  ``layers_out`` receives the residual rows
    after every layer as ``[layers, tokens, width]``."""
    W = {k: v.to(dtype) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    L = cfg["layers"]
    keys = [[] for _ in L]
    values = [[] for _ in L]
    states = [[torch.zeros(s["mixer"]["dim"], s["mixer"]["vdim"], dtype=dtype) for _ in range(s["mixer"]["heads"])]
              if s["type"] == "lightning" else None for s in L]
    per_layer = [[] for _ in L]
    logits = []
    for t, tok in enumerate(tokens):
        x = W["embed"][tok] * cfg["embedding"]["scale"]
        for i, spec in enumerate(L):
            m, pre = spec["mixer"], f"l{i}.mix."
            if spec["type"] == "lightning":
                y = lightning_mixer(W, pre, m, x, eps, states[i])
            else:
                src = m.get("kv_from")
                if src is None:
                    k, v = attention_keys_values(W, pre, m, x, t, eps)
                    keys[i].append(k)
                    values[i].append(v)
                    src = i
                y = attention_mixer(W, pre, m, x, t, eps, keys[src], values[src])
            x = x + rms(y, W[f"l{i}.norm1"], eps)
            mlp = spec.get("mlp")
            if mlp:
                y = dense_ff(W, f"l{i}.mlp.", x) if mlp["kind"] == "dense" else moe_ff(W, f"l{i}.mlp.", mlp, x)
                x = x + rms(y, W[f"l{i}.norm2"], eps)
            per_layer[i].append(x)
        logits.append(W["head"] @ rms(x, W["final.norm"], eps))
    if layers_out is not None:
        layers_out.append(torch.stack([torch.stack(rows) for rows in per_layer]))
    return torch.stack(logits)


def random_tensors(cfg: Dict[str, Any], seed: int = 0) -> Dict[str, torch.Tensor]:
    """Weights by checkpoint name for ``cfg``, rounded to bfloat16 values (kept in float32)."""
    g = torch.Generator().manual_seed(seed)
    C = cfg["width"]

    def mat(o: int, i: int, gain: float = 1.0) -> torch.Tensor:
        return torch.randn(o, i, generator=g) * gain / math.sqrt(i)

    def vec(n: int, mean: float = 0.0, std: float = 0.3) -> torch.Tensor:
        return mean + torch.randn(n, generator=g) * std

    W = {"embed": torch.randn(cfg["vocab"], C, generator=g), "head": mat(cfg["vocab"], C), "final.norm": vec(C, 1.0, 0.1)}

    def expert(pre: str, ff: int) -> None:
        W[pre + "gate"], W[pre + "up"], W[pre + "down"] = mat(ff, C, 2.0), mat(ff, C, 2.0), mat(C, ff)

    for i, spec in enumerate(cfg["layers"]):
        m, pre = spec["mixer"], f"l{i}.mix."
        W[f"l{i}.norm1"] = vec(C, 1.0, 0.1)
        if spec["type"] == "lightning":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            W[pre + "q"], W[pre + "k"], W[pre + "v"], W[pre + "g"] = mat(H * D, C), mat(H * D, C), mat(H * V, C), mat(H * V, C)
            W[pre + "o"], W[pre + "norm"] = mat(C, H * V), vec(H * V, 1.0, 0.1)
        else:
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            W[pre + "q"], W[pre + "q.b"], W[pre + "q.norm"] = mat(H * D, C), vec(H * D), vec(H * D, 1.0, 0.2)
            if m.get("kv_from") is None:
                W[pre + "k"], W[pre + "k.b"], W[pre + "k.norm"] = mat(G * D, C), vec(G * D), vec(G * D, 1.0, 0.2)
                W[pre + "v"], W[pre + "v.b"] = mat(G * V, C), vec(G * V)
            W[pre + "sink"], W[pre + "g"], W[pre + "o"] = vec(H, 0.0, 1.0), mat(H, C), mat(C, H * V)
        mlp = spec.get("mlp")
        if not mlp:
            continue
        W[f"l{i}.norm2"] = vec(C, 1.0, 0.1)
        pre = f"l{i}.mlp."
        if mlp["kind"] == "dense":
            W[pre + "up"], W[pre + "down"] = mat(mlp["ff"], C), mat(C, mlp["ff"])
            continue
        r = mlp["router"]
        n_out = r["experts"] + r.get("identity", 0)
        W[pre + "router"], W[pre + "correction"] = mat(n_out, C, 2.0), vec(n_out, 0.0, 0.05)
        for e in range(r["experts"]):
            expert(f"{pre}e{e}.", mlp["expert"]["ff"])
        if mlp.get("shared"):
            expert(pre + "shared.", mlp["shared"]["ff"])
            W[pre + "shared.sg"] = mat(1, C)
    return {k: v.to(torch.bfloat16).float() for k, v in W.items()}
