"""The hybrid model family: a residual stream through layers that each pick their own sequence mixer.

Mixers (all written against the packed-batch operations of :mod:`mdi_llm_b200.ops.hybrid`):

* :class:`LatentAttention` — softmax attention whose keys and values are expansions of one cached latent row per
  token plus a rotated key part shared by the heads.  Only that row is cached; the query is carried into the latent
  space (``q W_uk``) so that the attention kernel reads the cache directly, and the attended latent is expanded
  by ``W_uv`` afterwards.
* :class:`GatedLinearAttention` — ``S_t = diag(a_t) S_(t-1) + k_t v_t^T`` with a data-dependent decay per key
  channel.
* :class:`ChannelDelta` — the gated delta rule with a decay per key channel, short causal convolutions on q, k, v
  and unit-norm q, k.
* :class:`WindowAttention` — grouped-query softmax attention over a sliding window of cached keys and values, with
  interleaved rotary positions (optionally stretched by wavelength), weight-free RMS norm of q and k after the
  rotation, and one sigmoid output gate per head.

* :class:`LightningAttention` — ``S_t = decay_h S_(t-1) + k_t v_t^T`` with one fixed decay per head, SiLU on q, k, v,
  an RMS norm over all heads' read-outs together and a sigmoid gate per channel.

Feed-forwards: :class:`DenseFF` and :class:`MoEFF` (sigmoid router, top-k, the score scales the expert's *input*).

A layer is a *sandwich* block (``x += norm_b(f(norm_a(x)))`` for the mixer and again for the feed-forward), a
*pre-norm* block (``x += m f(norm(x))``, optionally followed by a gated per-layer token embedding), a *parallel* block
or a *post-norm* block (``x += norm(f(x))``: the sublayer reads the residual stream itself), chosen by the
architecture (``config.block``), with the residual stream kept in fp32.  A span of layers may be looped; each pass owns its own state and starts by
mixing the embedding output back in.  State lives in a :class:`StatePool` — slots like the KV pool of the
transformer family (``models/gpt.py:KVPool``), one entry per *layer run*.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import torch
import torch.nn as nn

from ..ops import hybrid as H
from .config import HybridConfig

__all__ = ["HybridLM", "StatePool", "SandwichBlock", "PreNormBlock", "ParallelBlock", "PostNormBlock", "LatentAttention",
           "GatedLinearAttention", "ChannelDelta", "WindowAttention", "LightningAttention", "DenseFF", "GatedFF", "MoEFF", "read_safetensors", "write_safetensors", "load_hybrid"]

_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path: Union[str, Path]) -> Dict[str, torch.Tensor]:
    """Minimal reader: 8-byte little-endian header length, JSON header, raw little-endian data."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    out: Dict[str, torch.Tensor] = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        buf = bytearray(raw[8 + n + a:8 + n + b])
        out[name] = (torch.frombuffer(buf, dtype=dt) if buf else torch.empty(0, dtype=dt)).view(info["shape"])
    return out


def write_safetensors(tensors: Dict[str, torch.Tensor], path: Union[str, Path]) -> None:
    names = {v: k for k, v in _ST_DTYPES.items()}
    header: Dict[str, Any] = {}
    blobs, off = [], 0
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        b = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""  # reshape: a scalar has no axis to view
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as fp:
        fp.write(struct.pack("<Q", len(hj)))
        fp.write(hj)
        for b in blobs:
            fp.write(b)


# =============================================================================================
# state
# =============================================================================================
class StatePool:
    """Slots of per-sequence state for every layer run of a hybrid model.

    A run of a latent-attention layer owns ``cache [slots, max_seq, kv_rank + rot_dim]`` (activation type); a run
    of a recurrent layer owns ``state [slots, heads, dim, vdim]`` in fp32 and, with a short convolution,
    ``conv [slots, taps - 1, channels]``.  ``alloc`` hands out a slot with zeroed recurrent and convolution state
    (attention rows need no clearing: a row is written before any query can see it); ``free`` returns it.
    The pool grows (doubling, contents kept) when more slots are asked for than it has.  A run of an attention layer
    that names ``kv_from`` owns nothing: its ``cache`` entry IS the cache of the latest earlier run of the layer it
    names (the same tensor), which that run has already extended by the step's tokens when this one reads it.
    """

    def __init__(self, config: HybridConfig, n_slots: int, max_seq_length: int, device: torch.device, dtype: torch.dtype) -> None:
        self.config, self.max_seq_length, self.device, self.dtype = config, int(max_seq_length), device, dtype
        self.n_slots = 0
        self.runs: List[Dict[str, torch.Tensor]] = [{} for _ in config.layer_runs()]
        self.free_slots: List[int] = []
        self.length: Dict[int, int] = {}
        self._grow(max(1, n_slots))

    def _shapes(self, spec: Dict[str, Any]) -> Dict[str, Tuple[Tuple[int, ...], torch.dtype]]:
        m = spec["mixer"]
        if spec["type"] == "latent_attention":
            return {"cache": ((self.max_seq_length, m["kv_rank"] + m["rot_dim"]), self.dtype)}
        if spec["type"] == "attention" and m.get("kv_from") is not None:
            return {}
        if spec["type"] == "attention":  # one row per position: the kv_heads keys, then the kv_heads values
            return {"cache": ((self.max_seq_length, m["kv_heads"] * (m["dim"] + m["vdim"])), self.dtype)}
        out = {"state": ((m["heads"], m["dim"], m["vdim"]), torch.float32)}
        if spec["type"] == "channel_delta" and m["conv"] > 1:
            ch = 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"]
            out["conv"] = ((m["conv"] - 1, ch), self.dtype)
        return out

    def _grow(self, n_slots: int) -> None:
        for run, (li, _) in zip(self.runs, self.config.layer_runs()):
            for key, (shape, dt) in self._shapes(self.config.layers[li]).items():
                new = torch.zeros((n_slots, *shape), device=self.device, dtype=dt)
                if key in run:
                    new[: self.n_slots] = run[key]
                run[key] = new
        order = self.config.layer_runs()
        for r, (li, _) in enumerate(order):
            src = self.config.layers[li]["mixer"].get("kv_from") if self.config.layers[li]["type"] == "attention" else None
            if src is not None:
                owner = max(j for j in range(r) if order[j][0] == int(src))
                self.runs[r]["cache"] = self.runs[owner]["cache"]
        self.free_slots += list(range(self.n_slots, n_slots))
        self.n_slots = n_slots

    def alloc(self) -> int:
        if not self.free_slots:
            self._grow(2 * self.n_slots)
        slot = self.free_slots.pop(0)
        for run in self.runs:
            for key in ("state", "conv"):
                if key in run:
                    run[key][slot].zero_()
        self.length[slot] = 0
        return slot

    def free(self, slot: int) -> None:
        if slot not in self.length:
            raise KeyError(f"slot {slot} is not in use")
        del self.length[slot]
        self.free_slots.append(slot)

    @property
    def nbytes(self) -> int:
        own = {t.data_ptr(): t for run in self.runs for t in run.values()}  # a borrowed cache counts once
        return sum(t.numel() * t.element_size() for t in own.values())


# =============================================================================================
# modules
# =============================================================================================
def _param(*shape: int) -> nn.Parameter:
    return nn.Parameter(torch.empty(*shape), requires_grad=False)


class _Fused:
    """Mixin: several projections that read the same input become one weight; the originals turn into row views."""

    def fuse(self, names: Sequence[str]) -> None:
        ws = [getattr(self, n) for n in names]
        fused = torch.cat([w.data for w in ws], 0).contiguous()
        self.w_in = fused
        self.cols: Dict[str, Tuple[int, int]] = {}
        r = 0
        for n, w in zip(names, ws):
            self.cols[n] = (r, r + w.size(0))
            w.data = fused[r:r + w.size(0)]
            r += w.size(0)

    def col(self, p: torch.Tensor, name: str) -> torch.Tensor:
        a, b = self.cols[name]
        return p[:, a:b]

    def rebase(self, rows: torch.Tensor) -> None:
        """Move the fused weight into ``rows`` (same shape, a slice of a larger matrix that already holds its values):
        the originals become views of that."""
        assert rows.shape == self.w_in.shape
        self.w_in = rows
        for n, (a, b) in self.cols.items():
            getattr(self, n).data = rows[a:b]


class LatentAttention(nn.Module, _Fused):
    tensor_names = {"dq": "dq", "dq.norm": "dq_norm", "uq": "uq", "dkv": "dkv", "dkv.norm": "dkv_norm", "uk": "uk",
                    "uv": "uv", "g": "g", "o": "o"}

    def __init__(self, width: int, m: Dict[str, Any], eps: float) -> None:
        super().__init__()
        self.H, self.D, self.R, self.V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
        self.L, self.QR, self.scale, self.eps = m["kv_rank"], m["q_rank"], float(m["scale"]), eps
        self.nrot, self.rot_base = int(m["rot"]["dims"]), float(m["rot"]["base"])
        if self.nrot > self.R or self.nrot % 2:
            raise ValueError("rot.dims must be even and at most rot_dim")
        H_, D, R, V, L = self.H, self.D, self.R, self.V, self.L
        self.dq, self.dq_norm, self.uq = _param(self.QR, width), _param(self.QR), _param(H_ * (D + R), self.QR)
        self.dkv, self.dkv_norm = _param(L + R, width), _param(L)
        self.uk, self.uv = _param(H_ * D, L), _param(H_ * V, L)
        self.g, self.o = _param(H_ * V, width), _param(width, H_ * V)
        self.inv_freq: Optional[torch.Tensor] = None

    def finalize(self) -> None:
        self.fuse(("dq", "dkv", "g"))
        self.inv_freq = H.rotary_inv_freq(self.nrot, self.rot_base, self.dq.device)

    def forward(self, h: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        N = h.size(0)
        Hh, D, R, V, L = self.H, self.D, self.R, self.V, self.L
        p = H.linear(h, self.w_in)
        cq = H.norm_rows(self.col(p, "dq"), self.dq_norm, None, self.eps, "rms", h.dtype)
        q = H.linear(cq, self.uq)
        H.latent_append(self.col(p, "dkv"), q, self.dkv_norm, self.inv_freq, st["cache"], plan, Hh, D, R, L, self.nrot, self.eps)
        if min(n for _, n, _, _ in plan.seqs) >= self.expand_from:
            o = self._expanded(q, st["cache"], plan)
        else:
            qlat = torch.bmm(q.view(N, Hh, D + R)[:, :, :D].transpose(0, 1), self.uk.view(Hh, D, L)).contiguous()
            olat = H.latent_attn(qlat, q, st["cache"], plan, Hh, D, R, L, self.scale)
            o = torch.bmm(olat, self.uv.view(Hh, V, L).transpose(1, 2)).contiguous()
        return H.linear(H.headmajor_gate(o, self.col(p, "g")), self.o)

    expand_from = 64   # a step whose every sequence brings at least this many tokens takes the expanded form
    query_block = 1024  # rows of the score matrix alive at a time

    def _expanded(self, q: torch.Tensor, cache: torch.Tensor, plan: H.BatchPlan) -> torch.Tensor:
        """Prompt form: keys and values are expanded from the cached latents once per step (two matrix products),
        scores and the weighted sum are batched matrix products over heads, the causal softmax runs on fp32 scores.
        Decoding instead carries the query into the latent space and reads the cache directly (``H.latent_attn``):
        per query that costs ``kv_rank`` instead of ``dim`` multiplies per key and head, which only pays when
        there is a single query.  Returns ``[heads, N, vdim]``."""
        Hh, D, R, V, L = self.H, self.D, self.R, self.V, self.L
        out = torch.empty(Hh, q.size(0), V, device=q.device, dtype=q.dtype)
        for r0, n, slot, p0 in plan.seqs:
            keys = p0 + n
            rows = cache[slot, :keys]
            lat = rows[:, :L]
            k = torch.empty(Hh, D + R, keys, device=q.device, dtype=q.dtype)  # K^T per head: [unrotated | shared rotated]
            k[:, :D] = H.linear(lat, self.uk).view(keys, Hh, D).permute(1, 2, 0)
            k[:, D:] = rows[:, L:].t()
            v = H.linear(lat, self.uv).view(keys, Hh, V).transpose(0, 1)  # [H, keys, V]
            qh = q[r0:r0 + n].view(n, Hh, D + R).transpose(0, 1)  # [H, n, D+R]
            for a in range(0, n, self.query_block):
                b = min(n, a + self.query_block)
                vis = p0 + b  # keys any row of this block can see
                s = H.matmul_f32(qh[:, a:b], k[:, :, :vis]).contiguous()
                pr = H.causal_softmax(s, p0 + a, self.scale, q.dtype)
                out[:, r0 + a:r0 + b] = torch.bmm(pr, v[:, :vis])
        return out


class GatedLinearAttention(nn.Module, _Fused):
    tensor_names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2.b": "a2_b"}

    def __init__(self, width: int, m: Dict[str, Any], eps: float, rank: int) -> None:
        super().__init__()
        self.H, self.D, self.V, self.tau, self.eps = m["heads"], m["dim"], m["vdim"], float(m["tau"]), eps
        Hh, D, V = self.H, self.D, self.V
        self.q, self.k, self.v, self.g = _param(Hh * D, width), _param(Hh * D, width), _param(Hh * V, width), _param(Hh * V, width)
        self.o, self.norm = _param(width, Hh * V), _param(V)
        self.a1, self.a2, self.a2_b = _param(rank, width), _param(Hh * D, rank), _param(Hh * D)

    def finalize(self) -> None:
        self.fuse(("q", "k", "v", "g", "a1"))

    def forward(self, h: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        p = H.linear(h, self.w_in)
        z = H.linear(self.col(p, "a1"), self.a2)
        y = H.gated_recurrence(self.col(p, "q"), self.col(p, "k"), self.col(p, "v"), z, self.col(p, "g"), self.norm,
                               st["state"], plan, heads=self.H, kv_heads=self.H, dim=self.D, vdim=self.V, mode="gla",
                               eps=self.eps, zb=self.a2_b, tau=self.tau)
        return H.linear(y, self.o)


class ChannelDelta(nn.Module, _Fused):
    tensor_names = {"q": "q", "q.conv": "q_conv", "k": "k", "k.conv": "k_conv", "v": "v", "v.conv": "v_conv", "b": "b",
                    "A_log": "A_log", "norm": "norm", "a1": "a1", "a2": "a2", "dt_bias": "dt_bias", "g1": "g1", "g2": "g2",
                    "o": "o"}

    def __init__(self, width: int, m: Dict[str, Any], eps: float, rank_a: int, rank_g: int) -> None:
        super().__init__()
        self.H, self.G, self.D, self.V, self.taps, self.eps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], eps
        if self.H % self.G:
            raise ValueError("heads must be a multiple of kv_heads")
        Hh, G, D, V, taps = self.H, self.G, self.D, self.V, self.taps
        self.q, self.k, self.v = _param(G * D, width), _param(G * D, width), _param(Hh * V, width)
        self.q_conv, self.k_conv, self.v_conv = _param(G * D, taps), _param(G * D, taps), _param(Hh * V, taps)
        self.b, self.A_log, self.norm = _param(Hh, width), _param(Hh), _param(V)
        self.a1, self.a2, self.dt_bias = _param(rank_a, width), _param(Hh * D, rank_a), _param(Hh * D)
        self.g1, self.g2, self.o = _param(rank_g, width), _param(Hh * V, rank_g), _param(width, Hh * V)

    def finalize(self) -> None:
        self.fuse(("q", "k", "v", "b", "a1", "g1"))
        self.conv_w = torch.cat((self.q_conv.data, self.k_conv.data, self.v_conv.data), 0).contiguous()

    def forward(self, h: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        GD, HV = self.G * self.D, self.H * self.V
        p = H.linear(h, self.w_in)
        if self.taps > 1:
            c = H.conv_silu(p[:, :2 * GD + HV], self.conv_w, st["conv"], plan)
        else:
            c = H.conv_silu(p[:, :2 * GD + HV], self.conv_w, p.new_zeros(1, 0, 2 * GD + HV), plan)
        z = H.linear(self.col(p, "a1"), self.a2)
        gate = H.linear(self.col(p, "g1"), self.g2)
        y = H.gated_recurrence(c[:, :GD], c[:, GD:2 * GD], c[:, 2 * GD:], z, gate, self.norm, st["state"], plan,
                               heads=self.H, kv_heads=self.G, dim=self.D, vdim=self.V, mode="delta", eps=self.eps,
                               zb=self.dt_bias, beta=self.col(p, "b"), a_log=self.A_log)
        return H.linear(y, self.o)


class WindowAttention(nn.Module, _Fused):
    """Grouped-query attention over cached keys and values of the slot, in the variants an architecture picks
    (``traits``, see ``models/config.py``): the mask is a sliding window of ``mask.size`` positions or the query's own
    block of ``mask.size`` positions (no mask entry: every earlier position); q and k are divided by their RMS after an
    optional rotation, with or without a learned weight per entry; q, k, v may have biases; the softmax may carry a
    zero-score sink; the output gate is one sigmoid per head or per channel.  A layer whose mixer entry says
    ``v_mix`` blends its values with those the first such layer computed for the same token,
    ``v <- (1 - lam) v + lam v_first`` (``lam`` the layer's ``vmix`` scalar; the first such layer keeps its own), and
    caches the blend.

    Further variants: ``qk_norm="full"`` norms the whole q projection (all heads at once) and the whole k projection
    with a weight per entry BEFORE the rotation; ``sink="learned"`` gives the sink a score per head (tensor ``sink``);
    a mixer entry may name ``softcap`` (scores become ``cap tanh(score / cap)`` after the scale) and ``kv_from``: the
    layer then has no key/value projections, prepares only its queries and reads the cache of the layer it names."""

    expand_from = 64   # a step whose every sequence brings at least this many tokens runs as batched matrix products
    query_block = 1024  # query rows per band
    score_bytes = 1 << 28  # fp32 scores alive at a time in the chunked prompt form

    def __init__(self, width: int, m: Dict[str, Any], eps: float, traits: Optional[Dict[str, Any]] = None) -> None:
        super().__init__()
        t = {"mask": "window", "sink": False, "qk_norm": "unit", "bias": False, "gate": "head", "p32": False, **(traits or {})}
        self.H, self.G, self.D, self.V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        self.scale, self.eps = float(m["scale"]), eps
        self.window = int((m.get("mask") or {}).get("size", 0) or 0)
        self.mask_kind, self.sink, self.p32 = str(t["mask"]), bool(t["sink"]), bool(t["p32"])
        self.v_mix = bool(m.get("v_mix"))
        self.softcap = float(m.get("softcap") or 0.0)
        self.borrows = m.get("kv_from") is not None
        self.full_norm = t["qk_norm"] == "full"
        if self.borrows and (self.v_mix or not self.full_norm):
            raise ValueError("kv_from is implemented for the full-projection q/k norm, without value mixing")
        rot = m.get("rot") or {}
        self.nrot, self.rot_base, self.rot_scaling = int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), rot.get("scaling")
        if self.nrot > self.D or self.nrot % 2:
            raise ValueError("rot.dims must be even and at most dim")
        Hh, G, D, V = self.H, self.G, self.D, self.V
        self.q = _param(Hh * D, width)
        self.g, self.o = _param(Hh if t["gate"] == "head" else Hh * V, width), _param(width, Hh * V)
        self.tensor_names = {"q": "q", "g": "g", "o": "o"}
        self.has_bias = bool(t["bias"])
        if self.has_bias:
            self.q_b = _param(Hh * D)
            self.tensor_names["q.b"] = "q_b"
        self.q_norm = self.k_norm = None
        if t["qk_norm"] in ("weight", "full"):
            self.q_norm = _param(Hh * D if self.full_norm else D)
            self.tensor_names["q.norm"] = "q_norm"
        if not self.borrows:
            self.k, self.v = _param(G * D, width), _param(G * V, width)
            self.tensor_names.update({"k": "k", "v": "v"})
            if self.has_bias:
                self.k_b, self.v_b = _param(G * D), _param(G * V)
                self.tensor_names.update({"k.b": "k_b", "v.b": "v_b"})
            if self.q_norm is not None:
                self.k_norm = _param(G * D if self.full_norm else D)
                self.tensor_names["k.norm"] = "k_norm"
        self.sink_w = None
        if t["sink"] == "learned":
            self.sink_w = _param(Hh)
            self.tensor_names["sink"] = "sink_w"
        self.sink32: Optional[torch.Tensor] = None
        if self.v_mix:
            self.vmix = nn.Parameter(torch.empty(()), requires_grad=False)
            self.tensor_names["vmix"] = "vmix"
        self.inv_freq: Optional[torch.Tensor] = None
        self.b_in: Optional[torch.Tensor] = None

    def finalize(self) -> None:
        self.fuse(("q", "g") if self.borrows else ("q", "k", "v", "g"))
        if self.has_bias:  # one bias vector for the fused projection; the gate has none
            kv = () if self.borrows else (self.k_b.data, self.v_b.data)
            self.b_in = torch.cat((self.q_b.data, *kv, torch.zeros_like(self.g.data[:, 0]))).contiguous()
        if self.sink_w is not None:
            self.sink32 = self.sink_w.data.float().contiguous()
        if self.v_mix:
            self.lam = self.vmix.data.reshape(1).contiguous()
        if self.nrot:
            self.inv_freq = H.scaled_inv_freq(self.nrot, self.rot_base, self.rot_scaling, self.q.device)

    def forward(self, h: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor],
                p: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``p``: the fused input projection of ``h`` when the caller has already computed it."""
        if p is None:
            p = H.linear(h, self.w_in, self.b_in)
        q, g = self.col(p, "q"), self.col(p, "g")
        if self.full_norm:
            k, v = (None, None) if self.borrows else (self.col(p, "k"), self.col(p, "v"))
            H.full_norm_append(q, k, v, self.inv_freq, st["cache"], plan, self.H, self.G, self.D, self.V, self.nrot,
                               self.eps, self.q_norm, self.k_norm)
            return self._attend(q, g, st["cache"], plan)
        v = self.col(p, "v")
        v_first = lam = None
        if self.v_mix:
            v_first = plan.shared.get("v_first")
            if v_first is None:
                plan.shared["v_first"] = v  # the first value-mixing layer of the step: later ones blend with these
            elif v_first.size(1) != v.size(1):
                raise ValueError("value-mixing layers must agree on kv_heads * vdim")
            else:
                lam = self.lam
        H.window_append(q, self.col(p, "k"), v, self.inv_freq, st["cache"], plan, self.H, self.G, self.D,
                        self.V, self.nrot, self.eps, self.q_norm, self.k_norm, v_first, lam)
        return self._attend(q, g, st["cache"], plan)

    def _attend(self, q: torch.Tensor, g: torch.Tensor, cache: torch.Tensor, plan: H.BatchPlan) -> torch.Tensor:
        """Prepared queries against the cache rows of each token's slot, gated and projected."""
        if min(n for _, n, _, _ in plan.seqs) >= self.expand_from:
            o = self._chunked(q, cache, plan) if self.mask_kind == "chunk" and self.window > 0 else self._banded(q, cache, plan)
            o = H.head_gate(o, g) if g.size(1) == self.H else H.headmajor_gate(o, g)
        else:
            o = H.window_attn(q, g, cache, plan, self.H, self.G, self.D, self.V, self.scale, self.window,
                              mask=self.mask_kind, sink=self.sink, cap=self.softcap, sink_vals=self.sink32)
        return H.linear(o, self.o)

    def _band(self, out: torch.Tensor, q: torch.Tensor, cache: torch.Tensor, slot: int, r0: int, p0: int, a: int, b: int,
              key0: int, window: int) -> None:
        """Rows ``a..b-1`` of the sequence at ``r0`` against the keys ``key0 .. p0+b-1`` of its slot: scores and the
        weighted sum as batched matrix products over the key/value heads (the group's query heads stacked as rows),
        the masked softmax on fp32 scores in between."""
        Hh, G, D, V = self.H, self.G, self.D, self.V
        rep, nb = Hh // G, b - a
        rows = cache[slot, key0:p0 + b]
        keys = rows.size(0)
        kt = rows[:, :G * D].view(keys, G, D).permute(1, 2, 0)   # [G, D, keys]
        vv = rows[:, G * D:].view(keys, G, V).transpose(0, 1)     # [G, keys, V]
        qh = q[r0 + a:r0 + b].view(nb, G, rep, D).permute(1, 2, 0, 3).reshape(G, rep * nb, D)
        s = H.matmul_f32(qh, kt).contiguous()
        if self.p32 and q.dtype != torch.float32:  # weights as two 16-bit halves: the sum stays on the tensor cores
            pr = H.causal_softmax(s.view(Hh, nb, keys), p0 + a, self.scale, q.dtype, window=window, key0=key0, sink=self.sink,
                                  split=True, cap=self.softcap, sink_vals=self.sink32)
            out[:, r0 + a:r0 + b] = H.matmul_f32(pr.view(G, rep * nb, 2 * keys), torch.cat((vv, vv), 1)).view(Hh, nb, V)
            return
        pdt = torch.float32 if self.p32 else q.dtype
        pr = H.causal_softmax(s.view(Hh, nb, keys), p0 + a, self.scale, pdt, window=window, key0=key0, sink=self.sink,
                              cap=self.softcap, sink_vals=self.sink32)
        out[:, r0 + a:r0 + b] = torch.bmm(pr.view(G, rep * nb, keys), vv.to(pdt)).view(Hh, nb, V)

    def _banded(self, q: torch.Tensor, cache: torch.Tensor, plan: H.BatchPlan) -> torch.Tensor:
        """Prompt form of the sliding window: per block of query rows, the band of keys the block can see.
        Returns ``[heads, N, vdim]``."""
        W = self.window
        out = torch.empty(self.H, q.size(0), self.V, device=q.device, dtype=q.dtype)
        for r0, n, slot, p0 in plan.seqs:
            for a in range(0, n, self.query_block):
                b = min(n, a + self.query_block)
                self._band(out, q, cache, slot, r0, p0, a, b, max(0, p0 + a - W + 1) if W > 0 else 0, W)
        return out

    def _chunked(self, q: torch.Tensor, cache: torch.Tensor, plan: H.BatchPlan) -> torch.Tensor:
        """Prompt form of the chunk mask.  Blocks of ``window`` positions are independent of one another, so the whole
        blocks a step brings are ONE pair of batched matrix products with (block, key/value head) as the batch and a
        ``window x window`` causal softmax per block; a step that starts inside a block, or ends inside one, runs
        that partial block as a band against the block's keys in the cache.  Returns ``[heads, N, vdim]``."""
        Hh, G, D, V, W = self.H, self.G, self.D, self.V, self.window
        rep = Hh // G
        out = torch.empty(Hh, q.size(0), V, device=q.device, dtype=q.dtype)
        pdt = torch.float32 if self.p32 else q.dtype
        split = self.p32 and q.dtype != torch.float32
        per = max(1, self.score_bytes // (Hh * W * W * 4))
        for r0, n, slot, p0 in plan.seqs:
            head = min(n, (-p0) % W)  # tokens that complete a block begun in an earlier step
            for a in range(0, head, self.query_block):
                self._band(out, q, cache, slot, r0, p0, a, min(head, a + self.query_block), (p0 // W) * W, 0)
            full = (n - head) // W
            for c0 in range(0, full, per):
                nc = min(per, full - c0)
                a = head + c0 * W
                rows = cache[slot, p0 + a:p0 + a + nc * W]
                kt = rows[:, :G * D].reshape(nc, W, G, D).permute(0, 2, 3, 1).reshape(nc * G, D, W)
                vv = rows[:, G * D:].reshape(nc, W, G, V).permute(0, 2, 1, 3).reshape(nc * G, W, V)
                qh = q[r0 + a:r0 + a + nc * W].reshape(nc, W, G, rep, D).permute(0, 2, 3, 1, 4).reshape(nc * G, rep * W, D)
                s = H.matmul_f32(qh, kt).contiguous()
                if split:
                    pr = H.causal_softmax(s.view(nc * Hh, W, W), 0, self.scale, q.dtype, sink=self.sink, split=True,
                                          cap=self.softcap, sink_vals=self.sink32)
                    o = H.matmul_f32(pr.view(nc * G, rep * W, 2 * W), torch.cat((vv, vv), 1))
                else:
                    pr = H.causal_softmax(s.view(nc * Hh, W, W), 0, self.scale, pdt, sink=self.sink, cap=self.softcap,
                                          sink_vals=self.sink32)
                    o = torch.bmm(pr.view(nc * G, rep * W, W), vv.to(pdt))  # [nc*G, rep*W, V]
                out[:, r0 + a:r0 + a + nc * W] = o.view(nc, G, rep, W, V).permute(1, 2, 0, 3, 4).reshape(Hh, nc * W, V)
            tail = head + full * W
            for a in range(tail, n, self.query_block):
                self._band(out, q, cache, slot, r0, p0, a, min(n, a + self.query_block), p0 + tail, 0)
        return out


class GatedFF(nn.Module, _Fused):
    """``down (act(gate h) * (up h))`` without biases; gate and up are one matrix product.  ``act="clamped"`` is the
    clamped product of :func:`mdi_llm_b200.ops.hybrid.glu` with ``limit``.  ``token_gate``: a projection ``sg [1, width]``
    gives one logit per token whose sigmoid weighs the output; it rides in the same matrix product as gate and up (its
    row, padded with zero rows to a multiple of 8 so the rows stay 16-byte aligned) and :meth:`gated` returns it."""

    def __init__(self, width: int, ff: int, act: str = "silu", limit: float = 0.0, token_gate: bool = False) -> None:
        super().__init__()
        self.act, self.limit, self.ff = act, float(limit), int(ff)
        self.gate, self.up, self.down = _param(ff, width), _param(ff, width), _param(width, ff)
        self.tensor_names = {"gate": "gate", "up": "up", "down": "down"}
        self.sg = None
        if token_gate:
            self.sg = _param(1, width)
            self.tensor_names["sg"] = "sg"

    def finalize(self) -> None:
        if self.sg is None:
            self.fuse(("gate", "up"))
            return
        self._pad = nn.Parameter(torch.zeros((-(2 * self.ff + 1)) % 8, self.sg.size(1), device=self.sg.device, dtype=self.sg.dtype),
                                 requires_grad=False)
        self.fuse(("gate", "up", "sg", "_pad"))

    def forward(self, h: torch.Tensor, gu: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``gu``: the gate and up projections of ``h`` side by side when the caller has already computed them."""
        return H.linear(H.act_mul(H.linear(h, self.w_in) if gu is None else gu, self.act, self.limit), self.down)

    def gated(self, h: torch.Tensor) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """(output before the token gate, the gate's logit per token ``[N, 1]`` or None)."""
        p = H.linear(h, self.w_in)
        if self.sg is None:
            return self.forward(h, p), None
        return self.forward(h, p[:, :2 * self.ff]), self.col(p, "sg")


class MoEFF(nn.Module):
    """A mixture of experts: fp32 router logits (optionally with a bias), the ``top`` largest per token, and

    * ``expert="relu2"``, ``router="sigmoid"``: ``sum_e down_e relu(up_e (s_e h))^2`` with ``s = sigmoid(logit)`` — the
      score scales the expert's *input*;
    * ``expert="gated_silu"``, ``router="softmax"``: ``sum_e s_e down_e (silu(gate_e h) * (up_e h))`` with ``s`` the
      softmax restricted to the selected logits — the score weighs the expert's *output*.

    * ``expert="clamped"``, ``router="softmax_all"``: scores are the softmax over all router outputs, the choice goes by
      score + ``correction``, the weights are the chosen scores over their sum; experts are the clamped gated product
      with ``limit``; the last ``identity`` router outputs have no tensors and return ``h`` itself.

    ``shared`` (a :class:`GatedFF`, optional) is an expert every token uses; the block adds its output.  The expert
    weights are stacked at load (``up [E, ff, C]``, or ``[E, 2 ff, C]`` with an expert's gate rows before its up rows;
    ``down [E, C, ff]``); the per-expert parameters the checkpoint names become views.  Few tokens (decoding) run two
    index-driven weight-streaming kernels; many tokens are sorted by expert and run as two grouped matrix products
    (bf16: one vendor call each, group sizes stay on the device; fp32: one product per expert that received any)."""

    gemv_max = 64  # token-expert pairs up to which the index-driven kernels are used

    def __init__(self, width: int, ff: int, experts: int, top: int, router: str = "sigmoid", router_bias: bool = False,
                 expert: str = "relu2", shared_ff: int = 0, identity: int = 0, limit: float = 0.0, shared_limit: float = 0.0,
                 shared_gate: bool = False) -> None:
        super().__init__()
        self.E, self.top, self.ff, self.identity = int(experts), int(top), int(ff), int(identity)
        self.mode, self.gated = router, expert in ("gated_silu", "clamped")
        self.act, self.limit = ("clamped" if expert == "clamped" else "silu"), float(limit)
        if self.identity and not self.gated:
            raise ValueError("identity experts are implemented for gated experts (the routing weight scales the output)")
        self.router = _param(self.E + self.identity, width)
        self.router_b = _param(self.E + self.identity) if router_bias else None
        self.correction = _param(self.E + self.identity) if router == "softmax_all" else None
        self.e_up = nn.ParameterList([_param(ff, width) for _ in range(self.E)])
        self.e_down = nn.ParameterList([_param(width, ff) for _ in range(self.E)])
        self.e_gate = nn.ParameterList([_param(ff, width) for _ in range(self.E)]) if self.gated else None
        self.shared = GatedFF(width, int(shared_ff), self.act, shared_limit, shared_gate) if shared_ff else None

    def names(self) -> Dict[str, nn.Parameter]:
        out = {"router": self.router}
        if self.correction is not None:
            out["correction"] = self.correction
        if self.router_b is not None:
            out["router.b"] = self.router_b
        for j in range(self.E):
            out[f"e{j}.up"], out[f"e{j}.down"] = self.e_up[j], self.e_down[j]
            if self.gated:
                out[f"e{j}.gate"] = self.e_gate[j]
        if self.shared is not None:
            for short, attr in self.shared.tensor_names.items():
                out[f"shared.{short}"] = getattr(self.shared, attr)
        return out

    def finalize(self) -> None:
        ff = self.ff
        if self.gated:
            self.up = torch.stack([torch.cat((g.data, u.data), 0) for g, u in zip(self.e_gate, self.e_up)]).contiguous()
        else:
            self.up = torch.stack([p.data for p in self.e_up]).contiguous()
        self.down = torch.stack([p.data for p in self.e_down]).contiguous()
        for j in range(self.E):
            self.e_down[j].data = self.down[j]
            if self.gated:
                self.e_gate[j].data, self.e_up[j].data = self.up[j, :ff], self.up[j, ff:]
            else:
                self.e_up[j].data = self.up[j]
        self.router32 = self.router.data.float().contiguous()
        self.router_b32 = None if self.router_b is None else self.router_b.data.float().contiguous()
        self.correction32 = None if self.correction is None else self.correction.data.float().contiguous()
        self.expert_ids = torch.arange(self.E, device=self.router.device)
        if self.shared is not None:
            self.shared.finalize()

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        N, top = h.size(0), self.top
        idx, wt = H.router_topk(H.linear_f32(h, self.router32, self.router_b32), top, self.mode, self.correction32)
        capturing = h.is_cuda and torch.cuda.is_current_stream_capturing()
        if N * top <= self.gemv_max or capturing:
            return H.moe_gemv(h, idx, wt, self.up, self.down, self.gated, self.act, self.limit)
        flat = idx.view(-1).long()
        order = torch.argsort(flat, stable=True)
        counts = (flat[:, None] == self.expert_ids[None, :]).sum(0)  # stays on the device
        rows = (order // top).to(torch.int32)
        where = torch.empty_like(order)
        where[order] = torch.arange(order.numel(), device=order.device)
        if self.gated:  # rows of identity experts sort behind the last group: no product touches them
            mid = H.act_mul(H.grouped_linear(H.gather_scale_rows(h, rows), self.up, counts), self.act, self.limit)
            ident = (idx, self.E, h) if self.identity else ()
            return H.combine_rows(H.grouped_linear(mid, self.down, counts), where.to(torch.int32), N, top, wt, *ident)
        xin = H.gather_scale_rows(h, rows, wt.view(-1)[order].contiguous())
        y = H.grouped_linear(H.relu2_(H.grouped_linear(xin, self.up, counts)), self.down, counts)
        return H.combine_rows(y, where.to(torch.int32), N, top)


class DenseFF(nn.Module):
    tensor_names = {"up": "up", "down": "down"}

    def __init__(self, width: int, ff: int, act: str = "gelu") -> None:
        super().__init__()
        self.act = act
        self.up, self.down = _param(ff, width), _param(width, ff)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        a = H.linear(h, self.up)
        return H.linear(H.relu2_(a) if self.act == "relu2" else H.gelu_(a), self.down)


class _LN(nn.Module):
    def __init__(self, width: int) -> None:
        super().__init__()
        self.w, self.b = _param(width), _param(width)


class SandwichBlock(nn.Module):
    """``x += norm1b(mixer(norm1(x)))``, then ``x += norm2b(ff(norm2(x)))`` when the layer has a feed-forward."""

    def __init__(self, width: int, mixer: nn.Module, ff: Optional[nn.Module], eps: float) -> None:
        super().__init__()
        self.mix, self.mlp, self.eps = mixer, ff, eps
        self.norm1, self.norm1b = _LN(width), _LN(width)
        if ff is not None:
            self.norm2, self.norm2b = _LN(width), _LN(width)

    side = None

    def norm_names(self) -> List[str]:
        return ["norm1", "norm1b"] + (["norm2", "norm2b"] if self.mlp is not None else [])

    def forward(self, x: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor], dtype: torch.dtype,
                tokens: Optional[torch.Tensor] = None, side_table: Optional[torch.Tensor] = None) -> None:
        h = H.norm_rows(x, self.norm1.w, self.norm1.b, self.eps, "layer", dtype)
        H.norm_accumulate(x, self.mix(h, plan, st), self.norm1b.w, self.norm1b.b, self.eps)
        if self.mlp is not None:
            h = H.norm_rows(x, self.norm2.w, self.norm2.b, self.eps, "layer", dtype)
            H.norm_accumulate(x, self.mlp(h), self.norm2b.w, self.norm2b.b, self.eps)


class _RMS(nn.Module):
    def __init__(self, width: int) -> None:
        super().__init__()
        self.w, self.b = _param(width), None


class TokenSide(nn.Module):
    """A per-layer embedding of the current token, gated by the residual stream: ``y = proj (gelu_tanh(gate x) * e)``
    with ``e`` this layer's slice of the shared side table; ``x += m * rms_norm(y) * norm``."""

    def __init__(self, width: int, dim: int, col0: int) -> None:
        super().__init__()
        self.dim, self.col0 = dim, col0
        self.gate, self.proj, self.norm = _param(dim, width), _param(width, dim), _param(width)

    def forward(self, x: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, eps: float, m: float, dtype: torch.dtype) -> None:
        xa = x if dtype == torch.float32 else torch.empty(x.shape, device=x.device, dtype=dtype)
        if xa is not x:
            H.cast_into(x, xa)
        g = H.token_side_gate(H.linear(xa, self.gate), table, tokens, self.col0)
        H.norm_accumulate(x, H.linear(g, self.proj), self.norm, None, eps, "rms", m)


class PreNormBlock(nn.Module):
    """``x += m * mixer(norm1(x))``, ``x += m * ff(norm2(x))`` when the layer has a feed-forward, then the gated
    per-layer token embedding when the model has one.  ``norm`` picks layer norm (weight and bias) or RMS norm."""

    def __init__(self, width: int, mixer: nn.Module, ff: Optional[nn.Module], eps: float, norm: str, mult: float,
                 side: Optional[TokenSide]) -> None:
        super().__init__()
        self.mix, self.mlp, self.eps, self.kind, self.mult, self.side = mixer, ff, eps, norm, float(mult), side
        mk = _LN if norm == "layer" else _RMS
        self.norm1 = mk(width)
        if ff is not None:
            self.norm2 = mk(width)

    def norm_names(self) -> List[str]:
        return ["norm1"] + (["norm2"] if self.mlp is not None else [])

    def forward(self, x: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor], dtype: torch.dtype,
                tokens: torch.Tensor, side_table: Optional[torch.Tensor]) -> None:
        h = H.norm_rows(x, self.norm1.w, self.norm1.b, self.eps, self.kind, dtype)
        H.norm_accumulate(x, self.mix(h, plan, st), None, None, self.eps, "none", self.mult)
        if self.mlp is not None:
            h = H.norm_rows(x, self.norm2.w, self.norm2.b, self.eps, self.kind, dtype)
            H.norm_accumulate(x, self.mlp(h), None, None, self.eps, "none", self.mult)
        if self.side is not None:
            self.side(x, tokens, side_table, self.eps, self.mult, dtype)


class LightningAttention(nn.Module, _Fused):
    """Linear attention with one fixed decay per head: ``q, k, v = silu(W h)``, ``S_t = decay_h S_(t-1) + k_t v_t^T``
    (fp32, one ``[dim, vdim]`` matrix per head and slot, zero for a fresh slot), ``o_t = S_t^T q_t`` without a scale; the
    heads' read-outs, side by side, get ONE RMS norm with the weight ``norm [heads * vdim]``, are multiplied by
    ``sigmoid(W_g h)`` and projected by ``W_o``.  q, k, v and the gate are one matrix product; the SiLU of q, k, v is
    taken inside the recurrence kernels, where they are read."""

    tensor_names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm"}

    def __init__(self, width: int, m: Dict[str, Any], eps: float) -> None:
        super().__init__()
        self.H, self.D, self.V, self.eps = int(m["heads"]), int(m["dim"]), int(m["vdim"]), eps
        self.decay_values = [float(x) for x in m["decay"]]
        Hh, D, V = self.H, self.D, self.V
        self.q, self.k, self.v, self.g = _param(Hh * D, width), _param(Hh * D, width), _param(Hh * V, width), _param(Hh * V, width)
        self.o, self.norm = _param(width, Hh * V), _param(Hh * V)

    def finalize(self) -> None:
        self.fuse(("q", "k", "v", "g"))
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.q.device)

    def forward(self, h: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor]) -> torch.Tensor:
        HD, HV = self.H * self.D, self.H * self.V
        p = H.linear(h, self.w_in)
        o = H.lightning_recurrence(self.col(p, "q"), self.col(p, "k"), self.col(p, "v"), self.decay, st["state"], plan,
                                   self.H, self.D, self.V, act=True)
        return H.linear(H.norm_gate_rows(o, self.norm, self.col(p, "g"), self.eps, h.dtype), self.o)


class PostNormBlock(nn.Module):
    """``x += norm1(mixer(x))``, then ``x += norm2(ff(x))`` when the layer has a feed-forward: the sublayers read the
    residual stream itself (rounded to the activation type), only their outputs are normed.  A mixture of experts with
    a shared expert adds ``sigmoid(sg) * shared(x)`` to the routed sum inside the same norm.  With 16-bit activations
    the kernel that adds a sublayer's normed output to the residual also writes the rounded copy the next sublayer
    reads (handed from block to block through the step's scratch), so the stream is not read again for a cast."""

    side = None

    def __init__(self, width: int, mixer: nn.Module, ff: Optional[nn.Module], eps: float, norm: str) -> None:
        super().__init__()
        self.mix, self.mlp, self.eps, self.kind = mixer, ff, eps, norm
        if norm != "rms":
            raise ValueError("post-norm blocks are implemented with RMS norms")
        self.norm1 = _RMS(width)
        if ff is not None:
            self.norm2 = _RMS(width)

    def norm_names(self) -> List[str]:
        return ["norm1"] + (["norm2"] if self.mlp is not None else [])

    @staticmethod
    def _read(x: torch.Tensor, dtype: torch.dtype, plan: Optional[H.BatchPlan] = None) -> torch.Tensor:
        """The stream as a sublayer reads it: itself in fp32, else the rounded copy the last update left, else a cast."""
        if dtype == torch.float32:
            return x
        h = plan.shared.pop("stream_copy", None) if plan is not None else None
        if h is None:
            h = torch.empty(x.shape, device=x.device, dtype=dtype)
            H.cast_into(x, h)
        return h

    def forward(self, x: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor], dtype: torch.dtype,
                tokens: Optional[torch.Tensor] = None, side_table: Optional[torch.Tensor] = None) -> None:
        h = self._read(x, dtype, plan)
        nxt = None if dtype == torch.float32 else torch.empty(x.shape, device=x.device, dtype=dtype)
        H.norm_accumulate(x, self.mix(h, plan, st), self.norm1.w, None, self.eps, self.kind, copy=nxt)
        if nxt is not None:
            plan.shared["stream_copy"] = nxt
        if self.mlp is None:
            return
        h = self._read(x, dtype, plan)
        nxt = None if dtype == torch.float32 else torch.empty(x.shape, device=x.device, dtype=dtype)
        y = self.mlp(h)
        shared = getattr(self.mlp, "shared", None)
        if shared is None:
            H.norm_accumulate(x, y, self.norm2.w, None, self.eps, self.kind, copy=nxt)
        else:
            y2, sg = shared.gated(h)
            H.gated_sum_norm_accumulate(x, y, y2, sg, self.norm2.w, self.eps, self.kind, copy=nxt)
        if nxt is not None:
            plan.shared["stream_copy"] = nxt


class ParallelBlock(nn.Module):
    """``x += ls1 * mixer(h) + ls2 * (ff(h) + shared(h))`` with ``h = norm1(x)``: one norm, read by both branches,
    each branch with a learned scale per channel when the architecture has them.  ``norm_offset`` is added to the
    norm weight (1: the weight is stored as its deviation from one)."""

    side = None

    def __init__(self, width: int, mixer: nn.Module, ff: Optional[nn.Module], eps: float, norm: str, norm_offset: float,
                 layer_scale: bool) -> None:
        super().__init__()
        self.mix, self.mlp, self.eps, self.kind, self.offset = mixer, ff, eps, norm, float(norm_offset)
        self.norm1 = _LN(width) if norm == "layer" else _RMS(width)
        self.ls1 = _param(width) if layer_scale else None
        self.ls2 = _param(width) if layer_scale and ff is not None else None
        self.w_all: Optional[torch.Tensor] = None
        self.b_all: Optional[torch.Tensor] = None
        self.n_mix = 0

    def norm_names(self) -> List[str]:
        return ["norm1"]

    def extra_tensors(self) -> Dict[str, nn.Parameter]:
        return {k: p for k, p in (("ls1", self.ls1), ("ls2", self.ls2)) if p is not None}

    def forward(self, x: torch.Tensor, plan: H.BatchPlan, st: Dict[str, torch.Tensor], dtype: torch.dtype,
                tokens: Optional[torch.Tensor] = None, side_table: Optional[torch.Tensor] = None) -> None:
        h = H.norm_rows(x, self.norm1.w, self.norm1.b, self.eps, self.kind, dtype, self.offset)
        shared = getattr(self.mlp, "shared", None)
        b = b2 = None
        if self.w_all is not None:
            pa = H.linear(h, self.w_all, self.b_all)
            a = self.mix(h, plan, st, pa[:, :self.n_mix])
            b2 = shared(h, pa[:, self.n_mix:])
        else:
            a = self.mix(h, plan, st)
            if shared is not None:
                b2 = shared(h)
        if self.mlp is not None:
            b = self.mlp(h)
        H.scaled_branches(x, a, self.ls1, b, b2, self.ls2)

    def finalize(self) -> None:
        """Both branches read the same normed rows: the mixer's fused input projection and the shared expert's gate
        and up projections become ONE matrix product (every output column is the same dot product as before).  The
        two fused weights turn into row ranges of one matrix; nothing is stored twice."""
        shared = getattr(self.mlp, "shared", None)
        if shared is None or not isinstance(self.mix, WindowAttention):
            return
        self.n_mix = self.mix.w_in.size(0)
        self.w_all = torch.cat((self.mix.w_in, shared.w_in), 0).contiguous()
        self.mix.rebase(self.w_all[:self.n_mix])
        shared.rebase(self.w_all[self.n_mix:])
        if self.mix.b_in is not None:
            self.b_all = torch.cat((self.mix.b_in, torch.zeros_like(shared.w_in[:, 0]))).contiguous()


def _rank_of(tensors: Optional[Dict[str, torch.Tensor]], key: str, default: int) -> int:
    return int(tensors[key].shape[0]) if tensors is not None and key in tensors else default


class HybridLM(nn.Module):
    """Embedding -> layer runs (with an optional looped span) -> final norm -> tied head -> soft cap.

    ``forward`` runs ONE step of a packed batch against a :class:`StatePool`; it is the step function for prompts
    and decoding alike.  Low-rank side projections (decay and gate bottlenecks) take their rank from the
    checkpoint's tensor shapes (``ranks``), since the configuration does not name them.
    """

    def __init__(self, config: HybridConfig, ranks: Optional[Dict[str, int]] = None) -> None:
        super().__init__()
        self.config = config
        ranks = ranks or {}
        C, eps = config.width, config.norm_eps
        self.embed = _param(config.vocab, C)
        self.pos = _param(config.max_positions, C) if config.positions == "learned" else None
        self.loop_in = _param(C, 2 * C) if config.loop is not None else None
        blocks = []
        for i, spec in enumerate(config.layers):
            m, kind = spec["mixer"], spec["type"]
            if kind == "latent_attention":
                mixer: nn.Module = LatentAttention(C, m, eps)
            elif kind == "attention":
                mixer = WindowAttention(C, m, eps, config.attention)
            elif kind == "lightning":
                mixer = LightningAttention(C, m, eps)
            elif kind == "gla":
                mixer = GatedLinearAttention(C, m, eps, ranks.get(f"l{i}.mix.a1", 16))
            else:
                mixer = ChannelDelta(C, m, eps, ranks.get(f"l{i}.mix.a1", 16), ranks.get(f"l{i}.mix.g1", 16))
            mlp = spec.get("mlp")
            if not mlp:
                ff: Optional[nn.Module] = None
            elif mlp["kind"] == "moe":
                sh = mlp.get("shared") or {}
                ff = MoEFF(C, mlp["expert"]["ff"], mlp["router"]["experts"], mlp["router"]["top"], config.moe["router"],
                           config.moe["router_bias"], config.moe["expert"], int(sh.get("ff", 0)),
                           int(mlp["router"].get("identity", 0) or 0), float(mlp["expert"].get("limit", 0.0)),
                           float(sh.get("limit", 0.0)), bool(config.moe["shared_gate"]))
            else:
                ff = DenseFF(C, mlp["ff"], config.dense_act)
            if config.block == "sandwich":
                blocks.append(SandwichBlock(C, mixer, ff, eps))
            elif config.block == "parallel":
                blocks.append(ParallelBlock(C, mixer, ff, eps, config.norm, config.norm_offset, config.layer_scale))
            elif config.block == "postnorm":
                blocks.append(PostNormBlock(C, mixer, ff, eps, config.norm))
            else:
                sd = int(config.token_side["dim"]) if config.token_side else 0
                side = TokenSide(C, sd, i * sd) if sd else None
                blocks.append(PreNormBlock(C, mixer, ff, eps, config.norm, config.residual_mult, side))
        self.blocks = nn.ModuleList(blocks)
        self.final_norm = _LN(C) if config.norm == "layer" else _RMS(C)
        self.side_embed = _param(config.vocab, len(config.layers) * int(config.token_side["dim"])) if config.token_side else None
        self.head_w = None if config.tied_head else _param(config.vocab, C)
        self.runs = config.layer_runs()

    # ---- weights -------------------------------------------------------------------------------
    def tensor_map(self) -> Dict[str, nn.Parameter]:
        """Checkpoint tensor name -> parameter."""
        out: Dict[str, nn.Parameter] = {"embed": self.embed, "final.norm": self.final_norm.w}
        if self.final_norm.b is not None:
            out["final.norm.b"] = self.final_norm.b
        if self.loop_in is not None:
            out["loop.in"] = self.loop_in
        if self.pos is not None:
            out["pos"] = self.pos
        if self.side_embed is not None:
            out["side.embed"] = self.side_embed
        if self.head_w is not None:
            out["head"] = self.head_w
        for i, blk in enumerate(self.blocks):
            for n in blk.norm_names():
                out[f"l{i}.{n}"] = getattr(blk, n).w
                if getattr(blk, n).b is not None:
                    out[f"l{i}.{n}.b"] = getattr(blk, n).b
            for short, attr in blk.mix.tensor_names.items():
                out[f"l{i}.mix.{short}"] = getattr(blk.mix, attr)
            if hasattr(blk, "extra_tensors"):
                for short, prm in blk.extra_tensors().items():
                    out[f"l{i}.{short}"] = prm
            if isinstance(blk.mlp, MoEFF):
                for short, prm in blk.mlp.names().items():
                    out[f"l{i}.mlp.{short}"] = prm
            elif blk.mlp is not None:
                for short, attr in blk.mlp.tensor_names.items():
                    out[f"l{i}.mlp.{short}"] = getattr(blk.mlp, attr)
            if blk.side is not None:
                out[f"l{i}.side.gate"], out[f"l{i}.side.proj"], out[f"l{i}.side.norm"] = blk.side.gate, blk.side.proj, blk.side.norm
        return out

    def load_tensors(self, tensors: Dict[str, torch.Tensor], device: Union[str, torch.device], dtype: torch.dtype) -> "HybridLM":
        tm = self.tensor_map()
        # a checkpoint may carry tensors a layer has no use for (a mixing factor where nothing is mixed, the scale of
        # a feed-forward the layer does not have)
        unused = (".mix.vmix", ".ls2")
        missing = sorted(set(tm) - set(tensors))
        extra = sorted(n for n in set(tensors) - set(tm) if not n.endswith(unused))
        if missing or extra:
            raise KeyError(f"checkpoint does not match the configuration: missing {missing[:5]}, unexpected {extra[:5]}")
        for name, p in tm.items():
            t = tensors[name]
            if p.dim() == 0 and t.numel() == 1:  # a scalar may be stored with shape [] or [1]
                t = t.reshape(())
            if tuple(t.shape) != tuple(p.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != expected {tuple(p.shape)}")
            p.data = t.to(device=device, dtype=dtype).contiguous()
        return self.finalize()

    def init_random(self, device: Union[str, torch.device], dtype: torch.dtype, seed: int = 0, std: float = 0.02) -> "HybridLM":
        """Random weights (benchmarks and tests): projections N(0, std * sqrt(width / fan_in)), norm weights near 1."""
        gen = torch.Generator().manual_seed(seed)
        for name, p in self.tensor_map().items():
            if p.dim() == 2 and not name.endswith(".conv"):
                t = torch.randn(p.shape, generator=gen) * (p.shape[1] ** -0.5)
            elif name.endswith(".conv"):
                t = torch.randn(p.shape, generator=gen) * 0.5
            elif name.endswith(".b") and p.dim() == 1 and "norm" in name:
                t = torch.randn(p.shape, generator=gen) * 0.1
            elif "norm" in name and not name.endswith((".q.norm", ".k.norm")):
                t = (1.0 - self.config.norm_offset) + torch.randn(p.shape, generator=gen) * 0.1
            elif "norm" in name or name.endswith((".ls1", ".ls2")):
                t = 1.0 + torch.randn(p.shape, generator=gen) * 0.1
            elif name.endswith(".vmix"):
                t = torch.rand(p.shape, generator=gen) * 0.5 + 0.25
            elif name.endswith(".correction"):
                t = torch.randn(p.shape, generator=gen) * 0.05
            else:
                t = torch.randn(p.shape, generator=gen) * 0.5
            if name == "embed":
                t = torch.randn(p.shape, generator=gen)
            p.data = t.to(torch.bfloat16).to(device=device, dtype=dtype).contiguous()
        return self.finalize()

    def finalize(self) -> "HybridLM":
        for blk in self.blocks:
            blk.mix.finalize()
            if isinstance(blk.mlp, (MoEFF, GatedFF)):
                blk.mlp.finalize()
            if isinstance(blk, ParallelBlock):
                blk.finalize()
        self.dtype, self.device = self.embed.dtype, self.embed.device
        return self

    def state_tensors(self) -> Dict[str, torch.Tensor]:
        return {k: v.data for k, v in self.tensor_map().items()}

    def new_pool(self, n_slots: int, max_seq_length: int) -> StatePool:
        return StatePool(self.config, n_slots, max_seq_length, self.device, self.dtype)

    # ---- the step function ---------------------------------------------------------------------
    @torch.inference_mode()
    def hidden(self, tokens: torch.Tensor, plan: H.BatchPlan, pool: StatePool,
               trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """Residual stream ``[N, width]`` (fp32) after the last layer for packed int32 ``tokens [N]``."""
        C, dt = self.config.width, self.dtype
        for _, n, slot, p0 in plan.seqs:
            if p0 + n > pool.max_seq_length:
                raise ValueError(f"sequence of {p0 + n} tokens exceeds the pool's max_seq_length {pool.max_seq_length}")
            if self.pos is not None and p0 + n > self.pos.size(0):
                raise ValueError(f"sequence of {p0 + n} tokens exceeds the model's {self.pos.size(0)} learned positions")
        plan.shared.clear()
        x0 = H.embed_rows(self.embed, tokens, self.pos, plan, self.config.embed_scale)
        x = x0.clone() if self.loop_in is not None else x0
        for run, (li, first) in enumerate(self.runs):
            if first:
                plan.shared.pop("stream_copy", None)  # the stream is about to change outside a block
                cat = torch.empty(x.size(0), 2 * C, device=x.device, dtype=dt)
                H.cast_into(x, cat[:, :C])
                H.cast_into(x0, cat[:, C:])
                y = H.linear(cat, self.loop_in)
                if dt == torch.float32:
                    x = y
                else:
                    H.cast_into(y, x)
            self.blocks[li](x, plan, pool.runs[run], dt, tokens, self.side_embed)
            if trace is not None:
                trace.append(x.clone())
        return x

    @torch.inference_mode()
    def head(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 logits of residual rows ``x [n, width]``: final norm, output head (tied or its own), soft cap."""
        h = H.norm_rows(x, self.final_norm.w, self.final_norm.b, self.config.norm_eps, self.config.norm, self.dtype,
                        self.config.norm_offset)
        return H.softcap(H.linear(h, self.embed if self.head_w is None else self.head_w), self.config.logit_softcap)

    def forward(self, tokens: torch.Tensor, plan: H.BatchPlan, pool: StatePool, rows: Optional[Sequence[int]] = None,
                trace: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        x = self.hidden(tokens, plan, pool, trace)
        if rows is not None:
            x = x.index_select(0, torch.as_tensor(list(rows), device=x.device, dtype=torch.long))
        return self.head(x)


def load_hybrid(checkpoint_dir: Union[str, Path], device: Union[str, torch.device], dtype: torch.dtype) -> HybridLM:
    """Build the model a checkpoint folder describes (``config.json`` + ``model.safetensors``) through the registry."""
    from .registry import architecture_of, model_classes

    d = Path(checkpoint_dir)
    cfg_cls, model_cls = model_classes(architecture_of(d))
    cfg = cfg_cls.from_file(d / "config.json")
    tensors = read_safetensors(d / "model.safetensors")
    ranks = {k: int(v.shape[0]) for k, v in tensors.items() if k.endswith((".a1", ".g1"))}
    return model_cls(cfg, ranks).load_tensors(tensors, device, dtype)
