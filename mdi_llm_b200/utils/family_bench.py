"""Throughput of the hybrid family beside the closest transformer of the same size (``bench.py --family hybrid``).

For each width a 4-layer hybrid model (latent attention, gated delta rule, gated linear attention, latent attention;
dense erf-GELU feed-forward of 4x width) and a 4-layer Llama-style transformer of the same width (GQA, gated MLP
sized to the same parameter count) are built with random weights.  Measured with CUDA events after warm-up:

* prefill: one prompt of ``prompt_len`` tokens, tokens/s;
* decode: one token per step at a context of ``prompt_len`` tokens, tokens/s, for one stream (what the transformer
  engine's recurrent pipeline runs per stage) and for a batch of streams (hybrid only: its runner batches);
* the hybrid family's own kernels one by one on the prefill shapes and on the decode shapes, with achieved bytes/s
  and FLOP/s against the measured peaks, beside the transformer's attention kernels on the same token counts.

An L2 flush (a write larger than L2) separates timed iterations of the single-kernel measurements.

``bench.py --family vudelix`` measures the pre-norm design of the family (windowed grouped-query attention, gated
delta rule, mixture-of-experts and dense feed-forwards, per-layer token embedding) the same way, beside the sandwich
design of the same width as the closest existing model, with its own kernels one by one.

``bench.py --family labepel`` measures the parallel-block design (chunk-masked attention with a softmax sink and value
mixing, softmax-routed gated experts plus a shared expert, layer scale, learned positions) beside the pre-norm design
of the same width, whose windowed attention and mixture of experts are the closest existing kernels.  Decoding is
timed inside one chunk (the prompt ends short of a chunk edge), so that a step sees about as many keys as the
windowed design does.

``bench.py --family zudovik`` measures the post-norm design (causal grouped-query attention with the norm over the
whole q and k projections, a score cap and learned sinks, a layer on another layer's keys and values, the fixed-decay
linear recurrence, clamped gated experts with identity experts and a token-gated shared expert) beside the
parallel-block design of the same width, whose attention and mixture of experts are the closest existing kernels; the
recurrence is set beside the gated linear attention of the sandwich design, timed in the same run.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, List

import torch

__all__ = ["run_family_compare", "hybrid_bench_config", "vudelix_bench_config", "labepel_bench_config", "zudovik_bench_config"]


def zudovik_bench_config(width: int) -> Dict[str, Any]:
    """4 layers: attention + dense (squared ReLU, ``4 * width``), recurrence + experts, attention + experts, attention on
    the third layer's keys and values + experts.  Two of eight clamped experts of width ``width`` plus two identity
    outputs in the router, and a token-gated shared expert of width ``width`` (the parallel-block design's expert sizes)."""
    h = width // 128
    att = {"heads": h, "kv_heads": max(1, h // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0,
           "rot": {"dims": 64, "base": 500000.0}}
    lit = {"heads": h, "dim": 128, "vdim": 128, "decay": [1.0 - 2.0 ** (-3 - 5 * i / max(1, h - 1)) for i in range(h)]}
    moe = {"kind": "moe", "expert": {"ff": width, "limit": 7.0}, "router": {"experts": 8, "identity": 2, "top": 2},
           "shared": {"ff": width, "limit": 7.0}}
    layers = [{"type": "attention", "mixer": dict(att), "mlp": {"kind": "dense", "ff": 4 * width}},
              {"type": "lightning", "mixer": lit, "mlp": dict(moe)}, {"type": "attention", "mixer": dict(att), "mlp": dict(moe)},
              {"type": "attention", "mixer": {**att, "kv_from": 2}, "mlp": dict(moe)}]
    return {"architecture": "Zudovik", "vocab": 32000, "width": width, "embedding": {"scale": 32.0}, "layers": layers,
            "norm": {"eps": 1e-6}}


def vudelix_bench_config(width: int, window: int = 1024) -> Dict[str, Any]:
    """4 layers: delta + dense, attention + experts, delta + experts, attention + dense.  Two of eight experts of
    width ``2 * width`` per token, so a token's feed-forward work equals the dense ``4 * width`` one."""
    h = width // 128
    dense = {"kind": "dense", "ff": 4 * width}
    moe = {"kind": "moe", "expert": {"ff": 2 * width}, "router": {"experts": 8, "top": 2}}
    att = {"heads": h, "kv_heads": max(1, h // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": window},
           "rot": {"dims": 128, "base": 500000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    delta = {"heads": h, "kv_heads": max(1, h // 2), "dim": 128, "vdim": 128, "conv": 4}
    layers = [{"type": "channel_delta", "mixer": dict(delta), "mlp": dense}, {"type": "attention", "mixer": dict(att), "mlp": moe},
              {"type": "channel_delta", "mixer": dict(delta), "mlp": moe}, {"type": "attention", "mixer": dict(att), "mlp": dense}]
    return {"architecture": "Vudelix", "vocab": 32000, "width": width, "layers": layers, "norm": {"eps": 1e-6},
            "residual_mult": 0.5, "token_side": {"dim": 64}}


def labepel_bench_config(width: int, chunk: int = 1024, positions: int = 8192) -> Dict[str, Any]:
    """4 attention layers with experts: two of eight gated experts of width ``width`` per token plus a shared expert of
    the same width (9 width^2 weights per token, the dense ``4 * width`` feed-forward has 8)."""
    h = width // 128
    att = {"heads": h, "kv_heads": max(1, h // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "mask": {"size": chunk},
           "v_mix": True}
    moe = {"kind": "moe", "expert": {"ff": width}, "router": {"experts": 8, "top": 2}, "shared": {"ff": width}}
    return {"architecture": "Labepel", "vocab": 32000, "width": width, "max_positions": positions, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": dict(att), "mlp": dict(moe)} for _ in range(4)]}


def hybrid_bench_config(width: int) -> Dict[str, Any]:
    h = width // 128
    lat = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": 4 * width},
           "mixer": {"heads": h, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 512, "q_rank": min(1536, width),
                     "scale": 192 ** -0.5, "rot": {"dims": 64, "base": 10000.0}}}
    delta = {"type": "channel_delta", "mlp": {"kind": "dense", "ff": 4 * width},
             "mixer": {"heads": h, "kv_heads": max(1, h // 2), "dim": 128, "vdim": 128, "conv": 4}}
    gla = {"type": "gla", "mlp": {"kind": "dense", "ff": 4 * width}, "mixer": {"heads": h, "dim": 64, "vdim": 128, "tau": 16.0}}
    return {"architecture": "Badapel", "vocab": 32000, "width": width, "layers": [lat, delta, gla, dict(lat)],
            "norm": {"eps": 1e-6}, "logit_softcap": 30.0}


def _time(fn: Callable[[], Any], iters: int, warmup: int, flush: Any = None) -> float:
    """Median milliseconds of ``fn`` over ``iters`` runs (CUDA events; optional L2 flush between runs)."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def _peaks() -> Dict[str, float]:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fp:
            d = json.load(fp)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _hybrid(width: int, prompt_len: int, batch: int, steps: int, warmup: int, design: str = "hybrid") -> Dict[str, Any]:
    from ..models.config import HybridConfig
    from ..models.hybrid import HybridLM
    from ..parallel.hybrid_runner import HybridRunner

    dev = torch.device("cuda")
    make = {"hybrid": hybrid_bench_config, "vudelix": vudelix_bench_config, "labepel": labepel_bench_config,
            "zudovik": zudovik_bench_config}[design]
    cfg = HybridConfig.from_dict(make(width))
    model = HybridLM(cfg, {}).init_random(dev, torch.bfloat16, seed=1)
    params = sum(p.numel() for p in model.tensor_map().values())
    out: Dict[str, Any] = {"params_m": round(params / 1e6, 1), "layer_params_m": round((params - model.embed.numel()) / 1e6, 1)}
    prompt = torch.randint(0, cfg.vocab, (prompt_len,)).tolist()
    S = prompt_len + steps + warmup + 8

    def prefill_once() -> None:
        r = HybridRunner(model, S, n_slots=1, use_graphs=False)
        prefill_once.r = r
        r.step([("p", prompt)])

    # the runner is rebuilt per run (a pool of zeros): its allocation is outside what a serving loop pays per
    # prompt, so time only the step by pre-building
    runners = [HybridRunner(model, S, n_slots=1, use_graphs=False) for _ in range(warmup + 5)]
    it = iter(runners)
    ms = _time(lambda: next(it).step([("p", prompt)]), 5, warmup)
    out["prefill_tok_s"] = round(prompt_len / ms * 1e3, 1)
    out["prefill_ms"] = round(ms, 3)
    del runners
    # the chunk-masked design decodes up to the end of the prompt's last chunk, not across its edge
    context = prompt if design != "labepel" else prompt[: max(1, prompt_len - steps - warmup - 8)]
    out["decode_context"] = len(context)
    for b in (1, batch):
        r = HybridRunner(model, S, n_slots=b)
        # every stream its own prompt and tokens: identical streams would all choose the same experts
        r.step([(i, torch.randint(0, cfg.vocab, (len(context),)).tolist()) for i in range(b)])
        tok = [(i, [1 + 37 * i]) for i in range(b)]
        ms = _time(lambda: r.step(tok), steps, warmup)
        out[f"decode_tok_s_b{b}"] = round(b / ms * 1e3, 1)
        out[f"decode_ms_b{b}"] = round(ms, 4)
        del r
    kernels = {"hybrid": _hybrid_kernels, "vudelix": _vudelix_kernels, "labepel": _labepel_kernels,
               "zudovik": _zudovik_kernels}[design]
    out["kernels"] = kernels(model, prompt_len, batch)
    return out


def _vudelix_kernels(model: Any, T: int, batch: int) -> List[Dict[str, Any]]:
    """The pre-norm design's own kernels alone, on the prompt shape and on the decode shape (see ``_hybrid_kernels``)."""
    from ..ops import hybrid as H

    pk = _peaks()
    dev, dt = model.device, model.dtype
    C = model.config.width
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows: List[Dict[str, Any]] = []

    def rec(name: str, phase: str, ms: float, nbytes: float, flops: float) -> None:
        rows.append({"kernel": name, "phase": phase, "ms": round(ms, 4), "gb_s": round(nbytes / ms / 1e6, 1),
                     "tflops": round(flops / ms / 1e9, 2),
                     "frac_of_roofline": round(max(nbytes / ms / 1e6 / pk["hbm_gbs"], flops / ms / 1e9 / pk["bf16_tflops"]), 4),
                     "peaks": pk["source"]})

    att, moe = model.blocks[1].mix, model.blocks[1].mlp
    Hh, G, D, V, W = att.H, att.G, att.D, att.V, att.window
    for phase, lengths, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [T] * batch)):
        n_seq, N = len(lengths), sum(lengths)
        pool = model.new_pool(n_seq, T + 8)
        plan = H.BatchPlan.make(lengths, list(range(n_seq)), starts, dev)
        cache = pool.runs[1]["cache"]
        cache.normal_()
        h = torch.randn(N, C, device=dev).to(dt)
        p = H.linear(h, att.w_in)
        q, g = att.col(p, "q"), att.col(p, "g")
        pairs = sum(min(W, s + i + 1) if W else s + i + 1 for n, s in zip(lengths, starts) for i in range(n))
        ms = _time(lambda: H.window_append(q, att.col(p, "k"), att.col(p, "v"), att.inv_freq, cache, plan, Hh, G, D, V,
                                           att.nrot, 1e-6), 5, 3, flush)
        rec("window_append", phase, ms, 2.0 * N * (2 * Hh * D + 2 * G * (D + V)), 0.0)
        if phase == "prefill":
            ms = _time(lambda: H.head_gate(att._banded(q, cache, plan), g), 5, 3, flush)
            rec("window_attn_banded(gemm+softmax)", phase, ms, 2.0 * N * (Hh * (D + V) + G * (D + V)), 2.0 * Hh * pairs * (D + V))
            nb = min(N, att.query_block)
            s32 = torch.randn(Hh, nb, nb + W - 1, device=dev)
            ms = _time(lambda: H.causal_softmax(s32, N - nb, att.scale, dt, window=W, key0=N - nb - W + 1), 5, 3, flush)
            rec("causal_softmax[window]", phase, ms, s32.numel() * 6.0, 0.0)
            del s32
        else:
            ms = _time(lambda: H.window_attn(q, g, cache, plan, Hh, G, D, V, att.scale, W), 5, 3, flush)
            keys = sum(min(W, s + 1) if W else s + 1 for s in starts)
            rec("window_attn", phase, ms, 2.0 * G * keys * (D + V) + 2.0 * N * Hh * (D + V), 2.0 * Hh * pairs * (D + V))
        z = H.linear_f32(h, moe.router32)
        ms = _time(lambda: H.router_topk(z, moe.top), 5, 3, flush)
        rec("router_topk", phase, ms, 4.0 * N * (moe.E + 2 * moe.top), 0.0)
        ms = _time(lambda: moe(h), 5, 3, flush)
        wbytes = 2.0 * 2 * C * moe.ff * min(moe.E, N * moe.top)
        rec("moe_experts[index-driven]" if N * moe.top <= moe.gemv_max else "moe_experts[grouped gemm]", phase, ms,
            wbytes + 2.0 * N * C * (1 + moe.top), 4.0 * N * moe.top * C * moe.ff)
        ff = model.blocks[0].mlp
        ms = _time(lambda: ff(h), 5, 3, flush)
        rec("dense_ff(gemm+gelu)", phase, ms, 2.0 * 2 * C * ff.up.size(0) + 4.0 * N * C, 4.0 * N * C * ff.up.size(0))
        side = model.blocks[0].side
        zs = H.linear(h, side.gate)
        tok = torch.randint(0, model.config.vocab, (N,), device=dev, dtype=torch.int32)
        ms = _time(lambda: H.token_side_gate(zs, model.side_embed, tok, 0), 5, 3, flush)
        rec("token_side_gate", phase, ms, 2.0 * N * 3 * side.dim, 0.0)
        x = torch.randn(N, C, device=dev)
        ms = _time(lambda: H.norm_rows(x, model.blocks[0].norm1.w, None, 1e-6, "rms", dt), 5, 3, flush)
        rec("rms_norm", phase, ms, N * C * 6.0, 0.0)
        y = torch.randn(N, C, device=dev).to(dt)
        ms = _time(lambda: H.norm_accumulate(x, y, None, None, 1e-6, "none", 0.5), 5, 3, flush)
        rec("scaled_residual_add", phase, ms, N * C * 10.0, 0.0)
        del pool
    return rows


def _zudovik_kernels(model: Any, T: int, batch: int) -> List[Dict[str, Any]]:
    """The post-norm design's own kernels alone, on the prompt shape and on the decode shape; ``like`` names the row of
    ``_labepel_kernels`` (or, for the recurrence, of ``_hybrid_kernels``) that does the corresponding work."""
    from ..ops import hybrid as H

    pk = _peaks()
    dev, dt = model.device, model.dtype
    C = model.config.width
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows: List[Dict[str, Any]] = []

    def rec(name: str, like: str, phase: str, ms: float, nbytes: float, flops: float) -> None:
        rows.append({"kernel": name, "like": like, "phase": phase, "ms": round(ms, 4), "gb_s": round(nbytes / ms / 1e6, 1),
                     "tflops": round(flops / ms / 1e9, 2),
                     "frac_of_roofline": round(max(nbytes / ms / 1e6 / pk["hbm_gbs"], flops / ms / 1e9 / pk["bf16_tflops"]), 4),
                     "peaks": pk["source"]})

    att, lit, moe, dense = model.blocks[2].mix, model.blocks[1].mix, model.blocks[2].mlp, model.blocks[0].mlp
    Hh, G, D, V = att.H, att.G, att.D, att.V
    for phase, lengths, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [T] * batch)):
        n_seq, N = len(lengths), sum(lengths)
        pool = model.new_pool(n_seq, T + 8)
        plan = H.BatchPlan.make(lengths, list(range(n_seq)), starts, dev)
        cache = pool.runs[2]["cache"]
        cache.normal_()
        tok = torch.randint(0, model.config.vocab, (N,), device=dev, dtype=torch.int32)
        ms = _time(lambda: H.embed_rows(model.embed, tok, None, plan, model.config.embed_scale), 5, 3, flush)
        rec("embed_rows[scale]", "embed_rows[positions]", phase, ms, N * C * 6.0, 0.0)
        x = torch.randn(N, C, device=dev)
        h = torch.randn(N, C, device=dev).to(dt)
        p = H.linear(h, att.w_in, att.b_in)
        q, g = att.col(p, "q"), att.col(p, "g")
        pairs = sum(s + i + 1 for n, s in zip(lengths, starts) for i in range(n))
        ms = _time(lambda: H.full_norm_append(q, att.col(p, "k"), att.col(p, "v"), att.inv_freq, cache, plan, Hh, G, D, V, att.nrot,
                                              1e-6, att.q_norm, att.k_norm), 5, 3, flush)
        rec("full_norm_append", "window_append[weights, value mixing]", phase, ms, 2.0 * N * (2 * Hh * D + 2 * G * (D + V)), 0.0)
        if phase == "prefill":
            ms = _time(lambda: H.head_gate(att._banded(q, cache, plan), g), 5, 3, flush)
            rec("causal_attn(gemm+softmax)", "chunk_attn(gemm+softmax)", phase, ms, 2.0 * N * (Hh * (D + 2 * V) + G * (D + V)),
                2.0 * Hh * pairs * (D + V))
            nb = min(N, att.query_block)
            s32 = torch.randn(Hh, nb, N, device=dev)
            ms = _time(lambda: H.causal_softmax(s32, N - nb, att.scale, dt, sink=True, split=True, cap=att.softcap,
                                                sink_vals=att.sink32), 5, 3, flush)
            rec("causal_softmax[cap, learned sink, split weights]", "causal_softmax[sink, split weights]", phase, ms,
                s32.numel() * 8.0, 0.0)
            del s32
        else:
            ms = _time(lambda: H.window_attn(q, g, cache, plan, Hh, G, D, V, att.scale, 0, sink=True, cap=att.softcap,
                                             sink_vals=att.sink32), 5, 3, flush)
            keys = sum(s + 1 for s in starts)
            rec("window_attn[causal, cap, learned sink]", "window_attn[chunk, sink, channel gate]", phase, ms,
                2.0 * G * keys * (D + V) + 2.0 * N * Hh * (D + V), 2.0 * Hh * pairs * (D + V))
        # the recurrent mixer
        LH, LD, LV = lit.H, lit.D, lit.V
        pl = H.linear(h, lit.w_in)
        state = pool.runs[1]["state"]
        ms = _time(lambda: H.lightning_recurrence(lit.col(pl, "q"), lit.col(pl, "k"), lit.col(pl, "v"), lit.decay, state,
                                                  plan, LH, LD, LV, act=True), 5, 3, flush)
        nbytes = 2.0 * N * (2 * LH * LD + LH * LV) + 4.0 * N * LH * LV + 8.0 * n_seq * LH * LD * LV
        rec("lightning_recurrence[chunks]" if phase == "prefill" else "lightning_recurrence[scan]", "gated_recurrence[gla]", phase,
            ms, nbytes, 4.0 * N * LH * LD * LV)
        o = torch.randn(N, LH * LV, device=dev)
        ms = _time(lambda: H.norm_gate_rows(o, lit.norm, lit.col(pl, "g"), 1e-6, dt), 5, 3, flush)
        rec("norm_gate_rows", "rms_norm[1 + w]", phase, ms, N * LH * LV * 8.0, 0.0)
        # feed-forwards
        z = H.linear_f32(h, moe.router32)
        ms = _time(lambda: H.router_topk(z, moe.top, "softmax_all", moe.correction32), 5, 3, flush)
        rec("router_topk[softmax over all, correction]", "router_topk[softmax]", phase, ms, 4.0 * N * (moe.E + moe.identity + 2 * moe.top), 0.0)
        ms = _time(lambda: moe(h), 5, 3, flush)
        wbytes = 2.0 * 3 * C * moe.ff * min(moe.E, N * moe.top)
        form = "index-driven" if N * moe.top <= moe.gemv_max else "grouped gemm"
        rec(f"moe_experts[{form}, clamped, identity]", f"moe_experts[{form}, gated]", phase, ms, wbytes + 2.0 * N * C * (1 + moe.top),
            6.0 * N * moe.top * C * moe.ff)
        sh = moe.shared
        ms = _time(lambda: sh.gated(h), 5, 3, flush)
        rec("shared_expert(gemm+clamped product)", "shared_expert(gemm+silu*up)", phase, ms, 2.0 * 3 * C * sh.ff + 4.0 * N * C,
            6.0 * N * C * sh.ff)
        gu = H.linear(h, sh.w_in)
        ms = _time(lambda: H.act_mul(gu[:, :2 * sh.ff], "clamped", sh.limit), 5, 3, flush)
        rec("act_mul[clamped]", "act_mul", phase, ms, 2.0 * N * 3 * sh.ff, 0.0)
        ms = _time(lambda: dense(h), 5, 3, flush)
        rec("dense_ff(gemm+relu2)", "shared_expert(gemm+silu*up)", phase, ms, 2.0 * 2 * C * dense.up.size(0) + 4.0 * N * C,
            4.0 * N * C * dense.up.size(0))
        ya, yb = (torch.randn(N, C, device=dev).to(dt) for _ in range(2))
        sg = torch.randn(N, 1, device=dev).to(dt)
        blk = model.blocks[2]
        cp = torch.empty(N, C, device=dev, dtype=dt)
        ms = _time(lambda: H.norm_accumulate(x, ya, blk.norm1.w, None, 1e-6, "rms", copy=cp), 5, 3, flush)
        rec("post_norm_accumulate[+ rounded copy]", "scaled_branches", phase, ms, N * C * 12.0, 0.0)
        ms = _time(lambda: H.gated_sum_norm_accumulate(x, ya, yb, sg, blk.norm2.w, 1e-6, copy=cp), 5, 3, flush)
        rec("gated_sum_norm_accumulate[+ rounded copy]", "scaled_branches", phase, ms, N * C * 14.0, 0.0)
        del pool
    return rows


def _labepel_kernels(model: Any, T: int, batch: int) -> List[Dict[str, Any]]:
    """The parallel-block design's own kernels alone, on the prompt shape and on the decode shape; ``like`` names the
    row of ``_vudelix_kernels`` that does the corresponding work in the pre-norm design."""
    from ..ops import hybrid as H

    pk = _peaks()
    dev, dt = model.device, model.dtype
    C = model.config.width
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows: List[Dict[str, Any]] = []

    def rec(name: str, like: str, phase: str, ms: float, nbytes: float, flops: float) -> None:
        rows.append({"kernel": name, "like": like, "phase": phase, "ms": round(ms, 4), "gb_s": round(nbytes / ms / 1e6, 1),
                     "tflops": round(flops / ms / 1e9, 2),
                     "frac_of_roofline": round(max(nbytes / ms / 1e6 / pk["hbm_gbs"], flops / ms / 1e9 / pk["bf16_tflops"]), 4),
                     "peaks": pk["source"]})

    blk = model.blocks[1]  # a layer that blends its values with the first layer's
    att, moe = blk.mix, blk.mlp
    Hh, G, D, V, W = att.H, att.G, att.D, att.V, att.window
    first = lambda pos: (pos // W) * W if W else 0  # noqa: E731 - first visible key of a position
    for phase, lengths, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [max(0, T - 8)] * batch)):
        n_seq, N = len(lengths), sum(lengths)
        pool = model.new_pool(n_seq, T + 8)
        plan = H.BatchPlan.make(lengths, list(range(n_seq)), starts, dev)
        cache = pool.runs[1]["cache"]
        cache.normal_()
        tok = torch.randint(0, model.config.vocab, (N,), device=dev, dtype=torch.int32)
        ms = _time(lambda: H.embed_rows(model.embed, tok, model.pos, plan), 5, 3, flush)
        rec("embed_rows[positions]", "", phase, ms, N * C * 8.0, 0.0)
        h = torch.randn(N, C, device=dev).to(dt)
        p = H.linear(h, att.w_in, att.b_in)
        q, g, v = att.col(p, "q"), att.col(p, "g"), att.col(p, "v")
        vf = torch.randn_like(v)
        pairs = sum(s + i + 1 - first(s + i) for n, s in zip(lengths, starts) for i in range(n))
        ms = _time(lambda: H.window_append(q, att.col(p, "k"), v, None, cache, plan, Hh, G, D, V, 0, 1e-6, att.q_norm,
                                           att.k_norm, vf, att.lam), 5, 3, flush)
        rec("window_append[weights, value mixing]", "window_append", phase, ms,
            2.0 * N * (2 * Hh * D + 2 * G * (D + V) + G * V), 0.0)
        if phase == "prefill":
            ms = _time(lambda: H.headmajor_gate(att._chunked(q, cache, plan), g), 5, 3, flush)
            rec("chunk_attn(gemm+softmax)", "window_attn_banded(gemm+softmax)", phase, ms,
                2.0 * N * (Hh * (D + 2 * V) + G * (D + V)), 2.0 * Hh * pairs * (D + V))
            nb = min(N, W) if W else min(N, att.query_block)
            s32 = torch.randn(max(1, N // nb) * Hh, nb, nb, device=dev)
            ms = _time(lambda: H.causal_softmax(s32, 0, att.scale, dt, sink=att.sink, split=True), 5, 3, flush)
            rec("causal_softmax[sink, split weights]", "causal_softmax[window]", phase, ms, s32.numel() * 8.0, 0.0)
            del s32
        else:
            ms = _time(lambda: H.window_attn(q, g, cache, plan, Hh, G, D, V, att.scale, W, mask=att.mask_kind, sink=att.sink),
                       5, 3, flush)
            keys = sum(s + 1 - first(s) for s in starts)
            rec("window_attn[chunk, sink, channel gate]", "window_attn", phase, ms,
                2.0 * G * keys * (D + V) + 2.0 * N * Hh * (D + 2 * V), 2.0 * Hh * pairs * (D + V))
        z = H.linear_f32(h, moe.router32, moe.router_b32)
        ms = _time(lambda: H.router_topk(z, moe.top, "softmax"), 5, 3, flush)
        rec("router_topk[softmax]", "router_topk", phase, ms, 4.0 * N * (moe.E + 2 * moe.top), 0.0)
        ms = _time(lambda: moe(h), 5, 3, flush)
        wbytes = 2.0 * 3 * C * moe.ff * min(moe.E, N * moe.top)
        form = "index-driven" if N * moe.top <= moe.gemv_max else "grouped gemm"
        rec(f"moe_experts[{form}, gated]", f"moe_experts[{form}]", phase, ms, wbytes + 2.0 * N * C * (1 + moe.top),
            6.0 * N * moe.top * C * moe.ff)
        sh = moe.shared
        ms = _time(lambda: sh(h), 5, 3, flush)
        rec("shared_expert(gemm+silu*up)", "dense_ff(gemm+gelu)", phase, ms, 2.0 * 3 * C * sh.down.size(1) + 4.0 * N * C,
            6.0 * N * C * sh.down.size(1))
        gu = H.linear(h, sh.w_in)
        ms = _time(lambda: H.act_mul(gu), 5, 3, flush)
        rec("act_mul", "", phase, ms, 2.0 * N * 3 * sh.down.size(1), 0.0)
        x = torch.randn(N, C, device=dev)
        ms = _time(lambda: H.norm_rows(x, blk.norm1.w, None, 1e-6, "rms", dt, 1.0), 5, 3, flush)
        rec("rms_norm[1 + w]", "rms_norm", phase, ms, N * C * 6.0, 0.0)
        ya, yb, yc = (torch.randn(N, C, device=dev).to(dt) for _ in range(3))
        ms = _time(lambda: H.scaled_branches(x, ya, blk.ls1, yb, yc, blk.ls2), 5, 3, flush)
        rec("scaled_branches", "scaled_residual_add", phase, ms, N * C * 14.0, 0.0)
        del pool
    return rows


def _hybrid_kernels(model: Any, T: int, batch: int) -> List[Dict[str, Any]]:
    """Each family kernel alone, on the prompt shape (1 x T tokens) and the decode shape (batch x 1 token at context T)."""
    from ..ops import hybrid as H

    pk = _peaks()
    dev, dt = model.device, model.dtype
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows: List[Dict[str, Any]] = []

    def rec(name: str, phase: str, ms: float, nbytes: float, flops: float) -> None:
        rows.append({"kernel": name, "phase": phase, "ms": round(ms, 4), "gb_s": round(nbytes / ms / 1e6, 1),
                     "tflops": round(flops / ms / 1e9, 2),
                     "frac_of_roofline": round(max(nbytes / ms / 1e6 / pk["hbm_gbs"], flops / ms / 1e9 / pk["bf16_tflops"]), 4),
                     "peaks": pk["source"]})

    for phase, lengths, starts in (("prefill", [T], [0]), ("decode", [1] * batch, [T] * batch)):
        n_seq, N = len(lengths), sum(lengths)
        pool = model.new_pool(n_seq, T + 8)
        plan = H.BatchPlan.make(lengths, list(range(n_seq)), starts, dev)
        for li, blk in enumerate(model.blocks[:3]):
            mix, st = blk.mix, pool.runs[li]
            h = torch.randn(N, model.config.width, device=dev).to(dt)
            p = H.linear(h, mix.w_in)
            if li == 0:
                Hh, D, R, V, L = mix.H, mix.D, mix.R, mix.V, mix.L
                st["cache"].normal_()
                q = H.linear(H.norm_rows(mix.col(p, "dq"), mix.dq_norm, None, 1e-6, "rms", dt), mix.uq)
                qlat = torch.randn(Hh, N, L, device=dev).to(dt)
                keys = sum((s + n) * n - n * (n - 1) // 2 for n, s in zip(lengths, starts))  # visible (query, key) pairs
                if phase == "prefill":  # prompts take the expanded form: GEMMs + the causal softmax kernel
                    ms = _time(lambda: mix._expanded(q, st["cache"], plan), 5, 3, flush)
                    total_keys = sum(s + n for n, s in zip(lengths, starts))
                    flops = 2.0 * total_keys * L * Hh * (D + V) + 2.0 * Hh * keys * (D + R + V)
                    rec("latent_attn_expanded(gemm+softmax)", phase, ms, 2.0 * N * Hh * (D + R + V), flops)
                    s32 = torch.randn(Hh, min(N, 1024), N, device=dev)
                    ms = _time(lambda: H.causal_softmax(s32, N - s32.size(1), mix.scale, dt), 5, 3, flush)
                    rec("causal_softmax", phase, ms, s32.numel() * 6.0, 0.0)
                    del s32
                else:
                    ms = _time(lambda: H.latent_attn(qlat, q, st["cache"], plan, Hh, D, R, L, mix.scale), 5, 3, flush)
                    nbytes = 2.0 * (2 * Hh * N * L + Hh * N * R) + 2.0 * (L + R) * sum(s + n for n, s in zip(lengths, starts))
                    rec("latent_attn", phase, ms, nbytes, 2.0 * Hh * keys * (2 * L + R))
                ms = _time(lambda: H.latent_append(mix.col(p, "dkv"), q, mix.dkv_norm, mix.inv_freq, st["cache"], plan, Hh, D,
                                                   R, L, mix.nrot, 1e-6), 5, 3, flush)
                rec("latent_append", phase, ms, 2.0 * N * (2 * (L + R) + 2 * Hh * R), 0.0)
            else:
                mode = "delta" if li == 1 else "gla"
                Hh, D, V = mix.H, mix.D, mix.V
                G = mix.G if mode == "delta" else Hh
                z = torch.randn(N, Hh * D, device=dev).to(dt)
                gate = torch.randn(N, Hh * V, device=dev).to(dt)
                if mode == "delta":
                    c = H.conv_silu(p[:, :2 * G * D + Hh * V], mix.conv_w, st["conv"], plan)
                    args = (c[:, :G * D], c[:, G * D:2 * G * D], c[:, 2 * G * D:], z, gate, mix.norm, st["state"], plan)
                    kw = dict(heads=Hh, kv_heads=G, dim=D, vdim=V, mode=mode, eps=1e-6, zb=mix.dt_bias, beta=mix.col(p, "b"),
                              a_log=mix.A_log)
                    ms = _time(lambda: H.conv_silu(p[:, :2 * G * D + Hh * V], mix.conv_w, st["conv"], plan), 5, 3, flush)
                    rec("conv_silu", phase, ms, 2.0 * N * 2 * (2 * G * D + Hh * V), 0.0)
                else:
                    args = (mix.col(p, "q"), mix.col(p, "k"), mix.col(p, "v"), z, gate, mix.norm, st["state"], plan)
                    kw = dict(heads=Hh, kv_heads=G, dim=D, vdim=V, mode=mode, eps=1e-6, zb=mix.a2_b, tau=mix.tau)
                ms = _time(lambda: H.gated_recurrence(*args, **kw), 5, 3, flush)
                nbytes = 2.0 * N * (2 * G * D + Hh * D + 3 * Hh * V) + 8.0 * n_seq * Hh * D * V
                rec(f"gated_recurrence[{mode}]", phase, ms, nbytes, (6.0 if mode == "delta" else 4.0) * N * Hh * D * V)
        x = torch.randn(N, model.config.width, device=dev)
        blk = model.blocks[0]
        ms = _time(lambda: H.norm_rows(x, blk.norm1.w, blk.norm1.b, 1e-6, "layer", dt), 5, 3, flush)
        rec("layer_norm", phase, ms, N * model.config.width * 6.0, 0.0)
        del pool
    return rows


def _transformer(width: int, prompt_len: int, steps: int, warmup: int, target_params: float) -> Dict[str, Any]:
    from ..models.config import Config
    from ..models.stage import build_stage
    from ..parallel.pipeline import DevicePipeline
    from ..parallel.scheduler import SamplingParams
    from ..utils.checkpoint import random_init_stage_

    n_head = width // 128
    groups = 8 if n_head % 8 == 0 else n_head
    attn = width * (n_head + 2 * groups) * 128 + width * width
    inter = int(max(256, round((target_params / 4 - attn) / (3 * width) / 256) * 256))  # equal parameters per layer
    cfg = Config(name="Llama-like-bench", block_size=prompt_len + steps + warmup + 64, vocab_size=32000, padded_vocab_size=32000,
                 n_layer=4, n_head=n_head, n_embd=width, n_query_groups=groups, rotary_percentage=1.0, parallel_residual=False,
                 bias=False, norm_class_name="RMSNorm", mlp_class_name="LLaMAMLP", intermediate_size=inter)
    stage = build_stage(cfg, "starter", cfg.n_layer, meta=True)
    random_init_stage_(stage, "cuda", torch.bfloat16)
    params = sum(p.numel() for p in stage.parameters())
    S = cfg.block_size
    pipe = DevicePipeline(stage, 0, 1, n_samples=1, max_seq_length=S, sampling=SamplingParams.greedy(), max_prompt_len=prompt_len)
    prompt = torch.randint(0, 32000, (prompt_len,), dtype=torch.int32)
    layer_params = sum(p.numel() for p in stage.transformer.h.parameters())
    out: Dict[str, Any] = {"params_m": round(params / 1e6, 1), "layer_params_m": round(layer_params / 1e6, 1), "intermediate_size": inter}

    def pre() -> None:
        pipe.prepare([prompt], steps + warmup + 8)
        torch.cuda.synchronize()

    ts = []
    for i in range(warmup + 5):
        pre()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        pipe.prefill()
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            ts.append(a.elapsed_time(b))
    ts.sort()
    ms = ts[len(ts) // 2]
    out["prefill_tok_s"] = round(prompt_len / ms * 1e3, 1)
    out["prefill_ms"] = round(ms, 3)
    pipe.decode_rounds(warmup)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    pipe.decode_rounds(steps)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    out["decode_tok_s_b1"] = round(1e3 / ms, 1)
    out["decode_ms_b1"] = round(ms, 4)
    pipe.close()
    return out


def run_family_compare(widths: List[int], prompt_len: int = 2048, batch: int = 8, steps: int = 64, warmup: int = 8,
                       family: str = "hybrid") -> Dict[str, Any]:
    torch.backends.cuda.matmul.allow_tf32 = False
    results = []
    if family == "vudelix":
        for w in widths:
            new = _hybrid(w, prompt_len, batch, steps, warmup, "vudelix")
            torch.cuda.empty_cache()
            old = _hybrid(w, prompt_len, batch, steps, warmup, "hybrid")
            torch.cuda.empty_cache()
            results.append({"width": w, "vudelix": new, "hybrid": old})
        return {"metric": "family_compare", "family": "vudelix", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
                "decode_batch": batch, "steps": steps, "warmup": warmup, "l2": "flushed between single-kernel timings",
                "results": results}
    if family == "zudovik":
        from ..models.config import HybridConfig
        from ..models.hybrid import HybridLM

        for w in widths:
            new = _hybrid(w, prompt_len, batch, steps, warmup, "zudovik")
            torch.cuda.empty_cache()
            old = _hybrid(w, prompt_len, batch, steps, warmup, "labepel")
            torch.cuda.empty_cache()
            # the recurrence's like kernel lives in the sandwich design: its kernels alone, no model-level timing
            sandwich = HybridLM(HybridConfig.from_dict(hybrid_bench_config(w)), {}).init_random(torch.device("cuda"), torch.bfloat16, seed=1)
            rec_rows = [k for k in _hybrid_kernels(sandwich, prompt_len, batch) if k["kernel"] == "gated_recurrence[gla]"]
            del sandwich
            torch.cuda.empty_cache()
            theirs = {(k["kernel"], k["phase"]): k["frac_of_roofline"] for k in old["kernels"] + rec_rows}
            for k in new["kernels"]:  # how far from its roofline, relative to the like kernel (above 1: this one is nearer)
                other = theirs.get((k["like"], k["phase"]))
                k["roofline_vs_like"] = round(k["frac_of_roofline"] / other, 3) if other else None
            results.append({"width": w, "zudovik": new, "labepel": old, "sandwich_recurrence": rec_rows})
        return {"metric": "family_compare", "family": "zudovik", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
                "decode_batch": batch, "steps": steps, "warmup": warmup, "l2": "flushed between single-kernel timings",
                "results": results}
    if family == "labepel":
        for w in widths:
            new = _hybrid(w, prompt_len, batch, steps, warmup, "labepel")
            torch.cuda.empty_cache()
            old = _hybrid(w, prompt_len, batch, steps, warmup, "vudelix")
            torch.cuda.empty_cache()
            theirs = {(k["kernel"], k["phase"]): k["frac_of_roofline"] for k in old["kernels"]}
            for k in new["kernels"]:  # how far from its roofline, relative to the like kernel of the other design
                other = theirs.get((k["like"], k["phase"]))
                k["roofline_vs_like"] = round(k["frac_of_roofline"] / other, 3) if other else None
            results.append({"width": w, "labepel": new, "vudelix": old})
        return {"metric": "family_compare", "family": "labepel", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
                "decode_batch": batch, "steps": steps, "warmup": warmup, "l2": "flushed between single-kernel timings",
                "results": results}
    for w in widths:
        hy = _hybrid(w, prompt_len, batch, steps, warmup)
        torch.cuda.empty_cache()
        try:
            tr = _transformer(w, prompt_len, steps, warmup, hy["layer_params_m"] * 1e6)
        except Exception as e:  # noqa: BLE001 - the comparison arm must not hide the family's own numbers
            tr = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()
        results.append({"width": w, "hybrid": hy, "transformer": tr})
    return {"metric": "family_compare", "family": "hybrid", "dtype": "bf16", "data": "synthetic", "prompt_len": prompt_len,
            "decode_batch": batch, "steps": steps, "warmup": warmup, "l2": "flushed between single-kernel timings",
            "results": results}
