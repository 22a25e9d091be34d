"""The Zudovik design (post-norm blocks of the hybrid family) against the plain oracle of ``zudovik_oracle.py``.

Every test builds its own small configuration with random weights.  Sizes are awkward on purpose: value width != key
width, rotated part shorter than the head and equal to it, one and several query heads per key head, a layer that
borrows another layer's keys and values with a scale, cap and sinks of its own, decays from nearly 0 to nearly 1,
mixtures with and without identity experts and shared expert, one and several experts per token, a layer without
feed-forward, an embedding scale that is not 1.  The same tests run on the CPU (PyTorch bodies of the operations) and,
marked ``gpu``, on the sm_100a kernels.
"""
from __future__ import annotations

import copy
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import zudovik_oracle as O
from mdi_llm_b200.models.config import HybridConfig
from mdi_llm_b200.models.hybrid import HybridLM, MoEFF, WindowAttention, load_hybrid, write_safetensors
from mdi_llm_b200.models.registry import model_classes
from mdi_llm_b200.ops import hybrid as H
from mdi_llm_b200.ops.hybrid import BatchPlan
from mdi_llm_b200.parallel.hybrid_runner import HybridRunner
from mdi_llm_b200.parallel.scheduler import SamplingParams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRAITS = {"mask": "window", "sink": "learned", "qk_norm": "full", "bias": True, "gate": "head", "p32": True}

DENSE = {"kind": "dense", "ff": 40}
MOE = {"kind": "moe", "expert": {"ff": 20, "limit": 1.5}, "router": {"experts": 5, "identity": 2, "top": 3},
       "shared": {"ff": 12, "limit": 0.7}}
MOE_BARE = {"kind": "moe", "expert": {"ff": 12, "limit": 2.5}, "router": {"experts": 3, "identity": 0, "top": 1}}


def attn(heads=4, kv=2, dim=12, vdim=10, scale=0.3, cap=8.0, rot=8, base=1000.0, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "softcap": cap,
         "rot": {"dims": rot, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": copy.deepcopy(mlp)}


def light(heads=3, dim=12, vdim=20, decay=(0.5, 0.93, 0.999), mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": copy.deepcopy(mlp)}


def cfg_dict(layers, width=24, vocab=50, eps=1e-3, scale=3.0):
    return {"architecture": "Zudovik", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "layers": copy.deepcopy(layers), "norm": {"eps": eps}}


def all_experts(d):
    """The same model with every router output chosen for every token: no routing decision that 8-bit mantissas could flip."""
    d = copy.deepcopy(d)
    for spec in d["layers"]:
        if spec["mlp"] and spec["mlp"]["kind"] == "moe":
            r = spec["mlp"]["router"]
            r["top"] = r["experts"] + r.get("identity", 0)
    return d


# attention + dense, recurrence + experts, attention with three heads per key head and the whole head rotated, a layer
# on layer 2's keys and values (other scale and cap) without feed-forward, a second recurrence with other sizes
FULL = cfg_dict([attn(mlp=DENSE), light(mlp=MOE), attn(heads=6, kv=2, dim=8, vdim=6, scale=0.8, cap=3.0, rot=8, base=50.0, mlp=MOE_BARE),
                 attn(heads=6, kv=2, dim=8, vdim=6, scale=0.2, cap=20.0, rot=8, base=50.0, kv_from=2, mlp=None),
                 light(heads=2, dim=5, vdim=36, decay=(0.05, 0.98), mlp=DENSE)])

DEVICES = [pytest.param(("cpu", torch.float32), id="cpu-f32"),
           pytest.param(("cuda", torch.float32), id="cuda-f32", marks=pytest.mark.gpu),
           pytest.param(("cuda", torch.bfloat16), id="cuda-bf16", marks=pytest.mark.gpu)]


def build(d, dev, seed=0):
    device, dtype = dev
    if device == "cuda":
        torch.backends.cuda.matmul.allow_tf32 = False
    if dtype == torch.bfloat16:
        d = all_experts(d)
    T = O.random_tensors(d, seed)
    return d, HybridLM(HybridConfig.from_dict(d)).load_tensors(T, device, dtype)


def oracle_logits(d, model, tokens, trace=None):
    W = {k: v.detach().float().cpu() for k, v in model.state_tensors().items()}
    return O.forward(d, W, list(tokens), layers_out=trace).float()


def close(got, want, dev, what=""):
    """fp32: every value within 2e-4.  bf16: per row, the error (root mean square over the row) relative to the row's
    own spread is below 8 % on average and 40 % at the worst row."""
    diff = got.float().cpu() - want
    if dev[1] == torch.float32:
        err = diff.abs().max().item()
        assert err < 2e-4 * max(1.0, want.abs().max().item()), f"{what}: max abs error {err}"
        return
    rel = diff.pow(2).mean(-1).sqrt() / want.std(-1).clamp_min(1e-3)
    assert rel.mean().item() < 0.08 and rel.max().item() < 0.4, f"{what}: relative rms error mean {rel.mean()} max {rel.max()}"


def toks(n, vocab=50, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def all_rows(n):
    return [list(range(n))]


# ---- each mechanism alone -----------------------------------------------------------------------------------
CASES = {
    "attention": [attn()],
    "one_head_per_key_head": [attn(heads=3, kv=3, dim=8, vdim=16, scale=1.5, rot=4)],
    "one_key_head_whole_head_rotated": [attn(heads=5, kv=1, dim=6, vdim=4, rot=6, base=7.0)],
    "tight_cap": [attn(scale=4.0, cap=0.5)],
    "borrowed_keys_and_values": [attn(), attn(scale=1.1, cap=2.0, kv_from=0)],
    "lightning": [light()],
    "lightning_one_head": [light(heads=1, dim=7, vdim=3, decay=(0.8,))],
    "dense": [light(heads=1, dim=4, vdim=4, decay=(0.9,), mlp=DENSE)],
    "experts_top1_no_identity_no_shared": [light(heads=1, dim=4, vdim=4, decay=(0.9,), mlp=MOE_BARE)],
    "experts_identity_shared": [light(heads=1, dim=4, vdim=4, decay=(0.9,), mlp=MOE)],
    "identity_only_choice": [light(heads=1, dim=4, vdim=4, decay=(0.9,),
                                   mlp={"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 1, "identity": 3, "top": 2}})],
}


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("case", list(CASES))
def test_each_mechanism_alone(dev, case):
    d, m = build(cfg_dict(CASES[case]), dev)
    t = toks(41)
    close(HybridRunner(m, 64).step([("a", t)], all_rows(len(t))), oracle_logits(d, m, t), dev, case)


def test_embedding_scale_and_traits():
    d, m = build(cfg_dict([light()], scale=1.0), ("cpu", torch.float32))
    d2, m2 = build(cfg_dict([light()], scale=5.0), ("cpu", torch.float32))
    t = toks(6)
    a, b = HybridRunner(m, 8).step([("a", t)], all_rows(6)), HybridRunner(m2, 8).step([("a", t)], all_rows(6))
    assert (a - b).abs().max() > 1e-3
    close(b, oracle_logits(d2, m2, t), ("cpu", torch.float32))
    c = m.config
    assert c.block == "postnorm" and c.norm == "rms" and not c.tied_head and c.dense_act == "relu2" and c.embed_scale == 1.0
    assert c.attention["sink"] == "learned" and c.attention["qk_norm"] == "full" and c.moe["router"] == "softmax_all"


# ---- row kernels against their plain forms ----------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_kernels_match_their_plain_forms(dtype):
    g = torch.Generator().manual_seed(0)
    N, C = 37, 72
    tol = 1e-5 if dtype == torch.float32 else 2e-2

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s).to(dtype)

    a, b, sg, w = rnd(N, C), rnd(N, C), rnd(N, 9), rnd(C) + 1
    for bb, ss in ((b, sg[:, 4:5]), (b, None), (None, None)):
        r0 = torch.randn(N, C, generator=g)
        rc, rg = r0.clone(), r0.clone().cuda()
        H.gated_sum_norm_accumulate(rc, a, bb, ss, w, 1e-3)
        H.gated_sum_norm_accumulate(rg, a.cuda(), None if bb is None else bb.cuda(), None if ss is None else sg.cuda()[:, 4:5], w.cuda(), 1e-3)
        assert (rg.cpu() - rc).abs().max() < tol
    o, gate = torch.randn(N, C, generator=g) * 3, rnd(N, 2 * C)
    want = H.norm_gate_rows(o, w, gate[:, C:], 1e-3, dtype)
    got = H.norm_gate_rows(o.cuda(), w.cuda(), gate.cuda()[:, C:], 1e-3, dtype)
    assert (got.float().cpu() - want.float()).abs().max() < tol * 4
    for bb, ss in ((b, sg[:, 4:5]), (None, None)):  # the rounded copy of the updated stream
        r0 = torch.randn(N, C, generator=g)
        rg, cp = r0.clone().cuda(), torch.empty(N, C, dtype=dtype, device="cuda")
        H.gated_sum_norm_accumulate(rg, a.cuda(), None if bb is None else bb.cuda(), None if ss is None else sg.cuda()[:, 4:5], w.cuda(),
                                    1e-3, copy=cp)
        assert torch.equal(cp, rg.to(dtype))
    gu = rnd(N, 2 * 24 + 8, s=2.0)
    for lim in (0.5, 7.0):
        want = H.act_mul(gu[:, :48], "clamped", lim)
        assert (H.act_mul(gu.cuda()[:, :48], "clamped", lim).float().cpu() - want.float()).abs().max() < tol * 4
    table, tk = rnd(11, C), torch.randint(0, 11, (N,), generator=g, dtype=torch.int32)
    assert torch.equal(H.embed_rows(table.cuda(), tk.cuda(), scale=2.5).cpu(), H.embed_rows(table, tk, scale=2.5))


def test_clamped_product_by_hand():
    g, u = torch.tensor([-3.0, 0.2, 5.0]), torch.tensor([4.0, -9.0, 0.3])
    lim = 1.0
    want = [min(a, lim) / (1 + math.exp(-1.702 * min(a, lim))) * (max(-lim, min(b, lim)) + 1) for a, b in zip(g.tolist(), u.tolist())]
    assert torch.allclose(H.glu(g, u, "clamped", lim), torch.tensor(want), atol=1e-6)
    assert torch.allclose(H.act_mul(torch.cat((g, u))[None], "clamped", lim)[0], torch.tensor(want), atol=1e-6)


# ---- query/key preparation: norm over the whole projection, then the rotation ---------------------------------
@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("borrow", [False, True])
def test_append_norms_the_whole_projection_then_rotates_and_writes_the_cache(dev, borrow):
    device, dtype = dev
    Hh, G, D, V, nrot, eps, base = 3, 2, 10, 7, 6, 1e-2, 40.0
    g = torch.Generator().manual_seed(3)
    lens, starts, slots = [5, 1, 9], [0, 17, 3], [2, 0, 1]
    N = sum(lens)
    q, k, v = torch.randn(N, Hh * D, generator=g) * 2, torch.randn(N, G * D, generator=g), torch.randn(N, G * V, generator=g)
    qw, kw = torch.rand(Hh * D, generator=g) + 0.5, torch.rand(G * D, generator=g) + 0.5
    q, k, v, qw, kw = (x.to(dtype).float() for x in (q, k, v, qw, kw))
    plan = BatchPlan.make(lens, slots, starts, torch.device(device))
    cache = torch.full((3, 32, G * (D + V)), 9.0, device=device, dtype=dtype)
    wide = torch.cat((q, k, v), 1).to(device=device, dtype=dtype)  # column slices of one matrix, as in the model
    qd = wide[:, :Hh * D]
    kd, vd = (None, None) if borrow else (wide[:, Hh * D:Hh * D + G * D], wide[:, Hh * D + G * D:])
    H.full_norm_append(qd, kd, vd, H.rotary_inv_freq(nrot, base, torch.device(device)), None if borrow else cache, plan,
                       Hh, G, D, V, nrot, eps, qw.to(device=device, dtype=dtype), None if borrow else kw.to(device=device, dtype=dtype))
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    row = 0
    for n, p0, slot in zip(lens, starts, slots):
        for i in range(n):
            wq = O.rms(q[row].double(), qw.double(), eps).view(Hh, D)
            wq = torch.stack([O.rotate_pairs(wq[a], p0 + i, nrot, base) for a in range(Hh)]).reshape(-1)
            assert (qd[row].float().cpu() - wq.float()).abs().max() < tol
            if not borrow:
                wk = O.rms(k[row].double(), kw.double(), eps).view(G, D)
                wk = torch.stack([O.rotate_pairs(wk[a], p0 + i, nrot, base) for a in range(G)]).reshape(-1)
                got = cache[slot, p0 + i].float().cpu()
                assert (got[:G * D] - wk.float()).abs().max() < tol and (got[G * D:] - v[row]).abs().max() < tol
            row += 1
    if borrow:
        assert bool((cache == 9.0).all())  # a borrowing layer writes nothing
    else:
        assert bool((cache[1, 12:] == 9.0).all()) and bool((cache[0, :17] == 9.0).all())


# ---- attention: sink, cap, far keys, the edge of what is visible ----------------------------------------------
def _plain_attention(q, k, v, pos, scale, cap, sink, rep):
    """q [H, D] at position pos over keys k [S, G, D], values v [S, G, V]: plain loops over heads and keys."""
    out = []
    for h in range(q.shape[0]):
        g = h // rep
        s = [float(q[h] @ k[j, g]) * scale for j in range(pos + 1)]
        if cap:
            s = [cap * math.tanh(x / cap) for x in s]
        mx = max(max(s), float(sink[h]))
        e = [math.exp(x - mx) for x in s]
        den = sum(e) + math.exp(float(sink[h]) - mx)
        out.append(sum(e[j] / den * v[j, g] for j in range(pos + 1)))
    return torch.cat(out)


def _attention_module(dev, Hh, G, D, V, scale, cap, sink):
    """A mixer whose output projection is the identity, with given sinks."""
    device, dtype = dev
    m = WindowAttention(Hh * V, {"heads": Hh, "kv_heads": G, "dim": D, "vdim": V, "scale": scale, "softcap": cap,
                                 "rot": {"dims": 0, "base": 10.0}}, 1e-3, TRAITS)
    for p in m.parameters():
        p.data = torch.zeros(p.shape)
    m.o.data = torch.eye(Hh * V)
    m.sink_w.data = sink.clone()
    m = m.to(device=device, dtype=dtype)
    m.finalize()
    return m


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("cap", [0.0, 6.0])
def test_one_key_stands_out_far_back_at_the_first_place_at_the_newest_and_never_a_later_one(dev, cap):
    device, dtype = dev
    S, G, D, V, rep, scale = 400, 2, 8, 6, 2, 0.5
    Hh = G * rep
    g = torch.Generator().manual_seed(4)
    k = torch.nn.functional.normalize(torch.randn(S, G, D, generator=g), dim=-1).to(dtype).float()
    v = torch.randn(S, G, V, generator=g).to(dtype).float()
    cache = torch.zeros(2, S, G * (D + V))
    cache[1, :, :G * D], cache[1, :, G * D:] = k.reshape(S, -1), v.reshape(S, -1)
    cache = cache.to(device=device, dtype=dtype)
    sink = torch.tensor([-1.0, 0.5, 2.0, -3.0])
    mod = _attention_module(dev, Hh, G, D, V, scale, cap, sink)
    tol = 2e-4 if dtype == torch.float32 else 4e-2
    aim = 24.0 if cap else 240.0  # without a cap the aimed-at key outweighs hundreds of others; with one, many scores saturate
    # decoding: one token at position pos, the query of every head aimed at one key
    for pos, target in ((399, 3), (399, 0), (399, 399), (200, 201), (64, 64), (65, 0), (0, 0), (0, 1)):
        q = torch.stack([k[target, h // rep] * aim for h in range(Hh)]).to(dtype).float()
        plan = BatchPlan.make([1], [1], [pos], torch.device(device))
        got = mod._attend(q.reshape(1, -1).to(device=device, dtype=dtype), torch.zeros(1, Hh, device=device, dtype=dtype), cache, plan)
        want = 0.5 * _plain_attention(q, k, v, pos, scale, cap, sink, rep)
        assert (got[0].float().cpu() - want).abs().max() < tol, (pos, target)
        if target <= pos and not cap:  # the aimed-at key takes nearly all the weight, whatever stands between
            assert (got[0].float().cpu() - 0.5 * v[target].repeat_interleave(rep, 0).reshape(-1)).abs().max() < 0.05
    # a prompt portion (the matrix-product form): rows 300..399 arrive together, each aimed at a key of its own
    n, p0 = 100, 300
    targets = [0, 299, 300, 7] + [p0 + i for i in range(4, n - 1)] + [p0 + n - 1 + 5 - S]  # the last aims past itself
    targets = [t % S for t in targets]
    q = torch.stack([torch.stack([k[t, h // rep] * aim for h in range(Hh)]) for t in targets]).to(dtype).float()
    plan = BatchPlan.make([n], [1], [p0], torch.device(device))
    got = mod._attend(q.reshape(n, -1).to(device=device, dtype=dtype), torch.zeros(n, Hh, device=device, dtype=dtype), cache, plan)
    for i in (0, 1, 2, 3, 4, 50, n - 2, n - 1):
        want = 0.5 * _plain_attention(q[i], k, v, p0 + i, scale, cap, sink, rep)
        assert (got[i].float().cpu() - want).abs().max() < tol, i


@pytest.mark.parametrize("dev", DEVICES)
def test_sink_takes_weight_without_a_value_and_differs_by_head(dev):
    device, dtype = dev
    S, G, D, V, rep = 70, 1, 4, 3, 3
    g = torch.Generator().manual_seed(5)
    k = (torch.randn(S, G, D, generator=g) * 0.1).to(dtype).float()
    v = (torch.ones(S, G, V) + torch.randn(S, G, V, generator=g) * 0.01).to(dtype).float()
    cache = torch.cat((k.reshape(S, -1), v.reshape(S, -1)), 1)[None].to(device=device, dtype=dtype)
    sink = torch.tensor([-30.0, math.log(S), 12.0])  # no weight; as much as all keys together; nearly everything
    mod = _attention_module(dev, rep, G, D, V, 1.0, 0.0, sink)
    for n, p0 in ((1, S - 1), (S, 0)):  # the one-token form and the matrix-product form
        q = torch.zeros(n, rep * D, device=device, dtype=dtype)
        plan = BatchPlan.make([n], [0], [p0], torch.device(device))
        got = mod._attend(q, torch.full((n, rep), 30.0, device=device, dtype=dtype), cache, plan)[-1].float().cpu().view(rep, V)
        assert (got[0] - 1).abs().max() < 0.05 and (got[1] - 0.5).abs().max() < 0.03 and got[2].abs().max() < 0.01


@pytest.mark.gpu
@pytest.mark.parametrize("keys", [37, 40, 1032, 2100])  # rows in registers (eight neighbours per thread or one) and re-read rows
@pytest.mark.parametrize("cap", [0.0, 2.5])
def test_softmax_kernel_with_cap_and_learned_sinks(keys, cap):
    g = torch.Generator().manual_seed(keys)
    heads, n = 3, 5
    s = torch.randn(2 * heads, n, keys, generator=g) * 6
    sink = torch.tensor([0.3, -2.0, 4.0])
    for out_dtype, split in ((torch.float32, False), (torch.bfloat16, True)):
        want = H.causal_softmax(s, keys - n, 0.7, out_dtype, sink=True, split=split, cap=cap, sink_vals=sink)
        got = H.causal_softmax(s.cuda(), keys - n, 0.7, out_dtype, sink=True, split=split, cap=cap, sink_vals=sink.cuda())
        assert (got.float().cpu() - want.float()).abs().max() < (1e-6 if out_dtype == torch.float32 else 1e-3)
    assert not torch.allclose(H.causal_softmax(s, keys - n, 0.7, torch.float32, sink=True, sink_vals=sink),
                              H.causal_softmax(s, keys - n, 0.7, torch.float32, sink=True))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_key_shares_of_the_decode_form_agree_with_cap_and_sinks(dtype):
    g = torch.Generator().manual_seed(1)
    S, Hh, G, D, V = 700, 4, 2, 16, 8
    cache = (torch.randn(1, S, G * (D + V), generator=g)).to(dtype).cuda()
    q, gate = (torch.randn(2, Hh * D, generator=g) * 2).to(dtype).cuda(), torch.randn(2, Hh, generator=g).to(dtype).cuda()
    plan = BatchPlan.make([2], [0], [S - 2], torch.device("cuda"))
    sink = torch.tensor([1.0, -1.0, 3.0, 0.0]).cuda()
    outs = [H.window_attn(q, gate, cache, plan, Hh, G, D, V, 0.4, 0, split=sp, sink=True, cap=5.0, sink_vals=sink) for sp in (1, 2, 7, 32)]
    want = H.window_attn(q.cpu(), gate.cpu(), cache.cpu(), BatchPlan.make([2], [0], [S - 2], torch.device("cpu")), Hh, G, D, V,
                         0.4, 0, sink=True, cap=5.0, sink_vals=sink.cpu())
    for o in outs:
        assert (o.float().cpu() - want.float()).abs().max() < (1e-5 if dtype == torch.float32 else 2e-2)


# ---- the fixed-decay recurrence ---------------------------------------------------------------------------------
def _plain_recurrence(q, k, v, decay, S0):
    """float64 loops: S <- decay S + k v^T; o = S^T q.  q, k [n, H, D], v [n, H, V]; returns o [n, H*V] and S."""
    S = S0.double().clone()
    out = []
    for t in range(q.shape[0]):
        row = []
        for h in range(q.shape[1]):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h].double(), v[t, h].double())
            row.append(S[h].T @ q[t, h].double())
        out.append(torch.cat(row))
    return torch.stack(out), S


RECURRENCE_DEVICES = [pytest.param(("cpu", 0), id="cpu"), pytest.param(("cuda", 1), id="cuda-scan", marks=pytest.mark.gpu),
                      pytest.param(("cuda", 2), id="cuda-chunks", marks=pytest.mark.gpu),
                      pytest.param(("cuda", 0), id="cuda-auto", marks=pytest.mark.gpu)]


@pytest.mark.parametrize("where", RECURRENCE_DEVICES)
@pytest.mark.parametrize("sizes", [(3, 12, 20), (1, 32, 32), (2, 16, 40), (2, 5, 36), (2, 40, 3), (1, 130, 70)], ids=str)
def test_recurrence_in_steps_of_every_size_with_state_carried_in_slots(where, sizes):
    """Three sequences in slots 2, 0, 1 advance together through steps of unequal sizes (one token, two, just below, at
    and above the chunk of 64 and the switch between the two kernels) and must match the plain loops at every token;
    decays from nearly nothing to exactly one."""
    device, variant = where
    Hh, D, V = sizes
    decay = torch.tensor([1e-3, 0.97, 1.0][:Hh] if Hh <= 3 else [0.5] * Hh)
    g = torch.Generator().manual_seed(7)
    steps = [[63, 1, 2], [1, 2, 15], [2, 64, 16], [64, 65, 17], [70, 1, 129], [1, 1, 1]]
    if D > 100:
        steps = steps[:4]
    slots = [2, 0, 1]
    state = torch.full((3, Hh, D, V), 0.0, device=device)
    ref = [torch.zeros(Hh, D, V, dtype=torch.float64) for _ in slots]
    worst = 0.0
    for lens in steps:
        N = sum(lens)
        q, k = torch.randn(N, Hh, D, generator=g) * 0.3, torch.randn(N, Hh, D, generator=g) * 0.3
        v = torch.randn(N, Hh, V, generator=g)
        plan = BatchPlan.make(lens, slots, [0] * 3, torch.device(device))
        act = N % 2 == 1  # some steps hand over pre-activations
        wide = torch.cat((q.reshape(N, -1), k.reshape(N, -1), v.reshape(N, -1)), 1).to(device)
        got = H.lightning_recurrence(wide[:, :Hh * D], wide[:, Hh * D:2 * Hh * D], wide[:, 2 * Hh * D:], decay.to(device), state, plan,
                                     Hh, D, V, variant=variant, act=act)
        if act:
            q, k, v = (torch.nn.functional.silu(x) for x in (q, k, v))
        r0 = 0
        for i, n in enumerate(lens):
            want, ref[i] = _plain_recurrence(q[r0:r0 + n], k[r0:r0 + n], v[r0:r0 + n], decay.tolist(), ref[i])
            worst = max(worst, ((got[r0:r0 + n].double().cpu() - want).abs().max() / want.abs().max().clamp_min(1.0)).item())
            r0 += n
    assert worst < 2e-5, worst
    for i, s in enumerate(slots):
        assert ((state[s].double().cpu() - ref[i]).abs().max() / ref[i].abs().max().clamp_min(1.0)).item() < 2e-5


@pytest.mark.parametrize("where", RECURRENCE_DEVICES)
def test_a_far_token_survives_a_slow_decay_and_not_a_fast_one(where):
    device, variant = where
    n, D, V = 300, 6, 4
    decay = torch.tensor([0.999, 0.8])
    q, k, v = torch.zeros(n, 2, D), torch.zeros(n, 2, D), torch.zeros(n, 2, V)
    k[3, :, 2], v[3, :, 1] = 5.0, 2.0   # written at position 3
    q[299, :, 2] = 1.0                  # asked for at position 299
    k[150, :, 4], v[150, :, 0] = 1.0, 1.0  # something else in between, on another key channel
    state = torch.zeros(1, 2, D, V, device=device)
    plan = BatchPlan.make([n], [0], [0], torch.device(device))
    o = H.lightning_recurrence(q.reshape(n, -1).to(device), k.reshape(n, -1).to(device), v.reshape(n, -1).to(device),
                               decay.to(device), state, plan, 2, D, V, variant=variant).cpu().view(n, 2, V)
    assert abs(o[299, 0, 1].item() - 10.0 * 0.999 ** 296) < 1e-3 and abs(o[299, 1, 1].item()) < 1e-20
    assert o[299, :, 0].abs().max() == 0 and o[:299].abs().max() == 0


# ---- router and experts ------------------------------------------------------------------------------------
def test_router_scores_all_outputs_corrects_the_choice_only_and_takes_the_lower_index_on_ties():
    z = torch.tensor([[1.0, 1.0, 0.0, 2.0, 1.0], [0.0, 0.0, 0.0, 0.0, 0.0]])
    s = torch.softmax(z, -1)
    idx, wt = H.router_topk(z, 2, "softmax_all")
    assert idx.tolist() == [[3, 0], [0, 1]]
    assert torch.allclose(wt[0], s[0, [3, 0]] / s[0, [3, 0]].sum())
    corr = torch.tensor([0.0, 0.0, 1.0, -1.0, 0.0])  # output 2 is chosen for its correction; its weight ignores it
    idx, wt = H.router_topk(z, 2, "softmax_all", corr)
    assert idx.tolist() == [[2, 0], [2, 0]]
    assert torch.allclose(wt[0], s[0, [2, 0]] / s[0, [2, 0]].sum()) and torch.allclose(wt.sum(-1), torch.ones(2))


@pytest.mark.gpu
def test_router_kernel_matches():
    g = torch.Generator().manual_seed(2)
    z = torch.randn(300, 11, generator=g) * 2
    z[5] = 0.0
    z[6, 3] = z[6, 8]
    corr = torch.randn(11, generator=g) * 0.1
    for c in (None, corr):
        ia, wa = H.router_topk(z, 4, "softmax_all", c)
        ib, wb = H.router_topk(z.cuda(), 4, "softmax_all", None if c is None else c.cuda())
        assert torch.equal(ia, ib.cpu()) and (wa - wb.cpu()).abs().max() < 1e-6


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("sizes", [(40, 24, 6, 2, 3), (33, 18, 4, 0, 1), (7, 8, 1, 3, 2), (1160, 1096, 3, 1, 2)],
                         ids=["identity", "plain", "mostly_identity", "long_rows"])
def test_expert_forms_agree_with_a_plain_loop(dev, sizes, monkeypatch):
    """The index-driven form (few tokens) and the sorted, grouped form (many) against plain loops, identity experts
    included; rows long enough for several chunks of the streamed kernel."""
    device, dtype = dev
    C, ff, E, ident, top = sizes
    g = torch.Generator().manual_seed(11)
    moe = MoEFF(C, ff, E, top, "softmax_all", False, "clamped", 0, ident, 1.2)
    for p in moe.parameters():
        p.data = (torch.randn(p.shape, generator=g) * (p.shape[-1] ** -0.5 if p.dim() == 2 else 0.05)).to(torch.bfloat16).float()
    moe = moe.to(device=device, dtype=dtype)
    moe.finalize()
    tol = 2e-4 if dtype == torch.float32 else 5e-2
    for N, gemv_max in ((5, 64), (90, 64), (90, 10 ** 6)):
        monkeypatch.setattr(MoEFF, "gemv_max", gemv_max)
        h = torch.randn(N, C, generator=g).to(dtype)
        got = moe(h.to(device)).float().cpu()
        W = {f"e{j}.{n}": getattr(moe, "e_" + n)[j].data.float().cpu() for j in range(E) for n in ("gate", "up", "down")}
        W["router"], W["correction"] = moe.router.data.float().cpu(), moe.correction.data.float().cpu()
        mlp = {"router": {"experts": E, "identity": ident, "top": top}, "expert": {"limit": 1.2}}
        if dtype == torch.float32:
            want = torch.stack([O.moe_ff(W, "", mlp, h[t].float()) for t in range(N)])
        else:  # 8-bit mantissas may flip a close choice: take the product's choice, check the arithmetic
            idx, wt = H.router_topk(H.linear_f32(h.to(device), moe.router32), top, "softmax_all", moe.correction32)
            want = torch.stack([sum(wt[t, j].item() * (O.clamped_expert(W, f"e{int(idx[t, j])}.", h[t].float(), 1.2) if int(idx[t, j]) < E
                                                      else h[t].float()) for j in range(top)) for t in range(N)])
        assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item()), (N, gemv_max)


# ---- whole models: prompts, decoding, portions, batches, slots ------------------------------------------------
@pytest.mark.parametrize("dev", DEVICES)
def test_whole_prompts_and_first_tokens(dev, monkeypatch):
    monkeypatch.setattr(WindowAttention, "query_block", 48)  # a prompt runs in several blocks of query rows
    d, m = build(FULL, dev)
    for n in (1, 2, 3, 15, 16, 17, 63, 64, 65, 150):  # the first tokens; the edges of both recurrence kernels and of the prompt form
        t = toks(n, seed=n)
        close(HybridRunner(m, 160).step([("a", t)], all_rows(n)), oracle_logits(d, m, t), dev, f"prompt of {n}")


@pytest.mark.parametrize("dev", DEVICES)
def test_residual_trace(dev):
    d, m = build(FULL, dev)
    t = toks(9)
    want = []
    oracle_logits(d, m, t, want)
    pool = m.new_pool(1, 16)
    plan = BatchPlan.make([len(t)], [pool.alloc()], [0], m.device)
    got = []
    m(torch.tensor(t, dtype=torch.int32, device=m.device), plan, pool, trace=got)
    assert len(got) == want[0].shape[0] == 5
    for i, g in enumerate(got):
        close(g, want[0][i].float(), dev, f"stream after layer {i}")


@pytest.mark.parametrize("dev", DEVICES)
def test_prefill_then_long_decode(dev):
    d, m = build(FULL, dev)
    t = toks(170, seed=3)
    want = oracle_logits(d, m, t)
    r = HybridRunner(m, 192)
    got = [r.step([("a", t[:30])], all_rows(30))]
    for p in range(30, 170):
        got.append(r.step([("a", [t[p]])]))
    close(torch.cat(got), want, dev, "decode")
    r2 = HybridRunner(m, 128)
    one = torch.cat([r2.step([("b", [x])]) for x in t[:20]])
    close(one, want[:20], dev, "token by token")


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("cuts", [(2, 3, 2, 64, 5, 70, 1, 2, 11), (66, 2, 92), (63, 65, 64, 16, 15, 17), (230,)],
                         ids=["small", "mixed", "kernel_edges", "whole"])
def test_portions_of_a_prompt(dev, cuts):
    d, m = build(FULL, dev)
    t = toks(sum(cuts), seed=5)
    want = oracle_logits(d, m, t)
    r = HybridRunner(m, 288)
    got, at = [], 0
    for c in cuts:
        got.append(r.step([("a", t[at:at + c])], all_rows(c)))
        at += c
    close(torch.cat(got), want, dev, f"portions {cuts}")


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("lengths", [(5, 19, 1, 9), (75, 64, 141)], ids=["short", "long"])
def test_unequal_batch_equals_each_alone_and_slots_are_reused(dev, lengths):
    d, m = build(FULL, dev)
    seqs = {f"s{i}": toks(n + 12, seed=10 + i) for i, n in enumerate(lengths)}
    want = {k: oracle_logits(d, m, v) for k, v in seqs.items()}
    r = HybridRunner(m, 192, n_slots=2)  # the pool has to grow; borrowed caches must follow
    live = list(seqs)
    out = r.step([(k, seqs[k][:n]) for k, n in zip(live, lengths)], [list(range(n)) for n in lengths])
    at = 0
    for k, n in zip(live, lengths):
        close(out[at:at + n], want[k][:n], dev, f"prompt {k}")
        at += n
    pos = dict(zip(live, lengths))
    for stepno in range(12):
        if stepno == 4:  # one request ends early; its slot goes back
            r.end_sample(live.pop(1))
        out = r.step([(k, [seqs[k][pos[k]]]) for k in live])
        for i, k in enumerate(live):
            close(out[i:i + 1], want[k][pos[k]:pos[k] + 1], dev, f"decode {k} at {pos[k]}")
            pos[k] += 1
    for k in live:
        r.end_sample(k)
    assert not r.pool.length
    t = toks(75, seed=99)  # freed slots serve a new request: nothing of the old cache or state shows
    close(r.step([("new", t)], all_rows(75)), oracle_logits(d, m, t), dev, "reused slot")
    for run, (li, _) in zip(r.pool.runs, m.config.layer_runs()):  # a borrowed cache is the lender's tensor, also after growth
        src = m.config.layers[li]["mixer"].get("kv_from")
        if src is not None:
            assert run["cache"] is r.pool.runs[src]["cache"]


@pytest.mark.parametrize("dev", DEVICES)
def test_pool_grows_while_requests_are_held(dev):
    d, m = build(FULL, dev)
    seqs = [toks(n, seed=20 + i) for i, n in enumerate((80, 66, 140, 71, 5))]
    want = [oracle_logits(d, m, t) for t in seqs]
    r = HybridRunner(m, 192, n_slots=2)
    r.step([(0, seqs[0][:70]), (1, seqs[1][:60])])
    for s in range(3):  # the third one-token step of this batch size runs as a captured graph on the GPU
        out = r.step([(0, [seqs[0][70 + s]]), (1, [seqs[1][60 + s]])])
        close(out, torch.stack((want[0][70 + s], want[1][60 + s])), dev, f"before growth {s}")
    out = r.step([(i, seqs[i]) for i in (2, 3, 4)])
    assert r.pool.n_slots >= 5
    close(out, torch.stack([want[i][-1] for i in (2, 3, 4)]), dev, "arrivals")
    for s in range(3, 6):
        out = r.step([(0, [seqs[0][70 + s]]), (1, [seqs[1][60 + s]])])
        close(out, torch.stack((want[0][70 + s], want[1][60 + s])), dev, f"after growth {s}")


@pytest.mark.parametrize("dev", DEVICES)
def test_greedy_generation_through_the_runner(dev):
    d, m = build(FULL, dev)
    prompts = [toks(5, seed=1), toks(11, seed=2)]
    r = HybridRunner(m, 32)
    out = r.generate(prompts, 6, SamplingParams.greedy())
    assert not r.pool.length
    if dev[1] == torch.float32:
        for p, o in zip(prompts, out):
            seq = list(p)
            for _ in range(6):
                seq.append(int(oracle_logits(d, m, seq)[-1].argmax()))
            assert o == seq


# ---- checkpoint, registry, command line ---------------------------------------------------------------------
def test_checkpoint_roundtrip_registry_and_trace_cli(tmp_path):
    d, m = build(FULL, ("cpu", torch.float32))
    ck = tmp_path / "ck"
    ck.mkdir()
    m.config.save(ck)
    tensors = {k: v.to(torch.bfloat16) for k, v in m.state_tensors().items()}
    assert "l3.mix.k" not in tensors and "l3.mix.v.b" not in tensors and "l3.mix.q.norm" in tensors
    assert tensors["l1.mlp.router"].shape[0] == 7 and "l1.mlp.e4.gate" in tensors and "l1.mlp.e5.gate" not in tensors
    write_safetensors(tensors, ck / "model.safetensors")
    cfg_cls, model_cls = model_classes("Zudovik")
    assert cfg_cls is HybridConfig and model_cls is HybridLM
    m2 = load_hybrid(ck, "cpu", torch.float32)
    c = m2.config
    assert c.block == "postnorm" and c.embed_scale == 3.0 and m2.head_w is not None
    assert HybridConfig.from_dict(c.asdict()).asdict() == c.asdict()
    with pytest.raises(KeyError):
        HybridLM(c).load_tensors({k: v for k, v in tensors.items() if k != "l2.mix.sink"}, "cpu", torch.float32)
    t = toks(12)
    want = oracle_logits(d, m2, t)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": t[:8], "want": [0, 7]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": t[8:9], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": t[9:10], "want": [0]}, ], "end": ["x"]},
             {"step": 3, "entries": [{"id": "y", "tokens": t, "want": [11]}], "end": ["y"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(ck), "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "16", "--device", "cpu"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    import numpy as np

    def rd(i):
        return torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, 50).copy())

    assert not (out / "1.f32").exists()
    close(rd(0), want[[0, 7]], ("cpu", torch.float32))
    close(rd(2), want[[9]], ("cpu", torch.float32))
    close(rd(3), want[[11]], ("cpu", torch.float32))


def test_sample_command_line_serves_the_checkpoint(tmp_path, capsys):
    from mdi_llm_b200.cli import sample

    d, m = build(all_experts(FULL), ("cpu", torch.float32))
    ck = tmp_path / "ck"
    ck.mkdir()
    m.config.save(ck)
    write_safetensors({k: v.to(torch.bfloat16) for k, v in m.state_tensors().items()}, ck / "model.safetensors")
    assert sample.main(["--ckpt", str(ck), "--prompt", "decays", "--n-samples", "2", "--n-tokens", "5", "--greedy",
                        "--device", "cpu", "--dtype", "float32"]) == 0
    out = capsys.readouterr().out
    ids = [b % 50 for b in b"decays"]
    want = []
    for _ in range(5):
        want.append(int(oracle_logits(d, m, ids + want)[-1].argmax()))
    assert out.count(" ".join(map(str, want))) == 2, out


def test_config_validation():
    with pytest.raises(ValueError):  # more choices than router outputs
        HybridConfig.from_dict(cfg_dict([light(mlp={"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 2, "identity": 1, "top": 4}})]))
    with pytest.raises(ValueError):  # clamped experts need their limit
        HybridConfig.from_dict(cfg_dict([light(mlp={"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "top": 1}})]))
    with pytest.raises(ValueError):  # one decay per head
        HybridConfig.from_dict(cfg_dict([light(heads=2, decay=(0.5,))]))
    with pytest.raises(ValueError):  # the lender comes first and lends its own keys
        HybridConfig.from_dict(cfg_dict([attn(kv_from=1), attn()]))
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([attn(), attn(kv_from=0), attn(kv_from=1)]))
    with pytest.raises(ValueError):  # a borrower has the lender's key and value sizes
        HybridConfig.from_dict(cfg_dict([attn(), attn(dim=16, kv_from=0)]))
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([light(), attn(kv_from=0)]))
    pool = HybridLM(HybridConfig.from_dict(cfg_dict([attn(), attn(kv_from=0)]))).init_random("cpu", torch.float32).new_pool(2, 8)
    assert pool.runs[1]["cache"] is pool.runs[0]["cache"] and pool.nbytes == pool.runs[0]["cache"].numel() * 4
