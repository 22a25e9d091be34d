"""The Labepel design (parallel blocks of the hybrid family) against the plain oracle of ``labepel_oracle.py``.

Every test builds its own small configuration with random weights.  Sizes are awkward on purpose: value width != key
width, chunk sizes that are neither the head size nor the threshold of the prompt form, chunks of one position and
chunks longer than any prompt, a layer without a mask, several query heads per key head and exactly one, one and several
experts per token, a feed-forward without the shared expert, a layer without feed-forward, value mixing that starts at a
later layer than the first.  The same tests run on the CPU (PyTorch bodies of the operations) and, marked ``gpu``, on
the sm_100a kernels.
"""
from __future__ import annotations

import copy
import json
import os
import subprocess
import sys

import pytest
import torch

import labepel_oracle as O
from mdi_llm_b200.models.config import HybridConfig
from mdi_llm_b200.models.hybrid import GatedFF, HybridLM, MoEFF, WindowAttention, load_hybrid, write_safetensors
from mdi_llm_b200.models.registry import model_classes
from mdi_llm_b200.ops import hybrid as H
from mdi_llm_b200.ops.hybrid import BatchPlan
from mdi_llm_b200.parallel.hybrid_runner import HybridRunner
from mdi_llm_b200.parallel.scheduler import SamplingParams

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRAITS = {"mask": "chunk", "sink": True, "qk_norm": "weight", "bias": True, "gate": "channel", "p32": True}

MOE = {"kind": "moe", "expert": {"ff": 20}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 28}}
MOE_BARE = {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 3, "top": 1}}


def att(heads=6, kv=2, dim=12, vdim=10, scale=0.4, size=7, v_mix=True, mlp=MOE):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix}
    if size:
        m["mask"] = {"size": size}
    return {"type": "attention", "mixer": m, "mlp": copy.deepcopy(mlp)}


def cfg_dict(layers, width=24, vocab=50, positions=300, eps=1e-3):
    return {"architecture": "Labepel", "vocab": vocab, "width": width, "max_positions": positions,
            "layers": copy.deepcopy(layers), "norm": {"eps": eps}}


def all_experts(d):
    """The same model with every expert chosen for every token: no routing decision that 8-bit mantissas could flip."""
    d = copy.deepcopy(d)
    for spec in d["layers"]:
        if spec["mlp"]:
            spec["mlp"]["router"]["top"] = spec["mlp"]["router"]["experts"]
    return d


# chunk 7 with mixing off, chunk 70 (above the prompt-form threshold) that starts the mixing, no feed-forward and one
# head per key head with chunk 1... and a layer whose chunk is longer than every prompt
FULL = cfg_dict([att(v_mix=False), att(heads=4, kv=2, dim=8, vdim=10, scale=1.3, size=70, mlp=MOE_BARE),
                 att(heads=2, kv=2, dim=16, vdim=10, scale=0.7, size=3, mlp=None), att(heads=2, kv=1, dim=8, vdim=20, size=500)])

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
    W = {k: v.detach().cpu() for k, v in model.state_tensors().items()}
    lg, layers = O.forward(W, d, list(tokens))
    if trace is not None:
        trace.extend(layers)
    return lg.float()


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
    "attention": [att(v_mix=False, mlp=None)],
    "one_head_per_key_head": [att(heads=3, kv=3, dim=8, vdim=16, scale=1.5, size=5, v_mix=False, mlp=None)],
    "no_mask": [att(size=0, v_mix=False, mlp=None)],
    "chunk_of_one": [att(size=1, v_mix=False, mlp=None)],
    "chunk_longer_than_prompt": [att(size=64, v_mix=False, mlp=None)],
    "value_mixing": [att(mlp=None), att(mlp=None, size=4), att(mlp=None, v_mix=False), att(mlp=None, size=9)],
    "experts": [att(heads=1, kv=1, dim=6, vdim=4, v_mix=False, mlp=MOE_BARE)],
    "experts_top3": [att(heads=1, kv=1, dim=6, vdim=4, v_mix=False,
                         mlp={"kind": "moe", "expert": {"ff": 9}, "router": {"experts": 7, "top": 3}})],
    "experts_and_shared": [att(heads=1, kv=1, dim=6, vdim=4, v_mix=False, mlp=MOE)],
}


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("case", list(CASES))
def test_each_mechanism_alone(dev, case):
    d, m = build(cfg_dict(CASES[case]), dev)
    t = toks(41)
    close(HybridRunner(m, 64).step([("a", t)], all_rows(len(t))), oracle_logits(d, m, t), dev, case)


@pytest.mark.parametrize("dev", DEVICES)
def test_positions_are_added_and_bounded(dev):
    d, m = build(cfg_dict([att(size=0, v_mix=False, mlp=None)], positions=12), dev)
    t = [7] * 12  # one token everywhere: without the position vectors every row would repeat the pattern of a constant
    got = HybridRunner(m, 64).step([("a", t)], all_rows(12))
    close(got, oracle_logits(d, m, t), dev, "positions")
    assert (got[0] - got[1]).abs().max() > 1e-2
    with pytest.raises(ValueError):
        HybridRunner(m, 64).step([("b", [7] * 13)])
    with pytest.raises(ValueError):
        HybridConfig.from_dict({**cfg_dict([att()]), "max_positions": 0})


def test_norm_weight_is_a_deviation_from_one():
    x = torch.randn(5, 16, generator=torch.Generator().manual_seed(0))
    w = torch.randn(16, generator=torch.Generator().manual_seed(1)) * 0.1
    got = H.norm_rows(x, w, None, 1e-2, "rms", torch.float32, w_offset=1.0)
    assert torch.allclose(got.double(), O.norm_one_plus(x.double(), w, 1e-2), atol=1e-6)
    assert torch.allclose(H.norm_rows(x, w, None, 1e-2, "rms", torch.float32).double(), O.norm_plain(x.double(), w, 1e-2), atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_kernels_match_their_plain_forms(dtype):
    g = torch.Generator().manual_seed(3)
    N, C, Fh = 37, 40, 22
    tol = 1e-5 if dtype == torch.float32 else 0.03
    dev = torch.device("cuda")
    # norm with an offset weight (bf16 weight, fp32 sum)
    x, w = torch.randn(N, C, generator=g), (torch.randn(C, generator=g) * 0.1).to(dtype)
    got = H.norm_rows(x.cuda(), w.cuda(), None, 1e-3, "rms", dtype, w_offset=1.0)
    assert (got.double().cpu() - O.norm_one_plus(x.double(), w, 1e-3)).abs().max() < tol
    # embedding + learned positions
    table, ptab = torch.randn(11, C, generator=g).to(dtype), torch.randn(30, C, generator=g).to(dtype)
    plan = BatchPlan.make([5, 3], [0, 1], [4, 27], dev)
    tk = torch.tensor([1, 9, 3, 3, 0, 10, 2, 2], dtype=torch.int32)
    got = H.embed_rows(table.cuda(), tk.cuda(), ptab.cuda(), plan)
    want = table[tk.long()].float() + ptab[[4, 5, 6, 7, 8, 27, 28, 29]].float()
    assert got.dtype == torch.float32 and torch.equal(got.cpu(), want)
    # gated activation on the two halves of a strided row
    wide = torch.randn(N, 2 * Fh + 6, generator=g).to(dtype)
    got = H.act_mul(wide.cuda()[:, 3:3 + 2 * Fh])
    a, b = wide[:, 3:3 + Fh].double(), wide[:, 3 + Fh:3 + 2 * Fh].double()
    assert (got.double().cpu() - a * torch.sigmoid(a) * b).abs().max() < tol * 4
    # residual update of a parallel block
    r = torch.randn(N, C, generator=g)
    ya, yb, yc = (torch.randn(N, C, generator=g).to(dtype) for _ in range(3))
    l1, l2 = (torch.randn(C, generator=g).to(dtype) for _ in range(2))
    for b_, c_, s2 in ((yb, yc, l2), (yb, None, l2), (None, None, None), (yb, yc, None)):
        rr = r.clone().cuda()
        H.scaled_branches(rr, ya.cuda(), l1.cuda(), None if b_ is None else b_.cuda(), None if c_ is None else c_.cuda(),
                          None if s2 is None else s2.cuda())
        want = r.double() + ya.double() * l1.double()
        if b_ is not None:
            want = want + (b_.double() + (c_.double() if c_ is not None else 0)) * (s2.double() if s2 is not None else 1.0)
        assert (rr.double().cpu() - want).abs().max() < 1e-5


# ---- the softmax with a sink -------------------------------------------------------------------------------------
@pytest.mark.parametrize("dev", DEVICES)
def test_softmax_with_a_sink(dev):
    device, dtype = dev
    g = torch.Generator().manual_seed(5)
    s = torch.randn(3, 9, 14, generator=g) * 4.0
    s[1, 4] = -40.0  # every visible score far below the sink's zero: the weights all but vanish
    s[2, 8, :3] = 30.0  # and far above: the sink all but vanishes
    first, key0, scale = 7, 2, 0.6
    got = H.causal_softmax(s.to(device).contiguous(), first, scale, torch.float32, key0=key0, sink=True).cpu()
    i = first + torch.arange(9)[:, None]
    j = key0 + torch.arange(14)[None, :]
    want = O.softmax_with_sink(s.double() * scale, (j <= i).expand(3, 9, 14))
    assert (got.double() - want).abs().max() < 1e-6
    assert got[1, 4].sum() < 1e-6 and abs(got[2, 8].sum() - 1.0) < 1e-5
    plain = H.causal_softmax(s.to(device).contiguous(), first, scale, torch.float32, key0=key0).cpu()
    assert torch.allclose(plain.sum(-1), torch.ones(3, 9), atol=1e-5) and (got.sum(-1) <= 1.0 + 1e-6).all() and got.sum(-1).mean() < 0.97
    # the weights as two halves of the 16-bit type: together they carry 16 bits of mantissa
    halves = H.causal_softmax(s.to(device).contiguous(), first, scale, torch.bfloat16, key0=key0, sink=True, split=True).double().cpu()
    assert halves.shape == (3, 9, 28)
    assert ((halves[..., :14] + halves[..., 14:] - want).abs() <= want * 2.0 ** -15 + 1e-30).all()


@pytest.mark.gpu
@pytest.mark.parametrize("keys", [37, 40, 1032, 2048, 2100],  # rows kept in registers (eight neighbours per thread when
                         ids=["odd", "short", "five_warps", "register_limit", "long"])  # they come in eights), and rows that are not
@pytest.mark.parametrize("sink", [False, True])
def test_softmax_kernel_matches_its_plain_form_for_short_and_long_rows(keys, sink):
    g = torch.Generator().manual_seed(keys)
    s = torch.randn(2, 6, keys, generator=g) * 3.0
    first, key0, window = keys - 9, 4, 37
    for kw in ({}, {"window": window}):
        want = H.causal_softmax(s, first, 0.5, torch.float32, key0=key0, sink=sink, **kw)
        got = H.causal_softmax(s.cuda(), first, 0.5, torch.float32, key0=key0, sink=sink, **kw).cpu()
        assert (got - want).abs().max() < 1e-6 and torch.equal(got == 0, want == 0)
        halves = H.causal_softmax(s.cuda(), first, 0.5, torch.bfloat16, key0=key0, sink=sink, split=True, **kw).float().cpu()
        assert ((halves[..., :keys] + halves[..., keys:] - want).abs() <= want * 2.0 ** -15 + 1e-30).all()
    # rows that see no key at all (they lie before the first column): zeros, not NaN
    got = H.causal_softmax(s.cuda(), 0, 0.5, torch.float32, key0=3, sink=sink).cpu()
    assert torch.equal(got[:, :3], torch.zeros(2, 3, keys)) and not got.isnan().any()


def test_router_softmax_over_the_chosen_lower_index_on_ties():
    z = torch.tensor([[0.1, 2.0, 2.0, -1.0], [3.0, -2.0, 0.5, 0.5]])
    idx, wt = H.router_topk(z, 3, "softmax")
    assert idx.tolist() == [[1, 2, 0], [0, 2, 3]]
    assert torch.allclose(wt, torch.softmax(torch.tensor([[2.0, 2.0, 0.1], [3.0, 0.5, 0.5]]), -1))
    for t in range(2):
        chosen, w = O.route(z[t].double(), 3)
        assert chosen == idx[t].tolist() and torch.allclose(w.float(), wt[t])
    idx1, wt1 = H.router_topk(z, 1, "softmax")
    assert idx1.tolist() == [[1], [0]] and wt1.tolist() == [[1.0], [1.0]]


@pytest.mark.gpu
def test_router_kernel_matches():
    z = torch.randn(300, 9, generator=torch.Generator().manual_seed(0)) * 3
    z[5, 3] = z[5, 7] = 9.0
    for top in (1, 4, 9):
        i0, w0 = H.router_topk(z, top, "softmax")
        i1, w1 = H.router_topk(z.cuda(), top, "softmax")
        assert torch.equal(i0, i1.cpu()) and torch.allclose(w0, w1.cpu(), atol=1e-6)
        assert torch.allclose(w1.sum(-1).cpu(), torch.ones(300), atol=1e-5)


# ---- prompts, decoding, portions, batches -------------------------------------------------------------------
@pytest.mark.parametrize("dev", DEVICES)
def test_whole_prompts_and_first_tokens(dev, monkeypatch):
    monkeypatch.setattr(WindowAttention, "score_bytes", 4 * 4 * 70 * 70)  # one chunk of the widest layer per product
    monkeypatch.setattr(WindowAttention, "query_block", 16)  # a partial chunk runs in several blocks of query rows
    d, m = build(FULL, dev)
    for n in (1, 2, 3, 4, 7, 8, 69, 70, 71, 150):  # the first tokens; the edges of the chunks of 3, 7 and 70
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
    assert len(got) == len(want) == 4
    for i, (g, w) in enumerate(zip(got, want)):
        close(g, w.float(), dev, f"stream after layer {i}")


@pytest.mark.parametrize("dev", DEVICES)
def test_prefill_then_long_decode(dev):
    d, m = build(FULL, dev)
    t = toks(170, seed=3)
    want = oracle_logits(d, m, t)
    r = HybridRunner(m, 192)
    got = [r.step([("a", t[:30])], all_rows(30))]
    for p in range(30, 170):  # decoding crosses the edges of the chunks of 3 and 7 many times, of 70 twice
        got.append(r.step([("a", [t[p]])]))
    close(torch.cat(got), want, dev, "decode")
    r2 = HybridRunner(m, 128)
    one = torch.cat([r2.step([("b", [x])]) for x in t[:20]])
    close(one, want[:20], dev, "token by token")


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("cuts", [(2, 3, 2, 64, 5, 70, 1, 2, 11), (66, 2, 92), (69, 71, 70, 64), (230,)],
                         ids=["small", "mixed", "chunk_edges", "whole"])
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
    r = HybridRunner(m, 192, n_slots=2)  # the pool has to grow
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
    t = toks(75, seed=99)  # freed slots serve a new request: nothing of the old cache shows
    close(r.step([("new", t)], all_rows(75)), oracle_logits(d, m, t), dev, "reused slot")


@pytest.mark.parametrize("dev", DEVICES)
def test_pool_grows_while_requests_are_held(dev):
    """Two requests decode (on the GPU: through a captured step), three more arrive as a batch of their own and the
    pool has to grow: the new ones start clean and the old ones go on from the state they had."""
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


# ---- chunk edges and far keys: one score made to stand out -------------------------------------------------------
def _sharp_case(dev, S=160, G=2, D=8, V=6):
    """A cache of unit keys and random values in slot 1 of 2."""
    device, dtype = dev
    g = torch.Generator().manual_seed(4)
    k = torch.nn.functional.normalize(torch.randn(S, G, D, generator=g), dim=-1)
    v = torch.randn(S, G, V, generator=g)
    cache = torch.zeros(2, S, G * (D + V))
    cache[1, :, :G * D] = k.reshape(S, -1)
    cache[1, :, G * D:] = v.reshape(S, -1)
    return k, v, cache.to(device=device, dtype=dtype)


def _plain_chunk(q, k, v, pos, W, scale, rep):
    """q [H, D] at position pos over keys k [S, G, D], values v [S, G, V]: plain loops, sink included."""
    first = (pos // W) * W
    out = []
    for h in range(q.shape[0]):
        g = h // rep
        e = [torch.exp((q[h] @ k[j, g]) * scale) for j in range(first, pos + 1)]
        den = 1.0 + sum(e)
        out.append(sum(e[j - first] / den * v[j, g] for j in range(first, pos + 1)))
    return torch.cat(out)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("W", [5, 33, 64])
def test_keys_just_inside_and_outside_the_chunk_and_far_back(dev, W):
    device, dtype = dev
    G, rep, D, V, S = 2, 3, 8, 6, 160
    Hh = G * rep
    k, v, cache = _sharp_case(dev)
    kq, vq = k.to(dtype).double(), v.to(dtype).double()
    tol = 1e-4 if dtype == torch.float32 else 0.05
    att_ = WindowAttention(16, {"heads": Hh, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.5, "mask": {"size": W}}, 1e-5, TRAITS)
    for target in ("chunk_start", "before_chunk", "first", "self"):
        pick = {"chunk_start": lambda p: (p // W) * W, "before_chunk": lambda p: max(0, (p // W) * W - 1), "first": lambda p: 0,
                "self": lambda p: p}[target]
        q = torch.stack([12.0 * k[pick(p)].repeat_interleave(rep, 0) for p in range(S)]).to(dtype)  # [S, H, D]
        want = torch.stack([_plain_chunk(q[p].double(), kq, vq, p, W, 0.5, rep) for p in range(S)]).float()
        qd = q.reshape(S, Hh * D).to(device)
        for p in (0, 1, W - 1, W, W + 1, 2 * W - 1, 2 * W, S - 1):  # decoding around the edges
            plan = BatchPlan.make([1], [1], [p], torch.device(device))
            got = H.window_attn(qd[p:p + 1].contiguous(), None, cache, plan, Hh, G, D, V, 0.5, W, mask="chunk", sink=True)
            assert (got.float().cpu() - want[p]).abs().max() < tol, (target, p)
        for p0, n in ((37, 100), (W, min(2 * W, S - W)), (3, S - 3)):  # portions that start inside a chunk and at its edge, both forms
            plan = BatchPlan.make([n], [1], [p0], torch.device(device))
            got = H.window_attn(qd[p0:p0 + n].contiguous(), None, cache, plan, Hh, G, D, V, 0.5, W, mask="chunk", sink=True)
            assert (got.float().cpu() - want[p0:p0 + n]).abs().max() < tol, target
            got = att_._chunked(qd[p0:p0 + n].contiguous(), cache, plan).permute(1, 0, 2).reshape(n, Hh * V)
            assert (got.float().cpu() - want[p0:p0 + n]).abs().max() < tol, target
    # the last key of the chunk before must not show although the query points at it
    p = 2 * W
    plan = BatchPlan.make([1], [1], [p], torch.device(device))
    q = (12.0 * k[p - 1].repeat_interleave(rep, 0)).reshape(1, -1).to(device=device, dtype=dtype)
    got = H.window_attn(q, None, cache, plan, Hh, G, D, V, 0.5, W, mask="chunk", sink=True).float().cpu().view(Hh, V)
    assert (got[0] - v[p - 1, 0]).abs().max() > 0.2


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("V", [6, 8, 136])  # one channel per lane; four per lane; a second pass of 128 channels
def test_key_shares_of_the_decode_form_agree(dtype, V):
    G, rep, D, W = 2, 3, 8, 70
    k, v, cache = _sharp_case(("cuda", dtype), V=V)
    g = torch.Generator().manual_seed(1)
    q = (torch.randn(3, G * rep * D, generator=g) * 3).to(device="cuda", dtype=dtype)
    gate = torch.randn(3, G * rep * V, generator=g).to(device="cuda", dtype=dtype)
    plan = BatchPlan.make([1, 1, 1], [1, 1, 1], [3, 70, 139], torch.device("cuda"))  # 4, 1 and 70 visible keys
    one = H.window_attn(q, gate, cache, plan, G * rep, G, D, V, 0.8, W, split=1, mask="chunk", sink=True)
    for split in (0, 2, 5):  # shares that get no tile at all
        got = H.window_attn(q, gate, cache, plan, G * rep, G, D, V, 0.8, W, split=split, mask="chunk", sink=True)
        assert (got.float() - one.float()).abs().max() < (1e-5 if dtype == torch.float32 else 0.02), split
    cpu = H.window_attn(q.cpu(), gate.cpu(), cache.cpu(), BatchPlan.make([1, 1, 1], [1, 1, 1], [3, 70, 139], torch.device("cpu")),
                        G * rep, G, D, V, 0.8, W, mask="chunk", sink=True)
    assert (one.float().cpu() - cpu.float()).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("dev", DEVICES)
def test_append_normalises_with_weights_mixes_values_and_writes_the_cache(dev):
    device, dtype = dev
    Hh, G, D, V, eps = 4, 2, 10, 6, 1e-3
    g = torch.Generator().manual_seed(2)
    N = 9
    q, k, v, vf = (torch.randn(N, n, generator=g) for n in (Hh * D, G * D, G * V, G * V))
    qw, kw = torch.randn(D, generator=g) + 1.5, torch.randn(D, generator=g) - 1.5
    lam = torch.tensor([0.3])
    plan = BatchPlan.make([4, 5], [2, 0], [3, 0], torch.device(device))
    to = lambda x: x.to(device=device, dtype=dtype)
    tol = 1e-5 if dtype == torch.float32 else 0.03
    for mix in (False, True):
        cache = torch.zeros(3, 12, G * (D + V), device=device, dtype=dtype)
        qd = to(q).clone()
        H.window_append(qd, to(k), to(v), None, cache, plan, Hh, G, D, V, 0, eps, to(qw), to(kw),
                        to(vf) if mix else None, to(lam) if mix else None)
        qr, kr, vr, vfr = (x.to(dtype).double() for x in (q, k, v, vf))
        for row, (slot, pos) in enumerate([(2, 3), (2, 4), (2, 5), (2, 6), (0, 0), (0, 1), (0, 2), (0, 3), (0, 4)]):
            for h in range(Hh):
                want = O.norm_plain(qr[row, h * D:(h + 1) * D], qw.to(dtype), eps)
                assert (qd[row, h * D:(h + 1) * D].double().cpu() - want).abs().max() < tol
            for h in range(G):
                want = O.norm_plain(kr[row, h * D:(h + 1) * D], kw.to(dtype), eps)
                assert (cache[slot, pos, h * D:(h + 1) * D].double().cpu() - want).abs().max() < tol
            lm = lam.to(dtype).double()
            want = (1 - lm) * vr[row] + lm * vfr[row] if mix else vr[row]
            assert (cache[slot, pos, G * D:].double().cpu() - want).abs().max() < tol
        assert cache[1].abs().sum() == 0 and cache[2, :3].abs().sum() == 0  # other slots and positions untouched


# ---- mixture of experts: the two forms against a plain loop -------------------------------------------------
@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("sizes", [(40, 24, 6, 3), (33, 18, 4, 1), (7, 8, 2, 2), (1160, 1096, 3, 2)],
                         ids=["top3", "top1", "all", "long_rows"])  # long rows: several chunks of a streamed weight row, the last partial
def test_expert_forms_agree_with_a_plain_loop(dev, sizes, monkeypatch):
    device, dtype = dev
    C, ff, E, top = sizes
    g = torch.Generator().manual_seed(7)
    moe = MoEFF(C, ff, E, top, "softmax", True, "gated_silu", shared_ff=ff + 3)
    for p in moe.parameters():
        p.data = (torch.randn(p.shape, generator=g) * p.shape[-1] ** -0.5).to(device=device, dtype=dtype)
    moe.finalize()
    N = 50
    h = torch.randn(N, C, generator=g).to(device=device, dtype=dtype)
    T = {"x." + n: p.detach().cpu() for n, p in moe.names().items()}
    hd = h.double().cpu()
    idx, wt = H.router_topk(H.linear_f32(h, moe.router32, moe.router_b32), top, "softmax")
    want = torch.zeros(N, C, dtype=torch.float64)
    for t in range(N):
        for j in range(top):
            want[t] += wt[t, j].double().cpu() * O.gated_expert(hd[t:t + 1], T, f"x.e{int(idx[t, j])}.")[0]
    tol = 1e-4 if dtype == torch.float32 else 0.08
    monkeypatch.setattr(MoEFF, "gemv_max", 10 ** 6)
    a = moe(h)
    monkeypatch.setattr(MoEFF, "gemv_max", 0)
    b = moe(h)
    for got, what in ((a, "index-driven"), (b, "grouped")):
        assert (got.double().cpu() - want).abs().max() < tol * max(1.0, want.abs().max().item()), what
    monkeypatch.setattr(MoEFF, "gemv_max", 10 ** 6)
    # a token's result does not depend on its neighbours in the batch beyond the rounding of the router's product
    assert (moe(h[3:4]).float() - a[3:4].float()).abs().max() < (1e-5 if dtype == torch.float32 else 0.02)
    assert isinstance(moe.shared, GatedFF)
    sh = moe.shared(h)
    assert (sh.double().cpu() - O.gated_expert(hd, T, "x.shared.")).abs().max() < tol * 4
    if dtype == torch.float32 and device == "cpu":  # the oracle's own routing agrees with the operation's
        z = O.lin(hd, T["x.router"], T["x.router.b"])
        for t in range(N):
            chosen, w = O.route(z[t], top)
            assert chosen == idx[t].tolist() and torch.allclose(w.float(), wt[t], atol=1e-5)


# ---- checkpoint, registry, command line ---------------------------------------------------------------------
def test_checkpoint_roundtrip_registry_and_trace_cli(tmp_path):
    d, m = build(FULL, ("cpu", torch.float32))
    ck = tmp_path / "ck"
    ck.mkdir()
    m.config.save(ck)
    tensors = {k: v.to(torch.bfloat16) for k, v in m.state_tensors().items()}
    # tensors a layer has no use for are tolerated: a mixing factor on a layer that mixes nothing, the
    # feed-forward scale of a layer without feed-forward
    tensors["l0.mix.vmix"] = torch.tensor(0.5, dtype=torch.bfloat16)
    tensors["l2.ls2"] = torch.ones(24, dtype=torch.bfloat16)
    write_safetensors(tensors, ck / "model.safetensors")
    cfg_cls, model_cls = model_classes("Labepel")
    assert cfg_cls is HybridConfig and model_cls is HybridLM
    m2 = load_hybrid(ck, "cpu", torch.float32)
    c = m2.config
    assert c.block == "parallel" and c.norm == "rms" and c.norm_offset == 1.0 and c.tied_head and m2.head_w is None
    assert c.positions == "learned" and c.max_positions == 300 and c.layer_scale and c.attention["sink"]
    assert HybridConfig.from_dict(c.asdict()).asdict() == c.asdict()
    with pytest.raises(KeyError):
        HybridLM(c).load_tensors({k: v for k, v in tensors.items() if k != "l1.mix.vmix"}, "cpu", torch.float32)
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
    """``sample --ckpt`` on a self-describing folder: registry -> loader -> runner -> greedy sampling; the printed ids
    continue the byte-level prompt exactly as the oracle's argmax does."""
    from mdi_llm_b200.cli import sample

    d, m = build(all_experts(FULL), ("cpu", torch.float32))
    ck = tmp_path / "ck"
    ck.mkdir()
    m.config.save(ck)
    write_safetensors({k: v.to(torch.bfloat16) for k, v in m.state_tensors().items()}, ck / "model.safetensors")
    assert sample.main(["--ckpt", str(ck), "--prompt", "chunks", "--n-samples", "2", "--n-tokens", "5", "--greedy",
                        "--device", "cpu", "--dtype", "float32"]) == 0
    out = capsys.readouterr().out
    ids = [b % 50 for b in b"chunks"]
    want = []
    for _ in range(5):
        want.append(int(oracle_logits(d, m, ids + want)[-1].argmax()))
    assert out.count(" ".join(map(str, want))) == 2, out


def test_config_validation():
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([att(mlp={"kind": "moe", "expert": {"ff": 8}, "router": {"experts": 2, "top": 3}})]))
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([att(mlp={**MOE, "shared": {"ff": 0}})]))
    with pytest.raises(ValueError):
        HybridConfig.from_dict(cfg_dict([att(heads=6, kv=4)]))
    with pytest.raises(ValueError):  # value-mixing layers share one value width
        _, m = build(cfg_dict([att(mlp=None), att(mlp=None, vdim=12)]), ("cpu", torch.float32))
        HybridRunner(m, 8).step([("a", [1, 2])])
