"""Model configuration (litGPT-compatible) for the B200 MDI engine.

Parity target: reference ``src/sub/model.py:94-273`` (``Config`` dataclass, ``from_name``,
``from_file``, ``from_checkpoint``, ``asdict``) and the registry in
``src/sub/config.py:170-1669``.  The field set and the ``model_config.yaml`` schema are kept
so checkpoints written by the reference load unchanged.  Two things are new:

* a GPT-2 family (learned positional embedding, LayerNorm with bias, tied ``lm_head``) can be
  expressed (``pos_embedding="learned"``, ``tie_embeddings=True``) — the reference needs a
  separate legacy tree for that (``old/GPT2/sub/model.py``);
* derived, kernel-facing quantities (``q_per_kv``, ``qkv_size``, ``kv_dim`` ...) are
  properties so the CUDA ops and the eager model agree on one definition.
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, Dict, Optional, Union

import yaml

__all__ = ["Config", "GPTConfig", "HybridConfig", "find_multiple"]


def find_multiple(n: int, k: int) -> int:
    """Smallest multiple of ``k`` that is >= ``n``."""
    if k <= 0:
        raise ValueError("k must be positive")
    return n if n % k == 0 else n + k - (n % k)


# Fields that exist in the reference's ``Config.asdict`` (model.py:245-273) — this is the
# on-disk ``model_config.yaml`` schema.  Extension fields are only emitted when they differ
# from their defaults so that reference-written/reference-read files stay valid.
_REFERENCE_FIELDS = (
    "name", "hf_config", "scale_embeddings", "block_size", "vocab_size", "padding_multiple",
    "padded_vocab_size", "n_layer", "n_head", "head_size", "n_embd", "rotary_percentage",
    "parallel_residual", "bias", "lm_head_bias", "n_query_groups", "shared_attention_norm",
    "norm_class_name", "norm_eps", "mlp_class_name", "gelu_approximate", "intermediate_size",
    "rope_condense_ratio", "rope_base", "n_expert", "n_expert_per_token",
)
_EXTENSION_DEFAULTS = {"pos_embedding": "rope", "tie_embeddings": False}


@dataclass
class Config:
    name: str = ""
    hf_config: dict = field(default_factory=dict)
    scale_embeddings: bool = False
    block_size: int = 4096
    vocab_size: int = 50254
    padding_multiple: int = 512
    padded_vocab_size: Optional[int] = None
    n_layer: int = 16
    n_head: int = 32
    head_size: Optional[int] = None
    n_embd: int = 4096
    rotary_percentage: float = 0.25
    parallel_residual: bool = True
    bias: bool = True
    lm_head_bias: bool = False
    n_query_groups: Optional[int] = None
    shared_attention_norm: bool = False
    norm_class_name: str = "LayerNorm"  # "LayerNorm" | "RMSNorm"
    norm_eps: float = 1e-5
    mlp_class_name: str = "GptNeoxMLP"  # GptNeoxMLP | LLaMAMLP | GemmaMLP | LLaMAMoE
    gelu_approximate: str = "none"
    intermediate_size: Optional[int] = None
    rope_condense_ratio: int = 1
    rope_base: int = 10000
    n_expert: int = 0
    n_expert_per_token: int = 0
    # ---- extensions (not in the reference schema) -------------------------------------
    pos_embedding: str = "rope"  # "rope" | "learned" (GPT-2 family: adds transformer.wpe)
    tie_embeddings: bool = False  # lm_head.weight is wte.weight (GPT-2 family)

    def __post_init__(self) -> None:
        if not self.name:
            self.name = self.hf_config.get("name", self.name)
        if self.head_size is None:
            if self.n_embd % self.n_head:
                raise ValueError("n_embd must be divisible by n_head when head_size is unset")
            self.head_size = self.n_embd // self.n_head
        if self.padded_vocab_size is None:
            self.padded_vocab_size = find_multiple(self.vocab_size, self.padding_multiple)
        else:
            self.vocab_size = min(self.vocab_size, self.padded_vocab_size)
        if self.n_query_groups is None:
            self.n_query_groups = self.n_head
        elif self.n_head % self.n_query_groups:
            raise ValueError("n_head must be a multiple of n_query_groups")
        if self.intermediate_size is None:
            if self.mlp_class_name == "LLaMAMLP":
                raise ValueError(f"config {self.name!r} must set `intermediate_size`")
            self.intermediate_size = 4 * self.n_embd
        if self.pos_embedding not in ("rope", "learned"):
            raise ValueError(f"unknown pos_embedding {self.pos_embedding!r}")
        self.rope_n_elem = int(self.rotary_percentage * self.head_size)
        if self.pos_embedding == "learned":
            self.rope_n_elem = 0

    # ---- derived quantities shared by eager model and CUDA ops -------------------------
    @property
    def q_per_kv(self) -> int:
        return self.n_head // self.n_query_groups

    @property
    def qkv_size(self) -> int:
        """Rows of the fused, group-interleaved QKV projection (model.py:644)."""
        return (self.n_head + 2 * self.n_query_groups) * self.head_size

    @property
    def kv_dim(self) -> int:
        return self.n_query_groups * self.head_size

    @property
    def attn_out_dim(self) -> int:
        return self.n_head * self.head_size

    @property
    def unit_offset_norm(self) -> bool:
        """Gemma adds 1 to the RMSNorm weight (model.py:242)."""
        return self.norm_class_name == "RMSNorm" and "Gemma" in self.name

    def block_param_count(self) -> int:
        """Parameters of one transformer block (used by the balanced stage planner)."""
        c, i = self.n_embd, self.intermediate_size
        attn = self.qkv_size * c + c * self.attn_out_dim
        if self.mlp_class_name in ("LLaMAMLP", "GemmaMLP"):
            mlp = 3 * c * i
        elif self.mlp_class_name == "LLaMAMoE":
            mlp = self.n_expert * 3 * c * i + c * self.n_expert
        else:
            mlp = 2 * c * i
        return attn + mlp + 2 * c

    def head_param_count(self) -> int:
        """Parameters the starter reads per token on top of its blocks (ln_f + lm_head)."""
        return self.padded_vocab_size * self.n_embd + self.n_embd

    # ---- constructors ------------------------------------------------------------------
    @classmethod
    def from_name(cls, name: str, **kwargs: Any) -> "Config":
        from .registry import lookup

        conf = dict(lookup(name))
        conf.update(kwargs)
        return cls(**conf)

    @classmethod
    def from_file(cls, path: Union[str, Path], **kwargs: Any) -> "Config":
        with open(path, encoding="utf-8") as fp:
            loaded = yaml.safe_load(fp)
        if loaded is None:
            raise ValueError(f"{path} is empty")
        known = {f.name for f in fields(cls)}
        loaded = {k: v for k, v in loaded.items() if k in known}
        loaded.update(kwargs)
        return cls(**loaded)

    @classmethod
    def from_checkpoint(cls, path: Union[str, Path], **kwargs: Any) -> "Config":
        path = Path(path)
        cfg_file = path / "model_config.yaml"
        if cfg_file.is_file():
            return cls.from_file(cfg_file, **kwargs)
        from .registry import name_to_config

        if path.name in name_to_config:
            return cls.from_name(path.name, **kwargs)
        raise FileNotFoundError(
            f"{str(path)!r}: neither 'model_config.yaml' nor a registry entry named {path.name!r}"
        )

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Config":
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})

    def asdict(self) -> Dict[str, Any]:
        out = {k: getattr(self, k) for k in _REFERENCE_FIELDS}
        for k, default in _EXTENSION_DEFAULTS.items():
            if getattr(self, k) != default:
                out[k] = getattr(self, k)
        return out

    def save(self, checkpoint_dir: Union[str, Path]) -> Path:
        """Write ``model_config.yaml`` (reference ``utils.py:608-611``)."""
        p = Path(checkpoint_dir) / "model_config.yaml"
        with open(p, "w", encoding="utf-8") as fp:
            yaml.safe_dump(self.asdict(), fp)
        return p


def GPTConfig(block_size: int = 1024, vocab_size: int = 50304, n_layer: int = 12, n_head: int = 12, n_embd: int = 768,
              dropout: float = 0.0, bias: bool = True, activation_function: str = "GELU", **extra: Any) -> Config:
    """The second-generation (GPT-2 / nanoGPT) configuration object as a factory for :class:`Config`
    (reference ``old/GPT2/sub/model.py:38-62``): learned positions, LayerNorm, GELU MLP, tied head.
    ``dropout`` is accepted and ignored (inference / the trainer here run without dropout)."""
    if activation_function.upper() != "GELU":
        raise ValueError("only the GELU MLP of GPT-2 is supported")
    return Config(name=extra.pop("name", f"gpt2-custom-{n_layer}l"), block_size=block_size, vocab_size=vocab_size,
                  padded_vocab_size=vocab_size, n_layer=n_layer, n_head=n_head, n_embd=n_embd, rotary_percentage=0.0,
                  parallel_residual=False, bias=bias, norm_class_name="LayerNorm", mlp_class_name="GptNeoxMLP",
                  gelu_approximate="tanh", pos_embedding="learned", tie_embeddings=True, **extra)


# =============================================================================================
# hybrid family: a list of heterogeneous layers (attention and recurrent mixers) read from config.json
# =============================================================================================
MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale", "rot"),
    "gla": ("heads", "dim", "vdim", "tau"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "lightning": ("heads", "dim", "vdim", "decay"),
}

# What an architecture of the family fixes beyond its config.json: the shape of a block ("sandwich": norms before and
# after each sublayer; "prenorm": one norm before, the sublayer output times ``residual_mult`` added; "parallel": one
# norm whose output both the mixer and the feed-forward read, their outputs summed into the residual), the kind of
# "postnorm": the sublayer reads the residual stream itself and its *output* is normed before it is added),
# its norms (``norm_offset`` is added to every block-level norm weight: 1 for weights stored as deviations from one),
# whether the output head is the embedding table or a tensor of its own, whether a learned position vector joins the
# token embedding (``positions``), whether each branch of a block has a learned scale per channel (``layer_scale``),
# and the variant of the grouped-query attention mixer and of the mixture of experts:
#   attention: mask "window" (the last mask.size positions) | "chunk" (the query's own block of mask.size positions);
#              sink: True (a zero-score slot in the softmax denominator) | "learned" (its score is a tensor, one number
#              per head); qk_norm "unit" (divide by the RMS) | "weight" (RMS norm with a learned weight per entry,
#              shared by the heads) | "full" (RMS norm over the WHOLE projection, all heads at once, with a weight per
#              entry, BEFORE the rotation); bias on q, k, v; gate "head" | "channel";
#              p32 (the prompt form sums the values with softmax weights of more than the activation type's mantissa:
#              fp32 weights, or with 16-bit activations their rounding and its remainder as two 16-bit operands)
#   moe:       router "sigmoid" (independent scores) | "softmax" (over the chosen logits) | "softmax_all" (scores are
#              the softmax over all router outputs, the choice goes by score + a ``correction`` tensor, the weights are
#              the chosen scores divided by their sum); router_bias; expert "relu2" (down relu(up x)^2, the score scales
#              the input) | "gated_silu" (down (silu(gate x) * up x), the score weighs the output) | "clamped" (gate and
#              up clamped by the entry's ``limit``, g sigmoid(1.702 g) (u + 1)); a ``shared`` always-on expert is read
#              from the layer's mlp entry; shared_gate: the shared expert's output is weighed by one sigmoid per token
#   dense_act: activation of a dense feed-forward, "gelu" (erf) | "relu2"
# Per layer, an attention mixer may also name ``softcap`` (scores pass through cap * tanh(score / cap)) and
# ``kv_from: j`` (no key/value projections: it reads the keys and values layer j cached); a mixture of experts may name
# ``router.identity`` (that many extra router outputs whose "expert" returns its input).
_ATTENTION_DEFAULT = {"mask": "window", "sink": False, "qk_norm": "unit", "bias": False, "gate": "head", "p32": False}
_MOE_DEFAULT = {"router": "sigmoid", "router_bias": False, "expert": "relu2", "shared_gate": False}
ARCHITECTURE_TRAITS = {
    "Badapel": {"block": "sandwich", "norm": "layer", "tied_head": True},
    "Vudelix": {"block": "prenorm", "norm": "rms", "tied_head": False},
    "Labepel": {"block": "parallel", "norm": "rms", "norm_offset": 1.0, "tied_head": True, "positions": "learned",
                "layer_scale": True,
                "attention": {"mask": "chunk", "sink": True, "qk_norm": "weight", "bias": True, "gate": "channel", "p32": True},
                "moe": {"router": "softmax", "router_bias": True, "expert": "gated_silu"}},
    "Zudovik": {"block": "postnorm", "norm": "rms", "tied_head": False, "dense_act": "relu2",
                "attention": {"mask": "window", "sink": "learned", "qk_norm": "full", "bias": True, "gate": "head", "p32": True},
                "moe": {"router": "softmax_all", "expert": "clamped", "shared_gate": True}},
}
FF_KINDS = ("dense", "moe")


@dataclass
class HybridConfig:
    """A decoder whose layers each name their own mixer and sizes (``config.json`` of the hybrid family).

    ``layers[i] = {"type": <mixer kind>, "mixer": {...sizes...}, "mlp": {"kind": "dense", "ff": n} | None}``.
    ``loop = {"start", "stop", "times"}`` repeats layers ``start..stop-1`` ``times`` times with shared weights and a
    state of its own per pass; each pass starts with a re-injection of the embedding output.  Everything a model
    of the family may vary is a field; nothing is assumed from a particular checkpoint.

    A feed-forward is ``{"kind": "dense", "ff": n}`` or a mixture of experts ``{"kind": "moe", "expert": {"ff": n},
    "router": {"experts": E, "top": k}}``.  ``residual_mult`` scales every sublayer output before it joins the
    residual stream (pre-norm blocks); ``token_side = {"dim": d}`` gives every layer a second, per-layer embedding of
    the current token (a ``d``-wide slice of one table) that is gated by the residual stream and added to it.
    ``block``, ``norm``, ``norm_offset``, ``tied_head``, ``positions``, ``layer_scale`` and the mixer variants
    ``attention`` / ``moe`` come from :data:`ARCHITECTURE_TRAITS` unless given.  ``max_positions`` is the length of the
    learned position table (``positions = "learned"``).  A mixture of experts may name a ``shared`` expert
    (``{"ff": n}``) that every token uses.  ``embed_scale`` (``embedding.scale``) multiplies the token embedding.
    """

    architecture: str = "Badapel"
    vocab: int = 0
    width: int = 0
    layers: list = field(default_factory=list)
    loop: Optional[dict] = None
    norm_eps: float = 1e-6
    logit_softcap: float = 0.0
    name: str = ""
    residual_mult: float = 1.0
    token_side: Optional[dict] = None
    block: str = ""
    norm: str = ""
    tied_head: Optional[bool] = None
    max_positions: int = 0
    norm_offset: Optional[float] = None
    positions: str = ""
    layer_scale: Optional[bool] = None
    attention: Optional[dict] = None
    moe: Optional[dict] = None
    embed_scale: float = 1.0
    dense_act: str = ""

    def __post_init__(self) -> None:
        traits = ARCHITECTURE_TRAITS.get(self.architecture, ARCHITECTURE_TRAITS["Badapel"])
        self.block = self.block or traits["block"]
        self.norm = self.norm or traits["norm"]
        if self.tied_head is None:
            self.tied_head = traits["tied_head"]
        if self.norm_offset is None:
            self.norm_offset = float(traits.get("norm_offset", 0.0))
        self.positions = self.positions or traits.get("positions", "none")
        if self.layer_scale is None:
            self.layer_scale = bool(traits.get("layer_scale", False))
        self.attention = {**_ATTENTION_DEFAULT, **traits.get("attention", {}), **(self.attention or {})}
        self.moe = {**_MOE_DEFAULT, **traits.get("moe", {}), **(self.moe or {})}
        self.dense_act = self.dense_act or traits.get("dense_act", "gelu")
        if self.dense_act not in ("gelu", "relu2"):
            raise ValueError(f"unknown dense feed-forward activation {self.dense_act!r}")
        if self.block not in ("sandwich", "prenorm", "parallel", "postnorm") or self.norm not in ("layer", "rms"):
            raise ValueError(f"unknown block {self.block!r} or norm {self.norm!r}")
        if self.positions not in ("none", "learned") or (self.positions == "learned" and self.max_positions < 1):
            raise ValueError("learned positions need max_positions >= 1")
        if self.attention["mask"] not in ("window", "chunk") or self.attention["qk_norm"] not in ("unit", "weight", "full") \
                or self.attention["gate"] not in ("head", "channel") or self.attention["sink"] not in (False, True, "learned") \
                or self.moe["router"] not in ("sigmoid", "softmax", "softmax_all") \
                or self.moe["expert"] not in ("relu2", "gated_silu", "clamped"):
            raise ValueError(f"unknown attention or mixture-of-experts variant: {self.attention} {self.moe}")
        if self.token_side is not None and int(self.token_side.get("dim", 0)) <= 0:
            raise ValueError("token_side needs a positive dim")
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("a hybrid config needs vocab, width and at least one layer")
        for i, spec in enumerate(self.layers):
            kind = spec.get("type")
            if kind not in MIXER_KEYS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            missing = [k for k in MIXER_KEYS[kind] if k not in spec.get("mixer", {})]
            if missing:
                raise ValueError(f"layer {i} ({kind}): missing mixer fields {missing}")
            mlp = spec.get("mlp")
            if mlp is not None and mlp.get("kind") not in FF_KINDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            if mlp is not None and mlp["kind"] == "moe":
                r = mlp.get("router", {})
                if not (1 <= int(r.get("top", 0)) <= int(r.get("experts", 0)) + int(r.get("identity", 0) or 0)) \
                        or int(r.get("experts", 0)) < 1 or int(mlp.get("expert", {}).get("ff", 0)) <= 0:
                    raise ValueError(f"layer {i}: a mixture of experts needs expert.ff and 1 <= router.top <= router.experts")
                if mlp.get("shared") and int(mlp["shared"].get("ff", 0)) <= 0:
                    raise ValueError(f"layer {i}: a shared expert needs a positive ff")
                if int(r.get("identity", 0) or 0) < 0 or int(r["top"]) > int(r["experts"]) + int(r.get("identity", 0) or 0):
                    raise ValueError(f"layer {i}: router.identity is a count of extra router outputs")
                if self.moe["expert"] == "clamped" and ("limit" not in mlp["expert"] or (mlp.get("shared") and "limit" not in mlp["shared"])):
                    raise ValueError(f"layer {i}: clamped experts need a limit")
            m = spec["mixer"]
            if kind in ("attention", "channel_delta") and int(m["heads"]) % int(m["kv_heads"]):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if kind == "lightning" and len(m["decay"]) != int(m["heads"]):
                raise ValueError(f"layer {i}: one decay per head")
            if kind == "attention" and m.get("kv_from") is not None:
                j = int(m["kv_from"])
                src = self.layers[j] if 0 <= j < i else None
                if src is None or src.get("type") != "attention" or src["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from names an earlier attention layer with projections of its own")
                if any(src["mixer"][k] != m[k] for k in ("kv_heads", "dim", "vdim")) or src["mixer"].get("rot") != m.get("rot"):
                    raise ValueError(f"layer {i}: kv_from needs the source layer's kv_heads, dim, vdim and rotation")
        if self.loop is not None:
            a, b, t = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not (0 <= a < b <= len(self.layers)) or t < 1:
                raise ValueError(f"bad loop {self.loop}")
        if not self.name:
            self.name = self.architecture

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def padded_vocab_size(self) -> int:
        return self.vocab

    def layer_runs(self) -> list:
        """Execution order as ``(layer index, starts a pass)``; a looped layer appears once per pass."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        runs = [(i, False) for i in range(a)]
        for _ in range(times):
            runs += [(i, i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, n)]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "HybridConfig":
        return cls(architecture=d.get("architecture", "Badapel"), vocab=int(d["vocab"]), width=int(d["width"]),
                   layers=[dict(x) for x in d["layers"]], loop=dict(d["loop"]) if d.get("loop") else None,
                   norm_eps=float(d.get("norm", {}).get("eps", 1e-6)),
                   logit_softcap=float(d.get("logit_softcap") or 0.0), name=d.get("name", ""),
                   residual_mult=float(d.get("residual_mult", 1.0)),
                   token_side=dict(d["token_side"]) if d.get("token_side") else None,
                   max_positions=int(d.get("max_positions") or 0),
                   embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)))

    @classmethod
    def from_file(cls, path: Union[str, Path]) -> "HybridConfig":
        import json

        with open(path, encoding="utf-8") as fp:
            return cls.from_dict(json.load(fp))

    def asdict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "layers": self.layers, "norm": {"eps": self.norm_eps}}
        if self.loop is not None:
            out["loop"] = self.loop
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.residual_mult != 1.0:
            out["residual_mult"] = self.residual_mult
        if self.token_side is not None:
            out["token_side"] = self.token_side
        if self.max_positions:
            out["max_positions"] = self.max_positions
        if self.embed_scale != 1.0:
            out["embedding"] = {"scale": self.embed_scale}
        return out

    def save(self, checkpoint_dir: Union[str, Path]) -> Path:
        import json

        p = Path(checkpoint_dir) / "config.json"
        with open(p, "w", encoding="utf-8") as fp:
            json.dump(self.asdict(), fp, indent=1)
        return p
