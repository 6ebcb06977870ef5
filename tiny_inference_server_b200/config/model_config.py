"""Typed model configuration, read from ``config.json``.

The upstream project keeps its model constants in one dataclass shared with training
(``Config/config.py:5-23``: ``D_MODEL, VOCAB_SIZE, MAX_CONTEXT, MAX_FREQ, N_HEAD,
NUM_LAYERS, FFN_HIDDEN_DIM, NUM_GROUPS, MTP_HEADS``) and has no ``config.json``.  Here
every size and constant of the model comes from ``config.json``; the upstream names
are accepted as aliases of the lower-case keys.  No size is written into code.
"""
from __future__ import annotations

import copy
import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import Any, ClassVar, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model; the message names every problem."""


# upstream Config field -> key of config.json  (Config/config.py:11-23)
UPSTREAM_ALIASES = {
    "D_MODEL": "hidden_size",
    "VOCAB_SIZE": "vocab_size",
    "MAX_CONTEXT": "max_context",
    "MAX_FREQ": "rope_theta",
    "N_HEAD": "num_heads",
    "NUM_LAYERS": "num_layers",
    "FFN_HIDDEN_DIM": "ffn_hidden",
    "MTP_HEADS": "num_mtp_heads",
}


@dataclass
class GqaMtpConfig:
    """Configuration of the bias-free pre-norm GQA decoder with MTP heads
    (``main_models_new.py:174-194``).

    Required keys have no default.  Defaults of the optional keys are the constants
    that the upstream code fixes: eps ``main_models_new.py:36``, RoPE base and table
    length ``Config/config.py:13-14``, end-of-sequence id ``server.py:12``.
    """

    architecture: ClassVar[str] = "gqa_mtp_transformer"

    vocab_size: int
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    ffn_hidden: int
    head_dim: Optional[int] = None            # default hidden_size // num_heads (main_models_new.py:91)
    rms_norm_eps: float = 2e-8
    rope_theta: float = 10000.0
    max_context: int = 8192
    tie_word_embeddings: bool = True
    num_mtp_heads: int = 0
    eos_token_id: Optional[int] = None
    # engine options that the upstream model does not have
    sliding_window: Optional[int] = None       # keys p-window+1..p instead of 0..p
    full_attention_layers: Optional[list] = None   # layers (0..L-1 trunk, L+i = MTP head i) exempt from the window
    layer_order: Optional[list] = None         # order in which trunk layers run; may name a layer twice
    cache_source: Optional[list] = None        # per entry of layer_order: None, or an earlier entry whose K/V it reads
    mixer_types: Optional[list] = None         # per trunk layer, a name of the mixer registry (default "gqa")
    ffn_types: Optional[list] = None           # per trunk layer, a name of the feed-forward registry (default "swiglu")
    norm_type: str = "rmsnorm_l2"
    position_type: str = "rope_half"
    torch_dtype: str = "bfloat16"              # dtype the weights are stored in

    def __post_init__(self):
        errs = []
        for name in ("vocab_size", "hidden_size", "num_layers", "num_heads", "num_kv_heads", "ffn_hidden"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                errs.append(f"{name} must be a positive integer, got {v!r}")
        if errs:
            raise ConfigError("; ".join(errs))
        if self.head_dim is None:
            if self.hidden_size % self.num_heads:
                errs.append(f"hidden_size {self.hidden_size} is not a multiple of num_heads {self.num_heads} "
                            f"and head_dim is not given")
            self.head_dim = self.hidden_size // self.num_heads
        if self.num_heads % self.num_kv_heads:
            errs.append(f"num_heads {self.num_heads} is not a multiple of num_kv_heads {self.num_kv_heads}")
        if self.head_dim % 2:
            errs.append(f"head_dim {self.head_dim} must be even for rotary position encoding")
        if not (self.rms_norm_eps >= 0):
            errs.append(f"rms_norm_eps must be >= 0, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            errs.append(f"rope_theta must be > 0, got {self.rope_theta}")
        if self.max_context <= 0:
            errs.append(f"max_context must be positive, got {self.max_context}")
        if self.num_mtp_heads < 0:
            errs.append(f"num_mtp_heads must be >= 0, got {self.num_mtp_heads}")
        if self.sliding_window is not None and self.sliding_window <= 0:
            errs.append(f"sliding_window must be positive or null, got {self.sliding_window}")
        n_all = self.num_layers + self.num_mtp_heads
        for l in self.full_attention_layers or []:
            if not (0 <= l < n_all):
                errs.append(f"full_attention_layers names layer {l}, outside 0..{n_all - 1}")
        order = self.layer_order if self.layer_order is not None else list(range(self.num_layers))
        for l in order:
            if not (isinstance(l, int) and 0 <= l < self.num_layers):
                errs.append(f"layer_order names layer {l!r}, outside 0..{self.num_layers - 1}")
        if self.cache_source is not None:
            if len(self.cache_source) != len(order):
                errs.append(f"cache_source has {len(self.cache_source)} entries, layer_order has {len(order)}")
            else:
                for e, s in enumerate(self.cache_source):
                    if s is None:
                        continue
                    if not (isinstance(s, int) and 0 <= s < e):
                        errs.append(f"cache_source[{e}]={s!r} must name an earlier entry")
                    elif self.cache_source[s] is not None:
                        errs.append(f"cache_source[{e}]={s} names an entry that has no cache of its own")
                    elif all(isinstance(l, int) and 0 <= l < self.num_layers for l in (order[e], order[s])):
                        # pages of the source's group are given back by the source's window: a reader
                        # that sees further back would walk pages that other requests hold by then
                        mine, theirs = self.window_of(order[e]), self.window_of(order[s])
                        if theirs is not None and (mine is None or mine > theirs):
                            errs.append(f"cache_source[{e}]={s}: layer {order[e]} sees "
                                        f"{'every key' if mine is None else f'{mine} keys'} but layer {order[s]}, "
                                        f"whose cache it reads, keeps only {theirs}")
        for key in ("mixer_types", "ffn_types"):
            v = getattr(self, key)
            if v is not None and len(v) != self.num_layers:
                errs.append(f"{key} has {len(v)} entries for {self.num_layers} layers")
        if self.torch_dtype not in ("bfloat16", "float32"):
            errs.append(f"torch_dtype must be bfloat16 or float32, got {self.torch_dtype!r}")
        if errs:
            raise ConfigError("; ".join(errs))

    # ---- derived ----
    @property
    def group_size(self) -> int:
        """Query heads per kv head (the upstream ``NUM_GROUPS``, Config/config.py:22)."""
        return self.num_heads // self.num_kv_heads

    def schedule(self):
        """[(layer index, entry whose cache is read or None)] in running order."""
        order = self.layer_order if self.layer_order is not None else list(range(self.num_layers))
        src = self.cache_source if self.cache_source is not None else [None] * len(order)
        return list(zip(order, src))

    def window_of(self, layer_index: int) -> Optional[int]:
        if self.sliding_window is None:
            return None
        if layer_index in (self.full_attention_layers or []):
            return None
        return int(self.sliding_window)

    # ---- (de)serialisation ----
    @classmethod
    def from_dict(cls, raw: dict) -> "GqaMtpConfig":
        d = {}
        for k, v in raw.items():
            d[UPSTREAM_ALIASES.get(k, k)] = v
        d.pop("architecture", None)
        if "NUM_GROUPS" in d:
            g = d.pop("NUM_GROUPS")
            if "num_heads" not in d:
                raise ConfigError("NUM_GROUPS given without N_HEAD / num_heads")
            if "num_kv_heads" not in d:
                if g <= 0 or d["num_heads"] % g:
                    raise ConfigError(f"N_HEAD {d['num_heads']} is not a multiple of NUM_GROUPS {g}")
                d["num_kv_heads"] = d["num_heads"] // g
        known = {f.name for f in dataclasses.fields(cls)}
        unknown = sorted(set(d) - known)
        required = [f.name for f in dataclasses.fields(cls)
                    if f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING]
        missing = [k for k in required if k not in d]
        if unknown or missing:
            parts = []
            if missing:
                parts.append("missing keys: " + ", ".join(missing))
            if unknown:
                parts.append("unknown keys: " + ", ".join(unknown))
            raise ConfigError(f"config for architecture {cls.architecture!r}: " + "; ".join(parts))
        return cls(**d)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture}
        for f in dataclasses.fields(self):
            d[f.name] = getattr(self, f.name)
        return d


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    with open(path) as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return raw


def write_config_json(folder: str, cfg: Any) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f, indent=1)


@dataclass
class KefisunConfig:
    """Configuration of the Kefisun decoder: pre-norm layers whose mixer is either windowed attention with a
    logarithmic distance bias or the delta rule with a decay per key channel, every mixer behind a short causal
    convolution of its input, a clamped gated feed-forward in the layers that have one, tied output matrix.

    ``config.json`` is nested: ``vocab``, ``width``, ``embedding.scale``, ``logit_scale``, ``norm.eps``,
    ``canon.taps`` (the taps of the convolution in front of every mixer; no ``canon``: none) and ``layers``, a
    list with, per layer, ``type`` (``attention`` | ``channel_delta``), ``mixer`` (its sizes and constants) and
    ``mlp`` (``kind``, ``ff``, ``limit``; null: the layer has no feed-forward).  The design has no position
    table and no context limit of its own: ``max_context`` (optional) bounds what the engine lays out.
    """

    architecture: ClassVar[str] = "Kefisun"
    MIXERS: ClassVar[tuple] = ("attention", "channel_delta")

    vocab_size: int
    hidden_size: int
    layers: list
    rms_norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    canon_taps: Optional[int] = None
    max_context: int = 1 << 17
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    def __post_init__(self):
        errs = []
        for name in ("vocab_size", "hidden_size"):
            v = getattr(self, name)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                errs.append(f"{name} must be a positive integer, got {v!r}")
        if not isinstance(self.layers, list) or not self.layers:
            errs.append("layers must be a non-empty list")
            raise ConfigError("; ".join(errs))
        if self.canon_taps is not None and not (isinstance(self.canon_taps, int) and 1 <= self.canon_taps <= 16):
            errs.append(f"canon.taps must be 1..16, got {self.canon_taps!r}")
        if not (self.rms_norm_eps >= 0):
            errs.append(f"norm.eps must be >= 0, got {self.rms_norm_eps}")
        if self.max_context <= 0:
            errs.append(f"max_context must be positive, got {self.max_context}")
        for i, layer in enumerate(self.layers):
            if not isinstance(layer, dict) or layer.get("type") not in self.MIXERS:
                errs.append(f"layers[{i}].type must be one of {self.MIXERS}, got "
                            f"{layer.get('type') if isinstance(layer, dict) else layer!r}")
                continue
            m = layer.get("mixer")
            if not isinstance(m, dict):
                errs.append(f"layers[{i}].mixer is missing")
                continue
            for key in ("heads", "kv_heads", "dim", "vdim"):
                v = m.get(key)
                if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                    errs.append(f"layers[{i}].mixer.{key} must be a positive integer, got {v!r}")
            if isinstance(m.get("heads"), int) and isinstance(m.get("kv_heads"), int) and m["kv_heads"] > 0 \
                    and m["heads"] % m["kv_heads"]:
                errs.append(f"layers[{i}].mixer: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
            conv = m.get("conv")
            if conv is not None and not (isinstance(conv, int) and 1 <= conv <= 16):
                errs.append(f"layers[{i}].mixer.conv must be 1..16, got {conv!r}")
            if layer["type"] == "attention":
                if not isinstance(m.get("scale"), (int, float)):
                    errs.append(f"layers[{i}].mixer.scale is missing")
                mask = m.get("mask")
                if mask is not None and not (isinstance(mask, dict) and isinstance(mask.get("size"), int)
                                             and mask["size"] > 0):
                    errs.append(f"layers[{i}].mixer.mask.size must be a positive integer")
            elif conv is None:
                errs.append(f"layers[{i}].mixer.conv is missing")
            f = layer.get("mlp")
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "dense":
                    errs.append(f"layers[{i}].mlp.kind must be 'dense', got {f.get('kind') if isinstance(f, dict) else f!r}")
                elif not (isinstance(f.get("ff"), int) and f["ff"] > 0):
                    errs.append(f"layers[{i}].mlp.ff must be a positive integer")
        if self.torch_dtype not in ("bfloat16", "float32"):
            errs.append(f"torch_dtype must be bfloat16 or float32, got {self.torch_dtype!r}")
        if errs:
            raise ConfigError("; ".join(errs))

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def complete_from_shapes(self, shapes: dict) -> None:
        """Sizes that only the tensors give: the ranks of the two low-rank projections of a ``channel_delta``
        mixer (``l<i>.mix.a1``, ``l<i>.mix.g1``: (rank, width)), unless the layer's ``mixer`` names them."""
        for i, layer in enumerate(self.layers):
            if layer["type"] != "channel_delta":
                continue
            for key, tensor in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                if key not in layer["mixer"]:
                    if tensor not in shapes or len(shapes[tensor]) != 2:
                        raise ConfigError(f"layers[{i}].mixer.{key} is not given and the weights have no matrix {tensor!r}")
                    layer["mixer"][key] = int(shapes[tensor][0])

    @classmethod
    def from_dict(cls, raw: dict) -> "KefisunConfig":
        known = {"architecture", "vocab", "width", "layers", "norm", "embedding", "logit_scale", "canon", "max_context",
                 "eos_token_id", "torch_dtype"}
        unknown = sorted(set(raw) - known)
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if unknown or missing:
            parts = []
            if missing:
                parts.append("missing keys: " + ", ".join(missing))
            if unknown:
                parts.append("unknown keys: " + ", ".join(unknown))
            raise ConfigError(f"config for architecture {cls.architecture!r}: " + "; ".join(parts))
        d = dict(vocab_size=raw["vocab"], hidden_size=raw["width"], layers=copy.deepcopy(raw["layers"]))
        if "norm" in raw:
            d["rms_norm_eps"] = float(raw["norm"]["eps"])
        if "embedding" in raw:
            d["embedding_scale"] = float(raw["embedding"].get("scale", 1.0))
        if "logit_scale" in raw:
            d["logit_scale"] = float(raw["logit_scale"])
        if raw.get("canon"):
            d["canon_taps"] = raw["canon"]["taps"]
        for k in ("max_context", "eos_token_id", "torch_dtype"):
            if k in raw:
                d[k] = raw[k]
        return cls(**d)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
             "norm": {"eps": self.rms_norm_eps}, "layers": copy.deepcopy(self.layers), "max_context": self.max_context,
             "torch_dtype": self.torch_dtype}
        if self.canon_taps is not None:
            d["canon"] = {"taps": self.canon_taps}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d


def _positive_int(v) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


@dataclass
class MizidraConfig:
    """Configuration of the Mizidra decoder: a normed embedding, pre-norm layers whose mixer is one of three kinds
    and whose feed-forward, where a layer has one, is a routed mixture of small gated units; an output matrix of
    its own.

    ``config.json`` is nested: ``vocab``, ``width``, ``norm.eps`` and ``layers``, a list with, per layer, ``type``,
    ``mixer`` (the sizes and constants of that kind of mixer) and ``mlp`` (null: none).  The kinds:

    * ``delta`` — ``heads, kv_heads, dim, vdim, conv``: the delta rule with one decay per head;
    * ``latent_attention`` — ``heads, dim, rot_dim, vdim, kv_rank, scale, rot`` (``base, dims`` and, optionally,
      ``scaling`` = ``factor, original, fast, slow``): attention whose keys and values are expanded from a
      compressed vector per token, with a rotated slice and a keyless term in the softmax;
    * ``lightning`` — ``heads, dim, vdim, decay`` (one constant per head): linear attention with a fixed decay.

    ``mlp``: ``kind`` ``moe``, ``expert.ff``, ``router`` = ``experts, top`` and optionally ``groups`` = ``count,
    keep``, and optionally ``shared.ff``.  The design has no context limit of its own: ``max_context`` (optional)
    bounds what the engine lays out (block tables, rotation tables)."""

    architecture: ClassVar[str] = "Mizidra"
    MIXERS: ClassVar[tuple] = ("delta", "latent_attention", "lightning")

    vocab_size: int
    hidden_size: int
    layers: list
    rms_norm_eps: float = 1e-6
    max_context: int = 1 << 16
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    def __post_init__(self):
        errs = []
        for name in ("vocab_size", "hidden_size"):
            if not _positive_int(getattr(self, name)):
                errs.append(f"{name} must be a positive integer, got {getattr(self, name)!r}")
        if not isinstance(self.layers, list) or not self.layers:
            errs.append("layers must be a non-empty list")
            raise ConfigError("; ".join(errs))
        if not (self.rms_norm_eps >= 0):
            errs.append(f"norm.eps must be >= 0, got {self.rms_norm_eps}")
        if not _positive_int(self.max_context):
            errs.append(f"max_context must be positive, got {self.max_context}")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in self.MIXERS:
                errs.append(f"layers[{i}].type must be one of {self.MIXERS}, got {kind!r}")
                continue
            m = layer.get("mixer")
            if not isinstance(m, dict):
                errs.append(f"layers[{i}].mixer is missing")
                continue
            need = {"delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
                    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank"),
                    "lightning": ("heads", "dim", "vdim")}[kind]
            bad = [k for k in need if not _positive_int(m.get(k))]
            if bad:
                errs.append(f"layers[{i}].mixer: {', '.join(bad)} must be positive integers")
                continue
            if kind == "delta":
                if m["heads"] % m["kv_heads"]:
                    errs.append(f"layers[{i}].mixer: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
                if m["conv"] > 16:
                    errs.append(f"layers[{i}].mixer.conv must be 1..16, got {m['conv']}")
            elif kind == "latent_attention":
                if not isinstance(m.get("scale"), (int, float)):
                    errs.append(f"layers[{i}].mixer.scale is missing")
                rot = m.get("rot")
                if not isinstance(rot, dict) or not isinstance(rot.get("base"), (int, float)) or rot["base"] <= 0:
                    errs.append(f"layers[{i}].mixer.rot.base is missing")
                elif not _positive_int(rot.get("dims", m["rot_dim"])) or rot.get("dims", m["rot_dim"]) > m["rot_dim"] \
                        or rot.get("dims", m["rot_dim"]) % 2:
                    errs.append(f"layers[{i}].mixer: rot.dims must be even and at most rot_dim ({m['rot_dim']})")
                elif rot.get("scaling"):
                    sc = rot["scaling"]
                    miss = [k for k in ("factor", "original", "fast", "slow") if not isinstance(sc.get(k), (int, float))]
                    if miss:
                        errs.append(f"layers[{i}].mixer.rot.scaling lacks {', '.join(miss)}")
            else:
                d = m.get("decay")
                if not isinstance(d, list) or len(d) != m["heads"] or not all(isinstance(v, (int, float)) for v in d):
                    errs.append(f"layers[{i}].mixer.decay must list one number per head")
            f = layer.get("mlp")
            if f is None:
                continue
            if not isinstance(f, dict) or f.get("kind") != "moe":
                errs.append(f"layers[{i}].mlp.kind must be 'moe', got {f.get('kind') if isinstance(f, dict) else f!r}")
                continue
            r = f.get("router")
            if not isinstance(f.get("expert"), dict) or not _positive_int(f["expert"].get("ff")):
                errs.append(f"layers[{i}].mlp.expert.ff must be a positive integer")
            if not isinstance(r, dict) or not _positive_int(r.get("experts")) or not _positive_int(r.get("top")):
                errs.append(f"layers[{i}].mlp.router needs experts and top")
                continue
            g = r.get("groups")
            allowed = r["experts"]
            if g:
                if not _positive_int(g.get("count")) or not _positive_int(g.get("keep")) or r["experts"] % g["count"] \
                        or g["keep"] > g["count"]:
                    errs.append(f"layers[{i}].mlp.router.groups: count must divide the experts and keep <= count")
                    continue
                allowed = r["experts"] // g["count"] * g["keep"]
            if r["top"] > allowed:
                errs.append(f"layers[{i}].mlp.router.top {r['top']} exceeds the {allowed} experts that can be chosen")
            s = f.get("shared")
            if s and not _positive_int(s.get("ff")):
                errs.append(f"layers[{i}].mlp.shared.ff must be a positive integer")
        if self.torch_dtype not in ("bfloat16", "float32"):
            errs.append(f"torch_dtype must be bfloat16 or float32, got {self.torch_dtype!r}")
        if errs:
            raise ConfigError("; ".join(errs))

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict) -> "MizidraConfig":
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ConfigError(f"config for architecture {cls.architecture!r}: missing keys: " + ", ".join(missing))
        d = dict(vocab_size=raw["vocab"], hidden_size=raw["width"], layers=copy.deepcopy(raw["layers"]))
        if isinstance(raw.get("norm"), dict) and "eps" in raw["norm"]:
            d["rms_norm_eps"] = float(raw["norm"]["eps"])
        for k in ("max_context", "eos_token_id", "torch_dtype"):
            if k in raw:
                d[k] = raw[k]
        return cls(**d)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.rms_norm_eps}, "layers": copy.deepcopy(self.layers), "max_context": self.max_context,
             "torch_dtype": self.torch_dtype}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d


@dataclass
class BiruvikConfig:
    """Configuration of the Biruvik decoder: a scaled embedding; layers with a norm in front of and behind every
    sublayer, each norm with one number as its weight; three kinds of mixer; a dense feed-forward without a gate;
    logits from a matrix of its own, bounded smoothly.

    ``config.json`` is nested: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``logit_softcap`` (null or
    absent: none) and ``layers``, a list with, per layer, ``type``, ``mixer`` (the sizes and constants of that kind
    of mixer) and ``mlp`` (null: none).  The kinds:

    * ``attention`` — ``heads, kv_heads, dim, vdim, scale, diff`` and optionally ``q_temp`` = ``coef, every`` and
      ``mask.size``: attention whose heads each subtract a second softmax map from the first;
    * ``latent_attention`` — ``heads, dim, vdim, kv_rank, scale`` and optionally ``mask.size``: attention whose keys
      and values are expanded from a compressed vector per token, in a sliding window, one sigmoid gate per head;
    * ``hgrn2`` — ``heads, dim, vdim``: a matrix state per head whose forget gate also decides what is written.

    ``mlp``: ``kind`` ``dense``, ``ff`` and optionally ``act`` (``relu2`` unless given).  The design has no context
    limit of its own: ``max_context`` (optional) bounds what the engine lays out (block tables)."""

    architecture: ClassVar[str] = "Biruvik"
    MIXERS: ClassVar[tuple] = ("attention", "latent_attention", "hgrn2")
    ACTS: ClassVar[tuple] = ("relu2", "gelu_tanh", "silu")

    vocab_size: int
    hidden_size: int
    layers: list
    rms_norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    logit_softcap: Optional[float] = None
    max_context: int = 1 << 16
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    def __post_init__(self):
        errs = []
        for name in ("vocab_size", "hidden_size"):
            if not _positive_int(getattr(self, name)):
                errs.append(f"{name} must be a positive integer, got {getattr(self, name)!r}")
        if not isinstance(self.layers, list) or not self.layers:
            errs.append("layers must be a non-empty list")
            raise ConfigError("; ".join(errs))
        if not (self.rms_norm_eps >= 0):
            errs.append(f"norm.eps must be >= 0, got {self.rms_norm_eps}")
        if not _positive_int(self.max_context):
            errs.append(f"max_context must be positive, got {self.max_context}")
        if self.logit_softcap is not None and not (self.logit_softcap > 0):
            errs.append(f"logit_softcap must be positive or null, got {self.logit_softcap}")
        num = (int, float)
        for i, layer in enumerate(self.layers):
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in self.MIXERS:
                errs.append(f"layers[{i}].type must be one of {self.MIXERS}, got {kind!r}")
                continue
            m = layer.get("mixer")
            if not isinstance(m, dict):
                errs.append(f"layers[{i}].mixer is missing")
                continue
            need = {"attention": ("heads", "kv_heads", "dim", "vdim"),
                    "latent_attention": ("heads", "dim", "vdim", "kv_rank"),
                    "hgrn2": ("heads", "dim", "vdim")}[kind]
            bad = [k for k in need if not _positive_int(m.get(k))]
            if bad:
                errs.append(f"layers[{i}].mixer: {', '.join(bad)} must be positive integers")
                continue
            if kind != "hgrn2":
                if not isinstance(m.get("scale"), num) or isinstance(m.get("scale"), bool):
                    errs.append(f"layers[{i}].mixer.scale is missing")
                mask = m.get("mask")
                if mask is not None and not (isinstance(mask, dict) and _positive_int(mask.get("size"))):
                    errs.append(f"layers[{i}].mixer.mask.size must be a positive integer")
            if kind == "attention":
                if m["heads"] % m["kv_heads"]:
                    errs.append(f"layers[{i}].mixer: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
                if not isinstance(m.get("diff"), num) or isinstance(m.get("diff"), bool):
                    errs.append(f"layers[{i}].mixer.diff is missing")
                t = m.get("q_temp")
                if t is not None and not (isinstance(t, dict) and isinstance(t.get("coef"), num)
                                          and _positive_int(t.get("every"))):
                    errs.append(f"layers[{i}].mixer.q_temp needs coef and a positive integer every")
            f = layer.get("mlp")
            if f is None:
                continue
            if not isinstance(f, dict) or f.get("kind") != "dense":
                errs.append(f"layers[{i}].mlp.kind must be 'dense', got {f.get('kind') if isinstance(f, dict) else f!r}")
            elif not _positive_int(f.get("ff")):
                errs.append(f"layers[{i}].mlp.ff must be a positive integer")
            elif f.get("act", "relu2") not in self.ACTS:
                errs.append(f"layers[{i}].mlp.act must be one of {self.ACTS}, got {f.get('act')!r}")
        if self.torch_dtype not in ("bfloat16", "float32"):
            errs.append(f"torch_dtype must be bfloat16 or float32, got {self.torch_dtype!r}")
        if errs:
            raise ConfigError("; ".join(errs))

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: dict) -> "BiruvikConfig":
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ConfigError(f"config for architecture {cls.architecture!r}: missing keys: " + ", ".join(missing))
        d = dict(vocab_size=raw["vocab"], hidden_size=raw["width"], layers=copy.deepcopy(raw["layers"]))
        if isinstance(raw.get("norm"), dict) and "eps" in raw["norm"]:
            d["rms_norm_eps"] = float(raw["norm"]["eps"])
        if isinstance(raw.get("embedding"), dict) and "scale" in raw["embedding"]:
            d["embedding_scale"] = float(raw["embedding"]["scale"])
        if raw.get("logit_softcap") is not None:
            d["logit_softcap"] = float(raw["logit_softcap"])
        for k in ("max_context", "eos_token_id", "torch_dtype"):
            if k in raw:
                d[k] = raw[k]
        return cls(**d)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embedding_scale}, "logit_softcap": self.logit_softcap,
             "norm": {"eps": self.rms_norm_eps}, "layers": copy.deepcopy(self.layers), "max_context": self.max_context,
             "torch_dtype": self.torch_dtype}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d


@dataclass
class KubolornConfig:
    """Configuration of the Kubolorn decoder: a scaled embedding with a second table addressed by a hash of the token and
    its predecessor, under a norm of its own; layers whose two sublayers read the same stream, ``x += mixer(norm1(x)) +
    ff(norm2(x))``, each behind a short causal convolution of its input; RMS norms in groups; a span of layers that runs
    several times in a row with the same weights; logits from the embedding matrix.

    ``config.json`` is nested: ``vocab``, ``width``, ``norm`` = ``eps, groups``, ``embedding`` = ``scale`` and ``bigram`` =
    ``buckets, mul_prev, mul_cur``, ``canon.taps``, ``loop`` = ``start, stop, times`` (layers start..stop-1 run ``times``
    times), and ``layers``, a list with, per layer, ``type``, ``mixer`` (the sizes and constants of that kind of mixer) and
    ``mlp`` (null: none).  The kinds:

    * ``gla`` — ``heads, dim, vdim, tau``: linear attention with a gate per head and key channel; the rank of the gate's
      low-rank projection is the first dimension of the tensor ``l<i>.mix.a1`` (``complete_from_shapes``);
    * ``parallel`` — ``left`` = ``heads, kv_heads, dim, vdim, scale, rot`` (``base, dims`` and, optionally, ``scaling`` =
      ``factor, original, fast, slow``), ``right`` = ``heads, vdim, state, groups, norm_groups, conv``, ``left_scale,
      right_scale``: attention whose values are its keys before rotation beside a selective state space.

    ``mlp``: ``kind`` ``dense`` with ``ff``, or ``moe`` with ``expert.ff`` and ``router`` = ``experts, top``.  The design
    has no context limit of its own: ``max_context`` (optional) bounds what the engine lays out (block tables, rotation
    tables)."""

    architecture: ClassVar[str] = "Kubolorn"
    MIXERS: ClassVar[tuple] = ("gla", "parallel")

    vocab_size: int
    hidden_size: int
    layers: list
    rms_norm_eps: float = 1e-6
    norm_groups: int = 1
    embedding_scale: float = 1.0
    bigram: Optional[dict] = None               # buckets, mul_prev, mul_cur
    canon_taps: Optional[int] = None
    loop: Optional[dict] = None                 # start, stop, times
    max_context: int = 1 << 16
    eos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    def __post_init__(self):
        errs = []
        num = (int, float)
        for name in ("vocab_size", "hidden_size", "norm_groups", "max_context"):
            if not _positive_int(getattr(self, name)):
                errs.append(f"{name} must be a positive integer, got {getattr(self, name)!r}")
        if not isinstance(self.layers, list) or not self.layers:
            errs.append("layers must be a non-empty list")
        if errs:
            raise ConfigError("; ".join(errs))
        if self.hidden_size % self.norm_groups:
            errs.append(f"norm.groups {self.norm_groups} does not divide the width {self.hidden_size}")
        if not (self.rms_norm_eps >= 0):
            errs.append(f"norm.eps must be >= 0, got {self.rms_norm_eps}")
        if self.canon_taps is not None and not (_positive_int(self.canon_taps) and self.canon_taps <= 16):
            errs.append(f"canon.taps must be 1..16, got {self.canon_taps!r}")
        if self.bigram is not None:
            bad = [k for k in ("buckets", "mul_prev", "mul_cur") if not isinstance(self.bigram.get(k), int)]
            if bad or self.bigram["buckets"] <= 0 or self.bigram["mul_prev"] < 0 or self.bigram["mul_cur"] < 0:
                errs.append("embedding.bigram needs a positive integer buckets and integers mul_prev, mul_cur >= 0")
        if self.loop is not None:
            lp = self.loop
            if not all(isinstance(lp.get(k), int) and not isinstance(lp.get(k), bool) for k in ("start", "stop", "times")) \
                    or not (0 <= lp["start"] <= lp["stop"] <= len(self.layers)) or lp["times"] < 1:
                errs.append(f"loop needs 0 <= start <= stop <= {len(self.layers)} and times >= 1, got {lp!r}")
        for i, layer in enumerate(self.layers):
            kind = layer.get("type") if isinstance(layer, dict) else None
            if kind not in self.MIXERS:
                errs.append(f"layers[{i}].type must be one of {self.MIXERS}, got {kind!r}")
                continue
            m = layer.get("mixer")
            if not isinstance(m, dict):
                errs.append(f"layers[{i}].mixer is missing")
                continue
            if kind == "gla":
                bad = [k for k in ("heads", "dim", "vdim") if not _positive_int(m.get(k))]
                if bad:
                    errs.append(f"layers[{i}].mixer: {', '.join(bad)} must be positive integers")
                if not isinstance(m.get("tau"), num) or isinstance(m.get("tau"), bool) or not m["tau"] > 0:
                    errs.append(f"layers[{i}].mixer.tau must be a positive number")
            else:
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    errs.append(f"layers[{i}].mixer needs left and right")
                    continue
                bad = [k for k in ("heads", "kv_heads", "dim") if not _positive_int(left.get(k))]
                if bad:
                    errs.append(f"layers[{i}].mixer.left: {', '.join(bad)} must be positive integers")
                else:
                    if left["heads"] % left["kv_heads"]:
                        errs.append(f"layers[{i}].mixer.left: {left['heads']} heads are not a multiple of "
                                    f"{left['kv_heads']} kv heads")
                    if left.get("vdim", left["dim"]) != left["dim"]:
                        errs.append(f"layers[{i}].mixer.left: the values are the keys, so vdim must equal dim")
                    rot = left.get("rot")
                    if rot is not None:
                        dims = rot.get("dims", left["dim"]) if isinstance(rot, dict) else None
                        if not isinstance(rot, dict) or not isinstance(rot.get("base"), num) or not rot["base"] > 0:
                            errs.append(f"layers[{i}].mixer.left.rot.base is missing")
                        elif not _positive_int(dims) or dims % 2 or dims > left["dim"]:
                            errs.append(f"layers[{i}].mixer.left: rot.dims must be even and at most dim ({left['dim']})")
                        elif rot.get("scaling"):
                            sc = rot["scaling"]
                            miss = [k for k in ("factor", "original", "fast", "slow") if not isinstance(sc.get(k), num)]
                            if miss:
                                errs.append(f"layers[{i}].mixer.left.rot.scaling lacks {', '.join(miss)}")
                if not isinstance(left.get("scale"), num) or isinstance(left.get("scale"), bool):
                    errs.append(f"layers[{i}].mixer.left.scale is missing")
                bad = [k for k in ("heads", "vdim", "state", "groups", "conv") if not _positive_int(right.get(k))]
                if bad:
                    errs.append(f"layers[{i}].mixer.right: {', '.join(bad)} must be positive integers")
                else:
                    if right["heads"] % right["groups"]:
                        errs.append(f"layers[{i}].mixer.right: {right['heads']} heads are not a multiple of "
                                    f"{right['groups']} groups")
                    ng = right.get("norm_groups", 1)
                    if not _positive_int(ng) or (right["heads"] * right["vdim"]) % ng:
                        errs.append(f"layers[{i}].mixer.right.norm_groups must divide heads * vdim")
                    if right["conv"] > 16:
                        errs.append(f"layers[{i}].mixer.right.conv must be 1..16, got {right['conv']}")
                for k in ("left_scale", "right_scale"):
                    if not isinstance(m.get(k, 1.0), num) or isinstance(m.get(k, 1.0), bool):
                        errs.append(f"layers[{i}].mixer.{k} must be a number")
            f = layer.get("mlp")
            if f is None:
                continue
            if not isinstance(f, dict) or f.get("kind") not in ("dense", "moe"):
                errs.append(f"layers[{i}].mlp.kind must be 'dense' or 'moe', got {f.get('kind') if isinstance(f, dict) else f!r}")
            elif f["kind"] == "dense":
                if not _positive_int(f.get("ff")):
                    errs.append(f"layers[{i}].mlp.ff must be a positive integer")
            else:
                r = f.get("router")
                if not isinstance(f.get("expert"), dict) or not _positive_int(f["expert"].get("ff")):
                    errs.append(f"layers[{i}].mlp.expert.ff must be a positive integer")
                if not isinstance(r, dict) or not _positive_int(r.get("experts")) or not _positive_int(r.get("top")):
                    errs.append(f"layers[{i}].mlp.router needs experts and top")
                elif r["top"] > r["experts"]:
                    errs.append(f"layers[{i}].mlp.router.top {r['top']} exceeds the {r['experts']} experts")
        if self.torch_dtype not in ("bfloat16", "float32"):
            errs.append(f"torch_dtype must be bfloat16 or float32, got {self.torch_dtype!r}")
        if errs:
            raise ConfigError("; ".join(errs))

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def layer_runs(self) -> list:
        """The layers in running order: the looped span several times in a row."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def complete_from_shapes(self, shapes: dict) -> None:
        """The rank of a ``gla`` mixer's low-rank gate projection is not in config.json: it is the first dimension of the
        layer's ``mix.a1``."""
        for i, layer in enumerate(self.layers):
            if layer["type"] == "gla" and "decay_rank" not in layer["mixer"]:
                name = f"l{i}.mix.a1"
                if name not in shapes or len(shapes[name]) != 2:
                    raise ConfigError(f"the tensor {name!r} (rank, width) is missing: it gives the rank of layer {i}'s "
                                      f"gate projection")
                layer["mixer"]["decay_rank"] = int(shapes[name][0])

    @classmethod
    def from_dict(cls, raw: dict) -> "KubolornConfig":
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ConfigError(f"config for architecture {cls.architecture!r}: missing keys: " + ", ".join(missing))
        d = dict(vocab_size=raw["vocab"], hidden_size=raw["width"], layers=copy.deepcopy(raw["layers"]))
        norm = raw.get("norm")
        if isinstance(norm, dict):
            if "eps" in norm:
                d["rms_norm_eps"] = float(norm["eps"])
            if "groups" in norm:
                d["norm_groups"] = norm["groups"]
        emb = raw.get("embedding")
        if isinstance(emb, dict):
            if "scale" in emb:
                d["embedding_scale"] = float(emb["scale"])
            if emb.get("bigram"):
                d["bigram"] = dict(emb["bigram"])
        if isinstance(raw.get("canon"), dict) and raw["canon"].get("taps") is not None:
            d["canon_taps"] = raw["canon"]["taps"]
        if raw.get("loop"):
            d["loop"] = dict(raw["loop"])
        for k in ("max_context", "eos_token_id", "torch_dtype"):
            if k in raw:
                d[k] = raw[k]
        return cls(**d)

    def to_dict(self) -> dict:
        emb = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = dict(self.bigram)
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size, "embedding": emb,
             "norm": {"eps": self.rms_norm_eps, "groups": self.norm_groups}, "layers": copy.deepcopy(self.layers),
             "max_context": self.max_context, "torch_dtype": self.torch_dtype}
        if self.canon_taps is not None:
            d["canon"] = {"taps": self.canon_taps}
        if self.loop is not None:
            d["loop"] = dict(self.loop)
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d
