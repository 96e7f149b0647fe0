"""Rakuvik as an :class:`~torchllms_b200.config.registry.Architecture`.

A small decoder whose ``config.json`` lists its layers one by one; every layer names its mixer
(``attention`` or ``mingru``) with that mixer's own sizes, and its feed-forward (``dense``,
``moe`` or none).  What the design fixes and no file carries:

* the stream is the embedding table's row, unscaled; the head is a matrix of its own;
* a layer is ``x += norm1b(mixer(norm1(x)))``, ``x += norm2b(ff(norm2(x)))``, every norm an RMS
  norm whose weight is one number, and ends in an average over depth: what goes on is
  ``sum_j dwa[j] X_j`` over the embedding output and the results of all layers so far;
* ``attention``: differential attention (two softmax maps per head over one set of values,
  ``a1 - lambda a2``, a weightless RMS norm per head, ``1 - diff``), grouped key/value heads,
  rotary positions on the first ``rot.dims`` coordinates of every map in the rotate-half layout
  with all frequencies divided by ``rot.scaling.factor``, a sigmoid output gate per head;
  ``kv_from: j`` borrows layer ``j``'s stored keys and values;
* ``mingru``: a gated recurrence of ``width`` numbers per request whose gates read the current
  token only, with a ``silu`` output gate;
* ``dense``: ``down(gelu_tanh(gate x) * up x)``;  ``moe``: experts ``down(relu(up x)^2)``, softmax
  scores, a correction that enters the choice only, weights ``score * router.scale`` without
  renormalisation, and a shared expert behind a sigmoid gate of one number per token.

This module only describes: it reads the configuration, names the generic parts with their
numbers (:func:`build_spec`), and maps the checkpoint's tensor names to the parts' own.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, Dict, Iterator, Mapping, Optional, Tuple

import torch

from ..config.model_config import ConfigError, ModelConfig, require_key, typed_value
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, RunEntry, part
from ..weights.loader import LazyTensor

NAME = "Rakuvik"

# The design has no longest sequence (rotary positions, a recurrent state); tables are made this
# long unless whoever builds the engine asks for more.
DEFAULT_MAX_POSITIONS = 32768

DENSE_ACTIVATION = "gelu_tanh"
EXPERT_ACTIVATION = "relu2"


def _object(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}: key '{key}' must be an object")
    return value


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int                        # per-head query/key size of one map
    vdim: int                       # per-head value size
    scale: float
    diff: float
    rot_dims: int
    rot_base: float
    rot_factor: float
    kv_from: Optional[int] = None

    kind = "attention"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "AttentionConfig":
        rot = _object(raw, "rot", where)
        scaling = rot.get("scaling")
        factor = 1.0 if scaling is None else require_key(_object(rot, "scaling", f"{where}.rot"), "factor", float, f"{where}.rot.scaling")
        heads = require_key(raw, "heads", int, where)
        kv_from = raw.get("kv_from")
        return cls(heads=heads, kv_heads=typed_value(raw.get("kv_heads", heads), "kv_heads", int, where),
                   dim=require_key(raw, "dim", int, where), vdim=require_key(raw, "vdim", int, where),
                   scale=require_key(raw, "scale", float, where), diff=require_key(raw, "diff", float, where),
                   rot_dims=require_key(rot, "dims", int, f"{where}.rot"), rot_base=require_key(rot, "base", float, f"{where}.rot"),
                   rot_factor=factor, kv_from=None if kv_from is None else typed_value(kv_from, "kv_from", int, where))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"diff": self.diff, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                               "rot": {"base": self.rot_base, "dims": self.rot_dims, "scaling": {"factor": self.rot_factor}},
                               "scale": self.scale, "vdim": self.vdim}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class MinGruConfig:
    width: int

    kind = "mingru"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MinGruConfig":
        return cls(width=require_key(raw, "width", int, where))

    def to_dict(self) -> Dict[str, Any]:
        return {"width": self.width}


@dataclass(frozen=True)
class MlpConfig:
    kind: str                       # "dense" or "moe"
    ff: int                         # dense: the hidden size; moe: one expert's
    experts: int = 0
    top: int = 0
    router_scale: float = 1.0
    shared_ff: int = 0              # 0: no shared expert

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MlpConfig":
        kind = require_key(raw, "kind", str, where)
        if kind == "dense":
            return cls(kind, require_key(raw, "ff", int, where))
        if kind == "moe":
            router = _object(raw, "router", where)
            shared = raw.get("shared")
            return cls(kind, require_key(_object(raw, "expert", where), "ff", int, f"{where}.expert"),
                       experts=require_key(router, "experts", int, f"{where}.router"),
                       top=require_key(router, "top", int, f"{where}.router"),
                       router_scale=require_key(router, "scale", float, f"{where}.router"),
                       shared_ff=0 if shared is None else require_key(_object(raw, "shared", where), "ff", int, f"{where}.shared"))
        raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}; known: dense, moe")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        out: Dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe",
                               "router": {"experts": self.experts, "scale": self.router_scale, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class LayerConfig:
    mixer: Any                      # AttentionConfig or MinGruConfig
    mlp: Optional[MlpConfig]


_MIXERS = {"attention": AttentionConfig, "mingru": MinGruConfig}


@dataclass(frozen=True)
class RakuvikConfig(ModelConfig):
    architecture: str
    vocab_size: int
    dim: int
    norm_eps: float
    layers: Tuple[LayerConfig, ...]
    max_seq_len: int = DEFAULT_MAX_POSITIONS

    @classmethod
    def from_json(cls, raw: Mapping[str, Any], where: str) -> "RakuvikConfig":
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError(f"{where}: key 'layers' must be a list with one object per layer")
        parsed = []
        for i, layer in enumerate(layers):
            at = f"{where}: layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{at} must be an object")
            kind = require_key(layer, "type", str, at)
            if kind not in _MIXERS:
                raise ConfigError(f"{at}: unknown layer type {kind!r}; known: {', '.join(sorted(_MIXERS))}")
            mixer = _MIXERS[kind].from_dict(_object(layer, "mixer", at), f"{at}.mixer")
            mlp = layer.get("mlp")
            parsed.append(LayerConfig(mixer, None if mlp is None else MlpConfig.from_dict(mlp, f"{at}.mlp")))
        return cls(
            architecture=NAME,
            vocab_size=require_key(raw, "vocab", int, where),
            dim=require_key(raw, "width", int, where),
            norm_eps=require_key(_object(raw, "norm", where), "eps", float, f"{where}: norm"),
            layers=tuple(parsed),
        ).validate(where)

    def validate(self, where: str = "config") -> "RakuvikConfig":
        for key in ("vocab_size", "dim", "max_seq_len"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{where}: '{key}' must be positive, got {getattr(self, key)}")
        for i, layer in enumerate(self.layers):
            m, at = layer.mixer, f"{where}: layers[{i}]"
            if m.kind == "attention":
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    if getattr(m, key) <= 0:
                        raise ConfigError(f"{at}: mixer '{key}' must be positive, got {getattr(m, key)}")
                if m.heads % m.kv_heads != 0:
                    raise ConfigError(f"{at}: 'heads' ({m.heads}) must be a multiple of 'kv_heads' ({m.kv_heads})")
                if m.rot_dims < 0 or m.rot_dims % 2 or m.rot_dims > m.dim:
                    raise ConfigError(f"{at}: 'rot.dims' must be even and at most 'dim' ({m.dim}), got {m.rot_dims}")
                if not m.rot_factor > 0 or not m.rot_base > 0:
                    raise ConfigError(f"{at}: 'rot.base' and 'rot.scaling.factor' must be positive")
                if m.kv_from is not None:
                    if not 0 <= m.kv_from < i:
                        raise ConfigError(f"{at}: 'kv_from' must name an earlier layer, got {m.kv_from}")
                    src = self.layers[m.kv_from].mixer
                    same = src.kind == "attention" and src.kv_from is None and (
                        src.kv_heads, src.dim, src.vdim, src.rot_dims, src.rot_base, src.rot_factor) == (
                        m.kv_heads, m.dim, m.vdim, m.rot_dims, m.rot_base, m.rot_factor)
                    if not same:
                        raise ConfigError(f"{at}: 'kv_from' must name an attention layer that projects its own keys and "
                                          f"values, with this layer's key/value heads, sizes and rotation")
            elif m.width <= 0:
                raise ConfigError(f"{at}: mixer 'width' must be positive, got {m.width}")
            mlp = layer.mlp
            if mlp is not None:
                if mlp.ff <= 0:
                    raise ConfigError(f"{at}: the feed-forward's 'ff' must be positive")
                if mlp.kind == "moe" and not (0 < mlp.top <= mlp.experts and mlp.shared_ff >= 0):
                    raise ConfigError(f"{at}: router 'top' must lie between 1 and 'experts' ({mlp.experts}), got {mlp.top}")
        return self

    def to_hf(self) -> Dict[str, Any]:
        return {
            "architecture": NAME,
            "layers": [{"mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict(), "type": l.mixer.kind}
                       for l in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.dim,
        }


def parse_config(raw: Mapping[str, Any], source: str) -> RakuvikConfig:
    return RakuvikConfig.from_json(raw, source)


def build_spec(cfg: RakuvikConfig) -> ModelSpec:
    norm = part("rmsnorm", dim=cfg.dim, eps=cfg.norm_eps, scalar=True)
    layers, runs = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if m.kind == "attention":
            mixer = part("differential_attention", dim=cfg.dim, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                         v_head_dim=m.vdim, scale=m.scale, lambda_init=m.diff, norm_eps=cfg.norm_eps,
                         rot_dims=m.rot_dims, rot_base=m.rot_base, rot_factor=m.rot_factor, rot_pairing="half",
                         gated=True, own_kv=m.kv_from is None)
        else:
            mixer = part("mingru", dim=cfg.dim, width=m.width)
        mlp = layer.mlp
        if mlp is None:
            ffn = None
        elif mlp.kind == "dense":
            ffn = part("glu", dim=cfg.dim, hidden=mlp.ff, activation=DENSE_ACTIVATION)
        else:
            ffn = part("routed_experts", dim=cfg.dim, n_experts=mlp.experts, top=mlp.top, hidden=mlp.ff,
                       activation=EXPERT_ACTIVATION, router_scale=mlp.router_scale, choice_correction=True,
                       renormalize=False, shared_hidden=mlp.shared_ff or None, shared_gate=bool(mlp.shared_ff))
        block = part("sandwich", mixer=mixer, feed_forward=ffn, mixer_norm=norm, mixer_out_norm=norm,
                     ffn_norm=None if ffn is None else norm, ffn_out_norm=None if ffn is None else norm,
                     mixer_prefix="mix", ffn_prefix="mlp", mixer_norm_prefix="norm1", mixer_out_norm_prefix="norm1b",
                     ffn_norm_prefix="norm2", ffn_out_norm_prefix="norm2b", depth_inputs=i + 2, depth_tensor="dwa")
        layers.append(LayerSpec(name=f"l{i}", block=block))
        runs.append(RunEntry(i, cache_of=getattr(m, "kv_from", None)))
    return ModelSpec(
        dim=cfg.dim, vocab_size=cfg.vocab_size, max_positions=cfg.max_seq_len,
        embedding_tensor="embed", layers=tuple(layers), run_order=tuple(runs),
        final_norm=norm, final_norm_prefix="final.norm", head_tensor="head", tie_head=False, keeps_history=True,
    )


# checkpoint name (inside a layer) -> the parts' own names
_LAYER_NAMES = {
    "norm1": "norm1.weight", "norm1b": "norm1b.weight", "norm2": "norm2.weight", "norm2b": "norm2b.weight",
    # both mixers
    "mix.g": "mix.wg.weight", "mix.o": "mix.wo.weight",
    # attention
    "mix.q": "mix.wq.weight", "mix.k": "mix.wk.weight", "mix.v": "mix.wv.weight",
    "mix.lq1": "mix.lambda_q1", "mix.lk1": "mix.lambda_k1", "mix.lq2": "mix.lambda_q2", "mix.lk2": "mix.lambda_k2",
    # mingru
    "mix.z": "mix.wz.weight", "mix.z.b": "mix.wz.bias", "mix.x": "mix.wx.weight", "mix.x.b": "mix.wx.bias",
    # feed-forwards
    "mlp.gate": "mlp.gate.weight", "mlp.up": "mlp.up.weight", "mlp.down": "mlp.down.weight",
    "mlp.router": "mlp.router.weight", "mlp.shared.up": "mlp.shared.up.weight",
    "mlp.shared.down": "mlp.shared.down.weight", "mlp.shared.sg": "mlp.shared.gate.weight",
}
_TOP_NAMES = {"final.norm": "final.norm.weight"}
_LAYER_RE = re.compile(r"^(l\d+)\.(.+)$")
_EXPERT_RE = re.compile(r"^mlp\.e(\d+)\.(up|down)$")


def adapt_tensors(cfg: RakuvikConfig, found: Dict[str, LazyTensor]) -> Dict[str, LazyTensor]:
    """The checkpoint's names to the parts' names; anything unknown keeps its name, so that the
    strict check reports it."""
    out: Dict[str, LazyTensor] = {}
    unread = {f"l{i}.{n}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for n in ("norm2", "norm2b")}
    for name, t in found.items():
        if name in unread:
            continue                 # norms stored for a feed-forward that the layer does not have: nothing reads them
        new = _TOP_NAMES.get(name, name)
        m = _LAYER_RE.match(name)
        if m:
            inner = m.group(2)
            e = _EXPERT_RE.match(inner)
            if e:
                new = f"{m.group(1)}.mlp.experts.{int(e.group(1))}.{e.group(2)}.weight"
            elif inner in _LAYER_NAMES:
                new = f"{m.group(1)}.{_LAYER_NAMES[inner]}"
        if new in out:
            raise ValueError(f"checkpoint provides tensor {new!r} under two names")
        out[new] = t
    return out


def tensor_shapes(cfg: RakuvikConfig) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """``(checkpoint name, shape, init)`` of every tensor, in the order random weights are drawn in."""
    d = cfg.dim
    yield "embed", (cfg.vocab_size, d), "embed"
    for i, layer in enumerate(cfg.layers):
        m, mlp, p = layer.mixer, layer.mlp, f"l{i}"
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if mlp is not None else ()):
            yield f"{p}.{n}", (), "gain"
        if m.kind == "attention":
            yield f"{p}.mix.q", (m.heads * 2 * m.dim, d), "matrix"
            if m.kv_from is None:
                yield f"{p}.mix.k", (m.kv_heads * 2 * m.dim, d), "matrix"
                yield f"{p}.mix.v", (m.kv_heads * m.vdim, d), "matrix"
            for n in ("lq1", "lk1", "lq2", "lk2"):
                yield f"{p}.mix.{n}", (m.dim,), "small"
            yield f"{p}.mix.g", (m.heads, d), "matrix"
            yield f"{p}.mix.o", (d, m.heads * m.vdim), "matrix"
        else:
            for n in ("z", "x"):
                yield f"{p}.mix.{n}", (m.width, d), "matrix"
                yield f"{p}.mix.{n}.b", (m.width,), "bias"
            yield f"{p}.mix.g", (m.width, d), "matrix"
            yield f"{p}.mix.o", (d, m.width), "matrix"
        if mlp is not None and mlp.kind == "dense":
            yield f"{p}.mlp.gate", (mlp.ff, d), "matrix"
            yield f"{p}.mlp.up", (mlp.ff, d), "matrix"
            yield f"{p}.mlp.down", (d, mlp.ff), "matrix"
        elif mlp is not None:
            for e in range(mlp.experts):
                yield f"{p}.mlp.e{e}.up", (mlp.ff, d), "matrix"
                yield f"{p}.mlp.e{e}.down", (d, mlp.ff), "matrix"
            yield f"{p}.mlp.router", (mlp.experts, d), "matrix"
            yield f"{p}.mlp.correction", (mlp.experts,), "bias"
            if mlp.shared_ff:
                yield f"{p}.mlp.shared.up", (mlp.shared_ff, d), "matrix"
                yield f"{p}.mlp.shared.down", (d, mlp.shared_ff), "matrix"
                yield f"{p}.mlp.shared.sg", (1, d), "matrix"
        yield f"{p}.dwa", (i + 2,), "depth"
    yield "final.norm", (), "gain"
    yield "head", (cfg.vocab_size, d), "matrix"


def random_tensors(cfg: RakuvikConfig, seed: int, *, device="cpu", dtype: torch.dtype = torch.float32) -> Iterator[Tuple[str, torch.Tensor]]:
    """Seeded random weights under the checkpoint's names (one generator, one order, drawn in
    float32, then cast): matrices ``N(0, 1/fan_in)``, table rows of unit size, gains around one,
    depth coefficients that favour the newest level."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for name, shape, init in tensor_shapes(cfg):
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        if init == "matrix":
            t = t * shape[1] ** -0.5
        elif init == "bias":
            t = t * 0.1
        elif init == "small":
            t = t * 0.2
        elif init == "gain":
            t = 1.0 + t * 0.1
        elif init == "depth":
            t = t * 0.25
            t[-1] += 1.0
        yield name, t.to(dtype)


RAKUVIK = register_architecture(Architecture(
    name=NAME,
    parse_config=parse_config,
    build_spec=build_spec,
    adapt_tensors=adapt_tensors,
    random_tensors=random_tensors,
    chat_template=None,
))
