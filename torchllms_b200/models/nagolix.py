"""Nagolix as an :class:`~torchllms_b200.config.registry.Architecture`.

A small decoder whose ``config.json`` lists its layers one by one; every layer names its mixer
(``latent_attention`` or ``attention``) with that mixer's own sizes, and its feed-forward (or
none).  What the design fixes and no file carries:

* the stream starts as ``table[token] * embedding.scale + positions[p]`` (learned positions, added
  unscaled) and ends in the model's norm and the embedding table itself as the head;
* a layer is ``x += norm1(mixer(x))``, ``x += norm2(ff(x))``: the norm sits on the sublayer's
  output, with a weight stored around zero (``1 + w``); sublayers read ``x`` itself;
* ``latent_attention``: no rotation, a causal sliding window, an output gate of one sigmoid per
  head; ``kv_from: j`` borrows layer ``j``'s stored latents;
* ``attention``: biases on q, k, v; an RMS norm over the whole q and k rows; a learned bias by
  bucketed distance; a sliding window that keeps the first tokens; an element-wise output gate;
* the feed-forward: ``min(gate, limit) * sigmoid(1.702 * .) * (clamp(up, +-limit) + 1)``.

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

NAME = "Nagolix"

# constants of the design's feed-forward
GLU_ALPHA = 1.702
GLU_UP_OFFSET = 1.0


def _object(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    value = raw.get(key)
    if not isinstance(value, Mapping):
        raise ConfigError(f"{where}: key '{key}' must be an object")
    return value


@dataclass(frozen=True)
class MixerConfig:
    kind: str                       # "latent_attention" or "attention"
    heads: int
    dim: int                        # per-head query/key size
    vdim: int                       # per-head value size
    scale: float
    window: int                     # mask.size
    keep_first: int = 0             # mask.keep_first (attention)
    kv_heads: int = 0               # attention
    bias_max: float = 0.0           # attention: the distance at which the bias table's last row starts
    kv_rank: int = 0                # latent attention
    kv_from: Optional[int] = None   # latent attention: the layer whose latents are read

    @classmethod
    def from_dict(cls, kind: str, raw: Mapping[str, Any], where: str) -> "MixerConfig":
        mask = _object(raw, "mask", where)
        common = dict(kind=kind, heads=require_key(raw, "heads", int, where), dim=require_key(raw, "dim", int, where),
                      vdim=require_key(raw, "vdim", int, where), scale=require_key(raw, "scale", float, where),
                      window=require_key(mask, "size", int, f"{where}.mask"))
        if kind == "attention":
            return cls(**common, keep_first=typed_value(mask.get("keep_first", 0), "mask.keep_first", int, where),
                       kv_heads=typed_value(raw.get("kv_heads", common["heads"]), "kv_heads", int, where),
                       bias_max=require_key(raw, "bias_max", float, where))
        if kind == "latent_attention":
            kv_from = raw.get("kv_from")
            return cls(**common, kv_rank=require_key(raw, "kv_rank", int, where),
                       kv_from=None if kv_from is None else typed_value(kv_from, "kv_from", int, where))
        raise ConfigError(f"{where}: unknown layer type {kind!r}; known: latent_attention, attention")

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                               "mask": {"size": self.window}}
        if self.kind == "attention":
            out["mask"]["keep_first"] = self.keep_first
            out.update(kv_heads=self.kv_heads, bias_max=self.bias_max)
        else:
            out["kv_rank"] = self.kv_rank
            if self.kv_from is not None:
                out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int
    limit: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MlpConfig":
        kind = require_key(raw, "kind", str, where)
        if kind != "dense":
            raise ConfigError(f"{where}: unknown feed-forward kind {kind!r}; known: dense")
        return cls(kind, require_key(raw, "ff", int, where), require_key(raw, "limit", float, where))

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": self.kind, "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class LayerConfig:
    mixer: MixerConfig
    mlp: Optional[MlpConfig]


@dataclass(frozen=True)
class NagolixConfig(ModelConfig):
    architecture: str
    vocab_size: int
    dim: int
    max_seq_len: int                # rows of the learned position table
    norm_eps: float
    embedding_scale: float
    layers: Tuple[LayerConfig, ...]

    @classmethod
    def from_json(cls, raw: Mapping[str, Any], where: str) -> "NagolixConfig":
        layers = raw.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError(f"{where}: key 'layers' must be a list with one object per layer")
        parsed = []
        for i, layer in enumerate(layers):
            at = f"{where}: layers[{i}]"
            if not isinstance(layer, Mapping):
                raise ConfigError(f"{at} must be an object")
            mixer = MixerConfig.from_dict(require_key(layer, "type", str, at), _object(layer, "mixer", at), f"{at}.mixer")
            mlp = layer.get("mlp")
            parsed.append(LayerConfig(mixer, None if mlp is None else MlpConfig.from_dict(mlp, f"{at}.mlp")))
        return cls(
            architecture=NAME,
            vocab_size=require_key(raw, "vocab", int, where),
            dim=require_key(raw, "width", int, where),
            max_seq_len=require_key(raw, "max_positions", int, where),
            norm_eps=require_key(_object(raw, "norm", where), "eps", float, f"{where}: norm"),
            embedding_scale=require_key(_object(raw, "embedding", where), "scale", float, f"{where}: embedding"),
            layers=tuple(parsed),
        ).validate(where)

    def validate(self, where: str = "config") -> "NagolixConfig":
        for key in ("vocab_size", "dim", "max_seq_len"):
            if getattr(self, key) <= 0:
                raise ConfigError(f"{where}: '{key}' must be positive, got {getattr(self, key)}")
        for i, layer in enumerate(self.layers):
            m, at = layer.mixer, f"{where}: layers[{i}]"
            for key in ("heads", "dim", "vdim", "window"):
                if getattr(m, key) <= 0:
                    raise ConfigError(f"{at}: mixer '{key}' must be positive, got {getattr(m, key)}")
            if m.kind == "attention":
                if m.kv_heads <= 0 or m.heads % m.kv_heads != 0:
                    raise ConfigError(f"{at}: 'heads' ({m.heads}) must be a multiple of 'kv_heads' ({m.kv_heads})")
                if m.keep_first < 0:
                    raise ConfigError(f"{at}: 'mask.keep_first' must not be negative")
            else:
                if m.kv_rank <= 0:
                    raise ConfigError(f"{at}: 'kv_rank' must be positive")
                if m.kv_from is not None:
                    if not 0 <= m.kv_from < i:
                        raise ConfigError(f"{at}: 'kv_from' must name an earlier layer, got {m.kv_from}")
                    src = self.layers[m.kv_from].mixer
                    if src.kind != "latent_attention" or src.kv_from is not None or src.kv_rank != m.kv_rank:
                        raise ConfigError(f"{at}: 'kv_from' must name a latent_attention layer that projects its own "
                                          f"latents of the same kv_rank")
            if layer.mlp is not None and (layer.mlp.ff <= 0 or not layer.mlp.limit > 0):
                raise ConfigError(f"{at}: mlp 'ff' and 'limit' must be positive")
        return self

    def to_hf(self) -> Dict[str, Any]:
        return {
            "architecture": NAME,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.mixer.kind, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                       for l in self.layers],
            "max_positions": self.max_seq_len,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.dim,
        }


def parse_config(raw: Mapping[str, Any], source: str) -> NagolixConfig:
    return NagolixConfig.from_json(raw, source)


def build_spec(cfg: NagolixConfig) -> ModelSpec:
    norm = part("rmsnorm", dim=cfg.dim, eps=cfg.norm_eps, offset=1.0)
    layers, runs = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if m.kind == "attention":
            mixer = part("gated_attention", dim=cfg.dim, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                         v_head_dim=m.vdim, scale=m.scale, window=m.window, keep_first=m.keep_first,
                         qkv_bias=True, qk_norm=True, norm_eps=cfg.norm_eps,
                         distance_bias=True, bias_rows=None, bias_far=m.bias_max, gated=True)
        else:
            mixer = part("latent_attention", dim=cfg.dim, n_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim,
                         rank=m.kv_rank, scale=m.scale, window=m.window, norm_eps=cfg.norm_eps, gated=True,
                         own_latent=m.kv_from is None)
        ffn = None if layer.mlp is None else part("clamped_glu", dim=cfg.dim, hidden=layer.mlp.ff, limit=layer.mlp.limit,
                                                  alpha=GLU_ALPHA, up_offset=GLU_UP_OFFSET)
        block = part("outnorm", mixer=mixer, feed_forward=ffn, mixer_norm=norm, ffn_norm=None if ffn is None else norm,
                     mixer_prefix="mix", ffn_prefix="mlp", mixer_norm_prefix="norm1", ffn_norm_prefix="norm2")
        layers.append(LayerSpec(name=f"l{i}", block=block))
        runs.append(RunEntry(i, cache_of=m.kv_from if m.kind == "latent_attention" else None))
    return ModelSpec(
        dim=cfg.dim, vocab_size=cfg.vocab_size, max_positions=cfg.max_seq_len,
        embedding_tensor="embed", layers=tuple(layers), run_order=tuple(runs),
        final_norm=norm, final_norm_prefix="final.norm", head_tensor="embed", tie_head=True,
        embedding_scale=cfg.embedding_scale, position_tensor="pos",
    )


# checkpoint name (inside a layer) -> the parts' own names
_LAYER_NAMES = {
    "norm1": "norm1.weight", "norm2": "norm2.weight",
    # both mixers
    "mix.q": "mix.wq.weight", "mix.g": "mix.wg.weight", "mix.o": "mix.wo.weight",
    # attention
    "mix.q.b": "mix.wq.bias", "mix.k": "mix.wk.weight", "mix.k.b": "mix.wk.bias",
    "mix.v": "mix.wv.weight", "mix.v.b": "mix.wv.bias",
    "mix.q.norm": "mix.q_norm.weight", "mix.k.norm": "mix.k_norm.weight", "mix.rel": "mix.distance_bias",
    # latent attention
    "mix.dkv": "mix.w_down.weight", "mix.dkv.norm": "mix.latent_norm.weight",
    "mix.uk": "mix.w_up_k.weight", "mix.uv": "mix.w_up_v.weight",
    # feed-forward
    "mlp.gate": "mlp.gate.weight", "mlp.up": "mlp.up.weight", "mlp.down": "mlp.down.weight",
}
_TOP_NAMES = {"final.norm": "final.norm.weight"}
_LAYER_RE = re.compile(r"^(l\d+)\.(.+)$")


def adapt_tensors(cfg: NagolixConfig, found: Dict[str, LazyTensor]) -> Dict[str, LazyTensor]:
    """The checkpoint's names to the parts' names; anything unknown keeps its name, so that the
    strict check reports it."""
    out: Dict[str, LazyTensor] = {}
    no_ffn = {f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.mlp is None}
    for name, t in found.items():
        if name in no_ffn:
            continue                 # a second norm stored for a layer that has no feed-forward: nothing reads it
        new = _TOP_NAMES.get(name, name)
        m = _LAYER_RE.match(name)
        if m and m.group(2) in _LAYER_NAMES:
            new = f"{m.group(1)}.{_LAYER_NAMES[m.group(2)]}"
        if new in out:
            raise ValueError(f"checkpoint provides tensor {new!r} under two names")
        out[new] = t
    return out


def tensor_shapes(cfg: NagolixConfig, bias_rows: int = 32) -> Iterator[Tuple[str, Tuple[int, ...], str]]:
    """``(checkpoint name, shape, init)`` of every tensor, in the order random weights are drawn in."""
    d = cfg.dim
    yield "embed", (cfg.vocab_size, d), "embed"
    yield "pos", (cfg.max_seq_len, d), "pos"
    for i, layer in enumerate(cfg.layers):
        m, p = layer.mixer, f"l{i}"
        yield f"{p}.norm1", (d,), "norm"
        if layer.mlp is not None:
            yield f"{p}.norm2", (d,), "norm"
        yield f"{p}.mix.q", (m.heads * m.dim, d), "matrix"
        if m.kind == "attention":
            yield f"{p}.mix.q.b", (m.heads * m.dim,), "bias"
            yield f"{p}.mix.k", (m.kv_heads * m.dim, d), "matrix"
            yield f"{p}.mix.k.b", (m.kv_heads * m.dim,), "bias"
            yield f"{p}.mix.v", (m.kv_heads * m.vdim, d), "matrix"
            yield f"{p}.mix.v.b", (m.kv_heads * m.vdim,), "bias"
            yield f"{p}.mix.q.norm", (m.heads * m.dim,), "gain"
            yield f"{p}.mix.k.norm", (m.kv_heads * m.dim,), "gain"
            yield f"{p}.mix.rel", (bias_rows, m.heads), "bias"
            yield f"{p}.mix.g", (m.heads * m.vdim, d), "matrix"
        else:
            if m.kv_from is None:
                yield f"{p}.mix.dkv", (m.kv_rank, d), "matrix"
                yield f"{p}.mix.dkv.norm", (m.kv_rank,), "gain"
            yield f"{p}.mix.uk", (m.heads * m.dim, m.kv_rank), "matrix"
            yield f"{p}.mix.uv", (m.heads * m.vdim, m.kv_rank), "matrix"
            yield f"{p}.mix.g", (m.heads, d), "matrix"
        yield f"{p}.mix.o", (d, m.heads * m.vdim), "matrix"
        if layer.mlp is not None:
            yield f"{p}.mlp.gate", (layer.mlp.ff, d), "matrix"
            yield f"{p}.mlp.up", (layer.mlp.ff, d), "matrix"
            yield f"{p}.mlp.down", (d, layer.mlp.ff), "matrix"
    yield "final.norm", (d,), "norm"


def random_tensors(cfg: NagolixConfig, seed: int, *, device="cpu", dtype: torch.dtype = torch.float32,
                   bias_rows: int = 32) -> Iterator[Tuple[str, torch.Tensor]]:
    """Seeded random weights under the checkpoint's names (one generator, one order, drawn in
    float32, then cast): matrices ``N(0, 1/fan_in)``, the table's rows of unit size over the
    embedding's scale, norm weights around zero, gains around one."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    for name, shape, init in tensor_shapes(cfg, bias_rows):
        t = torch.randn(shape, generator=gen, device=device, dtype=torch.float32)
        if init == "matrix":
            t = t * shape[1] ** -0.5
        elif init == "embed":
            t = t / cfg.embedding_scale
        elif init in ("norm", "bias"):
            t = t * 0.1
        elif init == "gain":
            t = 1.0 + t * 0.1
        yield name, t.to(dtype)


NAGOLIX = register_architecture(Architecture(
    name=NAME,
    parse_config=parse_config,
    build_spec=build_spec,
    adapt_tensors=adapt_tensors,
    random_tensors=random_tensors,
    chat_template=None,
))
