"""A plain, slow Nagolix: whole sequences, one function per mechanism, float64 by default.

Written from the design's equations and sharing nothing with the package: no cache, no pages, no
batching.  A sequence of ``n`` tokens is run as ``n`` rows at once; every mask is an explicit
``[n, n]`` table of who sees whom.  ``emulate_bf16=True`` rounds where a bfloat16 engine stores
bfloat16 (projections and activations), leaving norms, scores, probabilities and the residual
stream unrounded.

The design in short (``x`` is the residual stream, one row per token, position ``p`` from 0):

* ``x = E[token] * s_e + P[p]``
* every layer: ``x += N1(mixer(x))`` then, if it has one, ``x += N2(ff(x))`` where
  ``N(y) = y / sqrt(mean(y^2) + eps) * (1 + w)``: the norm sits on the sublayer's output.
* logits ``= E @ N_final(x)`` (the table itself, unscaled).
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Mapping, Optional

import torch


def rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + eps)


def norm_one_plus(y: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(y, eps) * (1.0 + w)


def norm_plain(y: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(y, eps) * w


def distance_bucket(n: int, n_rows: int, far: float) -> int:
    """Row of the distance table for a key ``n`` places back: exact below half the rows,
    logarithmic up to ``far``, the last row beyond."""
    half = n_rows // 2
    if n < half:
        return n
    return min(n_rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (n_rows - half))))


def window_mask(n: int, size: int, keep_first: int = 0) -> torch.Tensor:
    """``[n, n]`` bool: row i sees column j."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def masked_softmax(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    s = scores.masked_fill(~visible, float("-inf"))
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(-1, keepdim=True)


class Rounder:
    """Rounds to bfloat16 where a bfloat16 engine keeps bfloat16; the identity otherwise."""

    def __init__(self, emulate: bool):
        self.emulate = emulate

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.bfloat16).to(t.dtype) if self.emulate else t


def dense_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], limit: float, rd: Rounder) -> torch.Tensor:
    g = torch.clamp(rd(h @ w["gate"].T), max=limit)
    u = torch.clamp(rd(h @ w["up"].T), min=-limit, max=limit)
    y = rd(g * torch.sigmoid(1.702 * g) * (u + 1.0))
    return rd(y @ w["down"].T)


def attention_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], eps: float,
                    rd: Rounder) -> torch.Tensor:
    n = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rd(h @ w["q"].T + w["q.b"])
    k = rd(h @ w["k"].T + w["k.b"])
    v = rd(h @ w["v"].T + w["v.b"])
    q = rd(norm_plain(q, w["q.norm"], eps)).view(n, H, dk)        # one norm over the whole row, then heads
    k = rd(norm_plain(k, w["k.norm"], eps)).view(n, G, dk)
    v = v.view(n, G, dv)
    rel = w["rel"]                                                  # [rows, H]
    rows = rel.shape[0]
    dist = torch.tensor([[distance_bucket(i - j, rows, m["bias_max"]) if j <= i else 0 for j in range(n)]
                         for i in range(n)], dtype=torch.long)
    visible = window_mask(n, m["mask"]["size"], m["mask"].get("keep_first", 0))
    out = torch.empty(n, H, dv, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * m["scale"] + rel[dist, head]
        out[:, head] = masked_softmax(s, visible) @ v[:, kv]
    gate = torch.sigmoid(rd(h @ w["g"].T))
    return rd(rd(rd(out.reshape(n, H * dv)) * gate) @ w["o"].T)


def latent_of(h: torch.Tensor, w: Mapping[str, torch.Tensor], eps: float, rd: Rounder) -> torch.Tensor:
    return rd(norm_plain(rd(h @ w["dkv"].T), w["dkv.norm"], eps))


def latent_mixer(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping[str, Any], latent: torch.Tensor,
                 rd: Rounder) -> torch.Tensor:
    """``latent`` is this layer's own (``latent_of``) or the one of the layer it borrows from."""
    n = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = rd(h @ w["q"].T).view(n, H, dk)
    k = rd(latent @ w["uk"].T).view(n, H, dk)
    v = rd(latent @ w["uv"].T).view(n, H, dv)
    visible = window_mask(n, m["mask"]["size"])
    out = torch.empty(n, H, dv, dtype=h.dtype)
    for head in range(H):
        s = (q[:, head] @ k[:, head].T) * m["scale"]
        out[:, head] = masked_softmax(s, visible) @ v[:, head]
    gate = torch.sigmoid(rd(h @ w["g"].T))                          # [n, H]: one number per head
    out = rd(rd(out) * gate[:, :, None])
    return rd(out.reshape(n, H * dv) @ w["o"].T)


def sub(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], tokens: List[int], *,
            dtype=torch.float64, emulate_bf16: bool = False, layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits ``[n, vocab]`` of one whole sequence."""
    t = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    rd = Rounder(emulate_bf16)
    eps = config["norm"]["eps"]
    ids = torch.tensor(tokens, dtype=torch.long)
    x = t["embed"][ids] * config["embedding"]["scale"] + t["pos"][: len(tokens)]
    latents: Dict[int, torch.Tensor] = {}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        w = sub(t, p + "mix.")
        h = rd(x)
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(h, w, eps, rd)
                src = i
            y = latent_mixer(h, w, m, latents[src], rd)
        elif layer["type"] == "attention":
            y = attention_mixer(h, w, m, eps, rd)
        else:
            raise ValueError(layer["type"])
        x = x + norm_one_plus(y, t[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = dense_ff(rd(x), sub(t, p + "mlp."), layer["mlp"]["limit"], rd)
            x = x + norm_one_plus(y, t[p + "norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    y = rd(norm_one_plus(x, t["final.norm"], eps))
    return y @ t["embed"].T
