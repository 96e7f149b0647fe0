"""Rakuvik written out plainly: whole sequences, float64, explicit ``[n, n]`` masks and a token
by token recurrence, one function per mechanism.  It shares no code with the package; the tests
hold the engine to it.

``config`` is the design's ``config.json`` as a dict, ``tensors`` the checkpoint's tensors by
name.  ``rounding`` (``None`` or a torch dtype) rounds what a reduced-precision engine may round:
the results of projections and the activations between them; everything the design wants in
32-bit stays unrounded.
"""

from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Tuple

import torch

F = torch.float64


def _round(x: torch.Tensor, rounding) -> torch.Tensor:
    return x if rounding is None else x.to(rounding).to(F)


def _lin(x: torch.Tensor, w: torch.Tensor, rounding) -> torch.Tensor:
    """``W x`` for every row of ``x``; input and result rounded as a reduced-precision product's are."""
    return _round(_round(x, rounding) @ w.to(F).T, rounding)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is one number for all coordinates."""
    return unit_rms(x, eps) * float(g)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float, factor: float) -> torch.Tensor:
    """``x [n, heads, size]``: the first ``dims`` coordinates of every head turn by the position's
    angles, coordinate ``i`` paired with ``i + dims / 2``; the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    freq = base ** (-2.0 * i / dims) / factor
    ang = positions.to(F)[:, None] * freq[None, :]                  # [n, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attention_keys_values(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, rounding) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotated keys ``[n, G, 2, dim]`` and values ``[n, G, vdim]`` of a layer that projects its own."""
    n = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    pos = torch.arange(n)
    k = _lin(h, w["k"], rounding).view(n, G * 2, d)
    k = rotate(k, pos, rot["dims"], rot["base"], rot["scaling"]["factor"]).view(n, G, 2, d)
    v = _lin(h, w["v"], rounding).view(n, G, dv)
    return _round(k, rounding), v


def differential_attention(h: torch.Tensor, w: Mapping[str, torch.Tensor], m: Mapping, eps: float, rounding,
                           kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
    """Two softmax maps over the same values, combined as ``a1 - lambda a2``; returns the mixer's
    output and the keys and values it used (for a later layer that borrows them)."""
    n = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    pos = torch.arange(n)
    q = _lin(h, w["q"], rounding).view(n, H * 2, d)
    q = _round(rotate(q, pos, rot["dims"], rot["base"], rot["scaling"]["factor"]), rounding).view(n, H, 2, d)
    if kv is None:
        kv = attention_keys_values(h, w, m, rounding)
    k, v = kv
    lam = (math.exp(float((w["lq1"].to(F) * w["lk1"].to(F)).sum())) - math.exp(float((w["lq2"].to(F) * w["lk2"].to(F)).sum()))
           + m["diff"])
    hidden = pos[None, :] > pos[:, None]
    gate = torch.sigmoid(_lin(h, w["g"], rounding))                     # [n, H]
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        maps = []
        for mm in range(2):
            s = (q[:, hh, mm] @ k[:, g, mm].T) * m["scale"]
            p = torch.softmax(s.masked_fill(hidden, float("-inf")), dim=-1)
            maps.append(p @ v[:, g])
        o = maps[0] - lam * maps[1]
        o = unit_rms(o, eps) * (1.0 - m["diff"])
        heads.append(o * gate[:, hh:hh + 1])
    o = _round(torch.cat(heads, dim=-1), rounding)
    return _lin(o, w["o"], rounding), kv


def mingru(h: torch.Tensor, w: Mapping[str, torch.Tensor], rounding) -> torch.Tensor:
    """A gated recurrence whose gates read the current token only; the state starts at zero."""
    z = torch.sigmoid(_lin(h, w["z"], rounding) + w["z.b"].to(F))
    u = _lin(h, w["x"], rounding) + w["x.b"].to(F)
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    out_gate = _lin(h, w["g"], rounding)
    out_gate = out_gate * torch.sigmoid(out_gate)
    state = torch.zeros(z.shape[1], dtype=F)
    rows = []
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * cand[t]
        rows.append(state * out_gate[t])
    return _lin(_round(torch.stack(rows), rounding), w["o"], rounding)


def dense_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], rounding) -> torch.Tensor:
    y = gelu_tanh(_lin(h, w["gate"], rounding)) * _lin(h, w["up"], rounding)
    return _lin(_round(y, rounding), w["down"], rounding)


def squared_relu_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor, rounding) -> torch.Tensor:
    y = torch.relu(_lin(h, up, rounding)) ** 2
    return _lin(_round(y, rounding), down, rounding)


def route(h: torch.Tensor, w: Mapping[str, torch.Tensor], top: int, scale: float, rounding,
          margins: Optional[list] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts ``[n, top]`` and their weights: scores are a softmax over all experts, the
    choice adds a correction that the weights do not carry, and nothing is renormalised.
    ``margins`` collects, per token, how far the last chosen expert stood above the first one
    left out, as a share of the larger of their two scores (rounding moves a score by a share of
    itself; a test that wants no close call looks at this)."""
    s = torch.softmax(_round(h, rounding) @ w["router"].to(F).T, dim=-1)
    choice = s + w["correction"].to(F)
    chosen = torch.topk(choice, top, dim=-1).indices
    if margins is not None and top < choice.shape[1]:
        best = torch.topk(choice, top + 1, dim=-1)
        near = torch.gather(s, 1, best.indices[:, top - 1:top + 1]).max(-1).values
        margins.append((best.values[:, top - 1] - best.values[:, top]) / near)
    return chosen, torch.gather(s, 1, chosen) * scale


def moe_ff(h: torch.Tensor, w: Mapping[str, torch.Tensor], mlp: Mapping, rounding, margins: Optional[list] = None) -> torch.Tensor:
    r = mlp["router"]
    chosen, weights = route(h, w, r["top"], r["scale"], rounding, margins)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F)
    for e in range(r["experts"]):
        for slot in range(r["top"]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if rows.numel():
                y = squared_relu_expert(h[rows], w[f"e{e}.up"], w[f"e{e}.down"], rounding)
                out[rows] += weights[rows, slot:slot + 1] * y
    if mlp.get("shared") is not None:
        share = torch.sigmoid(_round(h, rounding) @ w["shared.sg"].to(F).T)          # [n, 1]
        out = out + share * squared_relu_expert(h, w["shared.up"], w["shared.down"], rounding)
    return out


def _sub(tensors: Mapping[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: Mapping, tensors: Mapping[str, torch.Tensor], tokens: List[int], rounding=None,
            return_layers: bool = False, margins: Optional[list] = None):
    """Logits ``[n, vocab]`` (float64) of every position of one sequence.  ``margins``: see :func:`route`."""
    eps = config["norm"]["eps"]
    x = tensors["embed"].to(F)[torch.tensor(tokens, dtype=torch.long)]
    history = [x]
    kept: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mw = _sub(tensors, p + "mix.")
        hin = scalar_norm(x, tensors[p + "norm1"], eps)
        if layer["type"] == "attention":
            src = layer["mixer"].get("kv_from")
            y, kv = differential_attention(hin, mw, layer["mixer"], eps, rounding, None if src is None else kept[src])
            kept[i] = kv
        elif layer["type"] == "mingru":
            y = mingru(hin, mw, rounding)
        else:
            raise ValueError(layer["type"])
        x = x + scalar_norm(y, tensors[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            fw = _sub(tensors, p + "mlp.")
            hin = scalar_norm(x, tensors[p + "norm2"], eps)
            y = dense_ff(hin, fw, rounding) if layer["mlp"]["kind"] == "dense" else moe_ff(hin, fw, layer["mlp"], rounding, margins)
            x = x + scalar_norm(y, tensors[p + "norm2b"], eps)
        history.append(x)
        coef = tensors[p + "dwa"].to(F)
        x = sum(coef[j] * history[j] for j in range(i + 2))
        after.append(x)
    x = scalar_norm(x, tensors["final.norm"], eps)
    logits = _round(x, rounding) @ tensors["head"].to(F).T
    return (logits, torch.stack(after)) if return_layers else logits
