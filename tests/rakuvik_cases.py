"""Small Rakuvik configurations with random weights for the tests, and the two ways of running
them: the plain implementation (``plain_rakuvik``) and the engine, either over the CUDA kernels or,
without a GPU, over their plain PyTorch twins (``torch_ops.TorchOps``), which still exercises the
package's parts, cache manager, step function and scheduler.

The configurations differ from each other in every size, so that nothing can lean on two numbers
being equal: grouped and ungrouped heads, key and value sizes that differ, rotations over a part
of a head and over all of it, a scaling factor of one, layers without a feed-forward, borrowed
keys and values, one expert per token and several, layers of experts with and without a shared
expert, recurrent widths below and above the stream's.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import torch

import plain_rakuvik as plain
from nagolix_cases import BACKENDS, feed, make_replayer, stored_dtype, tokens_for  # noqa: F401  (generic helpers)


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, diff=0.5, rot_dims=8, base=10000.0, factor=4.0, scale=None,
                    kv_from=None, mlp=None):
    mixer = {"diff": diff, "dim": dim, "heads": heads, "kv_heads": kv_heads,
             "rot": {"base": base, "dims": rot_dims, "scaling": {"factor": factor}},
             "scale": scale or dim ** -0.5, "vdim": vdim}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"mixer": mixer, "mlp": mlp, "type": "attention"}


def mingru_layer(width=48, mlp=None):
    return {"mixer": {"width": width}, "mlp": mlp, "type": "mingru"}


def dense(ff=80):
    return {"ff": ff, "kind": "dense"}


def moe(experts=6, top=2, ff=24, scale=1.3, shared=40):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "scale": scale, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def config(layers, width=64, vocab=97, eps=1e-5):
    return {"architecture": "Rakuvik", "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


# name -> (config, page size)
CASES = {
    # every kind of layer and feed-forward, sizes all different; the last attention layer borrows
    # the first one's keys and values
    "mixed": (config([
        mingru_layer(width=48, mlp=dense(80)),
        attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, factor=4.0, mlp=moe(6, 2, 24, 1.3, 40)),
        mingru_layer(width=80, mlp=None),
        attention_layer(heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, factor=4.0, diff=0.3, kv_from=1, mlp=moe(5, 3, 16, 0.7, 0)),
        mingru_layer(width=32, mlp=moe(4, 1, 40, 1.0, 24)),
    ], width=64, vocab=97), 8),
    # awkward sizes: a width that is no multiple of 8, one key/value head per head, heads of 24 over
    # values of 8, a rotation over the whole head with a factor of one, one expert per token, an
    # attention layer without a feed-forward, a recurrent width that is no multiple of 4
    "awkward": (config([
        attention_layer(heads=3, kv_heads=3, dim=24, vdim=8, rot_dims=24, base=300.0, factor=1.0, diff=0.8, mlp=None),
        mingru_layer(width=42, mlp=moe(7, 1, 20, 2.0, 12)),
        attention_layer(heads=6, kv_heads=1, dim=12, vdim=20, rot_dims=4, factor=2.5, diff=0.2, mlp=dense(50)),
    ], width=44, vocab=61, eps=1e-4), 4),
    # sizes the tensor-core kernels take, prompts longer than the scan's chunk
    "wide": (config([
        attention_layer(heads=4, kv_heads=1, dim=64, vdim=128, rot_dims=48, base=250000.0, factor=6.0, mlp=moe(8, 2, 96, 1.25, 160)),
        mingru_layer(width=288, mlp=dense(384)),
        attention_layer(heads=4, kv_heads=1, dim=64, vdim=128, rot_dims=48, base=250000.0, factor=6.0, kv_from=0, mlp=dense(192)),
    ], width=256, vocab=211), 16),
}


def tensors_for(cfg: dict, seed: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names.  ``sharp`` scales the query and key
    sides and the router, so that attention and routing are peaked and a single wrong key or
    expert moves the logits."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / cols ** 0.5)

    def vec(n, centre=0.0, spread=0.1):
        return centre + spread * torch.randn(n, generator=g)

    def one(centre=1.0, spread=0.1):
        return torch.tensor(centre) + spread * torch.randn((), generator=g)

    out = {"embed": torch.randn(cfg["vocab"], d, generator=g), "final.norm": one(), "head": mat(cfg["vocab"], d)}
    for i, layer in enumerate(cfg["layers"]):
        m, mlp, p = layer["mixer"], layer["mlp"], f"l{i}."
        out[p + "norm1"], out[p + "norm1b"] = one(), one(0.7)
        if layer["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out[p + "mix.q"] = mat(H * 2 * dk, d, sharp)
            if "kv_from" not in m:
                out[p + "mix.k"], out[p + "mix.v"] = mat(G * 2 * dk, d, sharp), mat(G * dv, d)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[p + "mix." + n] = vec(dk, 0.0, 0.25)
            out[p + "mix.g"], out[p + "mix.o"] = mat(H, d, 2.0), mat(d, H * dv)
        else:
            w = m["width"]
            out[p + "mix.z"], out[p + "mix.z.b"] = mat(w, d, 2.0), vec(w, -0.5, 0.5)
            out[p + "mix.x"], out[p + "mix.x.b"] = mat(w, d, 2.0), vec(w, 0.0, 0.5)
            out[p + "mix.g"], out[p + "mix.o"] = mat(w, d, 2.0), mat(d, w)
        if mlp is not None:
            out[p + "norm2"], out[p + "norm2b"] = one(), one(0.7)
            if mlp["kind"] == "dense":
                ff = mlp["ff"]
                out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = mat(ff, d, 2.0), mat(ff, d, 2.0), mat(d, ff)
            else:
                r, ff = mlp["router"], mlp["expert"]["ff"]
                for e in range(r["experts"]):
                    out[p + f"mlp.e{e}.up"], out[p + f"mlp.e{e}.down"] = mat(ff, d, 2.0), mat(d, ff)
                out[p + "mlp.router"] = mat(r["experts"], d, 6.0)      # decisive whatever the dtype: see clear_tokens
                out[p + "mlp.correction"] = vec(r["experts"], 0.0, 0.05)
                if mlp.get("shared"):
                    sf = mlp["shared"]["ff"]
                    out[p + "mlp.shared.up"], out[p + "mlp.shared.down"] = mat(sf, d, 2.0), mat(d, sf)
                    out[p + "mlp.shared.sg"] = mat(1, d, 2.0)
        coef = vec(i + 2, 0.0, 0.3)
        coef[-1] += 1.0
        out[p + "dwa"] = coef
    return out


def write_folder(tmp, name: str, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float32) -> Path:
    from safetensors.torch import save_file
    folder = Path(tmp) / f"rakuvik_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def stored(tensors: Dict[str, torch.Tensor], dtype) -> Dict[str, torch.Tensor]:
    """What the file stores is what both sides compute with."""
    return tensors if dtype == torch.float32 else {k: v.to(dtype).float() for k, v in tensors.items()}


def case_folder(tmp, name: str, sharp: Optional[float] = None, dtype=torch.float32):
    """In float32 the weights are sharp (peaked attention and routing: one wrong key or expert moves
    the logits far beyond the tolerance); in bfloat16 they are not, or rounding alone would
    scatter the logits."""
    cfg, page = CASES[name]
    if sharp is None:
        sharp = 3.0 if dtype == torch.float32 else 1.0
    tensors = stored(tensors_for(cfg, seed=sum(map(ord, name)), sharp=sharp), dtype)
    return cfg, tensors, write_folder(tmp, name, cfg, tensors, dtype), page


def clear_tokens(cfg: dict, tensors, n: int, seed: int = 0, dtype: str = "bfloat16") -> List[int]:
    """Random tokens on which no router of the model has a close call: everywhere the last chosen
    expert stands above the first one left out by at least a share of their scores (15 % for
    bfloat16, where the stream that the router reads carries the rounding of everything before it;
    0.1 % for float32).  A choice that rounding flips would move that row's logits, and through
    the caches and states all later rows', by far more than rounding does.  The sequence is grown
    eight tokens at a time, a block being drawn again until its own positions are clear (the model
    is causal: earlier positions stay as they were)."""
    margin = 0.15 if dtype == "bfloat16" else 1e-3
    rng = np.random.default_rng(1000 + seed)
    tokens: List[int] = []
    while len(tokens) < n:
        k = min(8, n - len(tokens))
        for _ in range(200):
            block = rng.integers(0, cfg["vocab"], size=k).tolist()
            margins: list = []
            plain.forward(cfg, tensors, tokens + block, margins=margins)
            if not margins or min(float(m[len(tokens):].min()) for m in margins) >= margin:
                break
        else:
            raise AssertionError("no tokens with clear routing found: make the router sharper")
        tokens += block
    return tokens


class Expected:
    """The plain logits of a sequence and how far an engine may be from them.  In float32: 5e-5 of
    the largest logit on every logit (2e-4 at least).  In bfloat16 the yardstick is what rounding
    itself does to this model: the plain implementation is run a second time with bfloat16 rounding
    of every projection and activation, and a row of the engine's logits may differ from the exact
    ones (root mean square over the vocabulary) by three times what that emulation differs, the
    typical row's figure standing in where a row's own is smaller; one row in twenty may pass
    that, by half at most."""

    def __init__(self, cfg, tensors, tokens, dtype: str):
        self.dtype = dtype
        self.logits = plain.forward(cfg, tensors, tokens).to(torch.float32).numpy()
        if dtype == "bfloat16":
            rounded = plain.forward(cfg, tensors, tokens, rounding=torch.bfloat16).to(torch.float32).numpy()
            noise = np.sqrt(((rounded - self.logits) ** 2).mean(-1))
            self.allowed = 3.0 * np.maximum(noise, np.median(noise))

    def __getitem__(self, rows):
        return self.logits[rows]

    def check(self, got: np.ndarray, what: str = "") -> None:
        assert got.shape == self.logits.shape, f"{what}: {got.shape} logits for {self.logits.shape}"
        if self.dtype == "float32":
            err = np.abs(got - self.logits).max()
            limit = 5e-5 * max(4.0, float(np.abs(self.logits).max()))
            assert err <= limit, f"{what}: logits differ by {err} (allowed {limit})"
        else:
            err = np.sqrt(((got - self.logits) ** 2).mean(-1))
            worst = int(np.argmax(err / self.allowed))
            assert err[worst] <= 1.5 * self.allowed[worst], \
                f"{what}: row {worst} differs by {err[worst]} (rms), rounding alone allows {self.allowed[worst]}"
            assert (err > self.allowed).mean() <= 0.05, f"{what}: {(err > self.allowed).sum()} of {len(err)} rows over their allowance"


def plain_logits(cfg, tensors, tokens, dtype: str) -> Expected:
    return Expected(cfg, tensors, tokens, dtype)
