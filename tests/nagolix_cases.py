"""Small Nagolix configurations with random weights for the tests, and the two ways of running
them: the plain implementation (``plain_nagolix``) and the engine, either over the CUDA kernels or,
without a GPU, over their plain PyTorch twins (``torch_ops.TorchOps``), which still exercises the
package's parts, cache manager, step function and scheduler.

The configurations differ from each other in every size, so that nothing can lean on two numbers
being equal: grouped and ungrouped heads, key and value sizes that differ, head sizes that are no
multiple of 16, windows and kept-first counts that are no multiple of the page size, a layer without
a feed-forward, a borrowed latent read through a wider and a narrower window than its owner's,
bias tables of other heights.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

import numpy as np
import pytest
import torch

import plain_nagolix as plain


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, size=12, keep_first=2, bias_max=40.0, scale=None, ff=48,
                    limit=2.0):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "bias_max": bias_max,
                      "mask": {"size": size, "keep_first": keep_first}, "scale": scale or dim ** -0.5},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def latent_layer(heads=2, dim=16, vdim=16, kv_rank=24, size=20, kv_from=None, scale=None, ff=48, limit=2.0):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": size},
             "scale": scale or dim ** -0.5}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer,
            "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


def config(layers, width=64, vocab=97, max_positions=256, eps=1e-5, scale=7.0):
    return {"architecture": "Nagolix", "embedding": {"scale": scale}, "layers": layers, "max_positions": max_positions,
            "norm": {"eps": eps}, "vocab": vocab, "width": width}


# name -> (config, page size, bias-table rows)
CASES = {
    # every kind of layer once, sizes all different; the second latent layer reads the first one's latents
    # through a wider window than the owner's
    "mixed": (config([
        latent_layer(heads=2, dim=16, vdim=8, kv_rank=24, size=10),
        attention_layer(heads=4, kv_heads=2, dim=16, vdim=32, size=12, keep_first=3, bias_max=50.0),
        latent_layer(heads=3, dim=8, vdim=16, kv_rank=24, size=17, kv_from=0, ff=None),
        attention_layer(heads=2, kv_heads=1, dim=32, vdim=16, size=7, keep_first=1, bias_max=30.0, ff=80, limit=0.7),
    ], width=64, vocab=97), 8, 12),
    # awkward sizes: a width that is no multiple of 4, heads of 24 and 40, windows across page borders,
    # a borrowed latent behind a narrower window, one kv head per head, a tall bias table
    "awkward": (config([
        attention_layer(heads=3, kv_heads=3, dim=24, vdim=40, size=9, keep_first=5, bias_max=100.0, ff=50),
        latent_layer(heads=5, dim=12, vdim=20, kv_rank=36, size=13, ff=30),
        latent_layer(heads=1, dim=20, vdim=12, kv_rank=36, size=6, kv_from=1),
    ], width=42, vocab=61, eps=1e-4, scale=3.0), 4, 20),
    # heads the tensor-core kernels like, a window longer than most prompts, nothing kept
    "wide": (config([
        attention_layer(heads=4, kv_heads=1, dim=64, vdim=64, size=300, keep_first=0, bias_max=200.0, ff=256),
        latent_layer(heads=4, dim=64, vdim=32, kv_rank=128, size=300, ff=320),
    ], width=128, vocab=211, max_positions=512), 16, 6),
}


def tensors_for(cfg: dict, seed: int, bias_rows: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random float32 tensors under the checkpoint's names.  ``sharp`` scales the query and key
    sides so that attention is peaked and a single wrong key moves the logits."""
    g = torch.Generator().manual_seed(seed)
    d = cfg["width"]

    def mat(rows, cols, gain=1.0):
        return torch.randn(rows, cols, generator=g) * (gain / cols ** 0.5)

    def vec(n, centre=0.0, spread=0.1):
        return centre + spread * torch.randn(n, generator=g)

    out = {"embed": torch.randn(cfg["vocab"], d, generator=g) / cfg["embedding"]["scale"],
           "pos": 0.5 * torch.randn(cfg["max_positions"], d, generator=g), "final.norm": vec(d)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = vec(d)
        out[p + "mix.q"] = mat(H * dk, d, sharp)
        out[p + "mix.o"] = mat(d, H * dv)
        if layer["type"] == "attention":
            G = m["kv_heads"]
            out[p + "mix.k"], out[p + "mix.v"] = mat(G * dk, d, sharp), mat(G * dv, d)
            out[p + "mix.q.b"], out[p + "mix.k.b"], out[p + "mix.v.b"] = vec(H * dk), vec(G * dk), vec(G * dv)
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = vec(H * dk, 1.0 * sharp), vec(G * dk, 1.0 * sharp)
            out[p + "mix.rel"] = torch.randn(bias_rows, H, generator=g)
            out[p + "mix.g"] = mat(H * dv, d)
        else:
            if "kv_from" not in m:
                out[p + "mix.dkv"] = mat(m["kv_rank"], d)
                out[p + "mix.dkv.norm"] = vec(m["kv_rank"], 1.0)
            out[p + "mix.uk"], out[p + "mix.uv"] = mat(H * dk, m["kv_rank"], sharp), mat(H * dv, m["kv_rank"])
            out[p + "mix.g"] = mat(H, d)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            out[p + "norm2"] = vec(d)
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = mat(ff, d, 2.0), mat(ff, d, 2.0), mat(d, ff)
    return out


def write_folder(tmp, name: str, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float32) -> Path:
    from safetensors.torch import save_file
    folder = Path(tmp) / f"nagolix_{name}"
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(dtype).contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def case_folder(tmp, name: str, sharp: Optional[float] = None, dtype=torch.float32):
    """In float32 the weights are sharp (peaked attention: one wrong key moves the logits far beyond
    the tolerance); in bfloat16 they are not, or rounding alone would scatter the logits."""
    cfg, page, rows = CASES[name]
    if sharp is None:
        sharp = 3.0 if dtype == torch.float32 else 1.0
    tensors = tensors_for(cfg, seed=sum(map(ord, name)), bias_rows=rows, sharp=sharp)
    if dtype != torch.float32:       # what the file stores is what both sides compute with
        tensors = {k: v.to(dtype).float() for k, v in tensors.items()}
    return cfg, tensors, write_folder(tmp, name, cfg, tensors, dtype), page


def tokens_for(cfg: dict, n: int, seed: int = 0) -> List[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


class Expected:
    """The plain logits of a sequence and how far an engine may be from them.  In float32: 5e-5 of the
    largest logit on every logit (2e-4 at least; the logits are of order one to ten).  In bfloat16 the yardstick is what rounding itself does to
    this model: the plain implementation is run a second time with bfloat16 rounding of every
    projection and activation, and a row of the engine's logits may differ from the exact ones
    (root mean square over the vocabulary) by three times what that emulation differs, the typical
    row's figure standing in where a row's own is smaller; one row in twenty may pass that, by half at most."""

    def __init__(self, cfg, tensors, tokens, dtype: str):
        self.dtype = dtype
        self.logits = plain.forward(cfg, tensors, tokens).to(torch.float32).numpy()
        if dtype == "bfloat16":
            rounded = plain.forward(cfg, tensors, tokens, emulate_bf16=True).to(torch.float32).numpy()
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
            # (the emulation is one draw of the rounding noise and the engine's another: a row may pass its
            # allowance by half, and one row in twenty may pass it at all)
            assert err[worst] <= 1.5 * self.allowed[worst], \
                f"{what}: row {worst} differs by {err[worst]} (rms), rounding alone allows {self.allowed[worst]}"
            assert (err > self.allowed).mean() <= 0.05, f"{what}: {(err > self.allowed).sum()} of {len(err)} rows over their allowance"


def plain_logits(cfg, tensors, tokens, dtype: str) -> Expected:
    return Expected(cfg, tensors, tokens, dtype)


# ---- the two ways to run the engine
BACKENDS = [pytest.param(("cpu", "float32"), id="twin-f32"),
            pytest.param(("cuda", "float32"), id="gpu-f32", marks=pytest.mark.gpu),
            pytest.param(("cuda", "bfloat16"), id="gpu-bf16", marks=pytest.mark.gpu)]


def make_replayer(folder, backend, max_tokens: int, page: int, max_num_seqs: int = 4):
    from torchllms_b200.engine.replay import Replayer
    device, dtype = backend
    if device == "cpu":
        from torch_ops import TorchOps
        return Replayer(folder, dtype, max_tokens, page_size=page, device="cpu", ops=TorchOps(), max_num_seqs=max_num_seqs)
    return Replayer(folder, dtype, max_tokens, page_size=page, max_num_seqs=max_num_seqs)


def stored_dtype(backend):
    return torch.bfloat16 if backend[1] == "bfloat16" else torch.float32


def feed(rp, rid: str, tokens: List[int], cuts: List[int], end: bool = True) -> np.ndarray:
    """One request alone, cut into portions of the given sizes (the rest one by one); all logits."""
    rows, at, step = [], 0, 0
    sizes = list(cuts)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
        last = at + n == len(tokens)
        out = rp.run_step({"step": step, "entries": [{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}],
                           "end": [rid] if (last and end) else []})
        rows.append(out)
        rp.engine.cache.check_invariants()
        at += n
        step += 1
    return np.concatenate(rows)
