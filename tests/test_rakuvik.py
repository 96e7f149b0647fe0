"""Rakuvik through the engine against the plain implementation (``plain_rakuvik``).

Every test runs three ways: over the kernels' plain PyTorch twins on the CPU (the package's
parts, cache manager, step function and scheduler are the ones under test there), and on the GPU
over the CUDA kernels in float32 and in bfloat16.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_rakuvik as plain
import rakuvik_cases as rc
from rakuvik_cases import BACKENDS


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", list(rc.CASES))
def test_whole_prompt_decoding_and_portions(tmp_path, backend, name):
    """A whole prompt in one step, the same tokens one by one from the first on, and portions of
    several sizes down to two tokens (cut inside pages and inside the recurrence's chunks) all
    give the plain logits."""
    cfg, tensors, folder, page = rc.case_folder(tmp_path, name, dtype=rc.stored_dtype(backend))
    n = 70 if name != "wide" else 200
    tokens = rc.clear_tokens(cfg, tensors, n, seed=1, dtype=backend[1])
    want = rc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = rc.make_replayer(folder, backend, 4 * 256, page)
    want.check(rc.feed(rp, "whole", tokens, [n]), "whole prompt")
    want.check(rc.feed(rp, "single", tokens, [] if n <= 70 else [n - 40]), "token by token")
    want.check(rc.feed(rp, "cut", tokens, [2, 3, 2, 7, 16, 2, 5, 9, 2, 11]), "portions")
    want.check(rc.feed(rp, "cut2", tokens, [page + 1, 2 * page - 1, 2, 2, 33]), "portions across pages")
    if n > 130:
        want.check(rc.feed(rp, "cut3", tokens, [64, 65, 2, 63]), "portions at the edges of the recurrence's chunks")
    assert rp.engine.cache.n_live() == 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_batches_of_unequal_requests(tmp_path, backend):
    """Four live requests of different lengths, portions beside single tokens, in a pool so small
    that pages and state slots are used again: every request's logits are those it gets alone."""
    cfg, tensors, folder, page = rc.case_folder(tmp_path, "mixed", dtype=rc.stored_dtype(backend))
    lengths = [61, 9, 34, 1, 47, 22, 80]
    reqs = {f"r{i}": rc.clear_tokens(cfg, tensors, n, seed=10 + i, dtype=backend[1]) for i, n in enumerate(lengths)}
    want = {rid: rc.plain_logits(cfg, tensors, toks, backend[1]) for rid, toks in reqs.items()}
    rp = rc.make_replayer(folder, backend, 4 * 128, page, max_num_seqs=4)
    rng = np.random.default_rng(0)
    waiting, live, at, got = list(reqs), [], {}, {rid: [] for rid in reqs}
    step = 0
    while waiting or live:
        while waiting and len(live) < 4:
            rid = waiting.pop(0)
            live.append(rid)
            at[rid] = 0
        entries, end = [], []
        for rid in live:
            if len(live) > 1 and rng.random() < 0.2:
                continue                                     # left out of this step
            left = len(reqs[rid]) - at[rid]
            n = 1 if (at[rid] > len(reqs[rid]) // 2) else int(min(left, rng.choice([2, 3, 5, 8, 13, 24])))
            entries.append({"id": rid, "tokens": reqs[rid][at[rid]:at[rid] + n], "want": list(range(n))})
            at[rid] += n
            if at[rid] == len(reqs[rid]):
                end.append(rid)
        if not entries:
            continue
        out = rp.run_step({"step": step, "entries": entries, "end": end})
        rp.engine.cache.check_invariants()
        row = 0
        for e in entries:
            got[e["id"]].append(out[row:row + len(e["tokens"])])
            row += len(e["tokens"])
        live = [rid for rid in live if rid not in end]
        step += 1
    for rid in reqs:
        want[rid].check(np.concatenate(got[rid]), rid)
    assert rp.engine.cache.n_live() == 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_and_a_slot_used_again(tmp_path, backend):
    """A short prompt and 250 tokens decoded one by one (recorded steps on the GPU), then another
    request in the same state slot and pages: its first tokens must not feel the state the first
    one left behind."""
    cfg, tensors, folder, page = rc.case_folder(tmp_path, "awkward", dtype=rc.stored_dtype(backend))
    tokens = rc.clear_tokens(cfg, tensors, 255, seed=3, dtype=backend[1])
    rp = rc.make_replayer(folder, backend, 256, page, max_num_seqs=1)
    rc.plain_logits(cfg, tensors, tokens, backend[1]).check(rc.feed(rp, "long", tokens, [5]), "long decoding")
    again = rc.clear_tokens(cfg, tensors, 20, seed=4, dtype=backend[1])
    rc.plain_logits(cfg, tensors, again, backend[1]).check(rc.feed(rp, "again", again, [1, 1, 3]), "the slot's next request")
    rp.engine.cache.check_invariants()


def test_layers_of_experts_as_one_matrix(tmp_path):
    """The form a decode batch takes on the GPU (every expert as one matrix each way, zeros where a
    token did not choose an expert), forced for every step over the kernels' twins: the same logits."""
    from torch_ops import TorchOps
    from torchllms_b200.engine.replay import Replayer
    cfg, tensors, folder, page = rc.case_folder(tmp_path, "mixed")
    tokens = rc.tokens_for(cfg, 40, seed=2)
    ops = TorchOps()
    ops.dense_experts = True
    rp = Replayer(folder, "float32", 256, page_size=page, device="cpu", ops=ops, max_num_seqs=2)
    rc.plain_logits(cfg, tensors, tokens, "float32").check(rc.feed(rp, "a", tokens, [17, 2]), "all experts as one matrix")


# ---------------------------------------------------------------- one mechanism at a time

def _one_layer(layer, **kw):
    return rc.config([layer], **kw)


def _marked(cfg, tensors, keys_at, query_at: int, n: int, score: float = 16.0, seed: int = 9):
    """Inputs and weights of a one-layer attention model made so that one query finds a few marked
    keys in its first map and next to nothing else.  The marked keys carry a token that no other
    position has, the query another such token; the first map's keys answer mostly to the marked
    token's direction, and its query projection has rank one: it
    answers the query token's (normed) embedding with the marked token's key, and any other input
    with little.  The scale makes the query score ``score`` against a marked key before rotation
    turns a part of it.  The query token's own key and value are its own, so what the query's first
    map returns is the marked keys' value: losing one of them, or reading a wrong page in its
    place, moves the query's logits by far more than any rounding.  Edits ``tensors`` and the
    configuration's scale in place; returns the tokens."""
    m = cfg["layers"][0]["mixer"]
    H, G, dk, d = m["heads"], m["kv_heads"], m["dim"], cfg["width"]
    key_token, query_token = cfg["vocab"] - 1, cfg["vocab"] - 2
    eps = cfg["norm"]["eps"]
    xa = plain.scalar_norm(tensors["embed"][key_token].double(), tensors["l0.norm1"].double(), eps)
    xb = plain.scalar_norm(tensors["embed"][query_token].double(), tensors["l0.norm1"].double(), eps)
    k = tensors["l0.mix.k"].double().view(G, 2, dk, d).clone()
    for g in range(G):          # the first map's keys answer mostly to the marked token's direction
        k[g, 0] = torch.outer(k[g, 0] @ xa, xa / (xa @ xa)) + 0.2 * k[g, 0]
    tensors["l0.mix.k"] = k.reshape(G * 2 * dk, d).float()
    q = tensors["l0.mix.q"].double().view(H, 2, dk, d).clone()
    for h in range(H):
        q[h, 0] = torch.outer(k[h // (H // G), 0] @ xa, xb / (xb @ xb))
    tensors["l0.mix.q"] = q.reshape(H * 2 * dk, d).float()
    ka = k[0, 0] @ xa
    m["scale"] = score / float(ka @ ka)
    tokens = np.random.default_rng(seed).integers(0, query_token, size=n).tolist()
    for p in keys_at:
        tokens[p] = key_token
    tokens[query_at] = query_token
    return tokens


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_far_key_that_stands_out(tmp_path, backend):
    """Hundreds of keys, one of them marked and far back, at a page's first and last place and in the
    middle: the query that is marked too must find it, in a prompt, decoded alone, and at the start of
    a portion.  The test first proves on the plain implementation that losing the key moves the logits."""
    page = 16
    for key_at in (0, 15, 16, 37):
        layer = rc.attention_layer(heads=2, kv_heads=1, dim=16, vdim=8, rot_dims=4, base=100.0, factor=4.0, diff=0.4, mlp=None)
        cfg = _one_layer(layer, width=32, vocab=50)
        tensors = rc.stored(rc.tensors_for(cfg, seed=key_at, sharp=1.0), rc.stored_dtype(backend))
        n, query_at = 300, 290
        tokens = _marked(cfg, tensors, (key_at,), query_at, n)
        tensors = rc.stored(tensors, rc.stored_dtype(backend))
        want = rc.plain_logits(cfg, tensors, tokens, backend[1])
        lost = list(tokens)
        lost[key_at] = 0
        assert np.abs(rc.plain_logits(cfg, tensors, lost, backend[1])[query_at] - want[query_at]).max() > 0.05, \
            "the test's inputs do not show the far key"
        folder = rc.write_folder(tmp_path, f"far{key_at}", cfg, tensors, rc.stored_dtype(backend))
        rp = rc.make_replayer(folder, backend, 640, page)
        want.check(rc.feed(rp, "p", tokens, [n]), f"prompt, key at {key_at}")
        want.check(rc.feed(rp, "d", tokens, [query_at - 3]), f"decoded, key at {key_at}")
        want.check(rc.feed(rp, "c", tokens, [page - 1, query_at - page + 1, 2, 2]), f"portion starting at the query, key at {key_at}")


@pytest.mark.parametrize("backend", BACKENDS)
def test_a_state_that_remembers_the_first_token(tmp_path, backend):
    """A recurrence whose gate stays nearly shut keeps its first tokens for hundreds of steps: the
    last logits depend on token 0 (proved on the plain implementation), so a state that is lost,
    zeroed or mixed up at the start of a portion or between steps shows."""
    cfg = _one_layer(rc.mingru_layer(width=40, mlp=None), width=64, vocab=50)
    tensors = rc.tensors_for(cfg, seed=2)
    # the gate is all but shut (z around 0.0003) except for one token that no other position has, which
    # opens it: what that token writes into the state at position 0 is still most of the state 200 steps on
    opener = cfg["vocab"] - 1
    x = plain.scalar_norm(tensors["embed"][opener].double(), tensors["l0.norm1"].double(), cfg["norm"]["eps"])
    tensors["l0.mix.z.b"].fill_(-8.0)
    tensors["l0.mix.z"] = (0.2 * tensors["l0.mix.z"].double() + 16.0 * (x / (x @ x))[None, :]).float()
    tensors = rc.stored(tensors, rc.stored_dtype(backend))
    n = 200
    tokens = [opener] + np.random.default_rng(5).integers(0, opener, size=n - 1).tolist()
    want = rc.plain_logits(cfg, tensors, tokens, backend[1])
    other = [0] + tokens[1:]
    assert np.abs(rc.plain_logits(cfg, tensors, other, backend[1])[n - 1] - want[n - 1]).max() > 0.05, \
        "the test's inputs do not show the first token at the end"
    folder = rc.write_folder(tmp_path, "memory", cfg, tensors, rc.stored_dtype(backend))
    rp = rc.make_replayer(folder, backend, 512, 16)
    want.check(rc.feed(rp, "p", tokens, [n]), "prompt")
    want.check(rc.feed(rp, "d", tokens, [1]), "decoded from the second token on")
    want.check(rc.feed(rp, "c", tokens, [63, 2, 64, 66]), "portions around the chunk size")


@pytest.mark.parametrize("backend", BACKENDS)
def test_rotation_far_from_the_start(tmp_path, backend):
    """Rotations over the whole head with a short base and a factor of one, and over a part of it
    with a large factor: positions in the hundreds, where a table that is off or angles taken in
    too few bits would show."""
    for rot_dims, base, factor in ((16, 50.0, 1.0), (6, 10000.0, 16.0), (0, 10.0, 1.0)):
        layer = rc.attention_layer(heads=2, kv_heads=2, dim=16, vdim=16, rot_dims=rot_dims, base=base, factor=factor, mlp=None)
        cfg = _one_layer(layer, width=32, vocab=50)
        tensors = rc.stored(rc.tensors_for(cfg, seed=rot_dims, sharp=3.0 if backend[1] == "float32" else 1.0), rc.stored_dtype(backend))
        tokens = rc.tokens_for(cfg, 400, seed=6)
        want = rc.plain_logits(cfg, tensors, tokens, backend[1])
        folder = rc.write_folder(tmp_path, f"rot{rot_dims}", cfg, tensors, rc.stored_dtype(backend))
        rp = rc.make_replayer(folder, backend, 512, 16)
        want.check(rc.feed(rp, "p", tokens, [400]), f"prompt, rot {rot_dims}")
        want.check(rc.feed(rp, "d", tokens, [380]), f"decoded, rot {rot_dims}")


def _ops_for(backend):
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        return TorchOps(), "cpu", torch.float32
    from torchllms_b200.kernels import get_ops
    return get_ops(), "cuda", (torch.float32 if backend[1] == "float32" else torch.bfloat16)


@pytest.mark.parametrize("backend", BACKENDS)
def test_small_kernels_against_the_plain_functions(backend):
    """The router, the experts, the recurrence, the gated and plain activations, the norm that adds
    and norms again, the average over depth, the rotation and the combination of two maps, each
    against the plain implementation's function, at sizes that are and are not multiples of four."""
    ops, dev, dtype = _ops_for(backend)
    g = torch.Generator().manual_seed(3)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    rounding = None if dtype == torch.float32 else dtype
    for T, dim in ((1, 64), (7, 42), (150, 256)):
        # router: a correction that decides the choice must not enter the weights
        E, top = 7, 3
        x = rnd(T, dim).to(dtype)
        w = {"router": 0.5 * rnd(E, dim), "correction": torch.tensor([0.0, 3.0, 0.0, -3.0, 0.0, 0.0, 0.0])}
        chosen, weights = plain.route(x.double(), w, top, 1.7, None)
        got_c, got_w, _ = ops.moe_route(x.to(dev), w["router"].to(dev), w["correction"].to(dev), n_experts=E, top=top, scale=1.7,
                                        renormalize=False, shared_gate=False)
        assert (chosen[:, 0] == 1).all() and not (chosen == 3).any()
        assert torch.equal(got_c.cpu().long().sort(-1).values, chosen.sort(-1).values)
        torch.testing.assert_close(got_w.cpu().sort(-1).values, weights.float().sort(-1).values, atol=1e-5, rtol=1e-5)
        # experts and the shared expert behind its gate
        ff = 24 if dim % 4 else 40
        ew = {f"e{e}.{n}": (rnd(ff, dim) * 2 / dim ** 0.5 if n == "up" else rnd(dim, ff) / ff ** 0.5).to(dtype).float()
              for e in range(E) for n in ("up", "down")}
        ew.update(w, **{"shared.up": (rnd(16, dim) / dim ** 0.5).to(dtype).float(), "shared.down": (rnd(dim, 16) / 4).to(dtype).float(),
                        "shared.sg": rnd(1, dim) / dim ** 0.5})
        mlp = {"router": {"experts": E, "top": top, "scale": 1.7}, "shared": {"ff": 16}}
        want = plain.moe_ff(x.double(), ew, mlp, rounding)
        router = torch.cat([w["router"], ew["shared.sg"]]).to(dev)
        c, wt, gate = ops.moe_route(x.to(dev), router, w["correction"].to(dev), n_experts=E, top=top, scale=1.7, renormalize=False,
                                    shared_gate=True)
        up = torch.stack([ew[f"e{e}.up"] for e in range(E)]).to(dtype).to(dev)
        down = torch.cat([ew[f"e{e}.down"] for e in range(E)], dim=1).to(dtype).to(dev)      # side by side: [dim, E * ff]
        u = ops.activation(ops.linear(x.to(dev), ew["shared.up"].to(dtype).to(dev)), "relu2")
        shared = ops.linear(u, ew["shared.down"].to(dtype).to(dev))
        got = ops.moe_experts(x.to(dev), c, wt, up, down, activation="relu2", shared=shared, shared_gate=gate)
        torch.testing.assert_close(got.float().cpu(), want.float(), atol=tol["atol"] * 4, rtol=tol["rtol"])
        # the same layer with all experts as one matrix each way (the form a decode batch takes)
        up_all = torch.cat([up.view(E * ff, dim), ew["shared.up"].to(dtype).to(dev)])
        down_all = torch.cat([down, ew["shared.down"].to(dtype).to(dev)], dim=1).contiguous()
        hidden_rows = ops.moe_dense_hidden(x.to(dev), c, wt, gate, up_all, n_experts=E, hidden=ff, activation="relu2")
        got = ops.linear(hidden_rows, down_all)
        torch.testing.assert_close(got.float().cpu(), want.float(), atol=tol["atol"] * 4, rtol=tol["rtol"])
        # the recurrence, with a state carried in and a fresh request beside it
        W = 20 if dim % 4 else 72
        lens = [T, 1, 3]
        proj, bias = rnd(sum(lens), 3 * W).to(dtype), 0.3 * rnd(3 * W)
        bias[2 * W:] = 0
        state = rnd(4, W)
        before = state.clone()
        q_start = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32)
        out = ops.mingru_scan(proj.to(dev), bias.to(dev), state.to(dev) if dev == "cuda" else state,
                              q_start.to(dev), torch.tensor([2, 0, 3], dtype=torch.int32).to(dev),
                              torch.tensor([0, 1, 0], dtype=torch.int32).to(dev), n_seqs=3, max_q_len=max(lens), out_dtype=dtype)
        x64 = proj.double() + bias.double()
        at = 0
        for b, (slot, fresh) in enumerate(((2, 0), (0, 1), (3, 0))):
            s = torch.zeros(W, dtype=torch.float64) if fresh else before[slot].double()
            for t in range(at, at + lens[b]):
                z, uu, gg = torch.sigmoid(x64[t, :W]), x64[t, W:2 * W], x64[t, 2 * W:]
                s = (1 - z) * s + z * torch.where(uu >= 0, uu + 0.5, torch.sigmoid(uu))
                torch.testing.assert_close(out[t].float().cpu(), (s * gg * torch.sigmoid(gg)).float(), **tol)
            at += lens[b]
        # gated and plain activations
        hidden = 50 if dim % 4 else 64
        gu = (2.0 * rnd(T, 2 * hidden)).to(dtype)
        want = (plain.gelu_tanh(gu.double()[:, :hidden]) * gu.double()[:, hidden:]).float()
        torch.testing.assert_close(ops.gated_act(gu.to(dev), "gelu_tanh").float().cpu(), want, **tol)
        torch.testing.assert_close(ops.activation(gu.to(dev), "relu2").float().cpu(), (torch.relu(gu.double()) ** 2).float(), **tol)
        # the output norm that adds to the stream and takes the next norm
        h, delta = rnd(T, dim), rnd(T, dim).to(dtype)
        w1, w2 = torch.full((dim,), 0.8), torch.full((dim,), 1.3)
        hh = h.clone().to(dev)
        rows = ops.norm_add(hh, delta.to(dev), w1.to(dev), 1e-5, out_dtype=dtype, then_weight=w2.to(dev), then_eps=1e-5)
        new = h.double() + plain.scalar_norm(delta.double(), torch.tensor(0.8), 1e-5)
        torch.testing.assert_close(hh.cpu(), new.float(), atol=2e-5, rtol=1e-5)
        torch.testing.assert_close(rows.float().cpu(), plain.scalar_norm(new, torch.tensor(1.3), 1e-5).float(), **tol)
        # the average over depth, written into the level after the ones it reads
        levels, coef = rnd(5, T, dim), rnd(4)
        hist = levels.clone().to(dev)
        ops.depth_mix(hist, coef.to(dev), 4, hist[4])
        torch.testing.assert_close(hist[4].cpu(), (levels[:4].double() * coef.double()[:, None, None]).sum(0).float(), atol=2e-5, rtol=1e-5)
        hist = levels.clone().to(dev)                   # ... and with the next layer's input norm from the same kernel
        rows = ops.depth_mix(hist, coef.to(dev), 4, hist[4], then_weight=w2.to(dev), then_eps=1e-5, out_dtype=dtype)
        mixed = (levels[:4].double() * coef.double()[:, None, None]).sum(0)
        torch.testing.assert_close(hist[4].cpu(), mixed.float(), atol=2e-5, rtol=1e-5)
        torch.testing.assert_close(rows.float().cpu(), plain.scalar_norm(mixed, torch.tensor(1.3), 1e-5).float(), **tol)
        # rotation of a part of every head, keys and values into pages of their own shapes
        nq, nk, nv, hd, vd, rot, page = 4, 2, 1, 12, 20, 8, 4
        proj = rnd(T, (nq + nk) * hd + nv * vd + 3).to(dtype)
        pos = torch.randint(0, 300, (T,), generator=g)
        from torchllms_b200.parts.rope import precise_rotary_table
        table = precise_rotary_table(rot, 100.0, 2.0, 300)
        n_pages = -(-T // page) + 2
        slots = torch.randperm(n_pages * page, generator=g)[:T].int()
        k_pages = torch.zeros(n_pages, nk, page, hd, dtype=dtype, device=dev)
        v_pages = torch.zeros(n_pages, nv, page, vd, dtype=dtype, device=dev)
        q, extra = ops.rope_store(proj.to(dev), pos.int().to(dev), table.to(dev), n_q_heads=nq, n_k_heads=nk, n_v_heads=nv,
                                  head_dim=hd, v_head_dim=vd, rot_dims=rot, interleaved=False, n_extra=3, k_pages=k_pages,
                                  v_pages=v_pages, slot_mapping=slots.to(dev), page_size=page, out_dtype=dtype)
        x64 = proj.double()
        qk = plain.rotate(x64[:, :(nq + nk) * hd].view(T, nq + nk, hd), pos, rot, 100.0, 2.0)
        torch.testing.assert_close(q.float().cpu(), qk[:, :nq].float(), **tol)
        sl = slots.long()
        torch.testing.assert_close(k_pages.cpu()[sl // page, :, sl % page].float(), qk[:, nq:].float(), **tol)
        torch.testing.assert_close(v_pages.cpu()[sl // page, :, sl % page].float().reshape(T, nv * vd),
                                   x64[:, (nq + nk) * hd:(nq + nk) * hd + nv * vd].float(), **tol)
        torch.testing.assert_close(extra.float().cpu(), torch.sigmoid(x64[:, -3:]).float(), **tol)
        # two maps into one result
        H, dv = 3, 20
        maps, gate = rnd(T, 2 * H, dv), torch.rand(T, H, generator=g).to(dtype)
        o = maps.double()[:, :H] - 0.37 * maps.double()[:, H:]
        want = (plain.unit_rms(o, 1e-5) * 0.6 * gate.double()[:, :, None]).reshape(T, H * dv)
        got = ops.differential_combine(maps.to(dev), 0.37, eps=1e-5, out_scale=0.6, gate=gate.to(dev), out_dtype=dtype)
        torch.testing.assert_close(got.float().cpu(), want.float(), **tol)


@pytest.mark.gpu
def test_gelu_gate_in_the_product_epilogue():
    """The one-kernel form (gelu(gate) * up in the tcgen05 product's epilogue) against product + gate kernel."""
    from torchllms_b200.kernels import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(8)
    for M, K, hidden in ((1, 256, 128), (8, 4096, 1024), (37, 512, 192), (64, 1024, 2048)):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(2 * hidden, K, generator=g) * (2.0 / K ** 0.5)).to(torch.bfloat16).cuda()
        two = ops.gated_act(ops.linear(x, w, partials_ok=True), "gelu_tanh", out_dtype=torch.bfloat16)
        one = ops.gemm_gated_gelu(x, w)
        ops.check_status()
        torch.testing.assert_close(one.float(), two.float(), atol=2e-2, rtol=2e-2)
        gu = x.double() @ w.double().T
        torch.testing.assert_close(one.double(), plain.gelu_tanh(gu[:, :hidden]) * gu[:, hidden:], atol=3e-2, rtol=3e-2)


def test_configuration_and_names(tmp_path):
    """The configuration reads back what it writes; a missing or misshapen tensor is refused; a
    borrowed cache must name a layer that owns one."""
    from torchllms_b200.config.model_config import ConfigError
    from torchllms_b200.config.registry import load_config
    from torchllms_b200.engine.loading import load_model
    from torchllms_b200.weights.loader import WeightError
    from torch_ops import TorchOps
    cfg, tensors, folder, _page = rc.case_folder(tmp_path, "mixed")
    arch, parsed = load_config(folder)
    assert arch.name == "Rakuvik" and parsed.to_hf() == cfg
    spec = arch.build_spec(parsed)
    assert [r.cache_of for r in spec.run_order] == [None, None, None, 1, None] and spec.keeps_history
    broken = dict(tensors)
    del broken["l1.mlp.correction"]
    broken["l0.mix.z.b"] = broken["l0.mix.z.b"][:-1]
    broken["l3.mix.k"] = tensors["l1.mix.k"].clone()      # a layer that borrows has no keys of its own
    bad = rc.write_folder(tmp_path, "broken", cfg, broken)
    with pytest.raises(WeightError) as e:
        load_model(bad, dtype="float32", device="cpu", ops=TorchOps())
    assert "l1.mlp.correction" in str(e.value) and "l0.mix.wz.bias" in str(e.value) and "l3.mix.wk.weight" in str(e.value)
    wrong = json_copy(cfg)
    wrong["layers"][3]["mixer"]["kv_from"] = 0            # a recurrent layer has nothing to lend
    (tmp_path / "wrong").mkdir()
    (tmp_path / "wrong" / "config.json").write_text(__import__("json").dumps(wrong))
    with pytest.raises(ConfigError):
        load_config(tmp_path / "wrong")


def json_copy(x):
    import json
    return json.loads(json.dumps(x))


@pytest.mark.parametrize("backend", BACKENDS[:2])
def test_greedy_generation_through_the_scheduler(tmp_path, backend):
    """``LLM.generate`` (scheduler, sampler, look-ahead) against a plain greedy loop."""
    from torchllms_b200.inference import LLM
    cfg, tensors, folder, page = rc.case_folder(tmp_path, "mixed")
    kw = {}
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        kw = dict(ops=TorchOps())
    llm = LLM(folder, max_len=128, max_bsz=3, device=backend[0], precision=backend[1], page_size=page,
              max_num_batched_tokens=24, **kw)
    prompts = [rc.tokens_for(cfg, n, seed=20 + n) for n in (3, 30, 11, 1)]
    results = llm.generate(prompt_token_ids=prompts, temperature=0.0, max_new_tokens=12, disable_tqdm=True)
    for prompt, r in zip(prompts, results):
        seq = list(prompt)
        for _ in range(12):
            logits = plain.forward(cfg, tensors, seq)[-1]
            top = torch.topk(logits, 2).values
            if float(top[0] - top[1]) < 1e-3:
                break                         # a near tie may fall either way: stop comparing this request
            seq.append(int(torch.argmax(logits)))
        made = seq[len(prompt):]
        assert r.error is None and r.token_ids[:len(made)] == made


def test_random_weights_mode_writes_a_folder_that_loads(tmp_path):
    """The framework's random-weights mode for this architecture: a folder under the checkpoint's
    names that loads like any other, and the same model built without a file."""
    from torchllms_b200.config.registry import load_config
    from torchllms_b200.engine.loading import load_model, random_model
    from torchllms_b200.weights.random_init import write_random_model
    from torchllms_b200.weights.safetensors_io import TensorSource
    from torch_ops import TorchOps
    _cfg, _tensors, folder, _page = rc.case_folder(tmp_path, "mixed")
    _arch, parsed = load_config(folder)
    out = write_random_model(tmp_path / "random", parsed, seed=3)
    names = set(TensorSource(out).names())
    assert {"embed", "head", "final.norm", "l0.mix.z.b", "l1.mix.lq1", "l1.mlp.e5.down", "l1.mlp.shared.sg", "l4.dwa"} <= names
    assert "l3.mix.k" not in names and "l2.norm2" not in names and "l3.mlp.shared.up" not in names
    _, _, from_file = load_model(out, dtype="float32", device="cpu", ops=TorchOps())
    _, _, direct = random_model(parsed, 3, dtype="float32", device="cpu", ops=TorchOps())
    assert torch.equal(from_file.embedding, direct.embedding)
    assert torch.equal(from_file.blocks[1].mixer.w_in, direct.blocks[1].mixer.w_in)
