"""Nagolix through the engine against the plain implementation (``plain_nagolix``).

Every test runs three ways: over the kernels' plain PyTorch twins on the CPU (the package's
parts, cache manager, step function and scheduler are the ones under test there), and on the GPU
over the CUDA kernels in float32 and in bfloat16.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

import nagolix_cases as nc
import plain_nagolix as plain
from nagolix_cases import BACKENDS


def check(got: np.ndarray, want: nc.Expected, backend, what: str = ""):
    want.check(got, what)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("name", list(nc.CASES))
def test_whole_prompt_decoding_and_portions(tmp_path, backend, name):
    """A whole prompt in one step, the same tokens one by one from the first on, and portions of
    several sizes down to two tokens (cut inside pages and windows) all give the plain logits."""
    cfg, tensors, folder, page = nc.case_folder(tmp_path, name, dtype=nc.stored_dtype(backend))
    n = 70 if name != "wide" else 150
    tokens = nc.tokens_for(cfg, n, seed=1)
    want = nc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = nc.make_replayer(folder, backend, 4 * 256, page)
    check(nc.feed(rp, "whole", tokens, [n]), want, backend, "whole prompt")
    check(nc.feed(rp, "single", tokens, []), want, backend, "token by token")
    check(nc.feed(rp, "cut", tokens, [2, 3, 2, 7, 16, 2, 5, 9, 2, 11]), want, backend, "portions")
    check(nc.feed(rp, "cut2", tokens, [page + 1, 2 * page - 1, 2, 2, 33]), want, backend, "portions across pages")
    assert rp.engine.cache.n_live() == 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_batches_of_unequal_requests(tmp_path, backend):
    """Four live requests of different lengths, portions beside single tokens, in a pool so small
    that pages and slots are used again: every request's logits are those it gets alone."""
    cfg, tensors, folder, page = nc.case_folder(tmp_path, "mixed", dtype=nc.stored_dtype(backend))
    lengths = [61, 9, 34, 1, 47, 22, 80]
    reqs = {f"r{i}": nc.tokens_for(cfg, n, seed=10 + i) for i, n in enumerate(lengths)}
    want = {rid: nc.plain_logits(cfg, tensors, toks, backend[1]) for rid, toks in reqs.items()}
    rp = nc.make_replayer(folder, backend, 4 * 128, page, max_num_seqs=4)
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
        check(np.concatenate(got[rid]), want[rid], backend, rid)
    assert rp.engine.cache.n_live() == 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_long_decoding_gives_pages_back(tmp_path, backend):
    """Decoding far past every window: pages behind the windows go back (the kept first ones stay)
    and the logits stay those of the plain implementation."""
    cfg, tensors, folder, page = nc.case_folder(tmp_path, "awkward", dtype=nc.stored_dtype(backend))
    tokens = nc.tokens_for(cfg, 140, seed=3)
    want = nc.plain_logits(cfg, tensors, tokens, backend[1])
    rp = nc.make_replayer(folder, backend, 192, page)
    got = nc.feed(rp, "long", tokens, [5], end=False)
    check(got, want, backend, "long decoding")
    cache = rp.engine.cache
    handle = rp.handles["long"]
    for gi, g in enumerate(cache.groups):
        held = [p for p in cache.pages_of(handle, gi) if p >= 0]
        need = g.need
        most = -(-need.keep_first // page) + -(-need.window // page) + 1
        assert len(held) <= most, f"group {gi} holds {len(held)} pages for a window of {need.window}"
        if need.keep_first:
            assert all(p >= 0 for p in cache.pages_of(handle, gi)[:-(-need.keep_first // page)])
    rp.engine.release(handle)
    cache.check_invariants()


# ---------------------------------------------------------------- one mechanism at a time

def _one_layer(layer, **kw):
    return nc.config([layer], **kw)


def _spiked(cfg, tensors, marked, n: int, amplitude: float = 4.0):
    """Inputs and weights made so that a few marked positions find each other and nothing else:
    queries are projected as keys are (so a score is a similarity), and the marked positions carry
    one large common vector.  A marked query then gives the marked keys it can see nearly all of its
    weight, and a window that is one key off moves its logits by far more than any rounding.
    Edits ``tensors`` in place; returns the tokens."""
    layer = cfg["layers"][0]
    m = layer["mixer"]
    if layer["type"] == "attention":
        tensors["l0.mix.q"] = torch.cat([tensors["l0.mix.k"]] * (m["heads"] // m["kv_heads"]))
        tensors["l0.mix.q.b"].zero_()
        tensors["l0.mix.k.b"].zero_()
        tensors["l0.mix.k.norm"].fill_(2.0)
        tensors["l0.mix.q.norm"].fill_(2.0)
    else:
        tensors["l0.mix.q"] = tensors["l0.mix.uk"] @ tensors["l0.mix.dkv"]
    mark = amplitude * torch.sign(torch.randn(cfg["width"], generator=torch.Generator().manual_seed(5)))
    # values must not carry the mark, or all marked keys would bring the same value: take its direction
    # out of the value projection, so that a marked key's value is its own token's
    if layer["type"] == "attention":
        u = mark / mark.norm()
        tensors["l0.mix.v"] -= torch.outer(tensors["l0.mix.v"] @ u, u)
    else:
        c = tensors["l0.mix.dkv.norm"] * (tensors["l0.mix.dkv"] @ mark)
        c = c / c.norm()
        tensors["l0.mix.uv"] -= torch.outer(tensors["l0.mix.uv"] @ c, c)
    tensors["pos"].mul_(0.1)
    for p in marked:
        tensors["pos"][p] = mark
    # the scale is chosen so that a marked query scores about 8 against a marked key (and so next to
    # nothing, after the softmax, against any other)
    eps, dk = cfg["norm"]["eps"], m["dim"]
    if layer["type"] == "attention":
        q = plain.norm_plain(tensors["l0.mix.q"] @ mark, tensors["l0.mix.q.norm"], eps)[:dk]
        k = plain.norm_plain(tensors["l0.mix.k"] @ mark, tensors["l0.mix.k.norm"], eps)[:dk]
    else:
        q = (tensors["l0.mix.q"] @ mark)[:dk]
        k = (tensors["l0.mix.uk"] @ plain.norm_plain(tensors["l0.mix.dkv"] @ mark, tensors["l0.mix.dkv.norm"], eps))[:dk]
    m["scale"] = 8.0 / float(q @ k)
    return nc.tokens_for(cfg, n, seed=9)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("kind", ["attention", "latent"])
def test_window_edges_with_a_key_that_stands_out(tmp_path, backend, kind):
    """One key carries a large mark.  Queries just inside its window must see it and those just
    outside must not, in a prompt and decoded one by one, with the key on a page border and with a
    kept first token: a window that is off by one moves the logits by far more than the tolerance."""
    size, keep = 11, 3
    page = 4
    for key_at in (1, 2, 3, 7, 8):        # kept (attention) and not kept; 3 and 7 sit at page borders
        layer = (nc.attention_layer(heads=2, kv_heads=1, dim=16, vdim=16, size=size, keep_first=keep, ff=None)
                 if kind == "attention" else nc.latent_layer(heads=2, dim=16, vdim=16, kv_rank=16, size=size, ff=None))
        cfg = _one_layer(layer, width=32, vocab=50, max_positions=64)
        tensors = nc.tensors_for(cfg, seed=key_at, bias_rows=8, sharp=4.0)
        if backend[1] == "bfloat16":
            tensors = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
        edge = key_at + size - 1                 # the last query that sees the key through the window
        kept = kind == "attention" and key_at < keep
        tokens = _spiked(cfg, tensors, (key_at, edge + 1) if kept else (key_at, edge, edge + 1), 40)
        if backend[1] == "bfloat16":
            tensors = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
        folder = nc.write_folder(tmp_path, f"{kind}{key_at}", cfg, tensors, nc.stored_dtype(backend))
        want = nc.plain_logits(cfg, tensors, tokens, backend[1])
        # the oracle itself must feel the edge: a window one shorter or longer moves these rows visibly
        if not kept:
            for row, other_size in ((edge, size - 1), (edge + 1, size + 1)):
                moved = dict(cfg, layers=[dict(layer, mixer=dict(layer["mixer"], mask=dict(layer["mixer"]["mask"], size=other_size)))])
                other = nc.plain_logits(moved, tensors, tokens, backend[1])
                assert np.abs(other[row] - want[row]).max() > 0.01, "the test's inputs do not show the edge"
        else:                                    # a kept key: without keeping it, the rows past the window move
            dropped = dict(cfg, layers=[dict(layer, mixer=dict(layer["mixer"], mask=dict(layer["mixer"]["mask"], keep_first=key_at)))])
            other = nc.plain_logits(dropped, tensors, tokens, backend[1])
            assert np.abs(other[edge + 1] - want[edge + 1]).max() > 0.01, "the test's inputs do not show the kept key"
        rp = nc.make_replayer(folder, backend, 256, page)
        check(nc.feed(rp, "p", tokens, [40]), want, backend, f"prompt, key at {key_at}")
        check(nc.feed(rp, "d", tokens, [key_at + 1]), want, backend, f"decoded, key at {key_at}")
        check(nc.feed(rp, "c", tokens, [edge, 2, 2]), want, backend, f"portion starting at the edge, key at {key_at}")


@pytest.mark.parametrize("backend", BACKENDS)
def test_far_keys_and_the_distance_table(tmp_path, backend):
    """A window wider than the prompt: every query sees hundreds of keys, the distance table is
    used along its whole logarithmic part and beyond its far end."""
    layer = nc.attention_layer(heads=2, kv_heads=2, dim=16, vdim=8, size=400, keep_first=0, bias_max=90.0, ff=None)
    cfg = _one_layer(layer, width=32, vocab=50, max_positions=320)
    tensors = nc.tensors_for(cfg, seed=4, bias_rows=10, sharp=3.0)
    tensors["l0.mix.rel"] *= 3.0
    if backend[1] == "bfloat16":
        tensors = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    tokens = _spiked(cfg, tensors, (2, 150, 290, 299), 300)
    if backend[1] == "bfloat16":
        tensors = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    folder = nc.write_folder(tmp_path, "far", cfg, tensors, nc.stored_dtype(backend))
    want = nc.plain_logits(cfg, tensors, tokens, backend[1])
    blind = nc.plain_logits(dict(cfg, layers=[dict(layer, mixer=dict(layer["mixer"], mask={"size": 297, "keep_first": 0}))]),
                            tensors, tokens, backend[1])
    assert np.abs(blind[299] - want[299]).max() > 0.01, "the test's inputs do not show the far key"
    rp = nc.make_replayer(folder, backend, 640, 16)
    check(nc.feed(rp, "p", tokens, [300]), want, backend, "prompt")
    check(nc.feed(rp, "d", tokens, [280]), want, backend, "decoded tail")


def test_distance_buckets_table():
    from torchllms_b200.parts.attention import distance_buckets
    for rows, far in ((16, 240.0), (12, 50.0), (7, 33.0), (2, 9.0)):
        table = distance_buckets(rows, far, 400).tolist()
        assert table == [plain.distance_bucket(n, rows, far) for n in range(400)]
        assert table[0] == 0 and max(table) == rows - 1 and all(b >= a for a, b in zip(table, table[1:]))


def test_configuration_and_names(tmp_path):
    """The configuration reads back what it writes; a missing or misshapen tensor is refused."""
    from torchllms_b200.config.registry import load_config
    from torchllms_b200.engine.loading import load_model
    from torchllms_b200.weights.loader import WeightError
    from torch_ops import TorchOps
    cfg, tensors, folder, _page = nc.case_folder(tmp_path, "mixed")
    arch, parsed = load_config(folder)
    assert arch.name == "Nagolix" and parsed.to_hf() == cfg
    spec = arch.build_spec(parsed)
    assert [r.cache_of for r in spec.run_order] == [None, None, 0, None]
    broken = dict(tensors)
    del broken["l1.mix.rel"]
    broken["l0.mix.uk"] = broken["l0.mix.uk"][:-1]
    bad = nc.write_folder(tmp_path, "broken", cfg, broken)
    with pytest.raises(WeightError) as e:
        load_model(bad, dtype="float32", device="cpu", ops=TorchOps())
    assert "l1.mix.distance_bias" in str(e.value) and "l0.mix.w_up_k.weight" in str(e.value)


@pytest.mark.parametrize("backend", BACKENDS[:2])
def test_greedy_generation_through_the_scheduler(tmp_path, backend):
    """``LLM.generate`` (scheduler, sampler, look-ahead) against a plain greedy loop."""
    from torchllms_b200.inference import LLM
    cfg, tensors, folder, page = nc.case_folder(tmp_path, "mixed")
    kw = {}
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        kw = dict(ops=TorchOps())
    llm = LLM(folder, max_len=128, max_bsz=3, device=backend[0], precision=backend[1], page_size=page,
              max_num_batched_tokens=24, **kw)
    prompts = [nc.tokens_for(cfg, n, seed=20 + n) for n in (3, 30, 11, 1)]
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


# ---------------------------------------------------------------- the attention kernels' options alone

def _paged_case(rng, seq_lens, q_lens, H, KV, hd, dv, P, dtype, shared):
    """Random queries, and random keys / values in a shuffled page pool (values of their own size,
    or the key pages themselves)."""
    g = torch.Generator().manual_seed(rng.randrange(1 << 30))
    B = len(seq_lens)
    blocks = [-(-L // P) for L in seq_lens]
    n_pages = sum(blocks) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((B, max(blocks) + 2), -1, dtype=torch.int32)
    it = iter(perm)
    for b in range(B):
        for j in range(blocks[b]):
            table[b, j] = next(it)
    k_pages = torch.randn((n_pages, KV, P, hd), generator=g).to(dtype).cuda()
    v_pages = k_pages if shared else torch.randn((n_pages, KV, P, dv), generator=g).to(dtype).cuda()
    q = (torch.randn((sum(q_lens), H, hd), generator=g) * 1.5).to(dtype).cuda()
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32).cuda()
    return dict(q=q, k_pages=k_pages, v_pages=v_pages, block_table=table.cuda(), q_start=q_start,
                kv_len=torch.tensor(seq_lens, dtype=torch.int32).cuda(), n_seqs=B, max_q_len=max(q_lens),
                max_kv_len=max(seq_lens), page_size=P)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_kernels_with_options_on_random_shapes(dtype):
    """Both kernels that take the options (CUDA cores; tensor cores in bfloat16) against the plain
    PyTorch twin: ragged batches of portions and single tokens late in their contexts, windows with
    and without kept first keys, distance tables, gates per head and per element, values of another
    size, keys read as values."""
    import random
    from torchllms_b200.kernels import get_ops
    from torchllms_b200.parts.attention import distance_buckets
    from torch_ops import TorchOps
    ops, twin = get_ops(), TorchOps()
    rng = random.Random(11)
    for case in range(40):
        H, KV = rng.choice([(4, 2), (3, 1), (8, 8), (6, 2), (20, 1), (1, 1)])
        hd = rng.choice([8, 16, 24, 32, 48, 64, 128] if dtype == torch.bfloat16 else [4, 12, 16, 40, 64])
        shared = rng.random() < 0.3
        dv = hd if shared else rng.choice([hd, 8, 16, 40, 64, 128])
        P = rng.choice([4, 8, 16, 64])
        B = rng.randint(1, 4)
        q_lens = [rng.choice([1, 1, rng.randint(2, 9), rng.randint(10, 150)]) for _ in range(B)]
        seq_lens = [ql + rng.choice([0, rng.randint(1, 40), rng.randint(100, 700)]) for ql in q_lens]
        window = rng.choice([None, rng.randint(1, 30), rng.randint(31, 400)])
        keep = rng.choice([0, 0, 1, 4, 19]) if window else 0
        a = _paged_case(rng, seq_lens, q_lens, H, KV, hd, dv, P, dtype, shared)
        T = sum(q_lens)
        kw = dict(scale=hd ** -0.5, window=window, keep_first=keep)
        if rng.random() < 0.6:
            rows = rng.choice([2, 6, 16, 21])
            kw["distance_bias"] = torch.randn(rows, H, generator=torch.Generator().manual_seed(case)).cuda()
            kw["distance_buckets"] = distance_buckets(rows, float(rng.choice([rows, 50, 300])) + 1.0, max(seq_lens) + 1).cuda()
        mode = rng.choice([0, 1, 2])
        if mode:
            kw["gate"] = torch.rand(T, H if mode == 1 else H * dv, generator=torch.Generator().manual_seed(case)).to(dtype).cuda()
        want = twin.paged_attention(**a, **kw).float()
        impls = ["general"]
        if dtype == torch.bfloat16 and hd % 8 == 0 and dv % 8 == 0 and max(hd, dv) <= 128:
            impls.append("mma")
        for impl in impls:
            got = ops.paged_attention(**a, **kw, impl=impl).float()
            tol = 2e-5 if dtype == torch.float32 else 2e-2
            torch.testing.assert_close(got, want, atol=tol, rtol=tol, msg=lambda m: (
                f"{impl} case {case}: seq {seq_lens} q {q_lens} H{H} KV{KV} hd{hd} dv{dv} P{P} window {window} keep {keep} "
                f"bias {'distance_bias' in kw} gate {mode} shared {shared}: {m}"))


def test_random_weights_mode_writes_a_folder_that_loads(tmp_path):
    """The framework's random-weights mode for this architecture: a folder under the checkpoint's
    names that loads like any other, and the same model built without a file."""
    from torchllms_b200.config.registry import load_config
    from torchllms_b200.engine.loading import load_model, random_model
    from torchllms_b200.weights.random_init import write_random_model
    from torchllms_b200.weights.safetensors_io import TensorSource
    from torch_ops import TorchOps
    cfg, _tensors, folder, _page = nc.case_folder(tmp_path, "mixed")
    _arch, parsed = load_config(folder)
    out = write_random_model(tmp_path / "random", parsed, seed=3)
    names = set(TensorSource(out).names())
    assert {"embed", "pos", "final.norm", "l0.mix.dkv", "l1.mix.rel", "l2.mix.uk", "l3.mlp.down"} <= names
    assert "l2.mix.dkv" not in names and "l2.norm2" not in names       # borrowed latents; no feed-forward
    _, _, from_file = load_model(out, dtype="float32", device="cpu", ops=TorchOps())
    _, _, direct = random_model(parsed, 3, dtype="float32", device="cpu", ops=TorchOps())
    assert torch.equal(from_file.embedding, direct.embedding)
    assert torch.equal(from_file.blocks[1].mixer.w_in, direct.blocks[1].mixer.w_in)


# ---------------------------------------------------------------- the small kernels against the plain functions

def _ops_for(backend):
    if backend[0] == "cpu":
        from torch_ops import TorchOps
        return TorchOps(), "cpu", torch.float32
    from torchllms_b200.kernels import get_ops
    return get_ops(), "cuda", (torch.float32 if backend[1] == "float32" else torch.bfloat16)


@pytest.mark.parametrize("backend", BACKENDS)
def test_small_kernels_against_the_plain_functions(backend):
    """Embedding with scale and positions, the norm of a sublayer's output with the residual sum
    (also from split-K partial sums), the clamped gate (both forms on the GPU), the stacked
    projection's kernel and the per-head products, each against the plain implementation's function,
    at widths that are and are not multiples of four, for one row and for many."""
    ops, dev, dtype = _ops_for(backend)
    g = torch.Generator().manual_seed(3)
    tol = dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    rnd = lambda *shape: torch.randn(*shape, generator=g)
    for T, dim in ((1, 64), (7, 42), (130, 256), (9, 1032)):
        # embedding
        table, pos = rnd(50, dim).to(dtype), rnd(40, dim).to(dtype)
        ids, at = torch.randint(0, 50, (T,), generator=g), torch.randint(0, 40, (T,), generator=g)
        got = ops.embed(ids.int().to(dev), table.to(dev), scale=3.5, positions=at.int().to(dev), position_table=pos.to(dev))
        torch.testing.assert_close(got.cpu(), table.float()[ids] * 3.5 + pos.float()[at], atol=1e-6, rtol=1e-6)
        # norm of the output + residual sum, from a tensor and from partial sums
        h, delta, w = rnd(T, dim), rnd(T, dim).to(dtype), 1.0 + 0.1 * rnd(dim)
        want = h + plain.norm_one_plus(delta.double(), (w - 1.0).double(), 1e-5).float()
        hh = h.clone().to(dev)
        rows = ops.norm_add(hh, delta.to(dev), w.to(dev), 1e-5, out_dtype=dtype)
        torch.testing.assert_close(hh.cpu(), want, atol=2e-5 if dtype == torch.float32 else 3e-2, rtol=1e-5)
        torch.testing.assert_close(rows.float().cpu(), hh.cpu().to(dtype).float(), atol=0, rtol=0)
        parts = rnd(3, T, dim)
        hh = h.clone().to(dev)
        ops.norm_add(hh, parts.to(dev), w.to(dev), 1e-5, out_dtype=dtype)
        want = h + plain.norm_one_plus(parts.sum(0).double(), (w - 1.0).double(), 1e-5).float()
        torch.testing.assert_close(hh.cpu(), want, atol=2e-5, rtol=1e-5)
        # clamped gate
        hidden = 64 if dim % 4 == 0 else 50
        gu = (2.0 * rnd(T, 2 * hidden)).to(dtype)
        gg, uu = gu.double()[:, :hidden].clamp(max=1.25), gu.double()[:, hidden:].clamp(-1.25, 1.25)
        want = (gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)).float()
        got = ops.glu(gu.to(dev), limit=1.25, alpha=1.702, up_offset=1.0)
        torch.testing.assert_close(got.float().cpu(), want, **tol)
        # the stacked projection: [q | k | v | extra], norms over whole rows, pages, sigmoid
        H, G, dk, dv, page = 3, 1, dim // 2 if dim <= 64 else 24, 8, 4
        n_q, n_k, n_v, n_e = H * dk, G * dk, G * dv, H * dv
        proj, bias = rnd(T, n_q + n_k + n_v + n_e).to(dtype), 0.3 * rnd(n_q + n_k + n_v + n_e)
        qw, kw = 1.0 + 0.2 * rnd(n_q), 1.0 + 0.2 * rnd(n_k)
        n_pages = -(-T // page) + 2
        slots = torch.randperm(n_pages * page, generator=g)[:T].int()
        k_pages = torch.zeros(n_pages, G, page, dk, dtype=dtype, device=dev)
        v_pages = torch.zeros(n_pages, G, page, dv, dtype=dtype, device=dev)
        q, extra = ops.project_and_store(proj.to(dev), n_q=n_q, n_k=n_k, n_v=n_v, n_extra=n_e, bias=bias.to(dev), q_norm=qw.to(dev),
                                         k_norm=kw.to(dev), eps=1e-5, k_pages=k_pages, v_pages=v_pages, slot_mapping=slots.to(dev),
                                         page_size=page, out_dtype=dtype)
        x = proj.double() + bias.double()
        xq, xk, xv, xe = x.split([n_q, n_k, n_v, n_e], dim=1)
        torch.testing.assert_close(q.float().cpu(), plain.norm_plain(xq, qw.double(), 1e-5).float(), **tol)
        torch.testing.assert_close(extra.float().cpu(), torch.sigmoid(xe).float(), **tol)
        sl = slots.long()
        torch.testing.assert_close(k_pages.cpu()[sl // page, :, sl % page].float().reshape(T, n_k),
                                   plain.norm_plain(xk, kw.double(), 1e-5).float(), **tol)
        torch.testing.assert_close(v_pages.cpu()[sl // page, :, sl % page].float().reshape(T, n_v), xv.float(), **tol)
        # per-head products
        K, N = dk, 20
        xh, wh = rnd(T, H, K).to(dtype), (rnd(H, N, K) / K ** 0.5).to(dtype)
        got = ops.head_linear(xh.to(dev), wh.to(dev))
        torch.testing.assert_close(got.float().cpu(), torch.einsum("thk,hnk->thn", xh.double(), wh.double()).float(), **tol)


@pytest.mark.gpu
def test_clamped_gate_in_the_product_epilogue():
    """The one-kernel form (gate in the tcgen05 product's epilogue) against product + gate kernel."""
    from torchllms_b200.kernels import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(8)
    for M, K, hidden in ((1, 256, 128), (8, 4096, 1024), (37, 512, 192), (64, 1024, 2048)):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(2 * hidden, K, generator=g) * (2.0 / K ** 0.5)).to(torch.bfloat16).cuda()
        two = ops.glu(ops.linear(x, w, partials_ok=True), out_dtype=torch.bfloat16, limit=1.5, alpha=1.702, up_offset=1.0)
        one = ops.gemm_gated_clamped(x, w, 1.5, 1.702, 1.0)
        ops.check_status()
        torch.testing.assert_close(one.float(), two.float(), atol=2e-2, rtol=2e-2)
        gu = x.double() @ w.double().T
        gg, uu = gu[:, :hidden].clamp(max=1.5), gu[:, hidden:].clamp(-1.5, 1.5)
        torch.testing.assert_close(one.double(), gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), atol=3e-2, rtol=3e-2)


@pytest.mark.gpu
def test_chat_command_line_in_token_ids(tmp_path, monkeypatch, capsys):
    """The chat program on a folder of this architecture (no tokenizer: it chats in token ids), with a
    longest sequence asked for that the learned position table cannot give."""
    from torchllms_b200.inference import chat
    cfg, tensors, folder, _page = nc.case_folder(tmp_path, "mixed")
    lines = iter(["5 17 3", "8"])

    def fake_input(_prompt=""):
        try:
            return next(lines)
        except StopIteration:
            raise EOFError
    monkeypatch.setattr("builtins.input", fake_input)
    chat.main(["--ckpt_paths", str(folder), "--precision", "float32", "--max_new_tokens", "4", "--max_len", "4096"])
    said = [l for l in capsys.readouterr().out.splitlines() if l.startswith("[assistant]: ")]
    assert len(said) == 2
    first = [int(t) for t in said[0].split(": ")[1].split()]
    seq = [5, 17, 3]
    for _ in range(4):
        seq.append(int(torch.argmax(plain.forward(cfg, tensors, seq)[-1])))
    assert first == seq[3:]
