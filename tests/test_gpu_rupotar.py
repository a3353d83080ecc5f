"""Rupotar on the GPU against the plain implementation (tests/plain_rupotar.py):
every mechanism alone, then whole models in every cutting of the same tokens
(whole prompts, token by token, portions down to two tokens, mixed batches),
slots and pages that are used again, keys at the edges of the window, of the
kept first tokens and of cache pages, long decoding, and greedy generation
through the engine's own loop and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_rupotar as plain
import rupotar_tiny as tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
DTYPES = [torch.float32, torch.bfloat16]


def rel_error(got, want):
    """Largest row error: rms of the difference over rms of the wanted values."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape and np.isfinite(got).all()
    scale = max(np.sqrt((want ** 2).mean()), 1e-12)
    return float(np.sqrt(((got - want) ** 2).mean(-1)).max() / scale)


def bound(dtype, loose=1.0):
    return (3e-5 if dtype in (torch.float32, "float32") else 4e-2) * loose


def double(weights):
    return {k: v.double() for k, v in weights.items()}


def make_ctx(cache, slots, counts, vocab=1000):
    from foundry_b200.engine import SequenceStep, build_context
    return build_context(cache, [SequenceStep(s, [0] * n, []) for s, n in zip(slots, counts)],
                         vocab, DEV)


def spec_of(name):
    from foundry_b200.config.rupotar import RupotarConfig, replace
    from foundry_b200.models.rupotar import build_rupotar_spec
    cfg = RupotarConfig.parse(tiny.CONFIGS[name])
    decay, gate = tiny.RANKS[name]
    cfg = replace(cfg, layers=tuple(replace(l, decay_rank=decay, gate_rank=gate) for l in cfg.layers))
    return build_rupotar_spec(cfg)


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_each_mixer_alone_in_two_cuttings(name, dtype):
    """Every mixer of both configurations with a cache of its own: two sequences of
    unequal lengths in one step, then the same rows as a prompt part, a portion of
    two tokens and single tokens."""
    from foundry_b200.cache import SequenceCache
    from foundry_b200.parts import MIXERS
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    spec = spec_of(name)
    torch.manual_seed(5)
    for i, layer in enumerate(cfg["layers"]):
        part = MIXERS.build(spec.layers[i].mixer, dtype=dtype, device=DEV)
        prefix = f"l{i}.mix"
        assert set(part.expected_tensors(prefix)) == {k for k in weights if k.startswith(prefix + ".")}
        part.load(prefix, lambda n: weights[n].to(DEV).to(dtype if weights[n].dim() > 1 else torch.float32))
        cache = SequenceCache({0: part.cache_request()}, 1024, 4, dtype, DEV)
        lens = [75, 6]
        xs = [torch.randn(n, cfg["width"]).to(dtype) for n in lens]
        fn = {"attention": plain.sink_attention, "wkv": plain.wkv_time_mix,
              "channel_delta": plain.gated_delta}[layer["type"]]
        want = torch.cat([fn(layer["mixer"], double(weights), prefix, x.double(), cfg["norm"]["eps"])
                          for x in xs])
        slots = [cache.open_sequence() for _ in lens]
        got = part.forward(make_ctx(cache, slots, lens), torch.cat(xs).to(DEV), cache.view(0, True))
        assert rel_error(got.float().cpu(), want) < bound(dtype), (name, i, layer["type"], "one step")
        for s in slots:
            cache.close_sequence(s)
        # the same slots again (their state and pages were used a moment ago), cut up
        slots = [cache.open_sequence() for _ in lens]
        cuts = [[70, 2, 1, 1, 1], [3, 2, 1]]
        pieces = [[], []]
        done = [0, 0]
        for step in range(5):
            live = [k for k in range(2) if step < len(cuts[k])]
            counts = [cuts[k][step] for k in live]
            x = torch.cat([xs[k][done[k]:done[k] + c] for k, c in zip(live, counts)]).to(DEV)
            out = part.forward(make_ctx(cache, [slots[k] for k in live], counts), x, cache.view(0, True))
            for k, rows in zip(live, torch.split(out, counts)):
                pieces[k].append(rows)
                done[k] += rows.shape[0]
        got = torch.cat([torch.cat(p) for p in pieces])
        assert rel_error(got.float().cpu(), want) < bound(dtype), (name, i, layer["type"], "cut up")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_feed_forwards_norm_embedding_and_junction_alone(name, dtype):
    from foundry_b200.parts import EMBEDDINGS, FEED_FORWARDS, JUNCTIONS, NORMS
    from foundry_b200.kernels import ops
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    spec, wd = spec_of(name), double(weights)
    W = cfg["width"]
    torch.manual_seed(6)
    x = torch.randn(37, W).to(dtype)
    fetch = lambda n: weights[n].to(DEV).to(dtype if weights[n].dim() > 1 else torch.float32)
    for i, layer in enumerate(cfg["layers"]):
        if not layer["mlp"]:
            continue
        part = FEED_FORWARDS.build(spec.layers[i].feed_forward, dtype=dtype, device=DEV)
        part.load(f"l{i}.mlp", fetch)
        got = part.forward(None, x.to(DEV))
        got = got.sum(torch.float32) if isinstance(got, ops.Planes) else got
        want = plain.dense_feed_forward(wd, f"l{i}.mlp", x.double()) if layer["mlp"]["kind"] == "dense" \
            else plain.routed_experts(layer["mlp"], wd, f"l{i}.mlp", x.double())
        assert rel_error(got.float().cpu(), want) < bound(dtype), (name, i, layer["mlp"]["kind"])
    # the norm on both sides of a sum: resid += LN(y); out = LN(resid)
    norm = NORMS.build(spec.final_norm, dtype=dtype, device=DEV)
    norm.load("l0.norm1", fetch)
    post = NORMS.build(spec.final_norm, dtype=dtype, device=DEV)
    post.load("l0.norm1b", fetch)
    resid = torch.randn(37, W, device=DEV) * 4 + 1
    y = torch.randn(37, W, device=DEV) * 2 - 3
    eps = cfg["norm"]["eps"]
    total = resid.double().cpu() + plain.layer_norm(y.double().cpu(), wd["l0.norm1b"], wd["l0.norm1b.b"], eps)
    out = norm.add_norm(resid, post.pending(y))
    assert rel_error(resid.cpu(), total) < 1e-6
    assert rel_error(out.float().cpu(), plain.layer_norm(total, wd["l0.norm1"], wd["l0.norm1.b"], eps)) \
        < bound(dtype, 0.3)
    # embedding at far positions
    from foundry_b200.cache import SequenceCache
    emb = EMBEDDINGS.build(spec.embedding, dtype=dtype, device=DEV)
    ids = torch.tensor([3, 0, cfg["vocab"] - 1, 7], dtype=torch.int32, device=DEV)
    pos = torch.tensor([0, 1, 5000, 123456], dtype=torch.int32, device=DEV)
    ctx = type("C", (), {"token_ids": ids, "positions": pos})
    out, copy = torch.empty(4, W, device=DEV), torch.empty(4, W, device=DEV)
    emb.forward(ctx, weights["embed"].to(DEV).to(dtype), out, copy)
    want = wd["embed"][ids.cpu().long()] * cfg["embedding"]["scale"] + \
        plain.position_vector(pos.cpu().tolist(), W)
    assert float((out.cpu().double() - want).abs().max()) < 2e-6 * float(want.abs().max())
    assert torch.equal(out, copy)
    if cfg.get("loop"):
        j = JUNCTIONS.build(spec.junctions[0], dtype=dtype, device=DEV)
        j.load("loop", fetch)
        resid, x0 = torch.randn(37, W, device=DEV), torch.randn(37, W, device=DEV)
        want = torch.cat([resid, x0], -1).double().cpu() @ wd["loop.in"].T + wd["loop.step"][2]
        assert j.forward(None, resid, None, x0, 2) is None
        assert rel_error(resid.cpu(), want) < bound(dtype, 0.3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens", [1, 5, 40])
def test_routed_experts_at_sizes_of_the_tensor_core_form(dtype, tokens):
    """Width 128 and 192 hidden units (multiples of 64): in bfloat16 the grouped
    products run on the tensor cores; 40 tokens over 6 experts give chunks of more than
    8 rows, 1 token leaves most experts without any."""
    from foundry_b200.config.spec import PartSpec
    from foundry_b200.parts import FEED_FORWARDS
    W, ff, E, top = 128, 192, 6, 2
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": 1.2}}
    gen = torch.Generator().manual_seed(21)
    weights = {"m.router": torch.randn(E, W, generator=gen) * 0.3,
               "m.router.b": torch.randn(E, generator=gen) * 0.2}
    for e in range(E):
        weights[f"m.e{e}.gate"] = torch.randn(ff, W, generator=gen) * 0.15
        weights[f"m.e{e}.up"] = torch.randn(ff, W, generator=gen) * 0.15
        weights[f"m.e{e}.down"] = torch.randn(W, ff, generator=gen) * 0.15
    weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    part = FEED_FORWARDS.build(PartSpec("routed_experts", {
        "width": W, "ff": ff, "experts": E, "top": top, "limit": 1.2, "alpha": 1.702}),
        dtype=dtype, device=DEV)
    part.load("m", lambda n: weights[n].to(DEV).to(dtype if weights[n].dim() > 1 else torch.float32))
    x = torch.randn(tokens, W, generator=gen).to(dtype)
    got = part.forward(None, x.to(DEV))
    want = plain.routed_experts(mlp, double(weights), "m", x.double())
    assert rel_error(got.float().cpu(), want) < bound(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_with_sizes_that_fit_no_vector(dtype):
    """Key size 12 and value size 20 (no multiple of 8), three heads on one key/value
    head, no window, no kept tokens: the scalar paths of the CUDA-core kernel."""
    from foundry_b200.cache import SequenceCache
    from foundry_b200.config.spec import PartSpec
    from foundry_b200.parts import MIXERS
    W, H, d, e = 40, 3, 12, 20
    m = {"heads": H, "kv_heads": 1, "dim": d, "vdim": e, "scale": 0.4}
    gen = torch.Generator().manual_seed(9)
    shapes = {"a.q": (H * d, W), "a.k": (d, W), "a.v": (e, W), "a.o": (W, H * e),
              "a.q.norm": (H * d,), "a.k.norm": (d,)}
    weights = {k: (torch.randn(s, generator=gen) * (0.3 if len(s) == 2 else 0.2)
                   + (0.0 if len(s) == 2 else 1.0)).to(torch.bfloat16).float()
               for k, s in shapes.items()}
    part = MIXERS.build(PartSpec("sink_window_attention", {
        "width": W, "heads": H, "kv_heads": 1, "dim": d, "vdim": e, "scale": 0.4, "eps": 1e-5,
        "window": None, "keep_first": 0, "steep": 8.0, "sink": True}), dtype=dtype, device=DEV)
    part.load("a", lambda n: weights[n].to(DEV).to(dtype if weights[n].dim() > 1 else torch.float32))
    cache = SequenceCache({0: part.cache_request()}, 512, 2, dtype, DEV)
    x = torch.randn(90, W, generator=gen).to(dtype)
    want = plain.sink_attention(m, double(weights), "a", x.double(), 1e-5)
    slot = cache.open_sequence()
    head = part.forward(make_ctx(cache, [slot], [88]), x[:88].to(DEV), cache.view(0, True))
    tail = [part.forward(make_ctx(cache, [slot], [1]), x[t:t + 1].to(DEV), cache.view(0, True))
            for t in (88, 89)]
    got = torch.cat([head] + tail)
    assert rel_error(got.float().cpu(), want) < bound(dtype)


# ------------------------------------------------------- the window's edges
def edge_case_inputs(query_at, marker_at, width=8):
    """Rows whose normalised query at `query_at` matches only the key at
    `marker_at`: that one score stands far above the rest, so an output that
    sees the marker differs plainly from one that does not."""
    gen = torch.Generator().manual_seed(query_at * 1000 + marker_at)
    x = torch.zeros(query_at + 1, width)
    x[:, 0] = 1.0
    x += 0.05 * torch.randn(x.shape, generator=gen)
    for t in (query_at, marker_at):
        x[t] = 0.05 * torch.randn(width, generator=gen)
        x[t, 1] = 1.0
    x[marker_at, 4:] += 3.0  # a value unlike every other (values read the upper half)
    return x.to(torch.bfloat16).float()


EDGES = [  # (query position, marker position, whether the window of 70 with 3 kept shows it)
    (69, 0, True), (70, 0, True), (70, 1, True), (72, 2, True), (73, 3, False), (73, 4, True),
    (133, 64, True), (133, 63, False), (134, 64, False), (127, 63, True), (128, 64, True),
    (300, 2, True), (300, 3, False), (300, 230, False), (300, 231, True), (63, 0, True),
    (64, 0, True), (65, 64, True),
]


@pytest.mark.parametrize("W", [8, 16])  # 16: a head size of the tensor-core prompt kernel
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_at_the_edges_of_window_kept_tokens_and_pages(dtype, W):
    """A crafted mixer (identity projections) in which one key dominates one
    query: just inside and just outside the window, at the first tokens that
    are kept and the next ones, on both sides of a page border, far back; as
    the last token of a prompt and as a token decoded alone."""
    from foundry_b200.cache import SequenceCache
    from foundry_b200.parts import MIXERS
    from foundry_b200.config.spec import PartSpec
    m = {"heads": 1, "kv_heads": 1, "dim": W, "vdim": W, "scale": 3.0 * 8 / W,
         "mask": {"size": 70, "keep_first": 3}}
    lower = torch.diag(torch.tensor([1.0] * 4 + [0.0] * (W - 4)))  # queries and keys read the first four
    upper = torch.diag(torch.tensor([0.0] * 4 + [1.0] * (W - 4)))  # values the rest of a row
    weights = {"a.q": lower, "a.k": lower, "a.v": upper, "a.o": torch.eye(W),
               "a.q.norm": torch.ones(W), "a.k.norm": torch.ones(W)}
    part = MIXERS.build(PartSpec("sink_window_attention", {
        "width": W, "heads": 1, "kv_heads": 1, "dim": W, "vdim": W, "scale": 3.0 * 8 / W, "eps": 1e-6,
        "window": 70, "keep_first": 3, "steep": 8.0, "sink": True}), dtype=dtype, device=DEV)
    part.load("a", lambda n: weights[n].to(DEV).to(dtype if weights[n].dim() > 1 else torch.float32))
    cache = SequenceCache({0: part.cache_request()}, 4096, 4, dtype, DEV)
    for query_at, marker_at, shown in EDGES:
        x = edge_case_inputs(query_at, marker_at, W)
        want = plain.sink_attention(m, double(weights), "a", x.double(), 1e-6)[-1]
        # the plain implementation itself must tell the two kinds of case apart
        assert (float(want[4:].mean()) > 0.3) == shown, (query_at, marker_at)
        for cut in ("prompt", "decoded"):
            slot = cache.open_sequence()
            if cut == "prompt":
                got = part.forward(make_ctx(cache, [slot], [query_at + 1]), x.to(DEV).to(dtype),
                                   cache.view(0, True))[-1]
            else:
                part.forward(make_ctx(cache, [slot], [query_at]), x[:-1].to(DEV).to(dtype),
                             cache.view(0, True))
                got = part.forward(make_ctx(cache, [slot], [1]), x[-1:].to(DEV).to(dtype),
                                   cache.view(0, True))[0]
            cache.close_sequence(slot)
            # (a score of 24 makes 16-bit keys and queries move the weights by several per
            # cent; a key wrongly seen or missed moves the output by all of it)
            assert rel_error(got.float().cpu()[None], want[None]) < bound(dtype, 5.0), \
                (query_at, marker_at, cut)


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("rupotar")
    return {name: tiny.write_folder(str(root / name), name) for name in tiny.CONFIGS}


def plain_logits(name, weights, tokens):
    return plain.forward(tiny.CONFIGS[name], double(weights), tokens).numpy()


def run_cutting(engine, prompts, cuts):
    """Feed `prompts` through `engine.step` in rounds; `cuts[k]` are the token
    counts sequence k brings round by round. Logits of every position."""
    from foundry_b200.engine import SequenceStep
    slots = [engine.open_sequence() for _ in prompts]
    done = [0] * len(prompts)
    rows = [[] for _ in prompts]
    for r in range(max(len(c) for c in cuts)):
        live = [k for k in range(len(prompts)) if r < len(cuts[k])]
        steps = [SequenceStep(slots[k], prompts[k][done[k]:done[k] + cuts[k][r]],
                              list(range(cuts[k][r]))) for k in live]
        logits = engine.step(steps).cpu().numpy()
        at = 0
        for k in live:
            n = cuts[k][r]
            rows[k].append(logits[at:at + n])
            at += n
            done[k] += n
            if done[k] == len(prompts[k]):
                engine.close_sequence(slots[k])
    assert done == [len(p) for p in prompts]
    return [np.concatenate(r) for r in rows]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_model_in_every_cutting(name, dtype, folders):
    """Whole prompts alone; token by token from the first token on; portions of
    several sizes down to two tokens; a batch of unequal requests decoded
    together while the shorter ones end; all on slots and pages that the
    earlier cuttings used and gave back."""
    import foundry_b200 as fb
    folder, weights = folders[name]
    vocab = tiny.CONFIGS[name]["vocab"]
    rng = np.random.default_rng(11)
    prompts = [[int(t) for t in rng.integers(0, vocab, n)] for n in (150, 1, 3, 81)]
    want = [plain_logits(name, weights, p) for p in prompts]
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_slots=6)
    results = {}
    results["whole, alone"] = [run_cutting(engine, [p], [[len(p)]])[0] for p in prompts]
    results["token by token"] = [run_cutting(engine, [prompts[k]], [[1] * len(prompts[k])])[0]
                                 for k in (2, 3)]
    results["portions"] = run_cutting(engine, [prompts[0], prompts[3]],
                                      [[2, 62, 1, 64, 2, 17, 2], [77, 2, 2]])
    results["batch, then decoded together"] = run_cutting(
        engine, prompts, [[120] + [1] * 30, [1], [2, 1], [70] + [1] * 11])
    wanted = {"whole, alone": want, "token by token": [want[2], want[3]],
              "portions": [want[0], want[3]], "batch, then decoded together": want}
    for cutting, got in results.items():
        for g, w in zip(got, wanted[cutting]):
            assert rel_error(g, w) < bound(dtype, 2.0), (name, dtype, cutting, len(w))
    if dtype == "float32":  # the cuttings agree with each other to rounding
        assert rel_error(results["portions"][0], results["whole, alone"][0]) < 2e-5
        assert rel_error(results["batch, then decoded together"][3], results["whole, alone"][3]) < 2e-5
    engine.cache.table.check()
    assert engine.free_slots() == 6


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_long_decoding_and_reused_slots(name, folders):
    """260 tokens decoded one by one behind a short prompt (across cache pages and
    far past every window), twice on the same slot with another sequence between."""
    import foundry_b200 as fb
    folder, weights = folders[name]
    vocab = tiny.CONFIGS[name]["vocab"]
    rng = np.random.default_rng(12)
    tokens = [int(t) for t in rng.integers(0, vocab, 265)]
    other = [int(t) for t in rng.integers(0, vocab, 40)]
    want = plain_logits(name, weights, tokens)
    engine = fb.Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=2)
    first = run_cutting(engine, [tokens], [[5] + [1] * 260])[0]
    run_cutting(engine, [other], [[40]])
    again = run_cutting(engine, [tokens], [[5] + [1] * 260])[0]
    assert rel_error(first, want) < bound("float32", 2.0)
    assert np.array_equal(first, again)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype, folders):
    """`Engine.generate` (the scheduler's batches, graphs, slot reuse) against the
    plain model's greedy tokens; five prompts through batches of two."""
    import foundry_b200 as fb
    folder, weights = folders["looped"]
    cfg = tiny.CONFIGS["looped"]
    rng = np.random.default_rng(13)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (9, 1, 30, 4, 17)]
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=512, max_slots=4)
    got = engine.generate(prompts, 8, eos_token_id=[], max_batch=2).token_ids
    wd = double(weights)
    for g, p in zip(got, prompts):
        w = plain.greedy_generate(cfg, wd, p, 8)
        if g == w:
            continue
        k = next(i for i, (a, b) in enumerate(zip(g, w)) if a != b)
        logits = plain.forward(cfg, wd, list(p) + w[:k])[-1]
        gap = float(logits[w[k]] - logits[g[k]])
        assert dtype == "bfloat16" and gap < 0.05 * float(logits.abs().max()), (g, w, gap)


def test_trace_replay_and_command_line(folders, tmp_path):
    """`bin/trace_run` on a Rupotar folder: a prompt step of two requests, then
    single tokens, one request ending early; and `foundry run` generating."""
    folder, weights = folders["straight"]
    cfg = tiny.CONFIGS["straight"]
    rng = np.random.default_rng(14)
    a = [int(t) for t in rng.integers(0, cfg["vocab"], 12)]
    b = [int(t) for t in rng.integers(0, cfg["vocab"], 5)]
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": [0, 9]},
                                     {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[10:11], "want": []},
                                     {"id": "b", "tokens": b[4:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[11:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", "float32", "--out", str(out), "--max-tokens", "128"],
                          input="".join(json.dumps(l) + "\n" for l in lines), capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = plain_logits("straight", weights, a), plain_logits("straight", weights, b)
    V = cfg["vocab"]
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    assert rel_error(got0, np.stack([wa[0], wa[9], wb[3]])) < bound("float32", 2.0)
    assert rel_error(got1, wb[4:5]) < bound("float32", 2.0)
    assert rel_error(got2, wa[11:12]) < bound("float32", 2.0)
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "run", "--model",
                          folder, "--dtype", "float32", "--prompt-ids", ",".join(map(str, a)),
                          "--max-new-tokens", "4", "--ignore-eos"], capture_output=True, text=True,
                         timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    want = plain.greedy_generate(cfg, double(weights), a, 4)
    assert json.loads(run.stdout.strip().split("\n")[-1]) == want


def test_command_line_bench_on_a_rupotar_folder(folders, tmp_path):
    """`foundry bench` (prompt step, decode steps, report with bytes and operations)
    on a model with state rows and routed experts."""
    folder, _ = folders["looped"]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "bench", "--model",
                           folder, "--prompt-tokens", "20", "--new-tokens", "5", "--runs", "2",
                           "--batch-size", "3", "--out", str(tmp_path)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads((tmp_path / "report.json").read_text())
    assert len(report["runs"]) == 2 and all(len(r) == 5 for r in report["runs"][0]["token_ids"])
    assert report["runs"][0]["token_ids"] == report["runs"][1]["token_ids"]
