"""Vonulorn on the GPU against the plain implementation (tests/plain_vonulorn.py):
every mechanism alone, then whole models in every cutting of the same tokens
(whole prompts, token by token, portions down to two tokens, mixed batches),
slots and pages that are used again, keys far back and at the borders of cache
pages, the sink, long decoding, and greedy generation through the engine's own
loop and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_vonulorn as plain
import vonulorn_tiny as tiny

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
DTYPES = [torch.float32, torch.bfloat16]
PLAIN = {"delta": plain.delta_mixer, "attention": plain.differential_attention,
         "latent_attention": plain.latent_attention}


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


def spec_of(doc):
    from foundry_b200.config.registry import resolve_architecture
    arch = resolve_architecture(doc)
    return arch.build_spec(arch.parse_config(doc))


def loader(weights, dtype):
    return lambda n: weights[n].to(DEV).to(dtype if weights[n].dim() > 1 else torch.float32)


def mixer_part(kind, m, W, eps, weights, dtype, prefix="a"):
    """A mixer of the library built the way the architecture builds it."""
    from foundry_b200.parts import MIXERS
    doc = {"architecture": "Vonulorn", "vocab": 8, "width": W, "norm": {"eps": eps},
           "residual_mult": 1.0, "layers": [{"type": kind, "mixer": m, "mlp": None}]}
    part = MIXERS.build(spec_of(doc).layers[0].mixer, dtype=dtype, device=DEV)
    assert set(part.expected_tensors(prefix)) == set(weights)
    part.load(prefix, loader(weights, dtype))
    return part


def run_mixer(part, cache, xs, cuts, dtype):
    """Feed the sequences `xs` through the mixer in rounds (`cuts[k]`: the rows sequence k
    brings round by round); every sequence's outputs in order."""
    slots = [cache.open_sequence() for _ in xs]
    pieces, done = [[] for _ in xs], [0] * len(xs)
    for step in range(max(len(c) for c in cuts)):
        live = [k for k in range(len(xs)) if step < len(cuts[k])]
        counts = [cuts[k][step] for k in live]
        x = torch.cat([xs[k][done[k]:done[k] + c] for k, c in zip(live, counts)]).to(DEV).to(dtype)
        out = part.forward(make_ctx(cache, [slots[k] for k in live], counts), x, cache.view(0, True))
        for k, rows in zip(live, torch.split(out, counts)):
            pieces[k].append(rows.float().cpu())
            done[k] += rows.shape[0]
    for s in slots:
        cache.close_sequence(s)
    return [torch.cat(p) for p in pieces]


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_each_mixer_alone_in_two_cuttings(name, dtype):
    """Every mixer of both configurations with a cache of its own: two sequences of
    unequal lengths in one step, then on the slots and pages that were just given
    back the same rows as a prompt part, portions of two tokens and single tokens."""
    from foundry_b200.cache import SequenceCache
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    eps = cfg["norm"]["eps"]
    torch.manual_seed(5)
    for i, layer in enumerate(cfg["layers"]):
        prefix = f"l{i}.mix"
        mine = {k: v for k, v in weights.items() if k.startswith(prefix + ".")}
        part = mixer_part(layer["type"], layer["mixer"], cfg["width"], eps, mine, dtype, prefix)
        cache = SequenceCache({0: part.cache_request()}, 1024, 4, dtype, DEV)
        lens = [139, 6]
        xs = [torch.randn(n, cfg["width"]).to(dtype).float() for n in lens]
        want = [PLAIN[layer["type"]](layer["mixer"], double(mine), prefix, x.double(), eps) for x in xs]
        for cuts in ([[139], [6]], [[70, 2, 1, 1, 63, 2], [3, 2, 1]]):
            got = run_mixer(part, cache, xs, cuts, dtype)
            for g, w in zip(got, want):
                assert rel_error(g, w) < bound(dtype), (name, i, layer["type"], cuts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_at_other_sizes(dtype):
    """Sizes neither configuration has: latent rows of more than 256 elements (several
    pieces a lane) and of a size that fits no vector; one key head for many heads; as
    many taps as 5; values that are no multiple of 8 beside keys that are."""
    from foundry_b200.cache import SequenceCache
    cases = [
        ("latent_attention", {"heads": 2, "dim": 24, "rot_dim": 32, "vdim": 40, "kv_rank": 288,
                              "q_rank": 64, "scale": 0.05, "rot": {"base": 500.0, "dims": 32}}),
        ("latent_attention", {"heads": 5, "dim": 8, "rot_dim": 6, "vdim": 12, "kv_rank": 21,
                              "q_rank": 17, "scale": 0.4, "rot": {"base": 10000.0, "dims": 6}}),
        ("attention", {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 12, "scale": 0.2,
                       "softcap": 1.0, "diff": 0.1, "q_temp": {"coef": 1.0, "every": 1}}),
        ("attention", {"heads": 1, "kv_heads": 1, "dim": 64, "vdim": 128, "scale": 0.125,
                       "softcap": 20.0, "diff": 0.4, "q_temp": {"coef": 0.25, "every": 32}}),
        ("delta", {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 72, "conv": 5}),
        ("delta", {"heads": 1, "kv_heads": 1, "dim": 128, "vdim": 64, "conv": 1}),
        # latent rows of 128 + 16, 256 + 32 and 512 + 64: in bfloat16 the heads-as-rows
        # tensor-core kernel (five heads: a block's 64 rows span 13 tokens)
        ("latent_attention", {"heads": 5, "dim": 16, "rot_dim": 16, "vdim": 24, "kv_rank": 128,
                              "q_rank": 40, "scale": 0.1, "rot": {"base": 10000.0, "dims": 16}}),
        ("latent_attention", {"heads": 3, "dim": 8, "rot_dim": 32, "vdim": 8, "kv_rank": 256,
                              "q_rank": 32, "scale": 0.07, "rot": {"base": 10000.0, "dims": 32}}),
        ("latent_attention", {"heads": 2, "dim": 8, "rot_dim": 64, "vdim": 16, "kv_rank": 512,
                              "q_rank": 32, "scale": 0.05, "rot": {"base": 1000.0, "dims": 64}}),
        # fewer rotated elements than the rotated part holds: the rest passes unchanged
        ("latent_attention", {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 16, "kv_rank": 32,
                              "q_rank": 24, "scale": 0.3, "rot": {"base": 50.0, "dims": 4}}),
    ]
    W, eps = 80, 1e-5
    torch.manual_seed(8)
    for n, (kind, m) in enumerate(cases):
        weights = tiny.random_mixer(kind, m, W, seed=n)
        part = mixer_part(kind, m, W, eps, weights, dtype)
        cache = SequenceCache({0: part.cache_request()}, 512, 2, dtype, DEV)
        x = torch.randn(90, W).to(dtype).float()
        want = PLAIN[kind](m, double(weights), "a", x.double(), eps)
        got = run_mixer(part, cache, [x], [[66, 2, 20, 1, 1]], dtype)[0]
        assert rel_error(got, want) < bound(dtype), (kind, m)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_feed_forward_and_scaled_residual_norm_alone(name, dtype):
    from foundry_b200.kernels import ops
    from foundry_b200.parts import FEED_FORWARDS, NORMS
    cfg, weights = tiny.CONFIGS[name], tiny.random_weights(name)
    spec, wd = spec_of(cfg), double(weights)
    W = cfg["width"]
    torch.manual_seed(6)
    for rows in (3, 37, 200):   # the products for few rows, some rows and many rows
        x = torch.randn(rows, W).to(dtype)
        for i, layer in enumerate(cfg["layers"]):
            if not layer["mlp"]:
                continue
            part = FEED_FORWARDS.build(spec.layers[i].feed_forward, dtype=dtype, device=DEV)
            part.load(f"l{i}.mlp", loader(weights, dtype))
            got = part.forward(None, x.to(DEV))
            got = got.sum(torch.float32) if isinstance(got, ops.Planes) else got
            want = plain.gated_feed_forward(wd, f"l{i}.mlp", x.double())
            assert rel_error(got.float().cpu(), want) < bound(dtype), (name, i, rows)
    # resid += m * y and the norm of the sum, in one pass
    norm = NORMS.build(spec.final_norm, dtype=dtype, device=DEV)
    norm.load("final.norm", loader(weights, dtype))
    resid = torch.randn(37, W, device=DEV) * 4 + 1
    y = torch.randn(37, W, device=DEV) * 2 - 3
    total = resid.double().cpu() + 0.37 * y.double().cpu()
    out = norm.add_norm(resid, ops.ScaledDelta(y, 0.37))
    assert rel_error(resid.cpu(), total) < 1e-6
    assert rel_error(out.float().cpu(), plain.rms_norm(total, wd["final.norm"], cfg["norm"]["eps"])) \
        < bound(dtype, 0.3)


# --------------------------------------------- one key that stands out, anywhere
def marked_inputs(query_at, marker_at, width, lift=3.0):
    """Rows in which the query of `query_at` (input 1) matches only the key of
    `marker_at` (input 2): that score stands far above the rest, so an output that
    sees the marker differs plainly from one that does not. The marker's value
    (inputs 4..8) is unlike every other."""
    gen = torch.Generator().manual_seed(query_at * 1000 + marker_at)
    x = torch.zeros(query_at + 1, width)
    x[:, 0] = 1.0
    x += 0.05 * torch.randn(x.shape, generator=gen)
    x[query_at] = 0.05 * torch.randn(width, generator=gen)
    x[query_at, 1] = 1.0
    x[marker_at] = 0.05 * torch.randn(width, generator=gen)
    x[marker_at, 2] = 1.0
    x[marker_at, 4:8] += lift
    return x.to(torch.bfloat16).float()


PLACES = [  # (query position, marker position): page borders, the first tokens, far back
    (5, 0), (63, 0), (64, 0), (64, 63), (65, 64), (127, 63), (128, 64), (129, 127), (200, 1),
    (700, 2), (700, 63), (700, 64), (700, 639), (700, 640), (700, 699),
]


def crafted_differential(W, d=4, e=4):
    """Map 1's query reads input 1 and its key input 2; map 2 reads nothing (all its
    scores are equal: the mean of the values); values are inputs 4..8."""
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": e, "scale": 24.0, "softcap": 40.0,
         "diff": 0.5, "q_temp": {"coef": 0.1, "every": 64}}
    q, k = torch.zeros(2 * d, W), torch.zeros(2 * d, W)
    q[0, 1] = k[0, 2] = 1.0
    val = torch.zeros(e, W)
    val[:4, 4:8] = torch.eye(4)
    out = torch.zeros(W, e)
    out[:4, :4] = torch.eye(4)
    z = torch.zeros(d)
    return m, {"a.q": q, "a.k": k, "a.v": val, "a.o": out, "a.lq1": z, "a.lk1": z,
               "a.lq2": z, "a.lk2": z}


def crafted_latent(W, d=4, c=4, e=4, r=8):
    """The query reads input 1 through its latent, the key input 2 of the cached latent,
    values the latent's elements 4..8; the rotated parts are idle in the scores (their
    query rows are zero) but are written and read all the same."""
    # (only 8 of the latent's r elements are fed: the norm over all r makes them
    # sqrt(r / 8) larger, which the scale takes back)
    m = {"heads": 1, "dim": d, "rot_dim": c, "vdim": e, "kv_rank": r, "q_rank": W,
         "scale": 5.0 * (8.0 / r) ** 0.5, "rot": {"base": 100.0, "dims": c}}
    uq = torch.zeros(d + c, W)
    uq[0, 1] = 1.0
    dkv = torch.zeros(r + c, W)
    dkv[:8, :8] = torch.eye(8)
    dkv[r:, 8:8 + c] = torch.eye(c)
    uk, uv = torch.zeros(d, r), torch.zeros(e, r)
    uk[0, 2] = 1.0
    uv[:4, 4:8] = torch.eye(4)
    out = torch.zeros(W, e)
    out[:4, :4] = torch.eye(4)
    return m, {"a.dq": torch.eye(W), "a.dq.norm": torch.ones(W), "a.uq": uq, "a.dkv": dkv,
               "a.dkv.norm": torch.ones(r), "a.uk": uk, "a.uv": uv, "a.sink": torch.tensor([2.0]),
               "a.o": out}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind, sizes", [
    ("attention", "small"), ("attention", "tensor-core"), ("latent_attention", "small"),
    ("latent_attention", "tensor-core"), ("latent_attention", "folded")])
def test_one_key_that_stands_out_is_found_wherever_it_lies(kind, sizes, dtype):
    """Crafted mixers in which one key dominates one query: at the first tokens, on both
    sides of page borders, hundreds of tokens back; as the last token of a prompt and
    as a token decoded alone. Once at sizes that only the CUDA-core kernel takes, once at
    sizes whose prompts run on the tensor cores in bfloat16."""
    from foundry_b200.cache import SequenceCache
    W = 32
    if kind == "attention":
        m, weights = crafted_differential(W) if sizes == "small" else crafted_differential(W, 16, 32)
    elif sizes == "folded":  # latent rows of 128 + 16: every bfloat16 step on the heads-as-rows kernel
        m, weights = crafted_latent(W, 8, 16, 24, 128)
    else:
        m, weights = crafted_latent(W) if sizes == "small" else crafted_latent(W, 32, 16, 16)
    part = mixer_part(kind, m, W, 1e-6, weights, dtype)
    cache = SequenceCache({0: part.cache_request()}, 2048, 2, dtype, DEV)
    for query_at, marker_at in PLACES:
        x = marked_inputs(query_at, marker_at, W, lift=3.0 if kind == "attention" else 1.0)
        want = PLAIN[kind](m, double(weights), "a", x.double(), 1e-6)[-1]
        # the plain implementation itself sees the marker: without it the output is another
        hidden = x.clone()
        hidden[marker_at] = hidden[max(0, marker_at - 1) if marker_at else 1]
        blind = PLAIN[kind](m, double(weights), "a", hidden.double(), 1e-6)[-1]
        assert float((want - blind).norm() / want.norm()) > 0.2, (query_at, marker_at)
        for cut in ([query_at + 1], [query_at, 1]):
            got = run_mixer(part, cache, [x], [cut], dtype)[0][-1]
            assert rel_error(got[None], want[None]) < bound(dtype, 5.0), (query_at, marker_at, cut)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_sink_that_takes_most_of_the_sum(dtype):
    """A sink score far above the keys' scores: the output shrinks by the sink's share,
    in a prompt, for its first token, and for tokens decoded alone (where the visible
    keys are cut into runs and the sink joins once, at the merge)."""
    from foundry_b200.cache import SequenceCache
    m = dict(tiny.CONFIGS["mixed"]["layers"][0]["mixer"])
    weights = tiny.random_mixer("latent_attention", m, 96, seed=4)
    weights["a.sink"] = torch.tensor([6.0, -3.0, 2.5])
    part = mixer_part("latent_attention", m, 96, 1e-5, weights, dtype)
    cache = SequenceCache({0: part.cache_request()}, 1024, 2, dtype, DEV)
    torch.manual_seed(2)
    x = torch.randn(300, 96).to(dtype).float()
    want = plain.latent_attention(m, double(weights), "a", x.double(), 1e-5)
    silent = dict(weights, **{"a.sink": torch.full((3,), -1e4)})
    assert rel_error(plain.latent_attention(m, double(silent), "a", x.double(), 1e-5), want) > 0.3
    for cuts in ([[300]], [[1] + [1] * 8 + [280] + [1] * 11]):
        got = run_mixer(part, cache, [x], cuts, dtype)[0]
        assert rel_error(got, want) < bound(dtype), cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_state_and_tail_survive_every_cutting(dtype):
    """Decays close to one, so that the first tokens still weigh on the last: the state
    and the convolution's tail carried through portions of one and two tokens equal
    the whole prompt's."""
    from foundry_b200.cache import SequenceCache
    m = {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "conv": 4}
    weights = tiny.random_mixer("delta", m, 48, seed=3)
    weights["a.A_log"] = torch.tensor([-6.0, -4.0])
    part = mixer_part("delta", m, 48, 1e-6, weights, dtype)
    cache = SequenceCache({0: part.cache_request()}, 1024, 3, dtype, DEV)
    torch.manual_seed(4)
    xs = [torch.randn(n, 48).to(dtype).float() for n in (150, 9)]
    want = [plain.delta_mixer(m, double(weights), "a", x.double(), 1e-6) for x in xs]
    # (the plain form itself: the first token still matters at the end)
    moved = xs[0].clone()
    moved[0] += 1.0
    assert rel_error(plain.delta_mixer(m, double(weights), "a", moved.double(), 1e-6)[-1:],
                     want[0][-1:]) > 1e-3
    for cuts in ([[150], [9]], [[1, 2, 1, 3, 2, 64, 2, 1] + [1] * 10 + [64], [2, 2, 2, 2, 1]]):
        got = run_mixer(part, cache, xs, cuts, dtype)
        for g, w in zip(got, want):
            assert rel_error(g, w) < bound(dtype, 2.0), cuts


# ---------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("vonulorn")
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
            # (bfloat16: the rounding of four layers with wide weights adds up; each mixer alone
            # stays within the single bound above)
            assert rel_error(g, w) < bound(dtype, 2.0 if dtype == "float32" else 3.0), \
                (name, dtype, cutting, len(w))
    if dtype == "float32":  # the cuttings agree with each other to rounding
        assert rel_error(results["portions"][0], results["whole, alone"][0]) < 2e-5
        assert rel_error(results["batch, then decoded together"][3], results["whole, alone"][3]) < 2e-5
    engine.cache.table.check()
    assert engine.free_slots() == 6


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_long_decoding_and_reused_slots(name, folders):
    """260 tokens decoded one by one behind a short prompt (across cache pages and
    the query temperature's steps), twice on the same slot with another sequence between."""
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


def test_a_width_that_fits_no_tensor_core_product(tmp_path):
    """Width 52 and inner sizes that are no multiples of 8: in bfloat16 every product takes
    the CUDA-core kernel and the feed-forward's activation runs behind its product."""
    import foundry_b200 as fb
    from foundry_b200.weights.safetensors_io import SINGLE_FILE, save_file
    doc = {"architecture": "Vonulorn", "vocab": 77, "width": 52, "norm": {"eps": 1e-5},
           "residual_mult": 0.25,
           "layers": [
               {"type": "delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 12, "vdim": 10, "conv": 3},
                "mlp": {"kind": "dense", "ff": 90}},
               {"type": "attention",
                "mixer": {"heads": 3, "kv_heads": 3, "dim": 10, "vdim": 14, "scale": 0.3,
                          "softcap": 3.0, "diff": 0.2, "q_temp": {"coef": 0.4, "every": 3}},
                "mlp": {"kind": "dense", "ff": 44}},
               {"type": "latent_attention",
                "mixer": {"heads": 2, "dim": 10, "rot_dim": 6, "vdim": 14, "kv_rank": 18, "q_rank": 20,
                          "scale": 0.25, "rot": {"base": 777.0, "dims": 6}}, "mlp": None}]}
    gen = torch.Generator().manual_seed(31)
    weights = {k: tiny.draw(k, shape, gen) for k, shape in tiny.tensor_shapes(doc).items()}
    folder = tmp_path / "odd"
    folder.mkdir()
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()}, str(folder / SINGLE_FILE),
              metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(doc))
    rng = np.random.default_rng(3)
    prompts = [[int(t) for t in rng.integers(0, 77, n)] for n in (70, 9)]
    want = [plain.forward(doc, double(weights), p).numpy() for p in prompts]
    for dtype in ("float32", "bfloat16"):
        engine = fb.Engine.from_folder(str(folder), dtype=dtype, max_tokens=512, max_slots=3)
        got = run_cutting(engine, prompts, [[66, 2, 1, 1], [5, 1, 2, 1]])
        for g, w in zip(got, want):
            assert rel_error(g, w) < bound(dtype, 2.0), dtype


def greedy(cfg, weights, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        tokens.append(int(plain.forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dtype, folders):
    """`Engine.generate` (the scheduler's batches, graphs, slot reuse) against the
    plain model's greedy tokens; five prompts through batches of two."""
    import foundry_b200 as fb
    folder, weights = folders["mixed"]
    cfg = tiny.CONFIGS["mixed"]
    rng = np.random.default_rng(13)
    prompts = [[int(t) for t in rng.integers(0, cfg["vocab"], n)] for n in (9, 1, 30, 4, 17)]
    engine = fb.Engine.from_folder(folder, dtype=dtype, max_tokens=512, max_slots=4)
    got = engine.generate(prompts, 8, eos_token_id=[], max_batch=2).token_ids
    wd = double(weights)
    for g, p in zip(got, prompts):
        w = greedy(cfg, wd, p, 8)
        if g == w:
            continue
        k = next(i for i, (a, b) in enumerate(zip(g, w)) if a != b)
        logits = plain.forward(cfg, wd, list(p) + w[:k])[-1]
        gap = float(logits[w[k]] - logits[g[k]])
        assert dtype == "bfloat16" and gap < 0.05 * float(logits.abs().max()), (g, w, gap)


def test_trace_replay_and_command_line(folders, tmp_path):
    """`bin/trace_run` on a Vonulorn folder: a prompt step of two requests, then
    single tokens, one request ending early; and `foundry run` generating."""
    folder, weights = folders["other"]
    cfg = tiny.CONFIGS["other"]
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
    wa, wb = plain_logits("other", weights, a), plain_logits("other", weights, b)
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
    want = greedy(cfg, double(weights), a, 4)
    assert json.loads(run.stdout.strip().split("\n")[-1]) == want


def test_command_line_bench_on_a_vonulorn_folder(folders, tmp_path):
    """`foundry bench` (prompt step, decode steps, report with bytes and operations)
    on a model with state rows, latent rows and two-map attention."""
    folder, _ = folders["mixed"]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "foundry"), "bench", "--model",
                           folder, "--prompt-tokens", "20", "--new-tokens", "5", "--runs", "2",
                           "--batch-size", "3", "--out", str(tmp_path)],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    report = json.loads((tmp_path / "report.json").read_text())
    assert len(report["runs"]) == 2 and all(len(r) == 5 for r in report["runs"][0]["token_ids"])
    assert report["runs"][0]["token_ids"] == report["runs"][1]["token_ids"]
