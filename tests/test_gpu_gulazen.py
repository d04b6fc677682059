"""The layered sequence engine on Gulazen models against the plain implementation (tests/gulazen_plain.py): every mechanism
alone, prompts against token-by-token decoding, portions, ragged batches, reuse of pages and state slots, one key that stands
out at the window's and the kept prefix's edges, at page borders and far back, the sink, the first tokens, long decoding, odd
sizes, and greedy generation through the engine's own generation loop and command line."""
import functools
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import gulazen_plain as plain
from gulazen_cases import build_engine, dense, layer, make_config, moe, plant_pair, random_weights, rel_err, row_errs, run_schedule, to_bf16_values

pytestmark = pytest.mark.gpu

# bf16 mode: products round their inputs to bf16 (relative 4e-3 each); fp32 mode is fp32 arithmetic against float64
TOL = {"float32": 2e-4, "bfloat16": 1e-1}


def tokens(n, vocab, seed=1):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def whole(m, toks):
    return run_schedule(m, {"a": toks}, [[("a", len(toks))]])["a"]


def check_logits(got, want, dtype):
    assert row_errs(got, want).max() < TOL[dtype]


def weights(cfg, seed, dtype, **kw):
    """In bf16 mode a rounding difference in front of a router could flip a close choice of experts: those comparisons use routers
    whose choice is fixed by their biases (the fp32 comparisons test the choice itself)."""
    return random_weights(cfg, seed=seed, decisive=(dtype == "bfloat16"), **kw)


# ---- each mechanism alone: residual stream after every layer, and the logits -----------------------------------------------------
MECHANISMS = {
    "attention_only": make_config([layer()]),
    "one_tap": make_config([layer(mlp=dense(24))], taps=1),
    "two_taps_odd_width": make_config([layer(heads=3, kv_heads=3, dim=10, vdim=7, window=5, keep=0)], width=37, taps=2, eps=1e-3),
    "five_taps": make_config([layer(window=9, keep=2), layer(window=200, keep=0)], taps=5),
    "one_head": make_config([layer(heads=1, kv_heads=1, dim=16, vdim=8, window=12, keep=1)]),
    "one_key_value_head": make_config([layer(heads=5, kv_heads=1, dim=8, vdim=24, window=17, keep=5)], width=40),
    "as_many_key_value_heads": make_config([layer(heads=4, kv_heads=4, dim=8, vdim=8, window=30, keep=2)]),
    "nine_heads": make_config([layer(heads=9, kv_heads=3, dim=8, vdim=12, window=40, keep=1)], width=64),
    "twenty_heads": make_config([layer(heads=20, kv_heads=5, dim=4, vdim=4, window=33, keep=4)], width=40),
    "forty_heads": make_config([layer(heads=40, kv_heads=8, dim=4, vdim=8, window=21, keep=2)], width=40),
    "window_one": make_config([layer(window=1, keep=0), layer(window=1, keep=2)]),
    "window_beyond_the_sequence": make_config([layer(window=500, keep=7)]),
    "kept_prefix_longer_than_window": make_config([layer(window=4, keep=11)]),
    "tight_cap": make_config([layer(softcap=1.5, scale=0.9)]),
    "wide_heads": make_config([layer(heads=2, kv_heads=1, dim=72, vdim=136, window=70, keep=3)], width=64),
    "dense_ff": make_config([layer(mlp=dense(56))]),
    "experts": make_config([layer(mlp=moe())]),
    "experts_one_choice_no_shared": make_config([layer(mlp=moe(experts=3, top=1, shared=0))]),
    "experts_all_chosen": make_config([layer(mlp=moe(experts=4, top=4, ff=8, shared=8))]),
    "experts_many": make_config([layer(mlp=moe(experts=37, top=9, ff=8, shared=0))]),
    "layers_that_differ": make_config([layer(mlp=dense(40)), layer(heads=2, kv_heads=1, dim=16, vdim=8, window=7, keep=0, mlp=moe()),
                                       layer(heads=6, kv_heads=3, dim=8, vdim=8, window=50, keep=9), layer(mlp=moe(experts=2, top=1, shared=16), window=3, keep=1, softcap=4.0)],
                                      vocab=101, width=56, taps=4),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_mechanism_layers_and_logits(name, dtype):
    cfg = MECHANISMS[name]
    W = weights(cfg, 3, dtype)
    toks = tokens(75, cfg["vocab"])
    want, layers = plain.run(cfg, W, toks)
    m = build_engine(cfg, W, dtype)
    m.debug_layers(True)
    got = whole(m, toks)
    got_layers = m.read_layers(len(toks))
    m.free()
    assert got_layers.shape == layers.shape
    for i in range(layers.shape[0]):
        scale = np.sqrt((layers[i] ** 2).mean())
        assert np.abs(got_layers[i] - layers[i]).max() / scale < TOL[dtype] * 5, f"layer {i}"
    check_logits(got, want, dtype)


def test_positions_enter_through_the_embedding_only():
    """Two equal tokens at different positions: their logits differ only because of the position vector (the attention has no
    rotation), and the engine's vector equals sin / cos of position x 10000^(-2i/width) also hundreds of tokens in."""
    cfg = make_config([layer(window=2, keep=0)], width=40, taps=1)
    W = random_weights(cfg, seed=4)
    toks = [5] * 300
    want, _ = plain.run(cfg, W, toks)
    assert row_errs(want[299:300], want[298:299])[0] > 100 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    got = whole(m, toks)
    m.free()
    check_logits(got, want, "float32")


# ---- prompts against decoding, portions, batches ---------------------------------------------------------------------------------
HYBRID = make_config([layer(mlp=dense(40)), layer(heads=8, kv_heads=2, dim=8, vdim=12, window=70, keep=5, mlp=moe()),
                      layer(heads=2, kv_heads=2, dim=16, vdim=8, window=9, keep=0), layer(window=130, keep=2, mlp=moe(experts=3, top=2, shared=0))], taps=3)
NO_ROUTER = make_config([layer(mlp=dense(40)), layer(heads=8, kv_heads=2, dim=8, vdim=12, window=70, keep=5), layer(window=9, keep=1, mlp=dense(16))], taps=4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_token_by_token(dtype):
    W = weights(HYBRID, 5, dtype)
    toks = tokens(150, HYBRID["vocab"], 2)
    want, _ = plain.run(HYBRID, W, toks)
    m = build_engine(HYBRID, W, dtype)
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 1)] for _ in toks])["a"]
    m.free()
    check_logits(a, want, dtype)
    check_logits(b, want, dtype)
    check_logits(b, a, dtype)


@pytest.mark.parametrize("sizes", [[2] * 40, [3, 61, 2, 64, 5, 65, 1, 63, 2], [64, 64, 64], [1, 127, 2, 2, 100], [129, 2, 33], [7, 1, 1, 8, 9, 1, 2, 31]])
def test_portions(sizes):
    """Portions down to two tokens and single tokens in between: the short convolution's state, the cache and the window all cross
    the cuts (portions of fewer than 8 rows take the row kernels, longer ones the tile kernels)."""
    toks = tokens(sum(sizes), HYBRID["vocab"], 7)
    W = random_weights(HYBRID, seed=6)
    want, _ = plain.run(HYBRID, W, toks)
    m = build_engine(HYBRID, W, "float32")
    got = run_schedule(m, {"a": toks}, [[("a", n)] for n in sizes])["a"]
    m.free()
    assert rel_err(got, want) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_ragged_batch_equals_each_alone(dtype):
    cfg = HYBRID if dtype == "float32" else NO_ROUTER
    W = random_weights(cfg, seed=8)
    reqs = {"a": tokens(90, cfg["vocab"], 11), "b": tokens(17, cfg["vocab"], 12), "c": tokens(130, cfg["vocab"], 13), "d": tokens(1, cfg["vocab"], 14)}
    m = build_engine(cfg, W, dtype, max_tokens=448)
    alone = {k: whole(m, v) for k, v in reqs.items()}
    sched = [[("a", 30), ("b", 2)], [("a", 1), ("b", 9), ("c", 64)], [("c", 2), ("a", 1), ("d", 1)], [("b", 6), ("a", 58), ("c", 64)]]
    got = run_schedule(m, reqs, sched)
    m.free()
    for k, v in reqs.items():
        assert rel_err(got[k], alone[k]) < TOL[dtype], k
        assert rel_err(got[k], plain.run(cfg, W, v)[0]) < TOL[dtype], k


def test_pages_and_slots_are_reused():
    """Two slots and three pages for five requests: later requests run in the slots and pages earlier ones gave back, and a stale
    convolution state or a stale cache row would show in their logits (a slot's state is not cleared: positions before 0 are
    never read)."""
    cfg = NO_ROUTER
    W = random_weights(cfg, seed=9)
    m = build_engine(cfg, W, "float32", max_tokens=192, max_seqs=2)
    seen_pages, seen_slots = [], []
    for i, n in enumerate([100, 70, 128, 5, 64]):
        toks = tokens(n, cfg["vocab"], 20 + i)
        s = m.open()
        other = m.open()   # a second live sequence holds the other slot and a page while this one runs
        m.step([(other, tokens(3, cfg["vocab"], 40 + i))], [[]])
        got = np.concatenate([m.step([(s, toks[:n // 2])], [list(range(n // 2))]), m.step([(s, toks[n // 2:])], [list(range(n - n // 2))])])
        seen_pages.append(tuple(m.pages(s)))
        seen_slots.append(s)
        assert rel_err(got, plain.run(cfg, W, toks)[0]) < TOL["float32"], i
        m.close(s)
        m.close(other)
    assert m.pool_info()["free_pages"] == 3 and m.pool_info()["free_slots"] == 2
    m.free()
    assert len(set(seen_slots)) <= 2
    assert len(set(p for ps in seen_pages for p in ps)) <= 3 and len(seen_pages) == 5


# ---- a key that stands out: at the window's edges, in the kept prefix, at page borders, far back -------------------------------------
@functools.lru_cache(maxsize=None)
def planted_case(window, keep, place, n, heads, kv_heads):
    """Token A sits at `place` among n - 1 other tokens, token B is last; head 0 of layer 0 gives B's query a large score against
    A's key.  Returns the model, the tokens, the true logits and how far the last row moves when the mask is off by that one key."""
    cfg = make_config([layer(heads=heads, kv_heads=kv_heads, dim=16, vdim=16, window=window, keep=keep, scale=0.75, softcap=40.0), layer(window=window + 3, keep=keep)], width=64)
    A, B = 7, 11
    W = plant_pair(cfg, random_weights(cfg, seed=13, sink=-1.0, talk_noise=0.15), A, B)
    rng = np.random.default_rng(place * 7 + n)
    fill = [t for t in range(cfg["vocab"]) if t not in (A, B)]
    toks = [fill[int(i)] for i in rng.integers(0, len(fill), n)]
    toks[place], toks[-1] = A, B
    last = n - 1
    # (the second layer's window is three longer, which tells the layers apart: only the first layer's mask is bent)
    hidden = plain.run(cfg, W, toks, sees=lambda i, j, w, k: plain.visible(i, j, w, k) and not (w == window and i == last and j == place))[0]
    shown = plain.run(cfg, W, toks, sees=lambda i, j, w, k: plain.visible(i, j, w, k) or (w == window and i == last and j == place))[0]
    want = shown if plain.visible(last, place, window, keep) else hidden
    return cfg, W, toks, want, row_errs(hidden[-1:], shown[-1:])[0]


def standing_out(window, keep, place, n, decode, dtype="float32", heads=4, kv_heads=2, tol=None):
    """Whether B sees A decides its logits (the plain implementation with a mask that is off by that one key differs by far more
    than the tolerance), so an engine whose window, kept prefix or page walk is one key off cannot pass."""
    cfg, W, toks, want, moved = planted_case(window, keep, place, n, heads, kv_heads)
    tol = tol or TOL[dtype]
    assert moved > 3 * tol and moved > 0.15, "the planted key does not decide the last logits"
    m = build_engine(cfg, W, dtype)
    if decode:
        got = run_schedule(m, {"a": toks}, [[("a", n - 4)]] + [[("a", 1)]] * 4)["a"]
    else:
        got = whole(m, toks)
    m.free()
    assert rel_err(got, want) < tol


EDGES = [  # (window, keep_first, place of the key, tokens)
    (20, 3, 99 - 19, 100),    # the last key inside the window
    (20, 3, 99 - 20, 100),    # the first key outside it
    (20, 3, 2, 100),          # the last kept first key
    (20, 3, 3, 100),          # the first one that is not kept
    (20, 3, 0, 100),          # position 0
    (64, 0, 199 - 63, 200),   # a window of exactly one page: inside ...
    (64, 0, 199 - 64, 200),   # ... and outside
    (65, 2, 192 - 64, 193),   # the window's edge on a page border, the row the first of its page
    (65, 2, 192 - 65, 193),
    (300, 1, 63, 330),        # far back, at the end of the first page
    (300, 1, 64, 330),        # ... and at the start of the second
    (300, 1, 329 - 299, 330), # the far edge of a long window among hundreds of keys
    (300, 1, 329 - 300, 330),
    (5, 70, 69, 200),         # a kept prefix that spans a page border: its last key ...
    (5, 70, 70, 200),         # ... and the first key behind it
    (5, 70, 63, 200),
    (5, 70, 64, 200),
]


@pytest.mark.parametrize("window,keep,place,n", EDGES)
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out(window, keep, place, n, decode):
    standing_out(window, keep, place, n, decode)


@pytest.mark.parametrize("window,keep,place,n", [(20, 3, 99 - 19, 100), (20, 3, 99 - 20, 100), (20, 3, 2, 100), (20, 3, 3, 100), (300, 1, 64, 330)])
def test_one_key_stands_out_bf16_nine_heads(window, keep, place, n):
    standing_out(window, keep, place, n, True, dtype="bfloat16", heads=9, kv_heads=3, tol=0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_counts_once_and_only_in_the_denominator(dtype):
    """A large sink takes most of the softmax mass: leaving it out (or giving it a value, or capping / scaling it) would change the
    attention output by several times."""
    cfg = make_config([layer(heads=2, kv_heads=1, window=6, keep=1, softcap=2.0)])
    W = random_weights(cfg, seed=14)
    W["l0.mix.sink"] = to_bf16_values(np.array([5.0, -1.0], np.float32))   # above the cap: a capped sink would be 2
    toks = tokens(70, cfg["vocab"], 3)
    want, _ = plain.run(cfg, W, toks)
    W0 = dict(W)
    W0["l0.mix.sink"] = np.array([2.0, -1.0], np.float32)
    tol = min(TOL[dtype], 0.05)
    assert row_errs(plain.run(cfg, W0, toks)[0], want).max() > 5 * tol
    m = build_engine(cfg, W, dtype)
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 1)]] * 70)["a"]
    m.free()
    assert rel_err(a, want) < tol and rel_err(b, want) < tol


def test_heads_are_mixed_before_the_mask_and_after_the_cap():
    """A mixing matrix far from the identity with negative entries, and a tight cap: mixing before the cap, or a softmax per head
    before the mixing, gives other logits."""
    cfg = make_config([layer(heads=3, kv_heads=1, dim=8, vdim=8, window=10, keep=1, softcap=1.0, scale=1.0)])
    W = random_weights(cfg, seed=15)
    W["l0.mix.talk"] = to_bf16_values(np.array([[0.5, -1.5, 1.0], [2.0, 0.25, -0.75], [-1.0, 1.0, 1.5]], np.float32))
    toks = tokens(40, cfg["vocab"], 6)
    want, _ = plain.run(cfg, W, toks)
    Wi = dict(W)
    Wi["l0.mix.talk"] = np.eye(3, dtype=np.float32)
    assert row_errs(plain.run(cfg, Wi, toks)[0], want).max() > 50 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 3)], [("a", 30)]] + [[("a", 1)]] * 7)["a"]
    m.free()
    assert rel_err(a, want) < TOL["float32"] and rel_err(b, want) < TOL["float32"]


def test_convolution_state_crosses_every_cut():
    """Five taps with large weights: a row's mixer input depends on the four rows before it, which lie in the same portion, in the
    portion before, two portions back (portions of one and two tokens) or before the sequence's start."""
    cfg = make_config([layer(window=3, keep=0)], taps=5)
    W = random_weights(cfg, seed=16)
    W["l0.canon1"] = to_bf16_values(np.random.default_rng(1).standard_normal((cfg["width"], 5)).astype(np.float32))
    toks = tokens(40, cfg["vocab"], 8)
    want, _ = plain.run(cfg, W, toks)
    W0 = dict(W)
    W0["l0.canon1"] = np.array(W["l0.canon1"], copy=True)
    W0["l0.canon1"][:, 0] = 0
    assert row_errs(plain.run(cfg, W0, toks)[0][4:], want[4:]).min() > 20 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    for sizes in ([1] * 40, [2, 1, 1, 3, 1, 2, 2, 9, 1, 1, 1, 1, 1, 14], [40], [3, 37]):
        got = run_schedule(m, {"a": toks}, [[("a", n)] for n in sizes])["a"]
        assert rel_err(got, want) < TOL["float32"], sizes
    m.free()


@pytest.mark.parametrize("heads,window,n", [(20, 900, 1000), (16, 1200, 1260)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_window_many_heads(dtype, heads, window, n):
    """A row's scores of all heads over a long window: 20 heads x 960 keys take the mixing pass that works out of shared memory
    (more than 16 heads); 16 heads x 1280 keys no longer fit beside the register form, which then keeps them in the score scratch
    between its two sweeps.  Prompt tiles and decoded rows."""
    cfg = make_config([layer(heads=heads, kv_heads=4, dim=16, vdim=8, window=window, keep=3, mlp=dense(32))], width=40)
    W = random_weights(cfg, seed=23)
    toks = tokens(n, cfg["vocab"], 9)
    want, _ = plain.run(cfg, W, toks)
    m = build_engine(cfg, W, dtype, max_tokens=(n + 63) // 64 * 64)
    got = run_schedule(m, {"a": toks}, [[("a", n - 300)], [("a", 3)], [("a", 290)]] + [[("a", 1)]] * 7)["a"]
    m.free()
    assert rel_err(got, want) < TOL[dtype]


def test_first_tokens_and_single_token_requests():
    W = random_weights(HYBRID, seed=16)
    m = build_engine(HYBRID, W, "float32")
    for n in (1, 2, 3):
        toks = tokens(n, HYBRID["vocab"], 30 + n)
        assert rel_err(whole(m, toks), plain.run(HYBRID, W, toks)[0]) < TOL["float32"]
    m.free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """The window (70) and the kept prefix pass over decoded tokens; 320 single-token steps."""
    cfg = NO_ROUTER
    W = random_weights(cfg, seed=17)
    toks = tokens(330, cfg["vocab"], 5)
    want, _ = plain.run(cfg, W, toks)
    m = build_engine(cfg, W, dtype)
    got = run_schedule(m, {"a": toks}, [[("a", 10)]] + [[("a", 1)]] * 320)["a"]
    m.free()
    assert rel_err(got, want) < TOL[dtype]


@pytest.mark.parametrize("rows", [1, 3, 8])
def test_wide_model_decode_rows_and_tiles(rows):
    """Widths in whole 32-element chunks (bf16 mode: the decode rows' products run on the tensor-core few-row kernel, prompt
    products on tcgen05), 16 heads of 32, a window of 100 behind 6 kept keys."""
    cfg = make_config([layer(heads=16, kv_heads=4, dim=32, vdim=32, window=100, keep=6, mlp=dense(264)),
                       layer(heads=8, kv_heads=2, dim=32, vdim=64, window=40, keep=0, mlp=moe(ff=64, shared=96))], vocab=203, width=256, taps=4)
    W = weights(cfg, 31, "bfloat16")
    lens = [150, 9, 33, 70, 21, 7, 12, 40][:rows]
    reqs = {"r%d" % i: tokens(n, 203, 60 + i) for i, n in enumerate(lens)}
    m = build_engine(cfg, W, "bfloat16", max_tokens=sum((n + 63) // 64 * 64 for n in lens), max_seqs=rows)
    alone = {k: whole(m, v) for k, v in reqs.items()}
    tail = 6
    got = run_schedule(m, reqs, [[(k, len(v) - tail) for k, v in reqs.items()]] + [[(k, 1) for k in reqs]] * tail)
    m.free()
    for k, v in reqs.items():
        check_logits(got[k], alone[k], "bfloat16")
        check_logits(alone[k], plain.run(cfg, W, v)[0], "bfloat16")


# ---- generation through the engine's own loop, and the command line ---------------------------------------------------------------
def plain_greedy(cfg, W, prompt, n_new):
    s = plain.Sequence(cfg, W)
    for t in prompt:
        z = s.feed(t)
    out = []
    for _ in range(n_new):
        out.append(int(np.argmax(z)))
        z = s.feed(out[-1])
    return out


def test_greedy_generation_continuous_batching():
    """Six requests through two slots and a pool that holds about two of them: admission, portions of prompts beside decoded
    tokens, and slots / pages handed on, all inside the engine's generation loop."""
    W = random_weights(HYBRID, seed=18)
    prompts = [tokens(n, HYBRID["vocab"], 70 + i) for i, n in enumerate([5, 40, 90, 1, 64, 23])]
    want = [plain_greedy(HYBRID, W, p, 12) for p in prompts]
    m = build_engine(HYBRID, W, "float32", max_tokens=256, max_seqs=2)
    got = m.generate(prompts, 12, step_tokens=48)
    m.free()
    assert got == want


def test_command_line_generate_and_trace_replay(tmp_path):
    from turboinfer_b200.safetensors_io import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = make_config([layer(mlp=moe()), layer(window=8, keep=2, mlp=dense(24)), layer(heads=2, kv_heads=1)], vocab=53)
    W = random_weights(cfg, seed=19)
    folder = os.path.join(tmp_path, "model")
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), W)
    prompts = [tokens(7, 53, 3), tokens(30, 53, 4)]
    want = [plain_greedy(cfg, W, p, 6) for p in prompts]
    cmd = [sys.executable, os.path.join(root, "bin", "generate"), "--model", folder, "--dtype", "float32", "--max-new", "6"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    assert [json.loads(line)["tokens"] for line in res.stdout.splitlines() if line.startswith("{")] == want
    out = os.path.join(tmp_path, "out")
    os.makedirs(out)
    p = prompts[1]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": p[:11], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": p[11:13], "want": []}, {"id": "b", "tokens": prompts[0], "want": [6]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": p[13:], "want": [0, len(p) - 14]}], "end": ["a"]}]
    res = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out,
                          "--max-tokens", "128"], input="".join(json.dumps(x) + "\n" for x in steps), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "0.f32"))
    ref_a, ref_b = plain.run(cfg, W, p)[0], plain.run(cfg, W, prompts[0])[0]
    l1 = np.fromfile(os.path.join(out, "1.f32"), "<f4").reshape(1, 53)
    l2 = np.fromfile(os.path.join(out, "2.f32"), "<f4").reshape(2, 53)
    assert rel_err(l1, ref_b[[6]]) < TOL["float32"]
    assert rel_err(l2, ref_a[[13, len(p) - 1]]) < TOL["float32"]


def test_errors_are_reported():
    cfg = make_config([layer(mlp=moe())])
    W = random_weights(cfg, seed=20)
    bad = dict(W)
    bad["l0.mix.talk"] = W["l0.mix.talk"][:-1]
    with pytest.raises(Exception):
        build_engine(cfg, bad)
    missing = {k: v for k, v in W.items() if k != "l0.mlp.router.b"}
    with pytest.raises(Exception):
        build_engine(cfg, missing)
    with pytest.raises(Exception):   # an unknown mixer type
        build_engine(make_config([dict(layer(), type="conv")]), W)
    with pytest.raises(Exception):   # more heads than the head-mixing attention holds
        build_engine(make_config([layer(heads=80, kv_heads=80, dim=4, vdim=4)], width=32), W)
