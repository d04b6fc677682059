"""The layered sequence engine on Zopipel models against the plain implementation (tests/zopipel_plain.py): every mechanism
alone, prompts against token-by-token decoding, portions, ragged batches, reuse of pages and state slots, one key that stands
out far back, at page borders and at the window's edges, the sink, the streams, both convolutions across cuts, the looped block,
the first tokens, long decoding, odd sizes, and greedy generation through the engine's own generation loop and command line."""
import functools
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import zopipel_plain as plain
from zopipel_cases import attn, build_engine, dense, latent, make_config, plant_pair, random_weights, rel_err, row_errs, run_schedule, to_bf16_values

pytestmark = pytest.mark.gpu

# bf16 mode: products round their inputs to bf16 (relative 4e-3 each); fp32 mode is fp32 arithmetic against float64
TOL = {"float32": 2e-4, "bfloat16": 1e-1}


def tokens(n, vocab, seed=1):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def whole(m, toks):
    return run_schedule(m, {"a": toks}, [[("a", len(toks))]])["a"]


def check_logits(got, want, dtype):
    assert row_errs(got, want).max() < TOL[dtype]


# ---- each mechanism alone: summed streams after every layer run, and the logits -------------------------------------------------
MECHANISMS = {
    "attention_only": make_config([attn()]),
    "latent_only": make_config([latent()]),
    "attention_with_ff": make_config([attn(mlp=dense(24))]),
    "latent_with_ff": make_config([latent(mlp=dense(56))]),
    "one_stream": make_config([attn(mlp=dense(24)), latent()], streams=1),
    "five_streams": make_config([latent(mlp=dense(24)), attn()], streams=5),
    "nine_streams": make_config([attn(mlp=dense(24)), latent(mlp=dense(16))], streams=9),
    "nine_taps": make_config([latent(mlp=dense(24)), attn(mlp=dense(16))], taps=9),
    "one_tap": make_config([attn(mlp=dense(24)), latent(mlp=dense(8))], taps=1),
    "two_taps_odd_width": make_config([attn(heads=3, kv_heads=3, dim=10, vdim=7, rot_dims=6), latent(heads=5, dim=6, rot_dim=2, vdim=5, kv_rank=9, q_rank=7)],
                                      width=37, taps=2, eps=1e-3),
    "six_taps": make_config([latent(window=9, mlp=dense(16)), attn(mlp=dense(16))], taps=6),
    "every_coordinate_turns": make_config([attn(dim=16, vdim=16, rot_dims=16, factor=None)]),
    "no_frequency_divisor_few_turn": make_config([attn(dim=16, rot_dims=2, factor=None, base=100.0)]),
    "large_frequency_divisor": make_config([attn(rot_dims=12, factor=8.0, base=500.0)]),
    "one_head": make_config([attn(heads=1, kv_heads=1, dim=16, vdim=8), latent(heads=1, dim=4, rot_dim=8, vdim=16, kv_rank=6, q_rank=3)]),
    "one_key_value_head": make_config([attn(heads=5, kv_heads=1, dim=8, vdim=24, rot_dims=4)], width=40),
    "as_many_key_value_heads": make_config([attn(heads=4, kv_heads=4, dim=8, vdim=8)]),
    "window_one": make_config([latent(window=1), latent(window=1, mlp=dense(16))]),
    "window_two": make_config([latent(window=2)]),
    "window_beyond_the_sequence": make_config([latent(window=500)]),
    "query_rank_above_width": make_config([latent(q_rank=70, kv_rank=60, heads=2)], width=40),
    "rotated_part_larger_than_plain": make_config([latent(dim=4, rot_dim=16, vdim=8, kv_rank=12)]),
    "wide_heads": make_config([attn(heads=2, kv_heads=1, dim=72, vdim=136, rot_dims=40)], width=64),
    "tensor_core_head_64": make_config([attn(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=64, mlp=dense(96))], width=128),
    "tensor_core_head_128": make_config([attn(heads=2, kv_heads=1, dim=128, vdim=128, rot_dims=32)], width=64),
    "latent_row_160": make_config([latent(heads=4, dim=16, rot_dim=32, vdim=16, kv_rank=128, q_rank=48, window=40, mlp=dense(64))], width=128),
    "latent_row_not_in_fours": make_config([latent(heads=2, dim=5, rot_dim=6, vdim=7, kv_rank=13, q_rank=5, window=11)]),
    "loop_of_one_layer": make_config([attn(mlp=dense(16)), latent(mlp=dense(16)), attn()], loop=(1, 2, 3)),
    "loop_over_everything": make_config([latent(window=7), attn(mlp=dense(16))], loop=(0, 2, 2)),
    "loop_once": make_config([attn(), latent(mlp=dense(16))], loop=(0, 1, 1)),
    "loop_at_the_end": make_config([latent(mlp=dense(16)), attn(mlp=dense(16)), latent(window=5)], loop=(1, 3, 2), streams=3),
    "layers_that_differ": make_config([attn(mlp=dense(40)), latent(heads=2, dim=16, rot_dim=8, vdim=8, window=7, mlp=dense(24)),
                                       attn(heads=6, kv_heads=3, dim=8, vdim=8, rot_dims=8, factor=4.0), latent(window=50, kv_rank=32, q_rank=24)],
                                      vocab=101, width=56, taps=4, streams=3),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_mechanism_layers_and_logits(name, dtype):
    cfg = MECHANISMS[name]
    W = random_weights(cfg, seed=3)
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
        assert np.abs(got_layers[i] - layers[i]).max() / scale < TOL[dtype] * 5, f"layer run {i}"
    check_logits(got, want, dtype)


# ---- prompts against decoding, portions, batches ---------------------------------------------------------------------------------
HYBRID = make_config([attn(mlp=dense(40)), latent(window=70, mlp=dense(24)), attn(heads=2, kv_heads=2, dim=16, vdim=8, rot_dims=16),
                      latent(heads=2, window=9, kv_rank=12, q_rank=16, mlp=dense(16))], taps=4, streams=3, loop=(1, 3, 2))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_token_by_token(dtype):
    W = random_weights(HYBRID, seed=5)
    toks = tokens(150, HYBRID["vocab"], 2)
    want, _ = plain.run(HYBRID, W, toks)
    m = build_engine(HYBRID, W, dtype)
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 1)] for _ in toks])["a"]
    m.free()
    check_logits(a, want, dtype)
    check_logits(b, want, dtype)
    check_logits(b, a, dtype)


def test_many_streams_and_taps_token_by_token():
    """More streams than the stream kernel keeps with a compile-time count, more taps than the prompt convolution keeps in
    registers: a prompt in one step, in portions, and token by token (the decode rows' convolution rides in the stream kernel)."""
    cfg = make_config([attn(mlp=dense(24)), latent(window=13, mlp=dense(16))], taps=9, streams=9, loop=(0, 2, 2))
    W = random_weights(cfg, seed=15, canon_amp=1.0)
    toks = tokens(90, cfg["vocab"], 4)
    want, _ = plain.run(cfg, W, toks)
    m = build_engine(cfg, W, "float32")
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 1)] for _ in toks])["a"]
    c = run_schedule(m, {"a": toks}, [[("a", n)] for n in (70, 2, 1, 1, 5, 1, 10)])["a"]
    m.free()
    for got in (a, b, c):
        check_logits(got, want, "float32")


@pytest.mark.parametrize("sizes", [[2] * 40, [3, 61, 2, 64, 5, 65, 1, 63, 2], [64, 64, 64], [1, 127, 2, 2, 100], [129, 2, 33], [7, 1, 1, 8, 9, 1, 2, 31]])
def test_portions(sizes):
    """Portions down to two tokens and single tokens in between: both convolutions' states, the caches and the window all cross
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
    cfg = HYBRID
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
    cfg = HYBRID
    W = random_weights(cfg, seed=9, canon_amp=0.8)
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


# ---- a key that stands out: far back, at page borders, at position 0, at the window's edges ----------------------------------------
@functools.lru_cache(maxsize=None)
def planted_case(kind, window, place, n):
    """Token A sits at `place` among n - 1 other tokens, token B is last; head 0 of layer 0 gives B's query a large score against
    A's key.  Returns the model, the tokens, the true logits and how far the last row moves when the mask is off by that one key."""
    if kind == "attention":
        first = attn(heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=8, scale=0.75)
        second = latent(window=window + 3)
    else:
        first = latent(heads=3, dim=16, rot_dim=4, vdim=16, kv_rank=24, q_rank=12, window=window, scale=0.5)
        second = attn()
    cfg = make_config([first, second], width=64)
    A, B = 7, 11
    W = plant_pair(cfg, random_weights(cfg, seed=13), A, B)
    rng = np.random.default_rng(place * 7 + n)
    fill = [t for t in range(cfg["vocab"]) if t not in (A, B)]
    toks = [fill[int(i)] for i in rng.integers(0, len(fill), n)]
    toks[place], toks[-1] = A, B
    last = n - 1
    true_sees = plain.sees_all if kind == "attention" else plain.sees_window
    key = "attention" if kind == "attention" else "latent_attention"
    hidden = plain.run(cfg, W, toks, sees={key: lambda i, j, w: true_sees(i, j, w) and not (i == last and j == place)})[0]
    shown = plain.run(cfg, W, toks, sees={key: lambda i, j, w: true_sees(i, j, w) or (i == last and j == place)})[0]
    want = shown if true_sees(last, place, window) else hidden
    return cfg, W, toks, want, row_errs(hidden[-1:], shown[-1:])[0]


def standing_out(kind, window, place, n, decode, dtype="float32", tol=None):
    """Whether B sees A decides its logits (the plain implementation with a mask that is off by that one key differs by far more
    than the tolerance), so an engine whose window or page walk is one key off, or that loses a far key, cannot pass."""
    cfg, W, toks, want, moved = planted_case(kind, window, place, n)
    tol = tol or TOL[dtype]
    assert moved > 3 * tol and moved > 0.1, "the planted key does not decide the last logits"
    m = build_engine(cfg, W, dtype)
    if decode:
        got = run_schedule(m, {"a": toks}, [[("a", n - 4)]] + [[("a", 1)]] * 4)["a"]
    else:
        got = whole(m, toks)
    m.free()
    assert rel_err(got, want) < tol


EDGES = [  # (mixer of layer 0, window, place of the key, tokens)
    ("attention", 0, 0, 400),          # position 0, hundreds of keys back
    ("attention", 0, 63, 330),         # the end of the first page
    ("attention", 0, 64, 330),         # the start of the second
    ("attention", 0, 17, 600),         # far back among hundreds
    ("attention", 0, 198, 200),        # the key right before the row
    ("latent", 20, 99 - 19, 100),      # the last key inside the window
    ("latent", 20, 99 - 20, 100),      # the first key outside it
    ("latent", 64, 199 - 63, 200),     # a window of exactly one page: inside ...
    ("latent", 64, 199 - 64, 200),     # ... and outside
    ("latent", 65, 192 - 64, 193),     # the window's edge on a page border, the row the first of its page
    ("latent", 65, 192 - 65, 193),
    ("latent", 300, 329 - 299, 330),   # the far edge of a long window among hundreds of keys
    ("latent", 300, 329 - 300, 330),
    ("latent", 300, 63, 330),          # inside a long window, at a page's end
    ("latent", 500, 0, 330),           # a window beyond the sequence: position 0
    ("latent", 1, 98, 100),            # a window of one: the key right before the row is already outside
]


@pytest.mark.parametrize("kind,window,place,n", EDGES)
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out(kind, window, place, n, decode):
    standing_out(kind, window, place, n, decode)


@pytest.mark.parametrize("kind,window,place,n", [("attention", 0, 64, 330), ("latent", 20, 99 - 19, 100), ("latent", 20, 99 - 20, 100), ("latent", 65, 192 - 65, 193)])
@pytest.mark.parametrize("decode", [False, True])
def test_one_key_stands_out_bf16(kind, window, place, n, decode):
    standing_out(kind, window, place, n, decode, dtype="bfloat16", tol=0.05)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_counts_once_with_score_zero(dtype):
    """Small scores: the sink's exp(0) = 1 is a large part of every denominator (all of 1/2 at position 0), so a softmax without
    it, or one that gives it a value, differs by far."""
    cfg = make_config([attn(heads=2, kv_heads=1, scale=0.05)])
    W = random_weights(cfg, seed=14)
    toks = tokens(70, cfg["vocab"], 3)
    want, _ = plain.run(cfg, W, toks)
    m = build_engine(cfg, W, dtype)
    m.debug_layers(True)
    a = whole(m, toks)
    first = m.read_layers(len(toks))[0, 0]
    b = run_schedule(m, {"a": toks}, [[("a", 1)]] * 70)["a"]
    m.free()
    tol = min(TOL[dtype], 0.05)
    assert rel_err(a, want) < tol and rel_err(b, want) < tol
    # at position 0 the only key gets exp(s) / (1 + exp(s)); without the sink it would get 1
    s = plain.Sequence(cfg, W)
    s.feed(toks[0])
    assert np.abs(first - s.layers_out[0][0]).max() < 5 * tol * np.abs(s.layers_out[0][0]).max()


def test_streams_are_rewritten_together_from_the_old_ones():
    """A mixing matrix far from the identity and not symmetric: using [to, from] instead of [from, to], or updating the streams one
    after the other, gives other logits."""
    cfg = make_config([attn(mlp=dense(16)), latent(mlp=dense(16))], streams=3)
    W = random_weights(cfg, seed=15)
    for nm in ("l0.hc1.mix", "l0.hc2.mix", "l1.hc1.mix", "l1.hc2.mix"):
        W[nm] = to_bf16_values(np.array([[0.5, -0.75, 1.0], [1.0, 0.25, -0.5], [-0.5, 0.5, 0.75]], np.float32))
    toks = tokens(40, cfg["vocab"], 6)
    want, _ = plain.run(cfg, W, toks)
    Wt = dict(W)
    Wt["l1.hc1.mix"] = np.ascontiguousarray(W["l1.hc1.mix"].T)
    assert row_errs(plain.run(cfg, Wt, toks)[0], want).max() > 50 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 3)], [("a", 30)]] + [[("a", 1)]] * 7)["a"]
    m.free()
    assert rel_err(a, want) < TOL["float32"] and rel_err(b, want) < TOL["float32"]


def test_convolution_states_cross_every_cut():
    """Five taps with large weights in front of BOTH sublayers of a looped layer: a row's input depends on the four rows before
    it, which lie in the same portion, in the portion before, two portions back or before the sequence's start; every pass of the
    loop has states of its own."""
    cfg = make_config([latent(window=3, mlp=dense(16)), attn()], taps=5, loop=(0, 1, 2))
    W = random_weights(cfg, seed=16)
    rng = np.random.default_rng(1)
    W["l0.canon1"] = to_bf16_values(rng.standard_normal((cfg["width"], 5)).astype(np.float32))
    W["l0.canon2"] = to_bf16_values(rng.standard_normal((cfg["width"], 5)).astype(np.float32))
    toks = tokens(40, cfg["vocab"], 8)
    want, _ = plain.run(cfg, W, toks)
    for nm in ("l0.canon1", "l0.canon2"):
        W0 = dict(W)
        W0[nm] = np.array(W[nm], copy=True)
        W0[nm][:, 0] = 0
        assert row_errs(plain.run(cfg, W0, toks)[0][4:], want[4:]).min() > 20 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    for sizes in ([1] * 40, [2, 1, 1, 3, 1, 2, 2, 9, 1, 1, 1, 1, 1, 14], [40], [3, 37]):
        got = run_schedule(m, {"a": toks}, [[("a", n)] for n in sizes])["a"]
        assert rel_err(got, want) < TOL["float32"], sizes
    m.free()


def test_biases_temperature_and_value_norm_matter_and_match():
    """Large biases, head factors far from 1 and values of very different sizes: dropping any of them moves the logits by far."""
    cfg = make_config([attn(heads=4, kv_heads=2, mlp=dense(16))])
    W = random_weights(cfg, seed=21)
    rng = np.random.default_rng(2)
    for nm in ("l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l0.mix.o.b"):
        W[nm] = to_bf16_values(rng.standard_normal(W[nm].shape).astype(np.float32) * 2.0)
    W["l0.mix.temp"] = to_bf16_values(np.array([0.25, 3.0, -1.0, 1.5], np.float32))
    W["l0.mix.v"] = to_bf16_values(W["l0.mix.v"] * np.repeat(np.array([8.0, 0.1], np.float32), cfg["layers"][0]["mixer"]["vdim"])[:, None])
    toks = tokens(50, cfg["vocab"], 4)
    want, _ = plain.run(cfg, W, toks)
    for nm in ("l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l0.mix.o.b", "l0.mix.temp"):
        W0 = dict(W)
        W0[nm] = np.ones_like(W[nm]) if nm.endswith("temp") else np.zeros_like(W[nm])
        assert row_errs(plain.run(cfg, W0, toks)[0], want).max() > 50 * TOL["float32"], nm
    m = build_engine(cfg, W, "float32")
    a = whole(m, toks)
    b = run_schedule(m, {"a": toks}, [[("a", 20)]] + [[("a", 1)]] * 30)["a"]
    m.free()
    assert rel_err(a, want) < TOL["float32"] and rel_err(b, want) < TOL["float32"]


def test_rotation_far_into_a_sequence():
    """Positions in the hundreds, angle = position x frequency in fp32: a frequency divisor that is off by two percent moves the late
    logits by far more than the tolerance, so the engine's frequencies and angles are the design's."""
    cfg = make_config([attn(dim=16, vdim=8, rot_dims=16, factor=2.0, base=10000.0), latent(dim=4, rot_dim=12, window=300)], taps=1)
    W = random_weights(cfg, seed=4)
    toks = tokens(700, cfg["vocab"], 12)
    want, _ = plain.run(cfg, W, toks)
    off = make_config([attn(dim=16, vdim=8, rot_dims=16, factor=2.04, base=10000.0), latent(dim=4, rot_dim=12, window=300)], taps=1)
    assert row_errs(plain.run(off, W, toks)[0][600:], want[600:]).max() > 10 * TOL["float32"]
    m = build_engine(cfg, W, "float32")
    got = run_schedule(m, {"a": toks}, [[("a", 690)]] + [[("a", 1)]] * 10)["a"]
    m.free()
    check_logits(got, want, "float32")


def test_first_tokens_and_single_token_requests():
    W = random_weights(HYBRID, seed=16)
    m = build_engine(HYBRID, W, "float32")
    for n in (1, 2, 3):
        toks = tokens(n, HYBRID["vocab"], 30 + n)
        assert rel_err(whole(m, toks), plain.run(HYBRID, W, toks)[0]) < TOL["float32"]
        assert rel_err(run_schedule(m, {"a": toks}, [[("a", 1)]] * n)["a"], plain.run(HYBRID, W, toks)[0]) < TOL["float32"]
    m.free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    """The windows (70 and 9) pass over decoded tokens; 320 single-token steps."""
    cfg = HYBRID
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
    products on tcgen05), attention heads of 64 on the tensor-core attention, a latent row of 128 + 32."""
    cfg = make_config([attn(heads=8, kv_heads=2, dim=64, vdim=64, rot_dims=32, mlp=dense(264)),
                       latent(heads=8, dim=32, rot_dim=32, vdim=32, kv_rank=128, q_rank=96, window=100, mlp=dense(320))], vocab=203, width=256, taps=4,
                      streams=4, loop=(0, 2, 2))
    W = random_weights(cfg, seed=31)
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
    cfg = make_config([attn(mlp=dense(24)), latent(window=8, mlp=dense(24)), attn(heads=2, kv_heads=1)], vocab=53, loop=(0, 2, 2))
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
    cfg = make_config([attn(mlp=dense(16)), latent()])
    W = random_weights(cfg, seed=20)
    bad = dict(W)
    bad["l0.hc1.mix"] = W["l0.hc1.mix"][:-1]
    with pytest.raises(Exception):
        build_engine(cfg, bad)
    for gone in ("l0.mix.temp", "l0.canon2", "l1.mix.dq.norm", "l1.hc1.in", "l0.mix.o.b"):
        with pytest.raises(Exception):
            build_engine(cfg, {k: v for k, v in W.items() if k != gone})
    with pytest.raises(Exception):   # an unknown mixer type
        build_engine(make_config([dict(attn(), type="conv")]), W)
    with pytest.raises(Exception):   # more streams than the engine keeps in registers
        build_engine(make_config([attn()], streams=40), W)
    with pytest.raises(Exception):   # the rotated part turns as a whole
        lat = latent()
        lat["mixer"]["rot"]["dims"] = 2
        build_engine(make_config([lat]), W)
