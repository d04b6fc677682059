"""CPU-side checks around the Gulazen model: the plain implementation's own invariants (each mechanism against a second, direct
formula), the configuration reader and the checkpoint reader.  No GPU, no engine library."""
import math

import numpy as np
import pytest

import gulazen_plain as plain
from gulazen_cases import dense, layer, make_config, moe, random_weights, rel_err


def toks(n, vocab, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def test_prefix_property():
    # causal: the logits of a prefix do not change when tokens are appended
    cfg = make_config([layer(mlp=moe()), layer(window=5, keep=2, mlp=dense(16)), layer(heads=2, kv_heads=1)])
    W = random_weights(cfg, seed=1)
    t = toks(30, cfg["vocab"])
    assert rel_err(plain.run(cfg, W, t)[0][:17], plain.run(cfg, W, t[:17])[0]) < 1e-12


def test_position_vector_interleaves_sine_and_cosine():
    v = plain.position_vector(7, 6)
    f = [7 * 10000.0 ** (-2.0 * i / 6) for i in range(3)]
    assert np.allclose(v, [math.sin(f[0]), math.cos(f[0]), math.sin(f[1]), math.cos(f[1]), math.sin(f[2]), math.cos(f[2])])
    assert np.allclose(plain.position_vector(0, 5), [0, 1, 0, 1, 0])


def test_short_conv_is_a_causal_filter_plus_the_input():
    rng = np.random.default_rng(2)
    D, taps, n = 5, 4, 9
    x, w = rng.standard_normal((n, D)), rng.standard_normal((D, taps))
    hist = [np.zeros(D)] * (taps - 1)
    for t in range(n):
        y = plain.short_conv(hist, x[t], w)
        want = x[t].copy()
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                want += w[:, j] * x[s]
        assert np.allclose(y, want)
        hist = (hist + [x[t]])[1:]
    # one tap: the newest input only
    assert np.allclose(plain.short_conv([], x[0], w[:, :1]), x[0] * (1 + w[:, 0]))


def test_xielu_branches_meet_and_match_their_formulas():
    p, q = 0.3, -0.7
    ap, an = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
    z = np.array([-3.0, -1e-9, 0.0, 1e-9, 2.0])
    y = plain.xielu(z, p, q)
    assert np.allclose(y[0], an * (math.exp(-3.0) + 2.0) - 1.5) and np.allclose(y[4], ap * 4 + 1.0)
    assert abs(y[1]) < 1e-8 and y[2] == 0.0 and abs(y[3]) < 1e-8


def test_mask_keeps_the_window_and_the_first_keys():
    seen = [j for j in range(50) if plain.visible(40, j, 6, 3)]
    assert seen == [0, 1, 2, 35, 36, 37, 38, 39, 40]
    assert [j for j in range(50) if plain.visible(4, j, 6, 3)] == [0, 1, 2, 3, 4]
    assert [j for j in range(50) if plain.visible(9, j, 1, 0)] == [9]


def test_route_takes_the_largest_logits_and_softmaxes_them_only():
    z = np.array([0.1, 2.0, -1.0, 2.0, 1.5])
    picks, w = plain.route(z, 3)
    assert picks == [1, 3, 4]
    e = np.exp(np.array([2.0, 2.0, 1.5]))
    assert np.allclose(w, e / e.sum()) and abs(w.sum() - 1) < 1e-12


def test_sink_only_adds_to_the_denominator():
    cfg = make_config([layer(heads=2, kv_heads=1, dim=4, vdim=4, window=50, keep=0)], width=8)
    W = {k: np.asarray(v, np.float64) for k, v in random_weights(cfg, seed=3).items()}
    mx, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    rng = np.random.default_rng(3)
    hs = rng.standard_normal((6, 8))

    def outs(sink):
        Wl = dict(W)
        Wl["l0.mix.sink"] = np.array(sink, np.float64)
        Wl["l0.mix.o"] = np.eye(8)
        cache = {"k": [], "v": []}
        return np.array([plain.attention_token(Wl, "l0.mix.", mx, eps, h, i, cache) for i, h in enumerate(hs)])

    a, b = outs([-40.0, -40.0]), outs([0.0, 1.0])
    ratio = a / b   # per head one factor > 1: the same weighted sum over a larger denominator
    for i in range(6):
        for h in range(2):
            r = ratio[i, 4 * h:4 * h + 4]
            assert np.allclose(r, r[0]) and r[0] > 1.0


def test_config_reader_takes_every_constant_from_the_configuration():
    from turboinfer_b200 import models, seq
    cfg = make_config([layer(heads=6, kv_heads=3, dim=10, vdim=14, window=33, keep=5, scale=0.21, softcap=17.0, mlp=dense(72)),
                       layer(mlp=moe(experts=7, top=3, ff=12, shared=20)), layer(mlp=moe(shared=0)), layer()], vocab=77, width=36, eps=3e-4, taps=5)
    m, L = models.gulazen_descs(cfg, seq.F32, 640, 3)
    assert (m.vocab, m.width, m.n_layers, m.max_tokens, m.max_seqs) == (77, 36, 4, 640, 3)
    assert abs(m.norm_eps - 3e-4) < 1e-9 and m.norm_kind == seq.NORM_ONE_PLUS and m.norm_place == seq.NORMS_BEHIND
    assert m.tied_head == 1 and m.pos_base == 10000.0 and m.loop_times == 0
    a = L[0]
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first) == (seq.MIXER_ATTENTION, 6, 3, 10, 14, 33, 5)
    assert abs(a.scale - 0.21) < 1e-7 and abs(a.softcap - 17.0) < 1e-6 and a.rot_dims == 0 and a.qk_norm == seq.QK_NORM_WHOLE
    assert (a.talk, a.sink, a.conv_taps, a.layer_scale, a.out_gate) == (1, 1, 5, 1, 0)
    assert (a.ff_kind, a.ff, a.ff_act) == (seq.FF_DENSE, 72, seq.ACT_XIELU)
    b = L[1]
    assert (b.ff_kind, b.ff, b.experts, b.top, b.shared_ff, b.shared_plain, b.route_kind, b.identity) == (seq.FF_EXPERTS, 12, 7, 3, 20, 1, seq.ROUTE_TOP_LOGITS, 0)
    assert L[2].shared_ff == 0 and L[3].ff == 0
    for bad in ({"type": "wkv"}, {"mlp": {"kind": "glu", "ff": 8}}):
        broken = make_config([dict(layer(), **bad)])
        with pytest.raises(ValueError):
            models.gulazen_descs(broken, seq.F32, 64, 1)
    with pytest.raises(ValueError):
        models.gulazen_descs({k: v for k, v in cfg.items() if k != "canon"}, seq.F32, 64, 1)
    assert "Gulazen" in models.REGISTRY


def test_checkpoint_round_trip(tmp_path):
    from turboinfer_b200.safetensors_io import read_safetensors, write_safetensors
    cfg = make_config([layer(mlp=moe(experts=2, top=1))])
    W = random_weights(cfg, seed=4)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, W)
    back = read_safetensors(path)
    assert set(back) == set(W)
    for k, v in W.items():
        assert np.array_equal(back[k].to_f32(), np.asarray(v, np.float32)), k
