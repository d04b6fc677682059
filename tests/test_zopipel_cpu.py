"""CPU-side checks around the Zopipel model: the plain implementation's own invariants (each mechanism against a second, direct
formula), the configuration reader and the checkpoint reader.  No GPU, no engine library."""
import math

import numpy as np
import pytest

import zopipel_plain as plain
from zopipel_cases import attn, dense, latent, make_config, random_weights, rel_err


def toks(n, vocab, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, n)]


def test_prefix_property():
    # causal: the logits of a prefix do not change when tokens are appended
    cfg = make_config([attn(mlp=dense(16)), latent(window=5, mlp=dense(16)), attn(heads=2, kv_heads=1)], loop=(0, 2, 2))
    W = random_weights(cfg, seed=1)
    t = toks(30, cfg["vocab"])
    assert rel_err(plain.run(cfg, W, t)[0][:17], plain.run(cfg, W, t[:17])[0]) < 1e-12


def test_layer_runs_repeat_the_looped_block_as_a_whole():
    cfg = make_config([attn()] * 5, loop=(1, 3, 3))
    assert plain.layer_runs(cfg) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert plain.layer_runs(make_config([attn()] * 3)) == [0, 1, 2]
    assert plain.layer_runs(make_config([attn()] * 3, loop=(0, 3, 1))) == [0, 1, 2]
    _, layers = plain.run(cfg, random_weights(cfg, seed=2), toks(4, cfg["vocab"]))
    assert layers.shape[0] == 9


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
    assert np.allclose(plain.short_conv([], x[0], w[:, :1]), x[0] * (1 + w[:, 0]))   # one tap: the newest input only


def test_rotation_pairs_the_two_halves_and_depends_on_the_distance_only():
    rot = {"base": 100.0, "dims": 6, "scaling": {"factor": 4.0}}
    rng = np.random.default_rng(3)
    q, k = rng.standard_normal(9), rng.standard_normal(9)
    r = plain.rotate_half(q, 5, rot)
    assert np.allclose(r[6:], q[6:])                      # behind rot.dims nothing turns
    for i in range(3):
        ang = 5 * 100.0 ** (-2.0 * i / 6) / 4.0
        assert np.allclose([r[i], r[i + 3]], [q[i] * math.cos(ang) - q[i + 3] * math.sin(ang), q[i + 3] * math.cos(ang) + q[i] * math.sin(ang)])
    a = plain.rotate_half(q, 40, rot) @ plain.rotate_half(k, 33, rot)
    b = plain.rotate_half(q, 7, rot) @ plain.rotate_half(k, 0, rot)
    assert abs(a - b) < 1e-12
    assert np.allclose(plain.rotate_half(q, 0, rot), q)
    assert not np.allclose(plain.rotate_half(q, 5, rot), plain.rotate_half(q, 5, {"base": 100.0, "dims": 6}))


def test_streams_with_identity_mixing_are_the_plain_residual():
    rng = np.random.default_rng(4)
    X = [rng.standard_normal(6) for _ in range(3)]
    y = rng.standard_normal(6)
    out = plain.streams_write(X, np.eye(3), np.ones(3), y)
    assert all(np.allclose(out[s], X[s] + y) for s in range(3))
    mix = rng.standard_normal((3, 3))
    out = plain.streams_write(X, mix, np.array([0.5, 0.0, -1.0]), y)
    assert np.allclose(out[1], mix[0, 1] * X[0] + mix[1, 1] * X[1] + mix[2, 1] * X[2])   # [from, to]
    assert np.allclose(plain.streams_read(X, np.array([1.0, 2.0, 0.0])), X[0] + 2 * X[1])


def test_windows():
    assert [j for j in range(50) if plain.sees_window(40, j, 6)] == [35, 36, 37, 38, 39, 40]
    assert [j for j in range(50) if plain.sees_window(3, j, 6)] == [0, 1, 2, 3]
    assert [j for j in range(50) if plain.sees_window(9, j, 1)] == [9]
    assert [j for j in range(12) if plain.sees_all(9, j, 0)] == list(range(10))


def test_sink_adds_one_to_the_denominator():
    cfg = make_config([attn(heads=2, kv_heads=1, dim=4, vdim=4, rot_dims=2)], width=8)
    W = {k: np.asarray(v, np.float64) for k, v in random_weights(cfg, seed=3).items()}
    W["l0.mix.o"], W["l0.mix.o.b"] = np.eye(8), np.zeros(8)
    mx, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    h = np.random.default_rng(3).standard_normal(8)
    out = plain.attention_token(W, "l0.mix.", mx, eps, h, 0, {"k": [], "v": []})
    q = plain.rotate_half((W["l0.mix.q"] @ h + W["l0.mix.q.b"]).reshape(2, 4), 0, mx["rot"])
    k = plain.rotate_half((W["l0.mix.k"] @ h + W["l0.mix.k.b"]).reshape(1, 4), 0, mx["rot"])
    v = plain.rms_div((W["l0.mix.v"] @ h + W["l0.mix.v.b"]).reshape(1, 4), eps)
    for hh in range(2):
        s = (q[hh] @ k[0]) * mx["scale"] * W["l0.mix.temp"][hh]
        assert np.allclose(out[4 * hh:4 * hh + 4], v[0] * math.exp(s) / (1.0 + math.exp(s)))
    assert np.allclose(np.sqrt((v * v).mean()), 1.0, atol=1e-3)


def test_latent_attention_equals_its_absorbed_form():
    """score = (Uk^T q) . c + qr . kr and out = Uv (sum p c): the form an engine with a low-rank cache computes."""
    cfg = make_config([latent(heads=2, dim=6, rot_dim=4, vdim=5, kv_rank=7, q_rank=3, window=4)], width=8)
    W = {k: np.asarray(v, np.float64) for k, v in random_weights(cfg, seed=5).items()}
    mx, eps, p = cfg["layers"][0]["mixer"], cfg["norm"]["eps"], "l0.mix."
    hs = np.random.default_rng(5).standard_normal((9, 8))
    cache = {"c": [], "kr": []}
    for pos, h in enumerate(hs):
        got = plain.latent_token(W, p, mx, eps, h, pos, cache)
        q = (W[p + "uq"] @ plain.norm(W[p + "dq"] @ h, W[p + "dq.norm"], eps)).reshape(2, 10)
        gate = 1.0 / (1.0 + np.exp(-(W[p + "g"] @ h)))
        outs = []
        for hh in range(2):
            Uk, Uv = W[p + "uk"][6 * hh:6 * hh + 6], W[p + "uv"][5 * hh:5 * hh + 5]
            qa, qr = Uk.T @ q[hh, :6], plain.rotate_half(q[hh, 6:], pos, mx["rot"])
            js = range(max(0, pos - 3), pos + 1)
            s = np.array([qa @ cache["c"][j] + qr @ cache["kr"][j] for j in js]) * mx["scale"]
            e = np.exp(s - s.max())
            outs.append(gate[hh] * (Uv @ sum(w * cache["c"][j] for w, j in zip(e / e.sum(), js))))
        assert np.allclose(got, W[p + "o"] @ np.concatenate(outs))


def test_config_reader_takes_every_constant_from_the_configuration():
    from turboinfer_b200 import models, seq
    cfg = make_config([attn(heads=6, kv_heads=3, dim=10, vdim=14, rot_dims=6, base=777.0, factor=3.0, scale=0.21, mlp=dense(72)),
                       latent(heads=5, dim=12, rot_dim=6, vdim=9, kv_rank=33, q_rank=21, window=17, base=1234.0, scale=0.3), attn(factor=None)],
                      vocab=77, width=36, eps=3e-4, taps=5, streams=4, loop=(1, 3, 3))
    m, L = models.zopipel_descs(cfg, seq.F32, 640, 3)
    assert (m.vocab, m.width, m.n_layers, m.max_tokens, m.max_seqs) == (77, 36, 3, 640, 3)
    assert abs(m.norm_eps - 3e-4) < 1e-9 and m.norm_kind == seq.NORM_VECTOR and m.norm_place == seq.NORMS_FRONT
    assert (m.streams, m.loop_start, m.loop_stop, m.loop_times, m.loop_plain, m.tied_head) == (4, 1, 3, 3, 1, 0)
    a = L[0]
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.window) == (seq.MIXER_ATTENTION, 6, 3, 10, 14, 0)
    assert (a.rot_dims, a.rot_half, a.proj_bias, a.v_norm, a.head_temp, a.sink, a.out_gate) == (6, 1, 1, 1, 1, seq.SINK_ZERO, 0)
    assert abs(a.scale - 0.21) < 1e-7 and abs(a.rot_base - 777.0) < 1e-3 and abs(a.rot_linear - 3.0) < 1e-6
    assert (a.conv_taps, a.conv_ff, a.ff_kind, a.ff, a.ff_act) == (5, 1, seq.FF_GLU, 72, seq.ACT_GELU_TANH)
    b = L[1]
    assert (b.mixer, b.heads, b.dim, b.rot_dims, b.vdim, b.kv_rank, b.q_rank, b.window) == (seq.MIXER_LATENT, 5, 12, 6, 9, 33, 21, 17)
    assert (b.out_gate, b.sink, b.rot_half, b.kv_from, b.ff) == (1, seq.SINK_NONE, 1, -1, 0) and abs(b.rot_base - 1234.0) < 1e-3 and b.rot_linear == 0.0
    assert L[2].rot_linear == 0.0
    once, _ = models.zopipel_descs(make_config([attn()], loop=(0, 1, 1)), seq.F32, 64, 1)
    assert once.loop_times == 0
    for bad in ({"type": "wkv"}, {"mlp": {"kind": "moe", "ff": 8}}):
        with pytest.raises(ValueError):
            models.zopipel_descs(make_config([dict(attn(), **bad)]), seq.F32, 64, 1)
    for gone in ("canon", "streams", "norm"):
        with pytest.raises(ValueError):
            models.zopipel_descs({k: v for k, v in cfg.items() if k != gone}, seq.F32, 64, 1)
    assert "Zopipel" in models.REGISTRY


def test_checkpoint_round_trip(tmp_path):
    from turboinfer_b200.safetensors_io import read_safetensors, write_safetensors
    cfg = make_config([attn(mlp=dense(8)), latent()])
    W = random_weights(cfg, seed=4)
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, W)
    back = read_safetensors(path)
    assert set(back) == set(W)
    for k, v in W.items():
        assert np.array_equal(back[k].to_f32(), np.asarray(v, np.float32)), k
