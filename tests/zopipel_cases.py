"""Small Zopipel configurations with random weights for the tests, and helpers that run them through the engine.

Weights are rounded to bfloat16-representable values, so the bf16 and the fp32 engine and the plain implementation all see
exactly the same numbers."""
from __future__ import annotations

import math

import numpy as np

from binusun_cases import rel_err, run_schedule, to_bf16_values  # noqa: F401  (re-exported for the tests)
from tudasun_cases import row_errs  # noqa: F401


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def attn(heads=4, kv_heads=2, dim=12, vdim=20, rot_dims=8, base=10000.0, factor=2.0, scale=None, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot,
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}}


def latent(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, q_rank=10, window=24, base=50000.0, scale=None, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "mask": {"size": window}, "rot": {"base": base, "dims": rot_dim},
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}}


def make_config(layers, vocab=131, width=48, eps=1e-5, taps=3, streams=2, loop=None):
    cfg = {"architecture": "Zopipel", "canon": {"taps": taps}, "layers": layers, "norm": {"eps": eps}, "streams": streams, "vocab": vocab,
           "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0, canon_amp=0.3, mix_noise=0.3):
    """canon_amp: size of the convolution weights; mix_noise: size of the off-identity part of the stream mixing matrices."""
    rng = np.random.default_rng(seed)
    D, V, taps, S = cfg["width"], cfg["vocab"], cfg["canon"]["taps"], cfg["streams"]
    W = {}

    def mat(o, i, amp=1.0):
        return to_bf16_values(rng.standard_normal((o, i)).astype(np.float32) * (amp / math.sqrt(i)))

    def vec(n, lo, hi):
        return to_bf16_values(rng.uniform(lo, hi, n).astype(np.float32))

    def noise(shape, amp):
        return to_bf16_values((rng.standard_normal(shape) * amp).astype(np.float32))

    W["embed"] = to_bf16_values(rng.standard_normal((V, D)).astype(np.float32))
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        mx = L["mixer"]
        H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
        for q in ("1", "2") if L.get("mlp") else ("1",):
            W[p + "norm" + q] = vec(D, 0.5, 1.5)
            W[p + "canon" + q] = noise((D, taps), canon_amp)
            W[p + f"hc{q}.in"] = vec(S, 0.3, 1.0)
            W[p + f"hc{q}.out"] = vec(S, 0.5, 1.2) * to_bf16_values(rng.choice([-1.0, 1.0], S).astype(np.float32))
            W[p + f"hc{q}.mix"] = to_bf16_values((np.eye(S) + mix_noise * rng.standard_normal((S, S))).astype(np.float32))
        if L["type"] == "attention":
            G = mx["kv_heads"]
            W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * d, D), mat(G * d, D), mat(G * dv, D)
            W[p + "mix.q.b"], W[p + "mix.k.b"], W[p + "mix.v.b"] = noise(H * d, 0.3), noise(G * d, 0.3), noise(G * dv, 0.3)
            W[p + "mix.temp"] = vec(H, 0.5, 2.0)
            W[p + "mix.o"], W[p + "mix.o.b"] = mat(D, H * dv), noise(D, 0.3)
        else:
            dr, rank, qr = mx["rot_dim"], mx["kv_rank"], mx["q_rank"]
            W[p + "mix.dq"], W[p + "mix.dq.norm"], W[p + "mix.uq"] = mat(qr, D), vec(qr, 0.5, 1.5), mat(H * (d + dr), qr)
            W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = mat(rank + dr, D), vec(rank, 0.5, 1.5)
            W[p + "mix.uk"], W[p + "mix.uv"] = mat(H * d, rank), mat(H * dv, rank)
            W[p + "mix.g"], W[p + "mix.o"] = mat(H, D, 2.0), mat(D, H * dv)
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"] = mat(F, D, 1.5), mat(F, D), mat(D, F)
    W["final.norm"] = vec(D, 0.5, 1.5)
    W["head"] = mat(V, D)
    return W


def build_engine(cfg, W, dtype="float32", max_tokens=1024, max_seqs=4):
    from turboinfer_b200 import models
    return models.REGISTRY["Zopipel"](cfg, W, dtype, max_tokens, max_seqs)


def plant_pair(cfg, W, a, b, gain=12.0):
    """Makes token `a` (as a key) and token `b` (as a query) stand out against each other in head 0 of layer 0, whatever their
    positions: both get a large embedding along one coordinate of their own that no other token uses; the convolution passes these
    two coordinates unchanged; the query of head 0 reads b's coordinate and the key of its key/value head reads a's coordinate with
    the same vector r, placed on coordinates that are NOT rotated (attention: the ones behind rot.dims; latent attention: the plain
    part of the head, reached through entry 0 of the two low-rank vectors; the head's output gate is opened for b)."""
    W = {k: np.array(v, np.float32, copy=True) for k, v in W.items()}
    L = cfg["layers"][0]
    mx = L["mixer"]
    d = mx["dim"]
    rng = np.random.default_rng(99)
    u, v = 0, 1   # the coordinates the two tokens own
    E = W["embed"]
    E[:, u] = 0.0
    E[:, v] = 0.0
    E[b] = 0.0
    E[a] = 0.0
    E[b, u] = gain
    E[a, v] = gain
    W["l0.norm1"][[u, v]] = 1.0
    W["l0.canon1"][[u, v]] = 0.0
    if L["type"] == "attention":
        rd = mx["rot"]["dims"]
        assert rd < d, "the planted direction lives on the coordinates that do not turn"
        r = np.zeros(d, np.float32)
        r[rd:] = rng.standard_normal(d - rd) * 1.5
        W["l0.mix.q"][:, [u, v]] = 0.0
        W["l0.mix.k"][:, [u, v]] = 0.0
        W["l0.mix.q"][:d, u] = r
        W["l0.mix.k"][:d, v] = r
        W["l0.mix.temp"][0] = 1.0
    else:
        r = rng.standard_normal(d).astype(np.float32)
        for nm, c in (("l0.mix.dq", u), ("l0.mix.dkv", v)):
            W[nm][:, [u, v]] = 0.0
            W[nm][0, c] = 4.0
        W["l0.mix.dq.norm"][0] = 1.0
        W["l0.mix.dkv.norm"][0] = 1.0
        W["l0.mix.uq"][:d, 0] = r
        W["l0.mix.uk"][:d, 0] = r
        W["l0.mix.g"][0, u] = 0.5   # head 0's gate is open at b
    return {k: to_bf16_values(x) for k, x in W.items()}
