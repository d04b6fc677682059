"""Small Gulazen configurations with random weights for the tests, and helpers that run them through the engine.

Weights are rounded to bfloat16-representable values, so the bf16 and the fp32 engine and the plain implementation all see
exactly the same numbers."""
from __future__ import annotations

import math

import numpy as np

from binusun_cases import rel_err, run_schedule, to_bf16_values  # noqa: F401  (re-exported for the tests)
from tudasun_cases import row_errs  # noqa: F401


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=5, top=2, ff=16, shared=24):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(heads=4, kv_heads=2, dim=12, vdim=20, window=24, keep=3, scale=None, softcap=30.0, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window, "keep_first": keep},
                      "scale": scale if scale is not None else 1.0 / math.sqrt(dim), "softcap": softcap}}


def make_config(layers, vocab=131, width=48, eps=1e-5, taps=3):
    return {"architecture": "Gulazen", "canon": {"taps": taps}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def random_weights(cfg, seed=0, decisive=False, sink=None, talk_noise=0.4):
    """decisive: the router's biases are four apart, so the choice of experts does not depend on the token (the weights still do)
    and a rounding difference in front of the router cannot flip it -- for comparisons in bf16 mode; sink: a fixed value for every
    head's sink (default: random); talk_noise: size of the off-diagonal part of the head-mixing matrices."""
    rng = np.random.default_rng(seed)
    D, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]
    W = {}

    def mat(o, i, amp=1.0):
        return to_bf16_values(rng.standard_normal((o, i)).astype(np.float32) * (amp / math.sqrt(i)))

    def vec(n, lo, hi):
        return to_bf16_values(rng.uniform(lo, hi, n).astype(np.float32))

    def around_zero(n):
        return to_bf16_values((rng.standard_normal(n) * 0.2).astype(np.float32))

    W["embed"] = to_bf16_values(rng.standard_normal((V, D)).astype(np.float32))
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        mx = L["mixer"]
        H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        W[p + "norm1"], W[p + "ls1"] = around_zero(D), vec(D, 0.3, 1.0)
        W[p + "canon1"] = to_bf16_values((rng.standard_normal((D, taps)) * 0.3).astype(np.float32))
        W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.v"] = mat(H * d, D), mat(G * d, D), mat(G * dv, D)
        W[p + "mix.q.norm"], W[p + "mix.k.norm"] = vec(H * d, 0.5, 1.5), vec(G * d, 0.5, 1.5)
        W[p + "mix.talk"] = to_bf16_values((np.eye(H) + talk_noise * rng.standard_normal((H, H))).astype(np.float32))
        W[p + "mix.sink"] = to_bf16_values(np.full(H, sink, np.float32)) if sink is not None else to_bf16_values(rng.standard_normal(H).astype(np.float32))
        W[p + "mix.o"] = mat(D, H * dv)
        mlp = L.get("mlp")
        if mlp:
            W[p + "norm2"], W[p + "ls2"] = around_zero(D), vec(D, 0.3, 1.0)
            if mlp["kind"] == "dense":
                W[p + "mlp.up"], W[p + "mlp.down"] = mat(mlp["ff"], D, 2.0), mat(D, mlp["ff"])
                W[p + "mlp.act"] = vec(2, -1.0, 1.0)
            else:
                r, F = mlp["router"], mlp["expert"]["ff"]
                n = r["experts"]
                for e in range(n):
                    q = p + "mlp.e%d." % e
                    W[q + "gate"], W[q + "up"], W[q + "down"] = mat(F, D, 1.5), mat(F, D, 1.5), mat(D, F, 1.5)
                W[p + "mlp.router"] = mat(n, D, 3.0)
                W[p + "mlp.router.b"] = to_bf16_values(rng.permutation(n).astype(np.float32) * 4.0) if decisive else vec(n, -0.5, 0.5)
                if mlp.get("shared"):
                    Fs = mlp["shared"]["ff"]
                    W[p + "mlp.shared.gate"], W[p + "mlp.shared.up"], W[p + "mlp.shared.down"] = mat(Fs, D), mat(Fs, D), mat(D, Fs)
    W["final.norm"] = around_zero(D)
    return W


def build_engine(cfg, W, dtype="float32", max_tokens=1024, max_seqs=4):
    from turboinfer_b200 import models
    return models.REGISTRY["Gulazen"](cfg, W, dtype, max_tokens, max_seqs)


def plant_pair(cfg, W, a, b, gain=12.0):
    """Makes token `a` (as a key) and token `b` (as a query) stand out against each other in head 0 of layer 0: both get a large
    embedding along one coordinate of their own, and the query rows of head 0 and the key rows of its key/value head read those
    coordinates with the same vector, so that q_0(b) and k_0(a) point the same way whatever the positions and neighbours add."""
    W = dict(W)
    mx = cfg["layers"][0]["mixer"]
    d, D = mx["dim"], cfg["width"]
    rng = np.random.default_rng(99)
    r = rng.standard_normal(d).astype(np.float32)
    E = np.array(W["embed"], np.float32, copy=True)
    u, v = 0, 1   # the coordinates the two tokens own
    E[:, u] = 0.0
    E[:, v] = 0.0
    E[b] = 0.0
    E[a] = 0.0
    E[b, u] = gain
    E[a, v] = gain
    Wq, Wk = np.array(W["l0.mix.q"], np.float32, copy=True), np.array(W["l0.mix.k"], np.float32, copy=True)
    Wq[:d, u] = r
    Wk[:d, v] = r
    qn, kn = np.array(W["l0.mix.q.norm"], np.float32, copy=True), np.array(W["l0.mix.k.norm"], np.float32, copy=True)
    qn[:d], kn[:d] = 1.0, 1.0
    W["embed"], W["l0.mix.q"], W["l0.mix.k"] = to_bf16_values(E), to_bf16_values(Wq), to_bf16_values(Wk)
    W["l0.mix.q.norm"], W["l0.mix.k.norm"] = to_bf16_values(qn), to_bf16_values(kn)
    return W
