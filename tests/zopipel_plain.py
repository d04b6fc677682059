"""Plain, slow implementation of the Zopipel decoder design (numpy, float64): the oracle of tests/test_gpu_zopipel.py.

One function per mechanism, written from the design's equations; nothing here is shared with the engine.  A model is a
configuration dictionary (the keys of config.json) and a dictionary name -> float array.  A sequence is processed one token
at a time through explicit caches (per layer RUN: keys / values or latent rows, and the last inputs of both sublayers' short
convolutions), so the same code answers "what are the logits at position p" whatever the engine's batching was.

  streams         n copies X[0 .. n) of the embedding output; sublayer q of a layer reads u = sum_s in_q[s] X[s] and writes
                  X'[t] = sum_s mix_q[s, t] X[s] + out_q[t] y for all t at once; the model's output is sum_s X[s]
  sublayer input  h = norm(u) = u / sqrt(mean(u^2) + eps) * w, then c(h)_t = h_t + sum_j k[:, j] h_(t - taps + 1 + j) (causal,
                  depth-wise, zeros before position 0) in front of the mixer AND in front of the feed-forward
  rotation        coordinate i of the first `dims` of a head pairs with i + dims / 2: (a, b) -> (a cos - b sin, b cos + a sin),
                  angle = pos * base^(-2i / dims) / factor
  attention       biased q, k, v; rotation of q and k; every value head divided by its RMS (cached so); score = q.k * scale *
                  temp[head]; all earlier positions; p_j = exp(s_j) / (1 + sum exp(s)); biased output projection
  latent          cq = norm(Dq h), q = Uq cq (per head: `dim` plain coordinates, then `rot_dim` rotated ones); Dkv h = [c | kr]:
                  c is normed, kr is rotated and shared by the heads; k_h = Uk_h c, v_h = Uv_h c; score = (q.k + qr.kr) * scale;
                  position i sees j with 0 <= i - j < window; softmax; head output times sigmoid(G h)[head]; output projection
  feed-forward    D (gelu_tanh(G h) * U h)
  loop            layers [start, stop) run `times` times in a row, each pass with caches of its own
  output          norm of the summed streams, then the head matrix
"""
from __future__ import annotations

import math

import numpy as np


def rms_div(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm(x, w, eps):
    return rms_div(x, eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def short_conv(history, h, w):
    """history: the taps - 1 inputs before h (oldest first, zeros before the sequence's start); w [width, taps]."""
    rows = list(history) + [h]
    assert len(rows) == w.shape[1]
    return h + sum(w[:, j] * rows[j] for j in range(w.shape[1]))


def rotate_half(v, pos, rot):
    """v [..., n]: the first rot['dims'] coordinates turn, coordinate i together with i + dims / 2."""
    dims = int(rot["dims"])
    half = dims // 2
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    out = np.array(v, dtype=np.float64, copy=True)
    for i in range(half):
        ang = pos * (float(rot["base"]) ** (-2.0 * i / dims) / factor)
        a, b = v[..., i], v[..., i + half]
        out[..., i] = a * math.cos(ang) - b * math.sin(ang)
        out[..., i + half] = b * math.cos(ang) + a * math.sin(ang)
    return out


def streams_read(X, w_in):
    return sum(w_in[s] * X[s] for s in range(len(X)))


def streams_write(X, mix, w_out, y):
    n = len(X)
    return [sum(mix[s, t] * X[s] for s in range(n)) + w_out[t] * y for t in range(n)]


def sees_all(i, j, window):
    return j <= i


def sees_window(i, j, window):
    return 0 <= i - j < window


def attention_token(W, p, mx, eps, h, pos, cache, sees=sees_all):
    """Grouped attention with a zero-score sink; cache = {"k": [...], "v": [...]} grows by this token."""
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (W[p + "q"] @ h + W[p + "q.b"]).reshape(H, d)
    k = (W[p + "k"] @ h + W[p + "k.b"]).reshape(G, d)
    v = (W[p + "v"] @ h + W[p + "v.b"]).reshape(G, dv)
    q, k = rotate_half(q, pos, mx["rot"]), rotate_half(k, pos, mx["rot"])
    cache["k"].append(k)
    cache["v"].append(rms_div(v, eps))
    seen = [j for j in range(pos + 1) if sees(pos, j, 0)]
    out = np.zeros((H, dv))
    for hh in range(H):
        g = hh // (H // G)
        s = np.array([cache["k"][j][g] @ q[hh] for j in seen]) * float(mx["scale"]) * float(W[p + "temp"][hh])
        m = max(s.max(), 0.0)
        e = np.exp(s - m)
        den = e.sum() + math.exp(-m)          # the sink: one more term exp(0) that has no value
        for a, j in zip(e / den, seen):
            out[hh] += a * cache["v"][j][g]
    return W[p + "o"] @ out.reshape(-1) + W[p + "o.b"]


def latent_token(W, p, mx, eps, h, pos, cache, sees=sees_window):
    """Latent attention in its direct form (per-head keys and values rebuilt from the cached rows)."""
    H, d, dr, dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    cq = norm(W[p + "dq"] @ h, W[p + "dq.norm"], eps)
    q = (W[p + "uq"] @ cq).reshape(H, d + dr)
    qn, qr = q[:, :d], rotate_half(q[:, d:], pos, mx["rot"])
    kv = W[p + "dkv"] @ h
    cache["c"].append(norm(kv[:rank], W[p + "dkv.norm"], eps))
    cache["kr"].append(rotate_half(kv[rank:], pos, mx["rot"]))
    win = int(mx["mask"]["size"])
    seen = [j for j in range(pos + 1) if sees(pos, j, win)]
    Uk, Uv = W[p + "uk"].reshape(H, d, rank), W[p + "uv"].reshape(H, dv, rank)
    gate = sigmoid(W[p + "g"] @ h)
    out = np.zeros((H, dv))
    for hh in range(H):
        s = np.array([(Uk[hh] @ cache["c"][j]) @ qn[hh] + cache["kr"][j] @ qr[hh] for j in seen]) * float(mx["scale"])
        e = np.exp(s - s.max())
        for a, j in zip(e / e.sum(), seen):
            out[hh] += a * (Uv[hh] @ cache["c"][j])
        out[hh] *= gate[hh]
    return W[p + "o"] @ out.reshape(-1)


def feed_forward(W, p, h):
    return W[p + "down"] @ (gelu_tanh(W[p + "gate"] @ h) * (W[p + "up"] @ h))


def layer_runs(cfg):
    """The order in which layers run: a looped block is repeated as a whole."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    a, b, times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


class Sequence:
    """Token-by-token evaluation of one sequence.  `sees` maps a mixer type to a visibility function (tests bend it to learn what a
    wrong mask would give)."""

    def __init__(self, cfg, weights, sees=None):
        self.cfg = cfg
        self.W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.sees = {"attention": sees_all, "latent_attention": sees_window}
        self.sees.update(sees or {})
        self.pos = 0
        self.runs = layer_runs(cfg)
        taps = int(cfg["canon"]["taps"])
        D = cfg["width"]
        self.cache = [{"k": [], "v": [], "c": [], "kr": []} for _ in self.runs]
        self.hist = [[[np.zeros(D) for _ in range(taps - 1)] for _ in range(2)] for _ in self.runs]
        self.layers_out = []

    def feed(self, token):
        cfg, W = self.cfg, self.W
        eps = float(cfg["norm"]["eps"])
        X = [W["embed"][token].copy() for _ in range(int(cfg["streams"]))]
        after = []
        for r, i in enumerate(self.runs):
            L, p = cfg["layers"][i], f"l{i}."
            h = norm(streams_read(X, W[p + "hc1.in"]), W[p + "norm1"], eps)
            hc = short_conv(self.hist[r][0], h, W[p + "canon1"])
            self.hist[r][0] = (self.hist[r][0] + [h])[1:]
            if L["type"] == "attention":
                y = attention_token(W, p + "mix.", L["mixer"], eps, hc, self.pos, self.cache[r], self.sees["attention"])
            elif L["type"] == "latent_attention":
                y = latent_token(W, p + "mix.", L["mixer"], eps, hc, self.pos, self.cache[r], self.sees["latent_attention"])
            else:
                raise ValueError(L["type"])
            X = streams_write(X, W[p + "hc1.mix"], W[p + "hc1.out"], y)
            if L.get("mlp"):
                h = norm(streams_read(X, W[p + "hc2.in"]), W[p + "norm2"], eps)
                hc = short_conv(self.hist[r][1], h, W[p + "canon2"])
                self.hist[r][1] = (self.hist[r][1] + [h])[1:]
                X = streams_write(X, W[p + "hc2.mix"], W[p + "hc2.out"], feed_forward(W, p + "mlp.", hc))
            after.append(sum(X))
        self.layers_out.append(after)
        self.pos += 1
        return W["head"] @ norm(sum(X), W["final.norm"], eps)


def run(cfg, weights, tokens, sees=None):
    """logits [len(tokens), vocab] and the summed streams after every layer run [runs, tokens, width]."""
    s = Sequence(cfg, weights, sees)
    logits = np.stack([s.feed(int(t)) for t in tokens])
    layers = np.transpose(np.array(s.layers_out), (1, 0, 2))
    return logits, layers
