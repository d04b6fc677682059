"""Plain, slow implementation of the Gulazen decoder design (numpy, float64): the oracle of tests/test_gpu_gulazen.py.

One function per mechanism, written from the design's equations; nothing here is shared with the engine.  A model is a
configuration dictionary (the keys of config.json) and a dictionary name -> float array.  A sequence is processed one token
at a time through explicit caches (keys / values of every attention layer, the last inputs of every layer's short
convolution), so the same code answers "what are the logits at position p" whatever the engine's batching was.

  embedding       x = E[token] + s(p), s(p)[2i] = sin(p * 10000^(-2i/width)), s(p)[2i + 1] = cos of the same angle
  layer           x <- x + ls1 * norm1(mixer(c(x))), then x <- x + ls2 * norm2(ff(x)): the norms sit BEHIND the sublayers only
  norm            y = x / sqrt(mean(x^2) + eps) * (1 + w)             (vector gain stored around zero)
  short conv      c(h)_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j), zeros before position 0 (depth-wise, causal)
  attention       q, k, v projections; q and k divided by the RMS over the WHOLE projection (all heads at once) times a plain
                  weight; no rotation; s = cap * tanh(scale * q.k / cap); the heads' scores are mixed, s'_h = sum_g T[h, g] s_g;
                  position i sees j <= i with i - j < window or j < keep_first; softmax whose denominator has one more term
                  exp(sink_h); weighted values; output projection
  dense ff        D act(U h), act(z) = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise
  expert ff       router logits R h + b; the `top` largest are chosen, weights = softmax over the chosen logits; experts are
                  D (silu(G h) * U h); a shared expert of the same form is added for every token
  output          norm, then the logits are the products with the embedding table
"""
from __future__ import annotations

import numpy as np


def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z / (1.0 + np.exp(-z))


def rms_div(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    return rms_div(x, eps) * (1.0 + w)


def position_vector(pos, width):
    """Entry 2i is sin(pos * 10000^(-2i/width)), entry 2i + 1 the cosine of the same angle."""
    out = np.zeros(width)
    for d in range(width):
        i = d // 2
        ang = pos * 10000.0 ** (-2.0 * i / width)
        out[d] = np.sin(ang) if d % 2 == 0 else np.cos(ang)
    return out


def short_conv(history, h, w):
    """history: the taps - 1 inputs before h (oldest first, zeros before the sequence's start); w [width, taps]."""
    taps = w.shape[1]
    rows = list(history) + [h]
    assert len(rows) == taps
    return h + sum(w[:, j] * rows[j] for j in range(taps))


def xielu(z, p, q):
    ap, an = softplus(p), 0.5 + softplus(q)
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, an * (np.exp(zn) - 1.0 - zn) + 0.5 * z)


def visible(i, j, window, keep_first):
    return j <= i and (i - j < window or j < keep_first)


def attention_scores(q, keys, mx):
    """q [H, d]; keys [n, G, d] -> capped scores [H, n] before the heads are mixed."""
    H, G = mx["heads"], mx["kv_heads"]
    K = np.array(keys)                                       # [n, G, d]
    s = np.zeros((H, len(keys)))
    for h in range(H):
        s[h] = (K[:, h // (H // G)] @ q[h]) * mx["scale"]   # query head h reads key/value head floor(h / (H / G))
    cap = mx["softcap"]
    return cap * np.tanh(s / cap)


def attention_token(W, p, mx, eps, h, pos, cache, sees=visible):
    """One token of the attention mixer; cache = {"k": [...], "v": [...]} grows by this token.  `sees` can be replaced by a test
    that wants to know what a wrong mask would give."""
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = rms_div(W[p + "q"] @ h, eps) * W[p + "q.norm"]
    k = rms_div(W[p + "k"] @ h, eps) * W[p + "k.norm"]
    v = W[p + "v"] @ h
    cache["k"].append(k.reshape(G, d))
    cache["v"].append(v.reshape(G, dv))
    s = attention_scores(q.reshape(H, d), cache["k"], mx)
    s = W[p + "talk"] @ s                                   # s'[h, j] = sum_g T[h, g] s[g, j]
    win, keep = mx["mask"]["size"], mx["mask"]["keep_first"]
    seen = [j for j in range(pos + 1) if sees(pos, j, win, keep)]
    out = np.zeros((H, dv))
    for hh in range(H):
        g = hh // (H // G)
        z = np.array([s[hh, j] for j in seen])
        sink = float(W[p + "sink"][hh])
        m = max(z.max(), sink)
        e = np.exp(z - m)
        den = e.sum() + np.exp(sink - m)
        for a, j in zip(e / den, seen):
            out[hh] += a * cache["v"][j][g]
    return W[p + "o"] @ out.reshape(-1)


def dense_ff(W, p, h):
    a = W[p + "act"]
    return W[p + "down"] @ xielu(W[p + "up"] @ h, float(a[0]), float(a[1]))


def gated_expert(W, p, h):
    return W[p + "down"] @ (silu(W[p + "gate"] @ h) * (W[p + "up"] @ h))


def route(z, top):
    """The `top` largest logits (the lower index wins a tie) and the softmax over them."""
    order = sorted(range(len(z)), key=lambda i: (-z[i], i))[:top]
    e = np.exp(np.array([z[i] for i in order]) - max(z[i] for i in order))
    return order, e / e.sum()


def expert_ff(W, p, mlp, h):
    z = W[p + "router"] @ h + W[p + "router.b"]
    picks, weights = route(z, int(mlp["router"]["top"]))
    out = np.zeros_like(h)
    for e, w in zip(picks, weights):
        out += w * gated_expert(W, f"{p}e{e}.", h)
    if mlp.get("shared"):
        out += gated_expert(W, p + "shared.", h)
    return out


class Sequence:
    """Token-by-token evaluation of one sequence."""

    def __init__(self, cfg, weights, sees=visible):
        self.cfg = cfg
        self.sees = sees
        self.W = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
        self.pos = 0
        self.kv = [{"k": [], "v": []} for _ in cfg["layers"]]
        taps = int(cfg["canon"]["taps"])
        self.hist = [[np.zeros(cfg["width"]) for _ in range(taps - 1)] for _ in cfg["layers"]]
        self.layers_out = []

    def feed(self, token):
        cfg, W = self.cfg, self.W
        eps = float(cfg["norm"]["eps"])
        x = W["embed"][token] + position_vector(self.pos, cfg["width"])
        after = []
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = short_conv(self.hist[i], x, W[p + "canon1"])
            self.hist[i] = (self.hist[i] + [x.copy()])[1:]
            if L["type"] != "attention":
                raise ValueError(L["type"])
            y = attention_token(W, p + "mix.", L["mixer"], eps, h, self.pos, self.kv[i], self.sees)
            x = x + W[p + "ls1"] * norm_one_plus(y, W[p + "norm1"], eps)
            mlp = L.get("mlp")
            if mlp:
                y = dense_ff(W, p + "mlp.", x) if mlp["kind"] == "dense" else expert_ff(W, p + "mlp.", mlp, x)
                x = x + W[p + "ls2"] * norm_one_plus(y, W[p + "norm2"], eps)
            after.append(x.copy())
        self.layers_out.append(after)
        self.pos += 1
        return W["embed"] @ norm_one_plus(x, W["final.norm"], eps)


def run(cfg, weights, tokens, sees=visible):
    """logits [len(tokens), vocab] and the residual stream after every layer [layers, tokens, width]."""
    s = Sequence(cfg, weights, sees)
    logits = np.stack([s.feed(int(t)) for t in tokens])
    layers = np.transpose(np.array(s.layers_out), (1, 0, 2))
    return logits, layers
