"""Throughput of a Binusun-style model on the layered sequence engine next to the library's closest existing model (the
INT4 Llama-style decoder of the persistent decode kernel) at equal width, depth and feed-forward size; random weights.

Used by `bench.py --arch-compare SIZE`.  Prompt throughput: one request's whole prompt in one step.  Decode throughput: single
tokens of B live sequences per step.  Times are CUDA-event times of the device work (L2 flushed between timed prompt steps; a
decode step streams more weight bytes than L2 holds at the larger sizes) and wall-clock times around the public call."""
from __future__ import annotations

import math
import statistics
import time

import numpy as np

from . import models, seq

SIZES = {
    # width, query heads x head size, kv heads, feed-forward, window; recurrence heads x size, decay rank
    "w1024": dict(width=1024, heads=8, kv_heads=2, dim=128, ff=2816, window=512, wkv_heads=16, wkv_dim=64, rank=32, vocab=32000),
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=5632, window=1024, wkv_heads=32, wkv_dim=64, rank=64, vocab=32000),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=11008, window=1024, wkv_heads=64, wkv_dim=64, rank=64, vocab=32000),
}


def config_for(size: str) -> dict:
    z = SIZES[size]
    attn = {"type": "attention", "mlp": {"kind": "dense", "ff": z["ff"]},
            "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "mask": {"size": z["window"]},
                      "rot": {"base": 10000.0, "dims": z["dim"] // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
                      "scale": 1.0 / math.sqrt(z["dim"])}}
    wkv = {"type": "wkv", "mlp": None, "mixer": {"heads": z["wkv_heads"], "dim": z["wkv_dim"]}}
    # wkv, attention, attention looped twice, then a closing wkv: 7 layer runs (4 attention + feed-forward, 3 recurrent)
    return {"architecture": "Binusun", "layers": [wkv, attn, attn, wkv], "loop": {"start": 0, "stop": 3, "times": 2}, "norm": {"eps": 1e-5},
            "logit_scale": 1.0, "vocab": z["vocab"], "width": z["width"]}


def tudasun_config_for(size: str) -> dict:
    """Seven layers in the order gla, latent attention, gla, hgrn2, latent attention on the second layer's cache, gla, hgrn2; dense
    feed-forwards at both ends, routed experts (8 of a quarter of the dense inner size, 2 identity experts, 2 chosen from the best of
    2 groups, a shared expert of half the dense size) in between.  The low-rank cache row is 256 + 64 wide."""
    z = SIZES[size]
    D, ff = z["width"], z["ff"]
    H = z["heads"]
    gla = {"type": "gla", "mixer": {"heads": H, "dim": 64, "vdim": 128, "tau": 16.0}}
    hg = {"type": "hgrn2", "mixer": {"heads": H, "dim": 128, "vdim": 128}}
    lat = {"type": "latent_attention", "mixer": {"heads": H, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 256, "rot": {"base": 10000.0, "dims": 64},
                                                 "scale": 1.0 / math.sqrt(192.0)}}
    lat2 = {"type": "latent_attention", "mixer": dict(lat["mixer"], kv_from=1)}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "expert": {"ff": ff // 4}, "router": {"experts": 8, "identity": 2, "top": 2, "groups": {"count": 2, "keep": 1}}, "shared": {"ff": ff // 2}}
    order = [(gla, dense), (lat, moe), (gla, moe), (hg, moe), (lat2, moe), (gla, dense), (hg, dense)]
    return {"architecture": "Tudasun", "layers": [dict(a, mlp=b) for a, b in order], "norm": {"eps": 1e-5}, "logit_softcap": 30.0,
            "token_side": {"dim": 64}, "vocab": z["vocab"], "width": D}


def gulazen_config_for(size: str) -> dict:
    """Seven attention layers behind a three-tap convolution: the size's heads and window with 8 kept first keys, capped and mixed
    scores; dense xIELU feed-forwards in layers 0, 2, 4, 6 and routed experts (8 of a quarter of the dense inner size, 2 chosen by
    logits, a shared expert of half the dense size) in layers 1, 3, 5."""
    z = SIZES[size]
    mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "mask": {"size": z["window"], "keep_first": 8},
             "scale": 1.0 / math.sqrt(z["dim"]), "softcap": 30.0}
    dense = {"kind": "dense", "ff": z["ff"]}
    moe = {"kind": "moe", "expert": {"ff": z["ff"] // 4}, "router": {"experts": 8, "top": 2}, "shared": {"ff": z["ff"] // 2}}
    return {"architecture": "Gulazen", "canon": {"taps": 3}, "layers": [{"type": "attention", "mixer": mixer, "mlp": dense if i % 2 == 0 else moe} for i in range(7)],
            "norm": {"eps": 1e-5}, "vocab": z["vocab"], "width": z["width"]}


def binusun_attention_config_for(size: str) -> dict:
    """The closest existing model to a Gulazen one: seven Binusun attention layers (same heads, window and feed-forward size, rotary,
    per-head unit norm, output gate, gated relu feed-forward), no recurrent layers, no looped block."""
    cfg = config_for(size)
    return {"architecture": "Binusun", "layers": [cfg["layers"][1]] * 7, "norm": cfg["norm"], "logit_scale": 1.0, "vocab": cfg["vocab"], "width": cfg["width"]}


def zopipel_config_for(size: str) -> dict:
    """Five layers, attention / latent attention in turn, the middle two run twice: 7 layer runs (4 attention, 3 latent attention), all
    with a gated gelu feed-forward of the size's inner width behind a four-tap convolution, four residual streams.  Attention: the
    size's heads over all earlier tokens, every coordinate turning; latent attention: a cached row of 256 + 64, queries through a
    vector of 3/8 of the width, the size's window."""
    z = SIZES[size]
    mlp = {"kind": "dense", "ff": z["ff"]}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"],
                     "rot": {"base": 10000.0, "dims": z["dim"], "scaling": {"factor": 2.0}}, "scale": 1.0 / math.sqrt(z["dim"])}}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 256, "q_rank": 3 * z["width"] // 8, "mask": {"size": z["window"]},
                     "rot": {"base": 500000.0, "dims": 64}, "scale": 1.0 / math.sqrt(192.0)}}
    return {"architecture": "Zopipel", "canon": {"taps": 4}, "layers": [att, lat, att, lat, att], "loop": {"start": 1, "stop": 3, "times": 2},
            "norm": {"eps": 1e-6}, "streams": 4, "vocab": z["vocab"], "width": z["width"]}


def build_synthetic(cfg: dict, rank: int, dtype: str, max_tokens: int, max_seqs: int) -> seq.SeqModel:
    mode = {"bfloat16": seq.BF16, "float32": seq.F32}[dtype]
    if cfg["architecture"] == "Gulazen":
        desc, layers = models.gulazen_descs(cfg, mode, max_tokens, max_seqs)
    elif cfg["architecture"] == "Zopipel":
        desc, layers = models.zopipel_descs(cfg, mode, max_tokens, max_seqs)
    elif cfg["architecture"] == "Tudasun":
        shapes = {f"l{i}.mix.a1": (rank, cfg["width"]) for i, L in enumerate(cfg["layers"]) if L["type"] == "gla"}
        shapes.update({f"l{i}.rg1": (cfg["width"], cfg["width"]) for i in range(len(cfg["layers"]))})
        desc, layers = models.tudasun_descs(cfg, mode, max_tokens, max_seqs, shapes)
    else:
        shapes = {f"l{i}.mix.w1": (rank, cfg["width"]) for i, L in enumerate(cfg["layers"]) if L["type"] == "wkv"}
        desc, layers = models.binusun_descs(cfg, mode, max_tokens, max_seqs, shapes)
    m = seq.SeqModel(desc, layers)
    for k, (name, shape) in enumerate(m.tensor_specs()):
        leaf = name.split(".")[-1]
        if cfg["architecture"] in ("Tudasun", "Gulazen") and (leaf in ("norm1", "norm1b", "norm2", "norm2b", "b", "correction") or name == "final.norm"):
            amp, off = 0.1, (1.0 if name.endswith("a2.b") else 0.0)   # gains stored around zero, biases, router corrections
        elif cfg["architecture"] == "Zopipel" and (leaf in ("norm1", "norm2", "temp") or name == "final.norm" or name.endswith(("dq.norm", "dkv.norm"))):
            amp, off = 0.25, 1.0   # plain gains and per-head score factors around one
        elif cfg["architecture"] == "Zopipel" and leaf == "b":
            amp, off = 0.1, 0.0
        elif leaf in ("in", "out") and ".hc" in name:
            amp, off = 0.2, 0.6
        elif leaf == "mix" and ".hc" in name:
            amp, off = 0.15, 1.0 / shape[-1]
        elif leaf == "canon2":
            amp, off = 0.2, 0.0
        elif leaf in ("ls1", "ls2"):
            amp, off = 0.25, 0.5
        elif leaf == "canon1":
            amp, off = 0.2, 0.0
        elif leaf == "talk":
            amp, off = 0.5 / math.sqrt(shape[-1]), 1.0 / shape[-1]
        elif leaf == "lower":
            amp, off = 0.45, 0.45
        elif leaf in ("sink", "act"):
            amp, off = 1.0, 0.0
        elif name == "side.embed":
            amp, off = 1.0, 0.0
        elif len(shape) == 0:
            amp, off = 0.25, 1.0
        elif ".mu." in name:
            amp, off = 0.5, 0.5
        elif leaf == "w0":
            amp, off = 1.0, -1.0
        elif leaf == "norm":
            amp, off = 0.5, 1.0
        elif leaf == "u":
            amp, off = 1.0, 0.0
        elif name == "embed":
            amp, off = 1.0, 0.0
        else:
            amp, off = math.sqrt(3.0 / shape[-1]), 0.0
        m.set_tensor_synthetic(name, shape, 1000 + k, amp, off)
    return m.finalize()


def prompt(n: int, vocab: int, offset: int = 0):
    return [int((7919 * i + 1 + offset) % vocab) for i in range(n)]


def measure_seq(size: str, dtype: str, n_prompt: int, n_new: int, batch: int, steps: int, warmup: int, design: str = "Binusun") -> dict:
    cfg = {"Tudasun": tudasun_config_for, "Gulazen": gulazen_config_for, "BinusunAttention": binusun_attention_config_for,
           "Zopipel": zopipel_config_for}.get(design, config_for)(size)
    m = build_synthetic(cfg, SIZES[size]["rank"], dtype, max_tokens=(n_prompt + n_new + 64) * max(batch, 1) + 64, max_seqs=max(batch, 1))
    V = cfg["vocab"]
    launches0 = seq.launch_count()
    # prompt: whole prompt in one step, first token sampled on the device
    pre_dev, pre_wall = [], []
    for it in range(warmup + steps):
        s = m.open()
        seq.flush_l2()
        t0 = time.perf_counter()
        m.step_sample([(s, prompt(n_prompt, V))])
        if it >= warmup:
            pre_wall.append(time.perf_counter() - t0)
            pre_dev.append(m.last_step_ms())
        m.close(s)
    # decode: `batch` live sequences, one token each per step
    ss = [m.open() for _ in range(batch)]
    toks, _ = m.step_sample([(s, prompt(64, V, b)) for b, s in enumerate(ss)])
    dec_dev, dec_wall = [], []
    for it in range(warmup + n_new):
        t0 = time.perf_counter()
        toks, _ = m.step_sample([(s, [int(toks[b])]) for b, s in enumerate(ss)])
        if it >= warmup:
            dec_wall.append(time.perf_counter() - t0)
            dec_dev.append(m.last_step_ms())
    by = m.bytes()
    for s in ss:
        m.close(s)
    launches = seq.launch_count() - launches0
    m.free()
    pre_ms, dec_ms = statistics.median(pre_dev), statistics.median(dec_dev)
    # routed experts: a decode step reads only the experts its rows chose; with one row that is at most `top` of them a layer
    idle = sum((L["mlp"]["router"]["experts"] - min(L["mlp"]["router"]["top"], L["mlp"]["router"]["experts"])) * 3.0 * L["mlp"]["expert"]["ff"] * cfg["width"] * 2.0
               for L in cfg["layers"] if L.get("mlp") and L["mlp"].get("kind") == "moe")
    extra = {}
    if idle and batch == 1:
        extra = {"weight_bytes_one_row": by["weights"] - idle, "decode_weight_GBps_one_row": (by["weights"] - idle) / (dec_ms * 1e-3) / 1e9}
    return {**extra, "prefill_tokens_per_s": n_prompt / (pre_ms * 1e-3), "prefill_ms": pre_ms, "prefill_e2e_tokens_per_s": n_prompt / statistics.median(pre_wall),
            "decode_tokens_per_s": batch / (dec_ms * 1e-3), "decode_ms_per_step": dec_ms,
            "decode_e2e_tokens_per_s": batch / statistics.median(dec_wall), "batch": batch, "weight_bytes": by["weights"],
            "decode_weight_GBps": by["weights"] / (dec_ms * 1e-3) / 1e9, "gpu_launches": launches}


def measure_llama(size: str, n_prompt: int, n_new: int, steps: int, warmup: int) -> dict:
    from . import capi
    z = SIZES[size]
    capi.init(0)
    meta = dict(vocab=z["vocab"], hidden=z["width"], layers=7, heads=z["heads"], inter=z["ff"])
    m = capi.Model(meta, capi.Q_INT4, attn_mode=1, rope_mode=1, max_seq=n_prompt + n_new + 64)
    m.load_synthetic()
    pr = prompt(n_prompt, z["vocab"])
    pre, dec, wall = [], [], []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        _, _, ms = m.generate_greedy(pr, n_new)
        if it >= warmup:
            wall.append(time.perf_counter() - t0)
            dec.append(ms)
            pre.append(m.last_prefill_ms())
    wb, _ = m.step_bytes(n_prompt)
    m.free()
    pre_ms, dec_ms = statistics.median(pre), statistics.median(dec) / max(1, n_new - 1)
    return {"prefill_tokens_per_s": n_prompt / (pre_ms * 1e-3), "prefill_ms": pre_ms, "decode_tokens_per_s": 1.0 / (dec_ms * 1e-3),
            "decode_ms_per_step": dec_ms, "weight_bytes": wb, "decode_weight_GBps": wb / (dec_ms * 1e-3) / 1e9,
            "e2e_s_per_generation": statistics.median(wall), "weights": "int4", "layers": 7}


def compare_tudasun(size: str, steps: int, warmup: int, n_prompt: int = 2048, n_new: int = 64) -> dict:
    """Tudasun next to the closest model of the library, the Binusun hybrid on the same engine (bf16 weights, 7 layer runs each)."""
    out = {"size": size, "shape": SIZES[size], "prompt_tokens": n_prompt, "decode_steps": n_new}
    for design in ("Tudasun", "Binusun"):
        key = design.lower() + "_bf16"
        out[key] = measure_seq(size, "bfloat16", n_prompt, n_new, 1, steps, warmup, design)
        out[key + "_batch4"] = {k: v for k, v in measure_seq(size, "bfloat16", 256, n_new, 4, 1, 1, design).items() if k.startswith("decode") or k == "batch"}
    return out


def compare_gulazen(size: str, steps: int, warmup: int, n_prompt: int = 2048, n_new: int = 64) -> dict:
    """Gulazen next to the closest model of the library, seven Binusun attention layers on the same engine (bf16 weights both)."""
    out = {"size": size, "shape": SIZES[size], "prompt_tokens": n_prompt, "decode_steps": n_new}
    for design, key in (("Gulazen", "gulazen_bf16"), ("BinusunAttention", "binusun_attention_bf16")):
        out[key] = measure_seq(size, "bfloat16", n_prompt, n_new, 1, steps, warmup, design)
        out[key + "_batch4"] = {k: v for k, v in measure_seq(size, "bfloat16", 256, n_new, 4, 1, 1, design).items() if k.startswith("decode") or k == "batch"}
    return out


def compare_zopipel(size: str, steps: int, warmup: int, n_prompt: int = 2048, n_new: int = 64) -> dict:
    """Zopipel next to the closest model of the library, seven Binusun attention layers on the same engine (bf16 weights both)."""
    out = {"size": size, "shape": SIZES[size], "prompt_tokens": n_prompt, "decode_steps": n_new}
    for design, key in (("Zopipel", "zopipel_bf16"), ("BinusunAttention", "binusun_attention_bf16")):
        out[key] = measure_seq(size, "bfloat16", n_prompt, n_new, 1, steps, warmup, design)
        out[key + "_batch4"] = {k: v for k, v in measure_seq(size, "bfloat16", 256, n_new, 4, 1, 1, design).items() if k.startswith("decode") or k == "batch"}
    return out


def compare(size: str, steps: int, warmup: int, n_prompt: int = 2048, n_new: int = 64, with_llama: bool = True) -> dict:
    out = {"size": size, "shape": SIZES[size], "prompt_tokens": n_prompt, "decode_steps": n_new,
           "binusun_bf16": measure_seq(size, "bfloat16", n_prompt, n_new, 1, steps, warmup),
           "binusun_bf16_batch4": {k: v for k, v in measure_seq(size, "bfloat16", 256, n_new, 4, 1, 1).items() if k.startswith("decode") or k == "batch"}}
    if with_llama:
        out["llama_int4_same_width_depth"] = measure_llama(size, n_prompt, n_new, steps, warmup)
    return out
