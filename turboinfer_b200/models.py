"""Model registry: config.json's "architecture" picks the class that turns the configuration into an engine.

    load_model(folder, dtype="bfloat16", max_tokens=..., max_seqs=...)

reads folder/config.json and folder/model.safetensors.  Registered architectures:
  * "Binusun"  -- layer list of windowed rotary attention / token-shifted linear recurrence (wkv) mixers with scalar-gain RMS
                  norms around every sublayer, an optional looped block of layers; runs on the layered sequence engine
                  (turboinfer_b200.seq, include/ti_b200_seq.h).
  * "Tudasun"  -- layer list of gated-linear-attention / HGRN2 recurrences and latent attention (low-rank key/value cache, rotated
                  key part shared by the heads, softmax sink, optional reuse of an earlier layer's cache), dense feed-forward with a
                  polynomial-norm activation or routed experts (group-limited choice, identity experts, shared expert), gated
                  residuals, a per-layer token side input and capped logits; runs on the layered sequence engine too.
  * "Gulazen"  -- attention layers that read the residual stream itself through a short causal convolution, with one norm and a
                  per-coordinate layer scale behind every sublayer: whole-projection query / key norm, capped scores mixed across
                  the heads, a sliding window that keeps the first keys, a softmax sink; dense feed-forward with the xIELU
                  activation or routed experts chosen by biased logits with a plain shared expert; sinusoidal positions added to
                  the embedding, logits tied to the embedding table; runs on the layered sequence engine too.
  * "Zopipel"  -- pre-norm layers on hyper-connections (several residual streams that every sublayer reads as one mixture and
                  rewrites together), a short causal convolution in front of BOTH sublayers, grouped attention with biased
                  projections, half-split rotation with linearly scaled frequencies, unit-RMS values, a per-head score factor and a
                  zero-score sink, latent attention with low-rank queries, a sliding window and a per-head output gate, a gated
                  gelu feed-forward, and a block of layers that is run several times in a row; on the layered sequence engine too.
  * "llama"    -- the quantized Llama-style decoder of the persistent decode kernel (turboinfer_b200.capi.Model); built from
                  {"hidden", "layers", "heads", "inter", "vocab"} and fp32 tensors under the reference's names.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, List, Tuple

from . import seq as _seq

REGISTRY: Dict[str, Callable] = {}


def register(name: str):
    def deco(fn):
        REGISTRY[name] = fn
        return fn
    return deco


def _req(d: dict, key: str, where: str):
    if key not in d:
        raise ValueError(f"config: {where} has no '{key}'")
    return d[key]


def binusun_descs(cfg: dict, mode: int, max_tokens: int, max_seqs: int, tensor_shapes: Dict[str, Tuple[int, ...]] = None):
    """config.json of a Binusun model -> (ModelDesc, [LayerDesc]).  Sizes the configuration does not carry (the inner size of the
    recurrence's decay projection) are taken from the checkpoint's tensor shapes."""
    layers: List[_seq.LayerDesc] = []
    for i, L in enumerate(_req(cfg, "layers", "the model")):
        mx = _req(L, "mixer", f"layer {i}")
        d = _seq.LayerDesc()
        kind = _req(L, "type", f"layer {i}")
        if kind == "attention":
            d.mixer = _seq.MIXER_ATTENTION
            d.heads, d.kv_heads = int(_req(mx, "heads", f"layer {i}")), int(_req(mx, "kv_heads", f"layer {i}"))
            d.dim, d.vdim = int(_req(mx, "dim", f"layer {i}")), int(_req(mx, "vdim", f"layer {i}"))
            d.window = int(_req(_req(mx, "mask", f"layer {i}"), "size", f"layer {i} mask"))
            rot = _req(mx, "rot", f"layer {i}")
            d.rot_dims, d.rot_base = int(_req(rot, "dims", f"layer {i} rot")), float(_req(rot, "base", f"layer {i} rot"))
            sc = rot.get("scaling")
            if sc:
                d.rot_scaled = 1
                d.rot_factor, d.rot_low = float(_req(sc, "factor", "rot.scaling")), float(_req(sc, "low", "rot.scaling"))
                d.rot_high, d.rot_original = float(_req(sc, "high", "rot.scaling")), float(_req(sc, "original", "rot.scaling"))
            d.qk_norm, d.out_gate = 1, 1
            d.scale = float(_req(mx, "scale", f"layer {i}"))
        elif kind == "wkv":
            d.mixer = _seq.MIXER_WKV
            d.heads, d.dim = int(_req(mx, "heads", f"layer {i}")), int(_req(mx, "dim", f"layer {i}"))
            d.kv_heads, d.vdim = d.heads, d.dim
            shape = (tensor_shapes or {}).get(f"l{i}.mix.w1")
            if not shape:
                raise ValueError(f"layer {i}: the decay projection l{i}.mix.w1 is missing from the checkpoint")
            d.decay_rank = int(shape[0])
        else:
            raise ValueError(f"layer {i}: unknown mixer type '{kind}'")
        mlp = L.get("mlp")
        if mlp:
            if mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind '{mlp.get('kind')}'")
            d.ff, d.ff_act = int(_req(mlp, "ff", f"layer {i} mlp")), _seq.ACT_RELU
        layers.append(d)
    m = _seq.ModelDesc()
    m.vocab, m.width, m.n_layers = int(_req(cfg, "vocab", "the model")), int(_req(cfg, "width", "the model")), len(layers)
    lp = cfg.get("loop")
    if lp and int(lp.get("times", 0)) > 0 and int(lp["stop"]) > int(lp["start"]):
        m.loop_start, m.loop_stop, m.loop_times = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    m.norm_eps = float(_req(_req(cfg, "norm", "the model"), "eps", "norm"))
    m.logit_scale = float(cfg.get("logit_scale", 1.0))
    m.mode, m.max_tokens, m.max_seqs = mode, int(max_tokens), int(max_seqs)
    return m, layers


@register("Binusun")
def _load_binusun(cfg: dict, weights: dict, dtype: str, max_tokens: int, max_seqs: int):
    mode = {"bfloat16": _seq.BF16, "float32": _seq.F32}[dtype]
    shapes = {k: tuple(getattr(v, "shape", ())) for k, v in weights.items()}
    desc, layers = binusun_descs(cfg, mode, max_tokens, max_seqs, shapes)
    return _seq.SeqModel(desc, layers).load(weights)


def tudasun_descs(cfg: dict, mode: int, max_tokens: int, max_seqs: int, tensor_shapes: Dict[str, Tuple[int, ...]] = None):
    """config.json of a Tudasun model -> (ModelDesc, [LayerDesc]).  The inner size of the gla decay projection, which the
    configuration does not carry, is the row count of the checkpoint's l<i>.mix.a1; the gated residual is on when the
    checkpoint has l<i>.rg1."""
    shapes = tensor_shapes or {}
    layers: List[_seq.LayerDesc] = []
    for i, L in enumerate(_req(cfg, "layers", "the model")):
        where = f"layer {i}"
        mx = _req(L, "mixer", where)
        d = _seq.LayerDesc()
        kind = _req(L, "type", where)
        d.heads, d.dim, d.vdim = int(_req(mx, "heads", where)), int(_req(mx, "dim", where)), int(_req(mx, "vdim", where))
        d.kv_heads = d.heads
        if kind == "gla":
            d.mixer = _seq.MIXER_GLA
            d.decay_tau = float(_req(mx, "tau", where))
            shape = shapes.get(f"l{i}.mix.a1")
            if not shape:
                raise ValueError(f"{where}: the decay projection l{i}.mix.a1 is missing from the checkpoint")
            d.decay_rank = int(shape[0])
        elif kind == "hgrn2":
            d.mixer = _seq.MIXER_HGRN2
        elif kind == "latent_attention":
            d.mixer = _seq.MIXER_LATENT
            d.kv_rank, d.rot_dims = int(_req(mx, "kv_rank", where)), int(_req(mx, "rot_dim", where))
            rot = _req(mx, "rot", where)
            if int(_req(rot, "dims", where + " rot")) != d.rot_dims:
                raise ValueError(f"{where}: rot.dims {rot['dims']} differs from rot_dim {d.rot_dims}; the rotated part turns as a whole")
            d.rot_base = float(_req(rot, "base", where + " rot"))
            d.scale = float(_req(mx, "scale", where))
            d.kv_from = int(mx["kv_from"]) if mx.get("kv_from") is not None else -1
            d.sink = 1
        else:
            raise ValueError(f"{where}: unknown mixer type '{kind}'")
        d.res_gate = 1 if (not shapes or f"l{i}.rg1" in shapes) else 0
        mlp = L.get("mlp")
        if mlp:
            fk = _req(mlp, "kind", where + " mlp")
            if fk == "dense":
                d.ff_kind, d.ff = _seq.FF_POLYNORM, int(_req(mlp, "ff", where + " mlp"))
            elif fk == "moe":
                r = _req(mlp, "router", where + " mlp")
                d.ff_kind, d.ff = _seq.FF_EXPERTS, int(_req(_req(mlp, "expert", where + " mlp"), "ff", where + " mlp.expert"))
                d.experts, d.top = int(_req(r, "experts", where + " router")), int(_req(r, "top", where + " router"))
                d.identity = int(r.get("identity") or 0)
                g = r.get("groups") or {}
                d.groups, d.groups_keep = int(g.get("count", 1)), int(g.get("keep", g.get("count", 1)))
                sh = mlp.get("shared")
                d.shared_ff = int(_req(sh, "ff", where + " mlp.shared")) if sh else 0
            else:
                raise ValueError(f"{where}: unknown feed-forward kind '{fk}'")
        layers.append(d)
    m = _seq.ModelDesc()
    m.vocab, m.width, m.n_layers = int(_req(cfg, "vocab", "the model")), int(_req(cfg, "width", "the model")), len(layers)
    m.norm_eps = float(_req(_req(cfg, "norm", "the model"), "eps", "norm"))
    m.norm_kind = _seq.NORM_ONE_PLUS
    m.logit_scale = 1.0
    m.logit_softcap = float(cfg.get("logit_softcap") or 0.0)
    ts = cfg.get("token_side")
    m.side_dim = int(_req(ts, "dim", "token_side")) if ts else 0
    m.mode, m.max_tokens, m.max_seqs = mode, int(max_tokens), int(max_seqs)
    return m, layers


@register("Tudasun")
def _load_tudasun(cfg: dict, weights: dict, dtype: str, max_tokens: int, max_seqs: int):
    mode = {"bfloat16": _seq.BF16, "float32": _seq.F32}[dtype]
    shapes = {k: tuple(getattr(v, "shape", ())) for k, v in weights.items()}
    desc, layers = tudasun_descs(cfg, mode, max_tokens, max_seqs, shapes)
    return _seq.SeqModel(desc, layers).load(weights)


def gulazen_descs(cfg: dict, mode: int, max_tokens: int, max_seqs: int, tensor_shapes: Dict[str, Tuple[int, ...]] = None):
    """config.json of a Gulazen model -> (ModelDesc, [LayerDesc]).  Every size and constant comes from the configuration; the base
    of the sinusoidal positions (10000) is fixed by the design."""
    taps = int(_req(_req(cfg, "canon", "the model"), "taps", "canon"))
    if taps < 1:
        raise ValueError(f"config: canon.taps {taps}")
    layers: List[_seq.LayerDesc] = []
    for i, L in enumerate(_req(cfg, "layers", "the model")):
        where = f"layer {i}"
        kind = _req(L, "type", where)
        if kind != "attention":
            raise ValueError(f"{where}: unknown mixer type '{kind}'")
        mx = _req(L, "mixer", where)
        d = _seq.LayerDesc()
        d.mixer = _seq.MIXER_ATTENTION
        d.heads, d.kv_heads = int(_req(mx, "heads", where)), int(_req(mx, "kv_heads", where))
        d.dim, d.vdim = int(_req(mx, "dim", where)), int(_req(mx, "vdim", where))
        mask = _req(mx, "mask", where)
        d.window, d.keep_first = int(_req(mask, "size", where + " mask")), int(_req(mask, "keep_first", where + " mask"))
        if d.window < 1:
            raise ValueError(f"{where}: mask.size {d.window}")
        d.scale, d.softcap = float(_req(mx, "scale", where)), float(_req(mx, "softcap", where))
        d.rot_dims, d.qk_norm, d.out_gate = 0, _seq.QK_NORM_WHOLE, 0
        d.talk, d.sink = 1, 1
        d.conv_taps, d.layer_scale = taps, 1
        mlp = L.get("mlp")
        if mlp:
            fk = _req(mlp, "kind", where + " mlp")
            if fk == "dense":
                d.ff_kind, d.ff, d.ff_act = _seq.FF_DENSE, int(_req(mlp, "ff", where + " mlp")), _seq.ACT_XIELU
            elif fk == "moe":
                r = _req(mlp, "router", where + " mlp")
                d.ff_kind, d.ff = _seq.FF_EXPERTS, int(_req(_req(mlp, "expert", where + " mlp"), "ff", where + " mlp.expert"))
                d.experts, d.top = int(_req(r, "experts", where + " router")), int(_req(r, "top", where + " router"))
                d.identity, d.groups, d.groups_keep = 0, 1, 1
                d.route_kind, d.shared_plain = _seq.ROUTE_TOP_LOGITS, 1
                sh = mlp.get("shared")
                d.shared_ff = int(_req(sh, "ff", where + " mlp.shared")) if sh else 0
            else:
                raise ValueError(f"{where}: unknown feed-forward kind '{fk}'")
        layers.append(d)
    m = _seq.ModelDesc()
    m.vocab, m.width, m.n_layers = int(_req(cfg, "vocab", "the model")), int(_req(cfg, "width", "the model")), len(layers)
    m.norm_eps = float(_req(_req(cfg, "norm", "the model"), "eps", "norm"))
    m.norm_kind, m.norm_place = _seq.NORM_ONE_PLUS, _seq.NORMS_BEHIND
    m.logit_scale, m.logit_softcap = 1.0, 0.0
    m.pos_base, m.tied_head = 10000.0, 1
    m.mode, m.max_tokens, m.max_seqs = mode, int(max_tokens), int(max_seqs)
    return m, layers


@register("Gulazen")
def _load_gulazen(cfg: dict, weights: dict, dtype: str, max_tokens: int, max_seqs: int):
    mode = {"bfloat16": _seq.BF16, "float32": _seq.F32}[dtype]
    desc, layers = gulazen_descs(cfg, mode, max_tokens, max_seqs)
    return _seq.SeqModel(desc, layers).load(weights)


def zopipel_descs(cfg: dict, mode: int, max_tokens: int, max_seqs: int, tensor_shapes: Dict[str, Tuple[int, ...]] = None):
    """config.json of a Zopipel model -> (ModelDesc, [LayerDesc]).  Every size and constant comes from the configuration."""
    taps = int(_req(_req(cfg, "canon", "the model"), "taps", "canon"))
    if taps < 1:
        raise ValueError(f"config: canon.taps {taps}")
    layers: List[_seq.LayerDesc] = []
    for i, L in enumerate(_req(cfg, "layers", "the model")):
        where = f"layer {i}"
        kind = _req(L, "type", where)
        mx = _req(L, "mixer", where)
        d = _seq.LayerDesc()
        d.heads = int(_req(mx, "heads", where))
        d.dim, d.vdim = int(_req(mx, "dim", where)), int(_req(mx, "vdim", where))
        d.scale = float(_req(mx, "scale", where))
        rot = _req(mx, "rot", where)
        d.rot_dims, d.rot_base, d.rot_half = int(_req(rot, "dims", where + " rot")), float(_req(rot, "base", where + " rot")), 1
        sc = rot.get("scaling")
        if sc:
            d.rot_linear = float(_req(sc, "factor", where + " rot.scaling"))
        mask = mx.get("mask")
        d.window = int(_req(mask, "size", where + " mask")) if mask else 0
        if mask and d.window < 1:
            raise ValueError(f"{where}: mask.size {d.window}")
        if kind == "attention":
            d.mixer = _seq.MIXER_ATTENTION
            d.kv_heads = int(_req(mx, "kv_heads", where))
            d.proj_bias, d.v_norm, d.head_temp, d.sink = 1, 1, 1, _seq.SINK_ZERO
        elif kind == "latent_attention":
            d.mixer = _seq.MIXER_LATENT
            d.kv_heads = d.heads
            d.kv_rank, d.q_rank = int(_req(mx, "kv_rank", where)), int(_req(mx, "q_rank", where))
            if int(_req(mx, "rot_dim", where)) != d.rot_dims:
                raise ValueError(f"{where}: rot.dims {d.rot_dims} differs from rot_dim {mx['rot_dim']}; the rotated part turns as a whole")
            d.out_gate, d.sink = 1, _seq.SINK_NONE
        else:
            raise ValueError(f"{where}: unknown mixer type '{kind}'")
        d.conv_taps, d.conv_ff = taps, 1
        mlp = L.get("mlp")
        if mlp:
            if _req(mlp, "kind", where + " mlp") != "dense":
                raise ValueError(f"{where}: unknown feed-forward kind '{mlp.get('kind')}'")
            d.ff_kind, d.ff, d.ff_act = _seq.FF_GLU, int(_req(mlp, "ff", where + " mlp")), _seq.ACT_GELU_TANH
        layers.append(d)
    m = _seq.ModelDesc()
    m.vocab, m.width, m.n_layers = int(_req(cfg, "vocab", "the model")), int(_req(cfg, "width", "the model")), len(layers)
    lp = cfg.get("loop")
    if lp and int(lp.get("times", 1)) > 1 and int(lp["stop"]) > int(lp["start"]):
        m.loop_start, m.loop_stop, m.loop_times, m.loop_plain = int(lp["start"]), int(lp["stop"]), int(lp["times"]), 1
    elif lp and int(lp.get("times", 1)) < 1:
        raise ValueError(f"config: loop.times {lp.get('times')}")
    m.norm_eps = float(_req(_req(cfg, "norm", "the model"), "eps", "norm"))
    m.norm_kind, m.norm_place = _seq.NORM_VECTOR, _seq.NORMS_FRONT
    m.streams = int(_req(cfg, "streams", "the model"))
    if m.streams < 1:
        raise ValueError(f"config: streams {m.streams}")
    m.logit_scale = 1.0
    m.mode, m.max_tokens, m.max_seqs = mode, int(max_tokens), int(max_seqs)
    return m, layers


@register("Zopipel")
def _load_zopipel(cfg: dict, weights: dict, dtype: str, max_tokens: int, max_seqs: int):
    mode = {"bfloat16": _seq.BF16, "float32": _seq.F32}[dtype]
    desc, layers = zopipel_descs(cfg, mode, max_tokens, max_seqs)
    return _seq.SeqModel(desc, layers).load(weights)


@register("llama")
def _load_llama(cfg: dict, weights: dict, dtype: str, max_tokens: int, max_seqs: int):
    import numpy as np

    from . import capi
    if dtype not in ("int4", "int8"):
        raise ValueError("the llama decoder of this library runs INT4 / INT8 weights (dtype 'int4' or 'int8')")
    capi.init(0)
    meta = {k: int(cfg[k]) for k in ("vocab", "hidden", "layers", "heads", "inter")}
    m = capi.Model(meta, capi.Q_INT4 if dtype == "int4" else capi.Q_INT8, attn_mode=1, rope_mode=1, max_seq=max_tokens)
    return m.load({k: (v.to_f32() if isinstance(v, _seq.Bf16Array) else np.asarray(v, np.float32)) for k, v in weights.items()})


def load_model(folder: str, dtype: str = "bfloat16", max_tokens: int = 4096, max_seqs: int = 4):
    from .safetensors_io import read_safetensors
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    arch = cfg.get("architecture")
    if arch not in REGISTRY:
        raise ValueError(f"config.json: architecture '{arch}' is not registered (known: {sorted(REGISTRY)})")
    weights = read_safetensors(os.path.join(folder, "model.safetensors"))
    return REGISTRY[arch](cfg, weights, dtype, max_tokens, max_seqs)
