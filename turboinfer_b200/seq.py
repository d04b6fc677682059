"""ctypes bindings of include/ti_b200_seq.h: the layered sequence engine (ragged steps over a paged cache and state slots).

numpy in / numpy out, no torch, no fallback: without a CUDA device `init` raises."""
from __future__ import annotations

import ctypes as C
import os
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BF16, F32 = 0, 1
MIXER_ATTENTION, MIXER_WKV, MIXER_GLA, MIXER_HGRN2, MIXER_LATENT = 0, 1, 2, 3, 4
ACT_RELU, ACT_SILU, ACT_GELU_TANH, ACT_XIELU = 0, 1, 2, 3
FF_GLU, FF_POLYNORM, FF_EXPERTS, FF_DENSE = 0, 1, 2, 3
NORM_SCALAR, NORM_ONE_PLUS, NORM_VECTOR = 0, 1, 2
SINK_NONE, SINK_LEARNED, SINK_ZERO = 0, 1, 2
ROUTE_SOFTMAX_ALL, ROUTE_TOP_LOGITS = 0, 1
QK_NORM_NONE, QK_NORM_HEAD, QK_NORM_WHOLE = 0, 1, 2
NORMS_AROUND, NORMS_BEHIND, NORMS_FRONT = 0, 1, 2


class SeqError(RuntimeError):
    pass


class LayerDesc(C.Structure):
    _fields_ = [("mixer", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32), ("dim", C.c_int32), ("vdim", C.c_int32),
                ("window", C.c_int32), ("rot_dims", C.c_int32), ("rot_base", C.c_float), ("rot_scaled", C.c_int32),
                ("rot_factor", C.c_float), ("rot_low", C.c_float), ("rot_high", C.c_float), ("rot_original", C.c_float),
                ("qk_norm", C.c_int32), ("out_gate", C.c_int32), ("scale", C.c_float), ("decay_rank", C.c_int32),
                ("ff", C.c_int32), ("ff_act", C.c_int32), ("decay_tau", C.c_float), ("kv_rank", C.c_int32), ("kv_from", C.c_int32),
                ("sink", C.c_int32), ("ff_kind", C.c_int32), ("experts", C.c_int32), ("identity", C.c_int32), ("top", C.c_int32),
                ("groups", C.c_int32), ("groups_keep", C.c_int32), ("shared_ff", C.c_int32), ("res_gate", C.c_int32),
                ("softcap", C.c_float), ("talk", C.c_int32), ("keep_first", C.c_int32), ("route_kind", C.c_int32),
                ("shared_plain", C.c_int32), ("conv_taps", C.c_int32), ("layer_scale", C.c_int32), ("conv_ff", C.c_int32),
                ("rot_half", C.c_int32), ("rot_linear", C.c_float), ("proj_bias", C.c_int32), ("v_norm", C.c_int32),
                ("head_temp", C.c_int32), ("q_rank", C.c_int32)]

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        if "kv_from" not in kw:
            self.kv_from = -1


class ModelDesc(C.Structure):
    _fields_ = [("vocab", C.c_int32), ("width", C.c_int32), ("n_layers", C.c_int32), ("loop_start", C.c_int32),
                ("loop_stop", C.c_int32), ("loop_times", C.c_int32), ("norm_eps", C.c_float), ("logit_scale", C.c_float),
                ("mode", C.c_int32), ("max_tokens", C.c_int32), ("max_seqs", C.c_int32), ("norm_kind", C.c_int32),
                ("logit_softcap", C.c_float), ("side_dim", C.c_int32), ("norm_place", C.c_int32), ("pos_base", C.c_float),
                ("tied_head", C.c_int32), ("loop_plain", C.c_int32), ("streams", C.c_int32)]


_i32 = C.POINTER(C.c_int32)
_i64 = C.POINTER(C.c_int64)
_f = C.POINTER(C.c_float)
_d = C.POINTER(C.c_double)
SYMBOLS = {
    "ti_seq_init": (C.c_int, [C.c_int]),
    "ti_seq_last_error": (C.c_char_p, []),
    "ti_seq_launch_count": (C.c_uint64, []),
    "ti_seq_model_new": (C.c_int, [C.POINTER(ModelDesc), C.POINTER(LayerDesc), C.POINTER(C.c_uint64)]),
    "ti_seq_model_set_tensor": (C.c_int, [C.c_uint64, C.c_char_p, C.c_int32, C.c_void_p, _i64, C.c_int32]),
    "ti_seq_model_set_tensor_synthetic": (C.c_int, [C.c_uint64, C.c_char_p, _i64, C.c_int32, C.c_uint64, C.c_float, C.c_float]),
    "ti_seq_model_tensor_count": (C.c_int, [C.c_uint64, _i32]),
    "ti_seq_model_tensor_info": (C.c_int, [C.c_uint64, C.c_int32, C.c_char_p, C.c_size_t, _i64, _i32]),
    "ti_seq_model_finalize": (C.c_int, [C.c_uint64]),
    "ti_seq_model_free": (C.c_int, [C.c_uint64]),
    "ti_seq_open": (C.c_int, [C.c_uint64, _i32]),
    "ti_seq_close": (C.c_int, [C.c_uint64, C.c_int32]),
    "ti_seq_length": (C.c_int, [C.c_uint64, C.c_int32, _i32]),
    "ti_seq_pool_info": (C.c_int, [C.c_uint64, _i32, _i32, _i32, _i32]),
    "ti_seq_pages": (C.c_int, [C.c_uint64, C.c_int32, _i32, C.c_int32, _i32]),
    "ti_seq_step": (C.c_int, [C.c_uint64, C.c_int32, _i32, _i32, _i32, C.c_int32, _i32, _f]),
    "ti_seq_step_sample": (C.c_int, [C.c_uint64, C.c_int32, _i32, _i32, _i32, C.c_float, C.c_int32, C.c_float, C.c_uint64, _i32, _i32, _f]),
    "ti_seq_generate": (C.c_int, [C.c_uint64, C.c_int32, _i32, _i32, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_float, C.c_uint64,
                                  C.c_int32, _i32, _i32]),
    "ti_seq_debug_layers": (C.c_int, [C.c_uint64, C.c_int32]),
    "ti_seq_debug_layers_read": (C.c_int, [C.c_uint64, _f, C.c_size_t, _i32, _i32]),
    "ti_seq_flush_l2": (C.c_int, []),
    "ti_seq_last_step_ms": (C.c_int, [C.c_uint64, _f]),
    "ti_seq_model_bytes": (C.c_int, [C.c_uint64, _d, _d, _d]),
}

_lib: Optional[C.CDLL] = None
_inited = False


def library_path() -> str:
    return os.path.join(HERE, "libturboinfer_b200_seq.so")


def lib() -> C.CDLL:
    """Loads the engine's library, compiling it first (nvcc, sm_100a) when the in-tree .so is missing or older than its sources."""
    global _lib
    if _lib is None:
        from . import build as _build
        if os.path.isdir(os.path.join(HERE, "csrc")) and os.path.exists(_build.NVCC):
            _build.build_seq()
        path = library_path()
        if not os.path.exists(path):
            raise SeqError(f"{path} is missing and cannot be built here (no CPU fallback exists)")
        L = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _ck(rc: int) -> None:
    if rc != 0:
        raise SeqError(lib().ti_seq_last_error().decode("utf-8", "replace"))


def init(device: int = 0) -> None:
    global _inited
    if not _inited:
        _ck(lib().ti_seq_init(device))
        _inited = True


def flush_l2() -> None:
    _ck(lib().ti_seq_flush_l2())


def launch_count() -> int:
    return int(lib().ti_seq_launch_count())


def _ints(a) -> Tuple[np.ndarray, "C._Pointer"]:
    arr = np.ascontiguousarray(np.asarray(a, dtype=np.int32).reshape(-1))
    return arr, arr.ctypes.data_as(_i32)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> bfloat16 bits (round to nearest even), as uint16."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class Bf16Array:
    """Raw bfloat16 bits with a shape: what a bf16 checkpoint tensor is handed over as."""

    def __init__(self, bits: np.ndarray, shape: Sequence[int]):
        self.bits = np.ascontiguousarray(bits, dtype=np.uint16).reshape(-1)
        self.shape = tuple(int(s) for s in shape)

    def to_f32(self) -> np.ndarray:
        return bf16_to_f32(self.bits).reshape(self.shape)


class SeqModel:
    """A decoder described layer by layer, its page pool and state slots, and the step / generate entry points."""

    def __init__(self, desc: ModelDesc, layers: Sequence[LayerDesc]):
        init()
        self.desc = desc
        self.layers = list(layers)
        arr = (LayerDesc * len(self.layers))(*self.layers)
        h = C.c_uint64(0)
        _ck(lib().ti_seq_model_new(C.byref(desc), arr, C.byref(h)))
        self.h = h.value
        self.vocab = int(desc.vocab)

    # -- weights ---------------------------------------------------------------------------------------------------
    def tensor_specs(self) -> List[Tuple[str, Tuple[int, ...]]]:
        n = C.c_int32(0)
        _ck(lib().ti_seq_model_tensor_count(self.h, C.byref(n)))
        out = []
        name = C.create_string_buffer(256)
        shape = (C.c_int64 * 8)()
        nd = C.c_int32(0)
        for i in range(n.value):
            _ck(lib().ti_seq_model_tensor_info(self.h, i, name, 256, shape, C.byref(nd)))
            out.append((name.value.decode(), tuple(int(shape[k]) for k in range(nd.value))))
        return out

    def set_tensor(self, name: str, value) -> None:
        if isinstance(value, Bf16Array):
            data, shape, dt = value.bits, value.shape, BF16
        else:
            a = np.asarray(value, dtype=np.float32)
            data, shape, dt = np.ascontiguousarray(a).reshape(-1), a.shape, F32   # (a 0-d array stays 0-d in `shape`)
        sh = (C.c_int64 * max(1, len(shape)))(*shape)
        _ck(lib().ti_seq_model_set_tensor(self.h, name.encode(), dt, data.ctypes.data_as(C.c_void_p), sh, len(shape)))

    def set_tensor_synthetic(self, name: str, shape: Sequence[int], seed: int, amp: float, offset: float = 0.0) -> None:
        sh = (C.c_int64 * max(1, len(shape)))(*shape)
        _ck(lib().ti_seq_model_set_tensor_synthetic(self.h, name.encode(), sh, len(shape), seed, amp, offset))

    def load(self, weights) -> "SeqModel":
        for name, _ in self.tensor_specs():
            if name not in weights:
                raise SeqError(f"checkpoint has no tensor {name}")
            self.set_tensor(name, weights[name])
        return self.finalize()

    def finalize(self) -> "SeqModel":
        _ck(lib().ti_seq_model_finalize(self.h))
        return self

    def free(self) -> None:
        if self.h:
            lib().ti_seq_model_free(self.h)
            self.h = 0

    # -- sequences -------------------------------------------------------------------------------------------------
    def open(self) -> int:
        s = C.c_int32(-1)
        _ck(lib().ti_seq_open(self.h, C.byref(s)))
        return s.value

    def close(self, seq: int) -> None:
        _ck(lib().ti_seq_close(self.h, seq))

    def length(self, seq: int) -> int:
        n = C.c_int32(0)
        _ck(lib().ti_seq_length(self.h, seq, C.byref(n)))
        return n.value

    def pool_info(self) -> dict:
        a, b, c, d = C.c_int32(0), C.c_int32(0), C.c_int32(0), C.c_int32(0)
        _ck(lib().ti_seq_pool_info(self.h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return {"free_pages": a.value, "total_pages": b.value, "free_slots": c.value, "page_tokens": d.value}

    def pages(self, seq: int) -> List[int]:
        buf = np.zeros(4096, np.int32)
        n = C.c_int32(0)
        _ck(lib().ti_seq_pages(self.h, seq, buf.ctypes.data_as(_i32), buf.size, C.byref(n)))
        return [int(x) for x in buf[:n.value]]

    # -- stepping --------------------------------------------------------------------------------------------------
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]] = None) -> np.ndarray:
        """entries: (sequence, its next tokens); want[e]: places among entry e's tokens whose logits are returned, in order."""
        seqs, sp = _ints([e[0] for e in entries])
        counts, cp = _ints([len(e[1]) for e in entries])
        toks, tp = _ints([t for e in entries for t in e[1]])
        rows: List[int] = []
        off = 0
        for i, e in enumerate(entries):
            if want is not None:
                rows += [off + int(w) for w in want[i]]
            off += len(e[1])
        wr, wp = _ints(rows if rows else [0])
        out = np.empty((len(rows), self.vocab), np.float32)
        _ck(lib().ti_seq_step(self.h, len(entries), sp, cp, tp, len(rows), wp, out.ctypes.data_as(_f)))
        return out

    def step_sample(self, entries: Sequence[Tuple[int, Sequence[int]]], temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                    seed: int = 0, sample_index: Optional[Sequence[int]] = None) -> Tuple[np.ndarray, np.ndarray]:
        seqs, sp = _ints([e[0] for e in entries])
        counts, cp = _ints([len(e[1]) for e in entries])
        toks, tp = _ints([t for e in entries for t in e[1]])
        idx, ip = _ints(sample_index if sample_index is not None else [0] * len(entries))
        out = np.zeros(len(entries), np.int32)
        lp = np.zeros(len(entries), np.float32)
        _ck(lib().ti_seq_step_sample(self.h, len(entries), sp, cp, tp, temperature, top_k, top_p, seed, ip, out.ctypes.data_as(_i32),
                                     lp.ctypes.data_as(_f)))
        return out, lp

    def generate(self, prompts: Sequence[Sequence[int]], max_new: int, step_tokens: int = 512, temperature: float = 0.0, top_k: int = 0,
                 top_p: float = 1.0, seed: int = 0, eos: int = -1) -> List[List[int]]:
        """Continuous batching over all prompts; returns the new tokens of every request."""
        flat, fp = _ints([t for p in prompts for t in p])
        lens, lp = _ints([len(p) for p in prompts])
        out = np.zeros((len(prompts), max_new), np.int32)
        n = np.zeros(len(prompts), np.int32)
        _ck(lib().ti_seq_generate(self.h, len(prompts), fp, lp, max_new, step_tokens, temperature, top_k, top_p, seed, eos,
                                  out.ctypes.data_as(_i32), n.ctypes.data_as(_i32)))
        return [[int(t) for t in out[i, :n[i]]] for i in range(len(prompts))]

    # -- inspection ------------------------------------------------------------------------------------------------
    def debug_layers(self, enable: bool = True) -> None:
        _ck(lib().ti_seq_debug_layers(self.h, 1 if enable else 0))

    def read_layers(self, rows: int) -> np.ndarray:
        r, t = C.c_int32(0), C.c_int32(0)
        n_runs = self.n_runs()
        buf = np.empty(n_runs * rows * int(self.desc.width), np.float32)
        _ck(lib().ti_seq_debug_layers_read(self.h, buf.ctypes.data_as(_f), buf.size, C.byref(r), C.byref(t)))
        return buf[:r.value * t.value * int(self.desc.width)].reshape(r.value, t.value, int(self.desc.width))

    def n_runs(self) -> int:
        d = self.desc
        n = int(d.n_layers)
        if d.loop_times > 0:
            n += (int(d.loop_times) - 1) * (int(d.loop_stop) - int(d.loop_start))
        return n

    def last_step_ms(self) -> float:
        ms = C.c_float(0)
        _ck(lib().ti_seq_last_step_ms(self.h, C.byref(ms)))
        return ms.value

    def bytes(self) -> dict:
        a, b, c = C.c_double(0), C.c_double(0), C.c_double(0)
        _ck(lib().ti_seq_model_bytes(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return {"weights": a.value, "kv_per_token": b.value, "state_per_seq": c.value}
