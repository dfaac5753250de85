"""ctypes binding of the CPU oracle (oracle/libpelica_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and
by bench.py's cpu_baseline / reference arm. The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libpelica_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile (gcc); returns the .so path."""
    srcs = [os.path.join(_HERE, f) for f in ("pelica_oracle.c", "pelica_oracle_fast.c", "pelica_oracle.h")]
    stale = (not os.path.exists(_SO)) or any(os.path.getmtime(s) > os.path.getmtime(_SO) for s in srcs)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "-s"])
    return _SO


class LayerDesc(C.Structure):
    """Mirror of pm_layer_desc (include/pelica_moe.h)."""

    _fields_ = [
        ("d", C.c_int32), ("ff", C.c_int32), ("n_exp", C.c_int32), ("top_k", C.c_int32),
        ("gating", C.c_int32), ("norm_w", C.c_int32), ("w_scale", C.c_float),
        ("n_group", C.c_int32), ("topk_group", C.c_int32),
        ("act", C.c_int32), ("act_limit", C.c_float), ("act_alpha", C.c_float),
        ("type_gate", C.c_int32), ("type_up", C.c_int32), ("type_down", C.c_int32),
        ("act_quant", C.c_int32), ("weight_fold", C.c_int32), ("has_expert_bias", C.c_int32),
        ("shared", C.c_int32), ("shared_ff", C.c_int32),
        ("first_local_expert", C.c_int32), ("n_exp_local", C.c_int32),
    ]


class ExpertW(C.Structure):
    _fields_ = [("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
                ("bias_gate", C.c_void_p), ("bias_up", C.c_void_p), ("bias_down", C.c_void_p)]


class PoLayer(C.Structure):
    _fields_ = [("desc", LayerDesc), ("router", C.c_void_p), ("logit_bias", C.c_void_p),
                ("select_bias", C.c_void_p), ("experts", C.POINTER(ExpertW)), ("shared", ExpertW),
                ("shared_gate_inp", C.c_void_p)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        f32p, u8p, i8p, i32p, u32p = (C.c_void_p,) * 5
        L.po_f16_to_f32.restype = C.c_float
        L.po_f16_to_f32.argtypes = [C.c_uint16]
        L.po_f32_to_f16.restype = C.c_uint16
        L.po_f32_to_f16.argtypes = [C.c_float]
        L.po_f32_to_bf16.restype = C.c_uint16
        L.po_f32_to_bf16.argtypes = [C.c_float]
        L.po_exp.restype = C.c_float
        L.po_exp.argtypes = [C.c_float]
        L.po_log1p.restype = C.c_float
        L.po_log1p.argtypes = [C.c_float]
        L.po_dot_f32.restype = C.c_float
        L.po_dot_f32.argtypes = [f32p, f32p, C.c_size_t]
        L.po_dot_bf16.restype = C.c_float
        L.po_dot_bf16.argtypes = [C.c_void_p, f32p, C.c_size_t]
        L.po_type_block_bytes.restype = C.c_size_t
        L.po_type_block_values.restype = C.c_size_t
        L.po_dequant.argtypes = [C.c_int, u8p, C.c_size_t, f32p]
        L.po_q8x.argtypes = [f32p, C.c_size_t, i8p, f32p, i32p]
        L.po_q8x.restype = None
        L.po_q8_32.argtypes = [f32p, C.c_size_t, i8p, f32p]
        L.po_q8_32.restype = None
        L.po_q8_32_f16.argtypes = [f32p, C.c_size_t, i8p, f32p]
        L.po_q8_32_f16.restype = None
        for name in ("po_row_q4k", "po_row_q4k_fast", "po_row_q4k_vnni"):
            fn = getattr(L, name)
            fn.restype = C.c_float
            fn.argtypes = [u8p, C.c_size_t, i8p, f32p, i32p]
        for name in ("po_row_q6k", "po_row_q6k_fast", "po_row_q8_0", "po_row_iq4nl", "po_row_iq4xs", "po_row_iq3s",
                     "po_row_q4k_q8_32"):
            fn = getattr(L, name)
            fn.restype = C.c_float
            fn.argtypes = [u8p, C.c_size_t, i8p, f32p]
        L.po_row_f32.restype = C.c_float
        L.po_row_f32.argtypes = [C.c_int, u8p, C.c_size_t, f32p]
        L.po_q4k_rows_multi.restype = None
        L.po_q4k_rows_multi.argtypes = [u8p, C.c_size_t, C.c_size_t, C.c_int, C.c_void_p, C.c_void_p,
                                        C.c_void_p, f32p, C.c_int]
        L.po_router_logits.restype = None
        L.po_router_logits.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, f32p]
        L.po_route.argtypes = [C.POINTER(LayerDesc), f32p, f32p, C.c_int, u32p, f32p]
        L.po_plan.argtypes = [u32p, C.c_int, C.c_int, C.c_int, u32p, u32p, u32p, u32p, u32p]
        L.po_experts.argtypes = [C.POINTER(PoLayer), f32p, C.c_int, u32p, f32p, f32p]
        L.po_combine.restype = None
        L.po_combine.argtypes = [C.POINTER(LayerDesc), f32p, u32p, f32p, f32p, f32p, C.c_int, f32p, C.c_int]
        L.po_moe_forward.argtypes = [C.POINTER(PoLayer), f32p, C.c_int, f32p, C.c_int, C.c_int]
        L.po_moe_forward_fast.argtypes = [C.POINTER(PoLayer), f32p, C.c_int, f32p, C.c_int]
        L.po_stack_forward.argtypes = [C.POINTER(PoLayer), C.c_int, C.c_float, f32p, C.c_int, f32p, C.c_int]
        L.po_rmsnorm.restype = None
        L.po_rmsnorm.argtypes = [f32p, C.c_int, C.c_float, f32p]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def f16_to_f32(h: int) -> float:
    return lib().po_f16_to_f32(h)


def f32_to_f16(x: float) -> int:
    return lib().po_f32_to_f16(x)


def exp(x: float) -> float:
    return lib().po_exp(x)


def log1p(x: float) -> float:
    return lib().po_log1p(x)


def dot_f32(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().po_dot_f32(_p(a), _p(b), a.size)


def dot_bf16(a_bits, b) -> float:
    a = np.ascontiguousarray(a_bits, dtype=np.uint16)
    b = _f32(b)
    return lib().po_dot_bf16(_p(a), _p(b), a.size)


def dequant(ggml_type: int, blocks, n_values: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n_values, dtype=np.float32)
    rc = lib().po_dequant(ggml_type, _p(blocks), n_values, _p(out))
    if rc:
        raise ValueError(f"po_dequant: {rc}")
    return out


def q8x(x):
    x = _f32(x).ravel()
    n = x.size
    q = np.empty(n, np.int8)
    d = np.empty(n // 256, np.float32)
    bsum = np.empty(n // 32, np.int32)
    lib().po_q8x(_p(x), n, _p(q), _p(d), _p(bsum))
    return q, d, bsum


def q8_32(x, f16_scale=False):
    x = _f32(x).ravel()
    q = np.empty(x.size, np.int8)
    d = np.empty(x.size // 32, np.float32)
    (lib().po_q8_32_f16 if f16_scale else lib().po_q8_32)(_p(x), x.size, _p(q), _p(d))
    return q, d


def row_q4k_q8_32(w, ncols, q, d32) -> float:
    return lib().po_row_q4k_q8_32(_p(w), ncols, _p(q), _p(d32))


def row_q4k(w, ncols, q, d, bsum, kind="scalar") -> float:
    fn = {"scalar": lib().po_row_q4k, "fast": lib().po_row_q4k_fast, "vnni": lib().po_row_q4k_vnni}[kind]
    w = np.ascontiguousarray(w, np.uint8)
    return fn(_p(w), ncols, _p(q), _p(d), _p(bsum))


def row_q6k(w, ncols, q, d, kind="scalar") -> float:
    fn = {"scalar": lib().po_row_q6k, "fast": lib().po_row_q6k_fast}[kind]
    w = np.ascontiguousarray(w, np.uint8)
    return fn(_p(w), ncols, _p(q), _p(d))


def row_q8_0(w, ncols, q, d32) -> float:
    w = np.ascontiguousarray(w, np.uint8)
    return lib().po_row_q8_0(_p(w), ncols, _p(q), _p(d32))


def row_iq4nl(w, ncols, q, d32) -> float:
    w = np.ascontiguousarray(w, np.uint8)
    return lib().po_row_iq4nl(_p(w), ncols, _p(q), _p(d32))


def row_iq4xs(w, ncols, q, d32) -> float:
    w = np.ascontiguousarray(w, np.uint8)
    return lib().po_row_iq4xs(_p(w), ncols, _p(q), _p(d32))


def row_iq3s(w, ncols, q, d32) -> float:
    w = np.ascontiguousarray(w, np.uint8)
    return lib().po_row_iq3s(_p(w), ncols, _p(q), _p(d32))


def row_f32(ggml_type, w, ncols, x) -> float:
    w = np.ascontiguousarray(w, np.uint8)
    x = _f32(x)
    return lib().po_row_f32(ggml_type, _p(w), ncols, _p(x))


def q4k_rows_multi(w, nrows, ncols, qs, canonical=False) -> np.ndarray:
    """qs: list of (q, d, bsum) per token; returns out[nrows, nt]."""
    w = np.ascontiguousarray(w, np.uint8)
    nt = len(qs)
    PT = C.c_void_p * nt
    qa = PT(*[q.ctypes.data for q, _, _ in qs])
    da = PT(*[d.ctypes.data for _, d, _ in qs])
    ba = PT(*[b.ctypes.data for _, _, b in qs])
    out = np.empty((nrows, nt), np.float32)
    lib().po_q4k_rows_multi(_p(w), nrows, ncols, nt, qa, da, ba, _p(out), int(canonical))
    return out


def rmsnorm(x, eps):
    x = _f32(x)
    out = np.empty_like(x)
    d = x.shape[-1]
    xf, of = x.reshape(-1, d), out.reshape(-1, d)
    for t in range(xf.shape[0]):
        lib().po_rmsnorm(_p(xf[t]), d, eps, _p(of[t]))
    return out


class Layer:
    """One MoE layer for the oracle, built from numpy arrays.

    weights: dict with router [E,d] f32, optional logit_bias/select_bias [E],
    gate/up/down: uint8 arrays [E, bytes], optional bias_gate/bias_up [E,ff],
    bias_down [E,d]; optional shared_gate/shared_up/shared_down (uint8),
    shared_gate_inp [d].
    """

    def __init__(self, desc: LayerDesc, weights: dict):
        self.desc = desc
        # a tensor family may also come as a per-expert list of byte arrays (a shard of a large layer)
        self.w = {k: ([np.ascontiguousarray(a) for a in v] if isinstance(v, list) else
                      np.ascontiguousarray(v) if v is not None else None) for k, v in weights.items()}
        w = self.w
        E = desc.n_exp
        self._experts = (ExpertW * E)()
        for e in range(E):
            ew = self._experts[e]
            if w.get("gate") is None:
                continue
            ew.gate = w["gate"][e].ctypes.data
            ew.up = w["up"][e].ctypes.data
            ew.down = w["down"][e].ctypes.data
            if w.get("bias_gate") is not None:
                ew.bias_gate = w["bias_gate"][e].ctypes.data
                ew.bias_up = w["bias_up"][e].ctypes.data
                ew.bias_down = w["bias_down"][e].ctypes.data
        self.c = PoLayer()
        self.c.desc = desc
        self.c.router = w["router"].ctypes.data
        if w.get("logit_bias") is not None:
            self.c.logit_bias = w["logit_bias"].ctypes.data
        if w.get("select_bias") is not None:
            self.c.select_bias = w["select_bias"].ctypes.data
        self.c.experts = self._experts
        if desc.shared:
            self.c.shared.gate = w["shared_gate"].ctypes.data
            self.c.shared.up = w["shared_up"].ctypes.data
            self.c.shared.down = w["shared_down"].ctypes.data
            if w.get("shared_gate_inp") is not None:
                self.c.shared_gate_inp = w["shared_gate_inp"].ctypes.data

    # --- split steps ---
    def router_logits(self, x):
        x = _f32(x)
        T = x.shape[0]
        D = self.desc
        out = np.empty((T, D.n_exp), np.float32)
        lib().po_router_logits(_p(self.w["router"]), _p(self.w.get("logit_bias")), _p(x), T, D.n_exp, D.d, _p(out))
        return out

    def route_logits(self, logits):
        logits = _f32(logits)
        T = logits.shape[0]
        ids = np.empty((T, self.desc.top_k), np.uint32)
        w = np.empty((T, self.desc.top_k), np.float32)
        rc = lib().po_route(C.byref(self.desc), _p(logits), _p(self.w.get("select_bias")), T, _p(ids), _p(w))
        if rc:
            raise ValueError(f"po_route: {rc}")
        return ids, w

    def route(self, x):
        return self.route_logits(self.router_logits(x))

    def plan(self, ids):
        return plan(ids, self.desc.n_exp)

    def experts(self, x, ids, w):
        x = _f32(x)
        T = x.shape[0]
        ids = np.ascontiguousarray(ids, np.uint32)
        w = _f32(w)
        out = np.empty((T * self.desc.top_k, self.desc.d), np.float32)
        rc = lib().po_experts(C.byref(self.c), _p(x), T, _p(ids), _p(w), _p(out))
        if rc:
            raise ValueError(f"po_experts: {rc}")
        return out

    def forward(self, x, threads=0, accumulate_into=None):
        x = _f32(x)
        T = x.shape[0]
        y = np.zeros((T, self.desc.d), np.float32) if accumulate_into is None else accumulate_into
        rc = lib().po_moe_forward(C.byref(self.c), _p(x), T, _p(y), int(accumulate_into is not None),
                                  threads or os.cpu_count() or 1)
        if rc:
            raise ValueError(f"po_moe_forward: {rc}")
        return y

    def forward_fast(self, x, threads=0):
        x = _f32(x)
        T = x.shape[0]
        y = np.zeros((T, self.desc.d), np.float32)
        rc = lib().po_moe_forward_fast(C.byref(self.c), _p(x), T, _p(y), threads or os.cpu_count() or 1)
        if rc:
            raise ValueError(f"po_moe_forward_fast: {rc}")
        return y


def plan(ids, n_exp):
    ids = np.ascontiguousarray(ids, np.uint32)
    T, K = ids.shape
    active = np.zeros(n_exp, np.uint32)
    offset = np.zeros(n_exp, np.uint32)
    count = np.zeros(n_exp, np.uint32)
    ptok = np.zeros(T * K, np.uint32)
    ppos = np.zeros(T * K, np.uint32)
    na = lib().po_plan(_p(ids), T, K, n_exp, _p(active), _p(offset), _p(count), _p(ptok), _p(ppos))
    return dict(n_active=na, active=active, offset=offset, count=count, pair_token=ptok, pair_pos=ppos)


def combine(desc, pair_out, pair_pos, w, shared_out=None, gate_logit=None, y=None):
    pair_out = _f32(pair_out)
    w = _f32(w)
    T = w.shape[0]
    acc = y is not None
    if y is None:
        y = np.zeros((T, desc.d), np.float32)
    pair_pos = np.ascontiguousarray(pair_pos, np.uint32)
    so = None if shared_out is None else _f32(shared_out)
    gl = None if gate_logit is None else _f32(gate_logit)
    lib().po_combine(C.byref(desc), _p(pair_out), _p(pair_pos), _p(w), _p(so), _p(gl), T, _p(y), int(acc))
    return y


def stack_forward(layers, eps, x, threads=0):
    x = _f32(x)
    T = x.shape[0]
    arr = (PoLayer * len(layers))(*[l.c for l in layers])
    out = np.empty_like(x)
    rc = lib().po_stack_forward(arr, len(layers), eps, _p(x), T, _p(out), threads or os.cpu_count() or 1)
    if rc:
        raise ValueError(f"po_stack_forward: {rc}")
    return out
