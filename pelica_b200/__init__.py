"""pelica_b200 - the B200 (sm_100a) mixture-of-experts FFN path of Pelica.

A thin host-side mirror of the C ABI in include/pelica_moe.h (ctypes). The
names follow the reference's operator seams: `route` / `plan` / `experts` /
`combine` are the pieces of its FFN op block (src/moe.rs:1377-1437), `forward`
is the whole block, `Stack` is the engines' layer loop reduced to its MoE part.

Everything computes on the GPU through libpelica_moe.so. There is no CPU
fallback: importing works anywhere, but creating a Context without the built
library or without a CUDA device raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import synth
from .synth import Config  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libpelica_moe.so")

PM_FWD_ACCUMULATE = 1


class PelicaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code


class LayerDesc(C.Structure):
    """pm_layer_desc"""

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


class PlanOut(C.Structure):
    """pm_plan_out"""

    _fields_ = [("n_active", C.c_void_p), ("active", C.c_void_p), ("offset", C.c_void_p),
                ("count", C.c_void_p), ("pair_token", C.c_void_p), ("pair_pos", C.c_void_p)]


# every symbol include/pelica_moe.h declares: name -> (restype, argtypes)
_VP = C.c_void_p
ABI = {
    "pm_last_error": (C.c_char_p, []),
    "pm_version": (C.c_char_p, []),
    "pm_type_block_bytes": (C.c_size_t, [C.c_int32]),
    "pm_type_block_values": (C.c_size_t, [C.c_int32]),
    "pm_ctx_create": (C.c_int32, [C.c_int32, C.POINTER(_VP)]),
    "pm_ctx_create_on_stream": (C.c_int32, [C.c_int32, _VP, C.POINTER(_VP)]),
    "pm_ctx_destroy": (C.c_int32, [_VP]),
    "pm_sync": (C.c_int32, [_VP]),
    "pm_ctx_set_tensor_core_min_tokens": (C.c_int32, [_VP, C.c_int32]),
    "pm_ctx_stream": (_VP, [_VP]),
    "pm_host_alloc": (C.c_int32, [_VP, C.c_size_t, C.POINTER(_VP)]),
    "pm_host_free": (C.c_int32, [_VP, _VP]),
    "pm_dev_alloc": (C.c_int32, [_VP, C.c_size_t, C.POINTER(_VP)]),
    "pm_dev_free": (C.c_int32, [_VP, _VP]),
    "pm_copy": (C.c_int32, [_VP, _VP, _VP, C.c_size_t]),
    "pm_layer_create": (C.c_int32, [_VP, C.POINTER(LayerDesc), C.POINTER(_VP)]),
    "pm_layer_destroy": (C.c_int32, [_VP]),
    "pm_layer_set_router": (C.c_int32, [_VP, _VP, C.c_int32, _VP, _VP]),
    "pm_layer_set_expert": (C.c_int32, [_VP, C.c_int32, _VP, _VP, _VP, _VP, _VP, _VP]),
    "pm_layer_set_shared": (C.c_int32, [_VP, _VP, _VP, _VP, _VP]),
    "pm_layer_read_usage": (C.c_int32, [_VP, _VP]),
    "pm_moe_forward": (C.c_int32, [_VP, _VP, C.c_int32, _VP, C.c_uint32]),
    "pm_router_logits": (C.c_int32, [_VP, _VP, C.c_int32, _VP]),
    "pm_route": (C.c_int32, [_VP, _VP, C.c_int32, _VP, _VP]),
    "pm_route_logits": (C.c_int32, [_VP, _VP, C.c_int32, _VP, _VP]),
    "pm_route_noalloc": (C.c_int32, [_VP, _VP, C.c_int32, _VP, _VP]),
    "pm_plan": (C.c_int32, [_VP, _VP, C.c_int32, C.POINTER(PlanOut)]),
    "pm_experts": (C.c_int32, [_VP, _VP, C.c_int32, _VP, _VP, _VP]),
    "pm_experts_rows": (C.c_int32, [_VP, _VP, C.c_int32, _VP, _VP, _VP]),
    "pm_shared": (C.c_int32, [_VP, _VP, C.c_int32, _VP]),
    "pm_combine": (C.c_int32, [_VP, _VP, _VP, _VP, _VP, C.c_int32, _VP, C.c_uint32]),
    "pm_ep_unique_id": (C.c_int32, [_VP]),
    "pm_ep_init": (C.c_int32, [_VP, _VP, C.c_int32, C.c_int32, C.POINTER(_VP)]),
    "pm_ep_destroy": (C.c_int32, [_VP]),
    "pm_ep_set_timeout_ms": (C.c_int32, [_VP, C.c_int64]),
    "pm_moe_forward_ep": (C.c_int32, [_VP, _VP, _VP, C.c_int32, _VP, C.c_uint32]),
    "pm_ep_last_stats": (C.c_int32, [_VP, _VP]),
    "pm_placement_create": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.POINTER(_VP)]),
    "pm_placement_destroy": (C.c_int32, [_VP]),
    "pm_placement_observe": (C.c_int32, [_VP, C.c_int32, _VP]),
    "pm_placement_plan": (C.c_int32, [_VP, C.c_uint64, C.c_uint64, _VP, C.c_int32, C.POINTER(C.c_int32)]),
    "pm_placement_slots": (C.c_int32, [_VP, C.c_int32, _VP]),
    "pm_placement_scores": (C.c_int32, [_VP, C.c_int32, _VP, _VP]),
    "pm_ep_set_slots": (C.c_int32, [_VP, _VP, _VP]),
    "pm_ep_get_slots": (C.c_int32, [_VP, _VP, _VP]),
    "pm_ep_swap_experts": (C.c_int32, [_VP, _VP, C.c_int32, C.c_int32]),
    "pm_dequant": (C.c_int32, [_VP, C.c_int32, _VP, C.c_size_t, _VP]),
    "pm_quant_act": (C.c_int32, [_VP, C.c_int32, _VP, C.c_size_t, _VP, _VP, _VP]),
    "pm_rmsnorm": (C.c_int32, [_VP, _VP, C.c_int32, C.c_int32, C.c_float, _VP]),
    "pm_stack_create": (C.c_int32, [_VP, C.POINTER(_VP), C.c_int32, C.c_float, C.POINTER(_VP)]),
    "pm_stack_destroy": (C.c_int32, [_VP]),
    "pm_stack_forward": (C.c_int32, [_VP, _VP, C.c_int32, _VP]),
    "pm_stack_set_mode": (C.c_int32, [_VP, C.c_int32]),
    "pm_stack_decode_kernel_available": (C.c_int32, [_VP]),
    "pm_stack_status": (C.c_int32, [_VP]),
    "pm_layer_fill_synthetic": (C.c_int32, [_VP, C.c_uint64, C.c_float, C.c_float, C.c_float]),
    "pm_layer_get_expert_bias": (C.c_int32, [_VP, C.c_int32, _VP, _VP, _VP]),
    "pm_layer_get_expert": (C.c_int32, [_VP, C.c_int32, C.c_int32, _VP]),
    "pm_layer_get_router": (C.c_int32, [_VP, _VP, _VP, _VP]),
}

# measurement and test hooks (include/pelica_moe_diag.h)
ABI_DIAG = {
    "pm_ctx_launch_count": (C.c_int64, [_VP]),
    "pm_ctx_path_counts": (C.c_int32, [_VP, _VP]),
    "pm_timer_start": (C.c_int32, [_VP]),
    "pm_timer_stop": (C.c_int32, [_VP, C.POINTER(C.c_float)]),
    "pm_flush_l2": (C.c_int32, [_VP]),
    "pm_profile_enable": (C.c_int32, [_VP, C.c_int32]),
    "pm_profile_phases": (C.c_int32, []),
    "pm_profile_phase_name": (C.c_char_p, [C.c_int32]),
    "pm_profile_read": (C.c_int32, [_VP, _VP, _VP]),
    "pm_stack_trace": (C.c_int32, [_VP, _VP, C.c_int32]),
    "pm_debug_set_wait_limit_ns": (C.c_int32, [_VP, C.c_uint64]),
    "pm_debug_stack_fault_next_call": (C.c_int32, [_VP]),
    "pm_debug_tc_fault_block": (C.c_int32, [_VP, C.c_int32]),
    "pm_debug_device_free_bytes": (C.c_int32, [_VP, C.POINTER(C.c_uint64)]),
}
PATHS = ("general", "tensor", "decode", "multi")

_lib = None


def load_library() -> C.CDLL:
    """dlopen the CUDA library and bind every declared entry point (fails loudly)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise PelicaError(-5, f"{LIB_PATH} is missing: run `python -m pelica_b200.build` "
                                  "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in {**ABI, **ABI_DIAG}.items():
            fn = getattr(lib, name)  # AttributeError = a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _check(rc: int):
    if rc != 0:
        raise PelicaError(rc, load_library().pm_last_error().decode())


class DevBuf:
    """A device allocation owned by a Context."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx = ctx
        self.nbytes = nbytes
        p = _VP()
        _check(ctx.lib.pm_dev_alloc(ctx.h, nbytes, C.byref(p)))
        self.ptr = p.value

    def upload(self, a: np.ndarray):
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        _check(self.ctx.lib.pm_copy(self.ctx.h, self.ptr, a.ctypes.data, a.nbytes))
        return self

    def download(self, dtype, shape) -> np.ndarray:
        out = np.empty(shape, dtype)
        assert out.nbytes <= self.nbytes
        _check(self.ctx.lib.pm_copy(self.ctx.h, out.ctypes.data, self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr:
            _check(self.ctx.lib.pm_dev_free(self.ctx.h, self.ptr))
            self.ptr = None


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, DevBuf):
        return a.ptr
    return a.ctypes.data


def _f32(a):
    return a if isinstance(a, DevBuf) else np.ascontiguousarray(a, dtype=np.float32)


def _u32(a):
    return a if isinstance(a, DevBuf) else np.ascontiguousarray(a, dtype=np.uint32)


class Context:
    """One GPU: a stream, a workspace and the layers created on it."""

    def __init__(self, device: int = 0, stream=None):
        """stream: a cudaStream_t handle (int) the caller owns, or None for a private stream."""
        self.lib = load_library()
        h = _VP()
        if stream is None:
            _check(self.lib.pm_ctx_create(device, C.byref(h)))
        else:
            _check(self.lib.pm_ctx_create_on_stream(device, stream, C.byref(h)))
        self.h = h.value
        self.device = device

    def close(self):
        if self.h:
            self.lib.pm_ctx_destroy(self.h)
            self.h = None

    def sync(self):
        _check(self.lib.pm_sync(self.h))

    def set_tensor_core_min_tokens(self, n: int):
        """Expert products use the tcgen05 kernels from n tokens per call (0 = never)."""
        _check(self.lib.pm_ctx_set_tensor_core_min_tokens(self.h, n))

    @property
    def launches(self) -> int:
        return self.lib.pm_ctx_launch_count(self.h)

    def path_counts(self) -> dict:
        """Launches of the expert-product kernels per family since the context was created."""
        out = np.zeros(len(PATHS), np.int64)
        _check(self.lib.pm_ctx_path_counts(self.h, out.ctypes.data))
        return dict(zip(PATHS, (int(v) for v in out)))

    def set_wait_limit_ns(self, ns: int):
        """Test hook: the time limit of every bounded device-side wait (default 2 s)."""
        _check(self.lib.pm_debug_set_wait_limit_ns(self.h, ns))

    def tc_fault_block(self, block: int):
        """Test hook: tensor-core kernels stop issuing products at this block (-1 = off)."""
        _check(self.lib.pm_debug_tc_fault_block(self.h, block))

    def device_free_bytes(self) -> int:
        v = C.c_uint64()
        _check(self.lib.pm_debug_device_free_bytes(self.h, C.byref(v)))
        return v.value

    def timer_start(self):
        _check(self.lib.pm_timer_start(self.h))

    def timer_stop(self) -> float:
        ms = C.c_float()
        _check(self.lib.pm_timer_stop(self.h, C.byref(ms)))
        return ms.value

    def flush_l2(self):
        _check(self.lib.pm_flush_l2(self.h))

    def alloc(self, nbytes: int) -> DevBuf:
        return DevBuf(self, nbytes)

    def pinned(self, shape, dtype=np.float32) -> np.ndarray:
        """A numpy array over page-locked host memory (kept alive by the context)."""
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        p = _VP()
        _check(self.lib.pm_host_alloc(self.h, n, C.byref(p)))
        buf = (C.c_uint8 * max(n, 1)).from_address(p.value)
        self._pinned = getattr(self, "_pinned", []) + [p.value]
        return np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)

    def profile(self, on: bool):
        _check(self.lib.pm_profile_enable(self.h, int(on)))

    def profile_read(self) -> dict:
        n = self.lib.pm_profile_phases()
        ms = np.zeros(n, np.float32)
        spans = np.zeros(n, np.int64)
        _check(self.lib.pm_profile_read(self.h, ms.ctypes.data, spans.ctypes.data))
        return {self.lib.pm_profile_phase_name(i).decode(): (float(ms[i]), int(spans[i])) for i in range(n)}

    # format checks
    def dequant(self, ggml_type: int, blocks: np.ndarray, n_values: int) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, np.uint8)
        out = np.empty(n_values, np.float32)
        _check(self.lib.pm_dequant(self.h, ggml_type, blocks.ctypes.data, n_values, out.ctypes.data))
        return out

    def quant_act_32(self, x: np.ndarray):
        """`Q8::new` (src/q4x_cpu.rs:23-37): returns (q int8[n], d f32[n/32])."""
        x = np.ascontiguousarray(x, np.float32).ravel()
        n = x.size
        q = np.empty(n, np.int8)
        d = np.empty(n // 32, np.float32)
        _check(self.lib.pm_quant_act(self.h, synth.AQ_Q8_32, x.ctypes.data, n, q.ctypes.data, d.ctypes.data, None))
        return q, d

    def quant_act(self, x: np.ndarray):
        """`Q8x::new` (src/ds4_cpu.rs:13-35): returns (q int8[n], d f32[n/256], bsum i32[n/32])."""
        x = np.ascontiguousarray(x, np.float32).ravel()
        n = x.size
        q = np.empty(n, np.int8)
        d = np.empty(n // 256, np.float32)
        b = np.empty(n // 32, np.int32)
        _check(self.lib.pm_quant_act(self.h, synth.AQ_Q8X_256, x.ctypes.data, n, q.ctypes.data, d.ctypes.data,
                                     b.ctypes.data))
        return q, d, b


class MoeLayer:
    """One MoE FFN layer resident on a GPU."""

    def __init__(self, ctx: Context, cfg):
        self.ctx = ctx
        self.lib = ctx.lib
        fields = cfg.desc_fields() if hasattr(cfg, "desc_fields") else dict(cfg)
        self.desc = LayerDesc(**fields)
        h = _VP()
        _check(self.lib.pm_layer_create(ctx.h, C.byref(self.desc), C.byref(h)))
        self.h = h.value

    def close(self):
        if self.h:
            self.lib.pm_layer_destroy(self.h)
            self.h = None

    # ---- weights ----
    def load(self, w: dict) -> "MoeLayer":
        """w: the dict synth.make_weights returns (raw GGUF block bytes per expert)."""
        D = self.desc
        lb = w.get("logit_bias")
        sb = w.get("select_bias")
        router = np.ascontiguousarray(w["router"], np.float32)
        _check(self.lib.pm_layer_set_router(self.h, router.ctypes.data, synth.F32, _ptr(lb), _ptr(sb)))
        first = D.first_local_expert if D.n_exp_local > 0 else 0
        n = D.n_exp_local if D.n_exp_local > 0 else D.n_exp
        for e in range(first, first + n):
            bias = [None, None, None]
            if D.has_expert_bias:
                bias = [np.ascontiguousarray(w[k][e], np.float32) for k in ("bias_gate", "bias_up", "bias_down")]
            g, u, dn = (np.ascontiguousarray(w[k][e], np.uint8) for k in ("gate", "up", "down"))
            _check(self.lib.pm_layer_set_expert(self.h, e, g.ctypes.data, u.ctypes.data, dn.ctypes.data,
                                                _ptr(bias[0]), _ptr(bias[1]), _ptr(bias[2])))
        if D.shared:
            g, u, dn = (np.ascontiguousarray(w[k], np.uint8) for k in ("shared_gate", "shared_up", "shared_down"))
            gi = w.get("shared_gate_inp")
            _check(self.lib.pm_layer_set_shared(self.h, g.ctypes.data, u.ctypes.data, dn.ctypes.data, _ptr(gi)))
        return self

    def fill_synthetic(self, seed: int, sigma: float = 0.02, logit_bias_sigma: float = 0.0,
                       select_bias_sigma: float = 0.0) -> "MoeLayer":
        """Seeded N(0, sigma) weights generated and quantised on the device."""
        _check(self.lib.pm_layer_fill_synthetic(self.h, seed, sigma, logit_bias_sigma, select_bias_sigma))
        self._has_lb = logit_bias_sigma > 0
        self._has_sb = select_bias_sigma > 0
        return self

    def get_expert(self, e: int, which: int) -> np.ndarray:
        """Raw GGUF bytes of expert e's gate (0) / up (1) / down (2); e = -1: the shared expert."""
        D = self.desc
        ff = D.shared_ff if e < 0 else D.ff
        ty = (D.type_gate, D.type_up, D.type_down)[which]
        rows, cols = ((ff, D.d), (ff, D.d), (D.d, ff))[which]
        out = np.empty(rows * synth.row_bytes(ty, cols), np.uint8)
        _check(self.lib.pm_layer_get_expert(self.h, e, which, out.ctypes.data))
        return out

    def get_weights(self, dense: bool = True) -> dict:
        """Everything back as the dict `load` takes (used to hand device-generated
        weights to a checker). dense=False: per-expert lists in which experts this context
        does not hold are one shared empty array (a shard of a large layer stays small)."""
        D = self.desc
        router = np.empty((D.n_exp, D.d), np.float32)
        lb = np.zeros(D.n_exp, np.float32)
        sb = np.zeros(D.n_exp, np.float32)
        _check(self.lib.pm_layer_get_router(self.h, router.ctypes.data, lb.ctypes.data, sb.ctypes.data))
        w = {"router": router}
        if getattr(self, "_has_lb", False):
            w["logit_bias"] = lb
        if getattr(self, "_has_sb", False):
            w["select_bias"] = sb
        first = D.first_local_expert if D.n_exp_local > 0 else 0
        n = D.n_exp_local if D.n_exp_local > 0 else D.n_exp
        for which, key in enumerate(("gate", "up", "down")):
            rows = [self.get_expert(e, which) if first <= e < first + n else None for e in range(D.n_exp)]
            size = next(r.size for r in rows if r is not None)
            if dense:
                w[key] = np.stack([r if r is not None else np.zeros(size, np.uint8) for r in rows])
            else:
                none = np.zeros(16, np.uint8)
                w[key] = [r if r is not None else none for r in rows]
        if D.has_expert_bias:
            bg = np.zeros((D.n_exp, D.ff), np.float32)
            bu = np.zeros((D.n_exp, D.ff), np.float32)
            bd = np.zeros((D.n_exp, D.d), np.float32)
            for e in range(first, first + n):
                _check(self.lib.pm_layer_get_expert_bias(self.h, e, bg[e].ctypes.data, bu[e].ctypes.data,
                                                         bd[e].ctypes.data))
            w.update(bias_gate=bg, bias_up=bu, bias_down=bd)
        if D.shared:
            for which, key in enumerate(("shared_gate", "shared_up", "shared_down")):
                w[key] = self.get_expert(-1, which)
        return w

    def usage(self) -> np.ndarray:
        out = np.empty(self.desc.n_exp, np.uint32)
        _check(self.lib.pm_layer_read_usage(self.h, out.ctypes.data))
        return out

    # ---- the operator ----
    def forward(self, x, out=None, accumulate: bool = False):
        """y[T,d] = sum_k w * expert(x) (+ shared(x)); x host array or DevBuf."""
        x = _f32(x)
        T = x.shape[0] if not isinstance(x, DevBuf) else out.nbytes // (4 * self.desc.d)
        if out is None:
            out = np.zeros((T, self.desc.d), np.float32)
        _check(self.lib.pm_moe_forward(self.h, _ptr(x), T, _ptr(out), PM_FWD_ACCUMULATE if accumulate else 0))
        return out

    def forward_dev(self, x: DevBuf, T: int, y: DevBuf, accumulate: bool = False):
        _check(self.lib.pm_moe_forward(self.h, x.ptr, T, y.ptr, PM_FWD_ACCUMULATE if accumulate else 0))

    def router_logits(self, x) -> np.ndarray:
        x = _f32(x)
        T = x.shape[0]
        out = np.empty((T, self.desc.n_exp), np.float32)
        _check(self.lib.pm_router_logits(self.h, _ptr(x), T, out.ctypes.data))
        return out

    def route(self, x):
        x = _f32(x)
        T = x.shape[0]
        ids = np.empty((T, self.desc.top_k), np.uint32)
        w = np.empty((T, self.desc.top_k), np.float32)
        _check(self.lib.pm_route(self.h, _ptr(x), T, ids.ctypes.data, w.ctypes.data))
        return ids, w

    def route_noalloc(self, x: DevBuf, T: int, ids: DevBuf, w: DevBuf):
        """pm_route_noalloc: device buffers in and out, no allocation inside, at most 256 tokens;
        queued on the context's stream (call ctx.sync() before reading the results)."""
        _check(self.lib.pm_route_noalloc(self.h, x.ptr, T, ids.ptr, w.ptr))

    def route_logits(self, logits):
        logits = _f32(logits)
        T = logits.shape[0]
        ids = np.empty((T, self.desc.top_k), np.uint32)
        w = np.empty((T, self.desc.top_k), np.float32)
        _check(self.lib.pm_route_logits(self.h, _ptr(logits), T, ids.ctypes.data, w.ctypes.data))
        return ids, w

    def plan(self, ids) -> dict:
        ids = _u32(ids)
        T, K = ids.shape
        E = self.desc.n_exp
        r = dict(n_active=np.zeros(1, np.int32), active=np.zeros(E, np.uint32), offset=np.zeros(E, np.uint32),
                 count=np.zeros(E, np.uint32), pair_token=np.zeros(T * K, np.uint32),
                 pair_pos=np.zeros(T * K, np.uint32))
        po = PlanOut(*[r[k].ctypes.data for k in ("n_active", "active", "offset", "count", "pair_token", "pair_pos")])
        _check(self.lib.pm_plan(self.h, _ptr(ids), T, C.byref(po)))
        r["n_active"] = int(r["n_active"][0])
        return r

    def experts(self, x, ids, w) -> np.ndarray:
        x, ids, w = _f32(x), _u32(ids), _f32(w)
        T = x.shape[0]
        out = np.empty((T * self.desc.top_k, self.desc.d), np.float32)
        _check(self.lib.pm_experts(self.h, _ptr(x), T, _ptr(ids), _ptr(w), out.ctypes.data))
        return out

    def experts_rows(self, x, eids, w) -> np.ndarray:
        """One expert per row (the serving side of expert parallelism)."""
        x, eids, w = _f32(x), _u32(eids), _f32(w)
        R = x.shape[0]
        out = np.empty((R, self.desc.d), np.float32)
        _check(self.lib.pm_experts_rows(self.h, _ptr(x), R, _ptr(eids), _ptr(w), out.ctypes.data))
        return out

    def shared(self, x) -> np.ndarray:
        x = _f32(x)
        out = np.empty((x.shape[0], self.desc.d), np.float32)
        _check(self.lib.pm_shared(self.h, _ptr(x), x.shape[0], out.ctypes.data))
        return out

    def combine(self, pair_out, ids, w, shared_out=None, y=None) -> np.ndarray:
        pair_out, ids, w = _f32(pair_out), _u32(ids), _f32(w)
        T = ids.shape[0]
        acc = y is not None
        if y is None:
            y = np.zeros((T, self.desc.d), np.float32)
        so = None if shared_out is None else _f32(shared_out)
        _check(self.lib.pm_combine(self.h, _ptr(pair_out), _ptr(ids), _ptr(w), _ptr(so), T, _ptr(y),
                                   PM_FWD_ACCUMULATE if acc else 0))
        return y


class Stack:
    """x <- x + moe_l(x / rms(x)) over a list of layers (the benchmark's unit)."""

    def __init__(self, ctx: Context, layers, eps: float = 1e-6):
        self.ctx = ctx
        self.lib = ctx.lib
        self.layers = list(layers)
        arr = (_VP * len(self.layers))(*[l.h for l in self.layers])
        h = _VP()
        _check(self.lib.pm_stack_create(ctx.h, arr, len(self.layers), eps, C.byref(h)))
        self.h = h.value
        self.d = self.layers[0].desc.d

    def close(self):
        if self.h:
            self.lib.pm_stack_destroy(self.h)
            self.h = None

    def forward(self, x, out=None):
        x = _f32(x)
        if out is None:
            out = np.empty_like(x)
        T = x.shape[0]
        _check(self.lib.pm_stack_forward(self.h, _ptr(x), T, _ptr(out)))
        return out

    def forward_dev(self, x: DevBuf, T: int, out: DevBuf):
        _check(self.lib.pm_stack_forward(self.h, x.ptr, T, out.ptr))

    def set_mode(self, general_only: bool):
        """True: always the general kernels; False: one-token calls use the persistent decode kernel."""
        _check(self.lib.pm_stack_set_mode(self.h, int(general_only)))

    @property
    def decode_kernel(self) -> bool:
        return bool(self.lib.pm_stack_decode_kernel_available(self.h))

    def status(self):
        _check(self.lib.pm_stack_status(self.h))

    def fault_next_call(self):
        """Test hook: the next decode-kernel call waits for an arrival that never comes."""
        _check(self.lib.pm_debug_stack_fault_next_call(self.h))

    def trace(self, enable: bool = False):
        """Decode-kernel phase stamps (global timer, ns) of the last call: array [CTAs, layers, 16]."""
        n = self.lib.pm_stack_trace(self.h, None, 0)
        if n < 0:
            _check(n)
        if enable:
            return None
        out = np.zeros(n, np.int64)
        r = self.lib.pm_stack_trace(self.h, out.ctypes.data, n)
        if r < 0:
            _check(r)
        return out.reshape(len(out) // (len(self.layers) * 16), len(self.layers), 16)


def ep_unique_id() -> bytes:
    """128 bytes naming a new expert-parallel communicator (rank 0 makes them, every rank passes them
    to ExpertParallel)."""
    buf = (C.c_uint8 * 128)()
    _check(load_library().pm_ep_unique_id(buf))
    return bytes(buf)


class ExpertParallel:
    """One rank of an expert-parallel group (pm_ep_*): experts sharded over the ranks' GPUs,
    NCCL dispatch and combine inside the library."""

    def __init__(self, ctx: Context, unique_id: bytes, rank: int, world: int):
        self.ctx = ctx
        self.lib = ctx.lib
        self.rank, self.world = rank, world
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        h = _VP()
        _check(self.lib.pm_ep_init(ctx.h, buf, rank, world, C.byref(h)))
        self.h = h.value

    def close(self):
        if self.h:
            self.lib.pm_ep_destroy(self.h)
            self.h = None

    def set_timeout_ms(self, ms: int):
        _check(self.lib.pm_ep_set_timeout_ms(self.h, ms))

    def forward_dev(self, layer: MoeLayer, x, T: int, y, accumulate: bool = False):
        """x, y: device pointers (DevBuf or int) of [T, d] f32."""
        xp = x.ptr if isinstance(x, DevBuf) else x
        yp = y.ptr if isinstance(y, DevBuf) else y
        _check(self.lib.pm_moe_forward_ep(self.h, layer.h, xp, T, yp, PM_FWD_ACCUMULATE if accumulate else 0))

    def forward(self, layer: MoeLayer, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        T, d = x.shape
        dx = self.ctx.alloc(max(x.nbytes, 4)).upload(x) if T else self.ctx.alloc(4)
        dy = self.ctx.alloc(max(x.nbytes, 4))
        self.forward_dev(layer, dx, T, dy)
        self.ctx.sync()
        out = dy.download(np.float32, (T, d)) if T else np.zeros((0, d), np.float32)
        dx.free()
        dy.free()
        return out

    def set_slots(self, layer: MoeLayer, slot_of_expert=None):
        """The layer's placement table (None: expert e in slot e). The weights must already sit in
        the slots it names."""
        if slot_of_expert is None:
            _check(self.lib.pm_ep_set_slots(self.h, layer.h, None))
        else:
            t = np.ascontiguousarray(slot_of_expert, np.int32)
            assert t.size == layer.desc.n_exp
            _check(self.lib.pm_ep_set_slots(self.h, layer.h, t.ctypes.data))

    def get_slots(self, layer: MoeLayer) -> np.ndarray:
        t = np.zeros(layer.desc.n_exp, np.int32)
        _check(self.lib.pm_ep_get_slots(self.h, layer.h, t.ctypes.data))
        return t

    def swap_experts(self, layer: MoeLayer, a: int, b: int):
        """Collective: experts a and b change places (every rank calls it, same arguments, same order)."""
        _check(self.lib.pm_ep_swap_experts(self.h, layer.h, a, b))

    def last_stats(self) -> dict:
        out = np.zeros(4, np.uint64)
        _check(self.lib.pm_ep_last_stats(self.h, out.ctypes.data))
        return dict(rows_sent=int(out[0]), rows_received=int(out[1]), bytes_sent=int(out[2]), bytes_received=int(out[3]))


class Placement:
    """The host-side planner of usage-driven expert placement (pm_placement_*): decayed use scores
    per (layer, expert) and rounds of swaps that even out what the ranks serve."""

    def __init__(self, n_layers: int, n_exp: int, world: int):
        self.lib = load_library()
        self.n_layers, self.n_exp, self.world = n_layers, n_exp, world
        h = _VP()
        _check(self.lib.pm_placement_create(n_layers, n_exp, world, C.byref(h)))
        self.h = h.value

    def close(self):
        if self.h:
            self.lib.pm_placement_destroy(self.h)
            self.h = None

    def observe(self, layer: int, usage):
        u = np.ascontiguousarray(usage, np.uint32)
        assert u.size == self.n_exp
        _check(self.lib.pm_placement_observe(self.h, layer, u.ctypes.data))

    def plan(self, expert_bytes: int, budget_bytes: int, max_swaps: int = 256) -> list:
        """One round: [(layer, hot expert, cold expert), ...] in the order to carry them out."""
        out = np.zeros(3 * max(max_swaps, 1), np.int32)
        n = C.c_int32(0)
        _check(self.lib.pm_placement_plan(self.h, expert_bytes, budget_bytes, out.ctypes.data, max_swaps, C.byref(n)))
        return [tuple(int(v) for v in out[3 * i:3 * i + 3]) for i in range(n.value)]

    def slots(self, layer: int) -> np.ndarray:
        t = np.zeros(self.n_exp, np.int32)
        _check(self.lib.pm_placement_slots(self.h, layer, t.ctypes.data))
        return t

    def scores(self, layer: int):
        s, r = np.zeros(self.n_exp, np.float32), np.zeros(self.world, np.float32)
        _check(self.lib.pm_placement_scores(self.h, layer, s.ctypes.data, r.ctypes.data))
        return s, r
