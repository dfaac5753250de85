"""GGUF files -> MoE layers of the library.

A reader for the GGUF container (the format the reference loads every model from,
src/gguf.rs:347-433: magic, version >= 2, key/value metadata, tensor directory, data
aligned to `general.alignment`), the MoE hyper-parameters the reference reads from it
(src/moe.rs:746-765) and the per-layer expert tensors it uploads (src/moe.rs:891-906:
`blk.N.ffn_gate_inp.weight`, `ffn_{gate,up,down}_exps.weight`, `exp_probs_b.bias`,
`ffn_*_shexp.weight`). The expert tensors are `[E][rows][cols]` blocks exactly as
`pm_layer_set_expert` takes them, so loading is a memory map and one call per expert.

A writer for the same container is included: the tests build small files with it, and
it is what turns synthetic weights into a file other GGUF tools can open.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np

from . import synth

MAGIC = b"GGUF"
# value types of the metadata section
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f",
           T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}
# ggml type id -> (values per block, bytes per block) of the types this library takes
BLOCK = {0: (1, 4), 1: (1, 2), 30: (1, 2), synth.Q8_0: (32, 34), synth.Q4_K: (256, 144), synth.Q6_K: (256, 210),
         synth.IQ4_NL: (32, 18), synth.IQ4_XS: (256, 136), synth.MXFP4: (32, 17)}


class GGUFError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    dims: tuple  # ne[0] (fastest, a row's values) first, as stored
    type: int
    offset: int  # absolute, in the file

    @property
    def n_values(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        if self.type not in BLOCK:
            raise GGUFError(f"tensor {self.name}: ggml type {self.type} is not handled")
        bv, bb = BLOCK[self.type]
        if self.dims[0] % bv:
            raise GGUFError(f"tensor {self.name}: rows of {self.dims[0]} values are not whole blocks of type {self.type}")
        return self.n_values // bv * bb


class _Reader:
    def __init__(self, buf):
        self.b, self.at = buf, 0

    def take(self, n):
        if self.at + n > len(self.b):
            raise GGUFError("unexpected end of file")
        v = self.b[self.at:self.at + n]
        self.at += n
        return v

    def scalar(self, t):
        fmt = _SCALAR[t]
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self):
        return bytes(self.take(self.scalar(T_U64))).decode("utf-8", "replace")

    def value(self, t):
        if t in _SCALAR:
            return self.scalar(t)
        if t == T_STR:
            return self.string()
        if t == T_ARR:
            et, n = self.scalar(T_U32), self.scalar(T_U64)
            return [self.value(et) for _ in range(n)]
        raise GGUFError(f"metadata value type {t}")


class GGUFFile:
    """A memory-mapped GGUF file: `.meta` (dict), `.tensors` (name -> TensorInfo)."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        r = _Reader(memoryview(self._map))
        if bytes(r.take(4)) != MAGIC:
            raise GGUFError(f"{path} is not a GGUF file")
        self.version = r.scalar(T_U32)
        if self.version < 2:
            raise GGUFError(f"GGUF version {self.version} is too old")  # src/gguf.rs:356
        nt, nkv = r.scalar(T_U64), r.scalar(T_U64)
        self.meta = {}
        for _ in range(nkv):
            k = r.string()
            self.meta[k] = r.value(r.scalar(T_U32))
        directory = []
        for _ in range(nt):
            name = r.string()
            nd = r.scalar(T_U32)
            dims = tuple(r.scalar(T_U64) for _ in range(nd))
            ty, off = r.scalar(T_U32), r.scalar(T_U64)
            directory.append((name, dims, ty, off))
        self.alignment = int(self.meta.get("general.alignment", 32))
        self.data_start = (r.at + self.alignment - 1) // self.alignment * self.alignment
        self.tensors = {}
        for name, dims, ty, off in directory:
            t = TensorInfo(name, dims, ty, self.data_start + off)
            if ty in BLOCK and t.offset + t.nbytes > len(self._map):
                raise GGUFError(f"tensor {name} runs past the end of the file")  # src/gguf.rs:385
            self.tensors[name] = t
        r.b.release()

    def close(self):
        """Unmaps the file, unless arrays returned by raw()/f32() still view it (then the map lives
        as long as they do)."""
        try:
            self._map.close()
        except BufferError:
            pass
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def arch(self) -> str:
        return self.meta.get("general.architecture", "")

    def tensor(self, name: str) -> TensorInfo:
        if name not in self.tensors:
            raise GGUFError(f"tensor {name} not in the GGUF file")
        return self.tensors[name]

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as stored (a view of the map)."""
        t = self.tensor(name)
        return np.frombuffer(self._map, np.uint8, t.nbytes, t.offset)

    def f32(self, name: str) -> np.ndarray:
        """An F32 / F16 / BF16 tensor as float32, shaped [..., ne1, ne0]."""
        t = self.tensor(name)
        raw = self.raw(name)
        if t.type == 0:
            a = raw.view(np.float32)
        elif t.type == 1:
            a = raw.view(np.float16).astype(np.float32)
        elif t.type == 30:
            a = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
        else:
            raise GGUFError(f"tensor {name}: type {t.type} is not a float type")
        return np.ascontiguousarray(a.reshape(tuple(reversed(t.dims))))


def moe_config(g: GGUFFile, layer: int = 0) -> synth.Config:
    """The layer descriptor fields the reference derives from the file (src/moe.rs:746-765)."""
    a = g.arch

    def key(k):
        return f"{a}.{k}"

    def need(k):
        if key(k) not in g.meta:
            raise GGUFError(f"GGUF key {key(k)} missing")
        return g.meta[key(k)]

    ff = g.meta.get(key("expert_feed_forward_length"), g.meta.get(key("feed_forward_length")))
    if ff is None:
        raise GGUFError(f"GGUF key {key('expert_feed_forward_length')} missing")
    gating_func = int(g.meta.get(key("expert_gating_func"), 1))  # 1 softmax, 2 sigmoid
    gate = g.tensor(f"blk.{layer}.ffn_gate_exps.weight")
    up = g.tensor(f"blk.{layer}.ffn_up_exps.weight")
    down = g.tensor(f"blk.{layer}.ffn_down_exps.weight")
    shared = f"blk.{layer}.ffn_up_shexp.weight" in g.tensors
    gated = f"blk.{layer}.ffn_gate_inp_shexp.weight" in g.tensors
    f32_acts = gate.type == synth.MXFP4
    return synth.Config(
        name=g.meta.get("general.name", a), d=int(need("embedding_length")), ff=int(ff), n_exp=int(need("expert_count")),
        top_k=int(need("expert_used_count")),
        gating=synth.GATE_SIGMOID if gating_func == 2 else synth.GATE_SOFTMAX_ALL,
        norm_w=int(bool(g.meta.get(key("expert_weights_norm"), a in ("qwen3moe", "llama", "mixtral")))),
        w_scale=float(g.meta.get(key("expert_weights_scale"), 0.0)),
        type_gate=gate.type, type_up=up.type, type_down=down.type,
        act_quant=synth.AQ_F32 if f32_acts else (synth.AQ_Q8_32 if gate.type in (synth.Q8_0, synth.IQ4_NL, synth.IQ4_XS) else synth.AQ_Q8X_256),
        weight_fold=synth.FOLD_IN_COMBINE if f32_acts else synth.FOLD_BEFORE_DOWN,
        shared=(synth.SHARED_SIGMOID_GATED if gated else synth.SHARED_PLAIN) if shared else synth.SHARED_NONE,
        shared_ff=int(g.tensor(f"blk.{layer}.ffn_up_shexp.weight").dims[1]) if shared else 0,
        n_layers=int(g.meta.get(key("block_count"), 1)))


def layer_weights(g: GGUFFile, layer: int, cfg: synth.Config | None = None) -> dict:
    """The weight dict `MoeLayer.load` / `oracle.Layer` take, as views of the file."""
    cfg = cfg or moe_config(g, layer)
    E = cfg.n_exp

    def t(n):
        return f"blk.{layer}.{n}"

    def experts(name, rows, cols, ty):
        info = g.tensor(name)
        if tuple(info.dims) != (cols, rows, E) or info.type != ty:
            raise GGUFError(f"{name}: dims {info.dims} type {info.type}, expected {(cols, rows, E)} type {ty}")
        return g.raw(name).reshape(E, -1)

    w = {"router": g.f32(t("ffn_gate_inp.weight")).reshape(E, cfg.d),
         "gate": experts(t("ffn_gate_exps.weight"), cfg.ff, cfg.d, cfg.type_gate),
         "up": experts(t("ffn_up_exps.weight"), cfg.ff, cfg.d, cfg.type_up),
         "down": experts(t("ffn_down_exps.weight"), cfg.d, cfg.ff, cfg.type_down)}
    if t("exp_probs_b.bias") in g.tensors:
        w["select_bias"] = g.f32(t("exp_probs_b.bias")).reshape(E)
    if cfg.shared:
        w["shared_gate"] = g.raw(t("ffn_gate_shexp.weight"))
        w["shared_up"] = g.raw(t("ffn_up_shexp.weight"))
        w["shared_down"] = g.raw(t("ffn_down_shexp.weight"))
        if cfg.shared == synth.SHARED_SIGMOID_GATED:
            w["shared_gate_inp"] = g.f32(t("ffn_gate_inp_shexp.weight")).reshape(cfg.d)
    return w


def load_moe_layer(ctx, g: GGUFFile, layer: int, **overrides):
    """A `MoeLayer` on `ctx` holding layer `layer` of the file. `overrides` replace fields of
    the derived configuration (e.g. `act_limit`, `n_group`, `first_local_expert`)."""
    from . import MoeLayer

    cfg = moe_config(g, layer).scaled(**overrides) if overrides else moe_config(g, layer)
    return MoeLayer(ctx, cfg).load(layer_weights(g, layer, cfg))


# ---- writer -------------------------------------------------------------------------
def _w_str(out, s):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _w_val(out, v):
    if isinstance(v, bool):
        out += struct.pack("<I?", T_BOOL, v)
    elif isinstance(v, int):
        out += struct.pack("<Iq", T_I64, v) if v < 0 else struct.pack("<II", T_U32, v) if v < 2 ** 32 else struct.pack("<IQ", T_U64, v)
    elif isinstance(v, float):
        out += struct.pack("<If", T_F32, v)
    elif isinstance(v, str):
        out += struct.pack("<I", T_STR)
        _w_str(out, v)
    else:
        raise GGUFError(f"metadata value {v!r}")


def write_gguf(path: str, meta: dict, tensors: dict, alignment: int = 32):
    """tensors: name -> (dims with ne[0] first, ggml type id, bytes-like)."""
    out = bytearray(MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta) + 1))
    _w_str(out, "general.alignment")
    _w_val(out, alignment)
    for k, v in meta.items():
        _w_str(out, k)
        _w_val(out, v)
    offs, off = {}, 0
    for name, (dims, ty, data) in tensors.items():
        offs[name] = off
        off = (off + len(memoryview(data).cast("B")) + alignment - 1) // alignment * alignment
    for name, (dims, ty, data) in tensors.items():
        _w_str(out, name)
        out += struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", ty, offs[name])
    out += b"\0" * (-len(out) % alignment)
    with open(path, "wb") as f:
        f.write(out)
        at = 0
        for name, (dims, ty, data) in tensors.items():
            f.write(b"\0" * (offs[name] - at))
            b = memoryview(data).cast("B")
            f.write(b)
            at = offs[name] + len(b)


def write_moe_layers(path: str, cfg: synth.Config, layers: list, arch: str = "qwen3moe"):
    """A GGUF file holding `layers` (weight dicts as `synth.make_weights` returns) of shape `cfg`."""
    meta = {"general.architecture": arch, "general.name": cfg.name, f"{arch}.block_count": len(layers),
            f"{arch}.embedding_length": cfg.d, f"{arch}.expert_feed_forward_length": cfg.ff,
            f"{arch}.expert_count": cfg.n_exp, f"{arch}.expert_used_count": cfg.top_k,
            f"{arch}.expert_gating_func": 2 if cfg.gating == synth.GATE_SIGMOID else 1,
            f"{arch}.expert_weights_norm": bool(cfg.norm_w), f"{arch}.expert_weights_scale": float(cfg.w_scale)}
    E, d, ff = cfg.n_exp, cfg.d, cfg.ff
    tensors = {}
    for i, w in enumerate(layers):
        p = f"blk.{i}."
        tensors[p + "ffn_gate_inp.weight"] = ((d, E), 0, np.ascontiguousarray(w["router"], np.float32))
        tensors[p + "ffn_gate_exps.weight"] = ((d, ff, E), cfg.type_gate, np.ascontiguousarray(w["gate"]))
        tensors[p + "ffn_up_exps.weight"] = ((d, ff, E), cfg.type_up, np.ascontiguousarray(w["up"]))
        tensors[p + "ffn_down_exps.weight"] = ((ff, d, E), cfg.type_down, np.ascontiguousarray(w["down"]))
        if "select_bias" in w:
            tensors[p + "exp_probs_b.bias"] = ((E,), 0, np.ascontiguousarray(w["select_bias"], np.float32))
        if cfg.shared:
            sf = cfg.shared_ff
            tensors[p + "ffn_gate_shexp.weight"] = ((d, sf), cfg.type_gate, np.ascontiguousarray(w["shared_gate"]))
            tensors[p + "ffn_up_shexp.weight"] = ((d, sf), cfg.type_up, np.ascontiguousarray(w["shared_up"]))
            tensors[p + "ffn_down_shexp.weight"] = ((sf, d), cfg.type_down, np.ascontiguousarray(w["shared_down"]))
            if "shared_gate_inp" in w:
                tensors[p + "ffn_gate_inp_shexp.weight"] = ((d,), 0, np.ascontiguousarray(w["shared_gate_inp"], np.float32))
    write_gguf(path, meta, tensors)
