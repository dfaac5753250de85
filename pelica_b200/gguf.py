"""GGUF files -> MoE layers of the library.

A reader for the GGUF container (the format the reference loads every model from,
src/gguf.rs:347-433: magic, version >= 2, key/value metadata, tensor directory, data
aligned to `general.alignment`), the MoE hyper-parameters the reference reads from it
(src/moe.rs:746-765) and the per-layer expert tensors it uploads (src/moe.rs:891-906:
`blk.N.ffn_gate_inp.weight`, `ffn_{gate,up,down}_exps.weight`, `exp_probs_b.bias`,
`ffn_*_shexp.weight`). The expert tensors are `[E][rows][cols]` blocks exactly as
`pm_layer_set_expert` takes them, so loading is a memory map and one call per expert.

Layers whose expert tensors are named `*_expm` hold each expert's gate, up and down rows
side by side (the layout `pelica repack` writes so that one read fetches an expert,
src/repack.rs:1-24; read back by src/ds4.rs:683-707, src/ds4_io.rs:54-87): `layer_weights`
reads both layouts, `repack` / `repack(undo=True)` convert a file in place.

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
         synth.IQ4_NL: (32, 18), synth.IQ4_XS: (256, 136), synth.MXFP4: (32, 17), synth.Q5_K: (256, 176),
         synth.IQ3_S: (256, 110)}
PIECES = ("ffn_gate", "ffn_up", "ffn_down")


class GGUFError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    dims: tuple  # ne[0] (fastest, a row's values) first, as stored
    type: int
    offset: int  # absolute, in the file
    name_at: int = 0  # where the name's bytes start in the header
    offset_at: int = 0  # where the u64 offset (relative to the data section) sits in the header

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
            name_at = r.at + 8
            name = r.string()
            nd = r.scalar(T_U32)
            dims = tuple(r.scalar(T_U64) for _ in range(nd))
            ty = r.scalar(T_U32)
            offset_at = r.at
            off = r.scalar(T_U64)
            directory.append((name, dims, ty, off, name_at, offset_at))
        self.alignment = int(self.meta.get("general.alignment", 32))
        self.data_start = (r.at + self.alignment - 1) // self.alignment * self.alignment
        self.tensors = {}
        for name, dims, ty, off, name_at, offset_at in directory:
            t = TensorInfo(name, dims, ty, self.data_start + off, name_at, offset_at)
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
    tag = "expm" if layer_is_repacked(g, layer) else "exps"
    gate = g.tensor(f"blk.{layer}.ffn_gate_{tag}.weight")
    up = g.tensor(f"blk.{layer}.ffn_up_{tag}.weight")
    down = g.tensor(f"blk.{layer}.ffn_down_{tag}.weight")
    shared = f"blk.{layer}.ffn_up_shexp.weight" in g.tensors
    gated = f"blk.{layer}.ffn_gate_inp_shexp.weight" in g.tensors
    f32_acts = gate.type in (synth.MXFP4, synth.Q5_K)
    q8_32 = (synth.Q8_0, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_S)
    return synth.Config(
        name=g.meta.get("general.name", a), d=int(need("embedding_length")), ff=int(ff), n_exp=int(need("expert_count")),
        top_k=int(need("expert_used_count")),
        gating=synth.GATE_SIGMOID if gating_func == 2 else synth.GATE_SOFTMAX_ALL,
        norm_w=int(bool(g.meta.get(key("expert_weights_norm"), a in ("qwen3moe", "llama", "mixtral")))),
        w_scale=float(g.meta.get(key("expert_weights_scale"), 0.0)),
        type_gate=gate.type, type_up=up.type, type_down=down.type,
        act_quant=synth.AQ_F32 if f32_acts else (synth.AQ_Q8_32 if gate.type in q8_32 else synth.AQ_Q8X_256),
        weight_fold=synth.FOLD_IN_COMBINE if f32_acts else synth.FOLD_BEFORE_DOWN,
        shared=(synth.SHARED_SIGMOID_GATED if gated else synth.SHARED_PLAIN) if shared else synth.SHARED_NONE,
        shared_ff=int(g.tensor(f"blk.{layer}.ffn_up_shexp.weight").dims[1]) if shared else 0,
        n_layers=int(g.meta.get(key("block_count"), 1)))


def layer_is_repacked(g: GGUFFile, layer: int) -> bool:
    """Whether the layer's expert tensors carry the `*_expm` names (`layer_state`,
    src/repack.rs:62-69); a layer with only some of them renamed was interrupted."""
    m = sum(f"blk.{layer}.{p}_expm.weight" in g.tensors for p in PIECES)
    if m not in (0, 3):
        raise GGUFError(f"layer {layer} was left half repacked: repack the file again to finish")
    return m == 3


def layer_weights(g: GGUFFile, layer: int, cfg: synth.Config | None = None) -> dict:
    """The weight dict `MoeLayer.load` / `oracle.Layer` take, as views of the file."""
    cfg = cfg or moe_config(g, layer)
    E = cfg.n_exp
    merged = layer_is_repacked(g, layer)

    def t(n):
        return f"blk.{layer}.{n}"

    shapes = ((cfg.ff, cfg.d, cfg.type_gate), (cfg.ff, cfg.d, cfg.type_up), (cfg.d, cfg.ff, cfg.type_down))
    infos = []
    for piece, (rows, cols, ty) in zip(PIECES, shapes):
        name = t(f"{piece}_{'expm' if merged else 'exps'}.weight")
        info = g.tensor(name)
        if tuple(info.dims) != (cols, rows, E) or info.type != ty:
            raise GGUFError(f"{name}: dims {info.dims} type {info.type}, expected {(cols, rows, E)} type {ty}")
        infos.append(info)
    if merged:
        # expert e's gate, up and down bytes follow one another from the region's start (the
        # lowest of the three tensor offsets, which repacking never changes): src/ds4.rs:697-704
        lens = [i.nbytes // E for i in infos]
        stride, base = sum(lens), min(i.offset for i in infos)
        if base + stride * E > len(g._map):
            raise GGUFError(f"layer {layer}: the repacked experts run past the end of the file")
        region = np.frombuffer(g._map, np.uint8, stride * E, base).reshape(E, stride)
        ex = [region[:, sum(lens[:i]):sum(lens[:i + 1])] for i in range(3)]
    else:
        ex = [g.raw(i.name).reshape(E, -1) for i in infos]
    w = {"router": g.f32(t("ffn_gate_inp.weight")).reshape(E, cfg.d), "gate": ex[0], "up": ex[1], "down": ex[2]}
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


# ---- repacking -----------------------------------------------------------------------
def _layer_region(g: GGUFFile, layer: int):
    """The layer's expert region as `layers` of src/repack.rs:118-205 describes it: the three
    tensor offsets and per-expert lengths, the gaps between the tensors as first written, and the
    other tensors that sit in those gaps."""
    tag = "expm" if layer_is_repacked(g, layer) else "exps"
    infos = [g.tensor(f"blk.{layer}.{p}_{tag}.weight") for p in PIECES]
    E = infos[0].dims[2]
    off = [i.offset for i in infos]
    lens = [i.nbytes // E for i in infos]
    base, total = min(off), sum(lens) * E
    holes, at = [], base
    for i in sorted(range(3), key=lambda i: off[i]):
        if off[i] > at:
            holes.append((at - base, off[i] - at))
        at = max(at, off[i] + lens[i] * E)
    span = at - base

    def packed_hole(h):
        return total + sum(x[1] for x in holes[:h])

    ok = span == total + sum(x[1] for x in holes) and all(
        a + n <= total and (packed_hole(h) - a) % g.alignment == 0 for h, (a, n) in enumerate(holes))
    movers = []
    if ok:
        mine = {i.name for i in infos}
        for name, t in g.tensors.items():
            r = t.offset - base
            if r < 0 or r >= span or name in mine:
                continue
            for h, (a, n) in enumerate(holes):
                if r >= a and r + t.nbytes <= a + n:
                    movers.append((t, h, False))
                    break
                pa = packed_hole(h)
                if r >= pa and r + t.nbytes <= pa + n:
                    movers.append((t, h, True))
                    break
            else:
                ok = False
    return dict(infos=infos, E=E, off=off, lens=lens, base=base, total=total, holes=holes, span=span,
                packed_hole=packed_hole, movers=movers, ok=ok, merged=tag == "expm")


def repack(path: str, undo: bool = False) -> int:
    """Rewrites a GGUF file in place so that every layer keeps each expert's gate, up and down bytes
    together (or, with `undo`, apart again), renaming `*_exps` <-> `*_expm` as `pelica repack` does
    (src/repack.rs:1-24): the tensors' recorded offsets never change, the bytes of other tensors
    that sat between the expert tensors follow the experts and their offsets move in the header.
    Returns the number of layers converted. (No journal: a tool for files that can be written
    again, not a crash-safe converter.)"""
    with GGUFFile(path) as g:
        layers = sorted({int(n.split(".")[1]) for n in g.tensors
                         if n.startswith("blk.") and n.endswith(("_exps.weight", "_expm.weight"))})
        plans = [(l, _layer_region(g, l)) for l in layers]
        data_start = g.data_start
    done = 0
    with open(path, "r+b") as f:
        for l, y in plans:
            if not y["ok"] or y["merged"] != undo:
                continue
            base, E, lens, off, total = y["base"], y["E"], y["lens"], y["off"], y["total"]
            f.seek(base)
            old = f.read(y["span"])
            new = bytearray(y["span"])
            stride = sum(lens)
            for e in range(E):
                for i in range(3):
                    apart = off[i] - base + e * lens[i]
                    together = e * stride + sum(lens[:i])
                    src, dst = (together, apart) if undo else (apart, together)
                    new[dst:dst + lens[i]] = old[src:src + lens[i]]
            for h, (a, n) in enumerate(y["holes"]):
                pa = y["packed_hole"](h)
                src, dst = (pa, a) if undo else (a, pa)
                new[dst:dst + n] = old[src:src + n]
            f.seek(base)
            f.write(new)
            for t, h, packed in y["movers"]:
                if packed != undo:
                    continue  # already where this direction puts it
                shift = y["packed_hole"](h) - y["holes"][h][0]
                f.seek(t.offset_at)
                f.write(struct.pack("<Q", t.offset - data_start + (-shift if undo else shift)))
            for i in y["infos"]:
                f.seek(i.name_at + i.name.index("_expm" if undo else "_exps") + 1)
                f.write(b"exps" if undo else b"expm")
            done += 1
    return done


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


def write_moe_layers(path: str, cfg: synth.Config, layers: list, arch: str = "qwen3moe", router_between: bool = False):
    """A GGUF file holding `layers` (weight dicts as `synth.make_weights` returns) of shape `cfg`.
    `router_between` writes a layer's router after its gate tensor, between the expert tensors (as
    the reference's Qwen3.8 files hold it, src/repack.rs:10-13)."""
    meta = {"general.architecture": arch, "general.name": cfg.name, f"{arch}.block_count": len(layers),
            f"{arch}.embedding_length": cfg.d, f"{arch}.expert_feed_forward_length": cfg.ff,
            f"{arch}.expert_count": cfg.n_exp, f"{arch}.expert_used_count": cfg.top_k,
            f"{arch}.expert_gating_func": 2 if cfg.gating == synth.GATE_SIGMOID else 1,
            f"{arch}.expert_weights_norm": bool(cfg.norm_w), f"{arch}.expert_weights_scale": float(cfg.w_scale)}
    E, d, ff = cfg.n_exp, cfg.d, cfg.ff
    tensors = {}
    for i, w in enumerate(layers):
        p = f"blk.{i}."
        if not router_between:
            tensors[p + "ffn_gate_inp.weight"] = ((d, E), 0, np.ascontiguousarray(w["router"], np.float32))
        tensors[p + "ffn_gate_exps.weight"] = ((d, ff, E), cfg.type_gate, np.ascontiguousarray(w["gate"]))
        if router_between:
            tensors[p + "ffn_gate_inp.weight"] = ((d, E), 0, np.ascontiguousarray(w["router"], np.float32))
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
