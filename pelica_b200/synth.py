"""Synthetic MoE layers: the named config shapes, seeded weights and the GGUF
block encoders (Q4_K, Q5_K, Q6_K, MXFP4, Q8_0, IQ4_NL, IQ4_XS, IQ3_S) that quantise them.

Pelica has no quantiser for these formats (it only reads them from GGUF files,
src/gguf.rs:85-121), so the encoders here are this repository's own. Any valid
encoder serves: the CUDA path and its checker consume the same bytes. The block
layouts follow the decoders they must round-trip through
(src/ds4_cpu.rs:45-83, src/moe_kernels.rs:73,75,80).
"""
from __future__ import annotations

import dataclasses

import numpy as np

# ggml type ids (src/gguf.rs:85-121)
F32, F16, Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL, IQ3_S, IQ4_XS, BF16, MXFP4 = 0, 1, 8, 12, 13, 14, 20, 21, 23, 30, 39
GLM_Q4 = 1064  # not a ggml id: the reference's int4 container, groups of 64 with f32 scales (src/quant.rs:9-11)
BLOCK = {Q8_0: (32, 34), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), IQ4_NL: (32, 18), IQ3_S: (256, 110),
         IQ4_XS: (256, 136), MXFP4: (32, 17), GLM_Q4: (64, 36)}
# the IQ4_NL codebook, a constant of the format (src/iq_tables.rs:72)
KV_IQ4NL = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.int8)

GATE_SOFTMAX_ALL, GATE_SIGMOID, GATE_SQRT_SOFTPLUS, GATE_SOFTMAX_SELECTED = 0, 1, 2, 3
ACT_SILU, ACT_SILU_CLAMP, ACT_OSS_GLU = 0, 1, 2
AQ_F32, AQ_Q8X_256, AQ_Q8_32, AQ_Q8_32_F16 = 0, 1, 2, 3
FOLD_BEFORE_DOWN, FOLD_IN_COMBINE = 0, 1
SHARED_NONE, SHARED_PLAIN, SHARED_SIGMOID_GATED = 0, 1, 2


def row_bytes(ggml_type: int, ncols: int) -> int:
    v, b = BLOCK[ggml_type]
    assert ncols % v == 0
    return ncols // v * b


# --------------------------------------------------------------------------
# encoders
# --------------------------------------------------------------------------

def _round_half_away(x):
    return np.sign(x) * np.floor(np.abs(x) + 0.5)


def encode_q4_k(x: np.ndarray) -> np.ndarray:
    """f32 [..., n] (n % 256 == 0) -> uint8 [..., n/256*144]."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 8, 32)
    nb = xb.shape[0]
    mn = np.minimum(xb.min(-1), 0.0)
    mx = xb.max(-1)
    scale = np.maximum(mx - mn, 0.0) / 15.0
    mins = -mn
    d = (scale.max(-1) / 63.0).astype(np.float16)
    dmin = (mins.max(-1) / 63.0).astype(np.float16)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df[:, None] > 0, _round_half_away(scale / df[:, None]), 0.0)
        m = np.where(dmf[:, None] > 0, _round_half_away(mins / dmf[:, None]), 0.0)
        sc = np.clip(sc, 0, 63)
        m = np.clip(m, 0, 63)
        step = df[:, None] * sc
        q = np.where(step[..., None] > 0,
                     _round_half_away((xb + (dmf[:, None] * m)[..., None]) / step[..., None]), 0.0)
    q = np.clip(q, 0, 15).astype(np.uint8)
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.zeros((nb, 144), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
    s = out[:, 4:16]
    s[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    s[:, 4:8] = m[:, 0:4] | ((m[:, 4:8] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:8] & 15) | ((m[:, 4:8] & 15) << 4)
    qq = q.reshape(nb, 4, 2, 32)
    out[:, 16:144] = (qq[:, :, 0, :] | (qq[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(*lead, -1)


def encode_q6_k(x: np.ndarray) -> np.ndarray:
    """f32 [..., n] (n % 256 == 0) -> uint8 [..., n/256*210]."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 16, 16)
    nb = xb.shape[0]
    gs = np.abs(xb).max(-1) / 31.0
    d = (gs.max(-1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df[:, None] > 0, _round_half_away(gs / df[:, None]), 0.0)
        sc = np.clip(sc, 0, 127)
        step = df[:, None] * sc
        q = np.where(step[..., None] > 0, _round_half_away(xb / step[..., None]), 0.0)
    q = (np.clip(q, -32, 31) + 32).astype(np.uint8).reshape(nb, 256)
    out = np.zeros((nb, 210), np.uint8)
    # value v = 128 n + 32 qt + l  (src/moe_kernels.rs:75)
    qv = q.reshape(nb, 2, 4, 32)  # [n][qt][l]
    lo = qv & 15
    hi = qv >> 4
    ql = out[:, 0:128].reshape(nb, 2, 2, 32)  # byte 64n + 32*(qt&1) + l
    ql[:, :, 0, :] = lo[:, :, 0, :] | (lo[:, :, 2, :] << 4)
    ql[:, :, 1, :] = lo[:, :, 1, :] | (lo[:, :, 3, :] << 4)
    qh = out[:, 128:192].reshape(nb, 2, 32)
    qh[:] = hi[:, :, 0, :] | (hi[:, :, 1, :] << 2) | (hi[:, :, 2, :] << 4) | (hi[:, :, 3, :] << 6)
    out[:, 192:208] = sc.astype(np.int8).view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
    return out.reshape(*lead, -1)


_MX_TABLE = np.array([0, 1, 2, 3, 4, 6, 8, 12], np.float32)  # doubled E2M1 (src/moe_kernels.rs:109)


def encode_mxfp4(x: np.ndarray) -> np.ndarray:
    """f32 [..., n] (n % 32 == 0) -> uint8 [..., n/32*17]."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 32)
    nb = xb.shape[0]
    amax = np.abs(xb).max(-1)
    with np.errstate(divide="ignore"):
        ex = np.where(amax > 0, np.floor(np.log2(np.maximum(amax, 1e-38))) - 3, -126.0)
    e = np.clip(ex + 128, 2, 254).astype(np.int32)  # scale = 2^(e-128) (src/oss_kernels.rs:42-45)
    s = np.exp2((e - 128).astype(np.float32))
    mag = np.abs(xb) / s[:, None]
    code = np.abs(mag[..., None] - _MX_TABLE).argmin(-1).astype(np.uint8)
    code |= ((xb < 0) & (code > 0)).astype(np.uint8) << 3
    out = np.zeros((nb, 17), np.uint8)
    out[:, 0] = e.astype(np.uint8)
    out[:, 1:17] = code[:, 0:16] | (code[:, 16:32] << 4)
    return out.reshape(*lead, -1)


def encode_q8_0(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 32)
    nb = xb.shape[0]
    d = (np.abs(xb).max(-1) / 127.0).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(df[:, None] > 0, _round_half_away(xb / df[:, None]), 0.0)
    q = np.clip(q, -127, 127).astype(np.int8)
    out = np.zeros((nb, 34), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:34] = q.view(np.uint8)
    return out.reshape(*lead, -1)


def encode_iq4_nl(x: np.ndarray) -> np.ndarray:
    """32 values -> f16 d + 16 bytes: byte j = codebook index of value j (low nibble) and of
    value j + 16 (high nibble) (src/q4x_cpu.rs:453-461). d = amax / 127 (by the sign of the largest
    value, so that it lands on the codebook's -127), indices = nearest codebook entry."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 32)
    nb = xb.shape[0]
    imax = np.abs(xb).argmax(-1)
    vmax = xb[np.arange(nb), imax]
    d = (vmax / -127.0).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        t = np.where(df[:, None] != 0, xb / df[:, None], 0.0)
    idx = np.abs(t[:, :, None] - KV_IQ4NL.astype(np.float32)[None, None, :]).argmin(-1).astype(np.uint8)
    out = np.zeros((nb, 18), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:18] = idx[:, :16] | (idx[:, 16:] << 4)
    return out.reshape(*lead, -1)


def encode_iq4_xs(x: np.ndarray) -> np.ndarray:
    """256 values -> f16 d, u16 high scale bits, 4 bytes of low scale nibbles, 128 index bytes
    (src/q4x_cpu.rs:462-476): sub-block scale = d * (ls - 32), ls six bits; sub-block ib's byte i holds
    the codebook index of value i (low nibble) and of value i + 16 (high nibble)."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 8, 32)
    nb = xb.shape[0]
    amax = np.abs(xb).max(-1)                      # [nb, 8]
    d = (amax.max(-1) / 127.0 / 31.0).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        l = np.where(df[:, None] > 0, np.rint(amax / 127.0 / df[:, None]), 0.0)
    l = np.clip(l, 0, 31).astype(np.int32)
    l = np.where((amax > 0) & (l == 0), 1, l)
    ls = (l + 32).astype(np.uint32)                # 32..63
    dl = df[:, None] * l.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        t = np.where(dl[:, :, None] != 0, xb / dl[:, :, None], 0.0)
    idx = np.abs(t[..., None] - KV_IQ4NL.astype(np.float32)).argmin(-1).astype(np.uint8)  # [nb, 8, 32]
    out = np.zeros((nb, 136), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    sh = np.zeros(nb, np.uint32)
    for ib in range(8):
        sh |= ((ls[:, ib] >> 4) & 3) << (2 * ib)
        out[:, 4 + ib // 2] |= ((ls[:, ib] & 15) << (4 * (ib % 2))).astype(np.uint8)
    out[:, 2] = (sh & 0xFF).astype(np.uint8)
    out[:, 3] = (sh >> 8).astype(np.uint8)
    out[:, 8:136] = (idx[:, :, :16] | (idx[:, :, 16:] << 4)).reshape(nb, 128)
    return out.reshape(*lead, -1)


def encode_q5_k(x: np.ndarray) -> np.ndarray:
    """f32 [..., n] (n % 256 == 0) -> uint8 [..., n/256*176]: Q4_K's header (f16 d, f16 dmin, 12 bytes
    of six-bit scales and mins), 32 bytes of fifth bits (byte l, bit 2c + hi = value 64c + 32hi + l),
    128 bytes of low nibbles as in Q4_K (src/moe_kernels.rs:74)."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 8, 32)
    nb = xb.shape[0]
    mn = np.minimum(xb.min(-1), 0.0)
    mx = xb.max(-1)
    scale = np.maximum(mx - mn, 0.0) / 31.0
    mins = -mn
    d = (scale.max(-1) / 63.0).astype(np.float16)
    dmin = (mins.max(-1) / 63.0).astype(np.float16)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.clip(np.where(df[:, None] > 0, _round_half_away(scale / df[:, None]), 0.0), 0, 63)
        m = np.clip(np.where(dmf[:, None] > 0, _round_half_away(mins / dmf[:, None]), 0.0), 0, 63)
        step = df[:, None] * sc
        q = np.where(step[..., None] > 0,
                     _round_half_away((xb + (dmf[:, None] * m)[..., None]) / step[..., None]), 0.0)
    q = np.clip(q, 0, 31).astype(np.uint8)
    sc = sc.astype(np.uint8)
    m = m.astype(np.uint8)
    out = np.zeros((nb, 176), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
    s = out[:, 4:16]
    s[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
    s[:, 4:8] = m[:, 0:4] | ((m[:, 4:8] >> 4) << 6)
    s[:, 8:12] = (sc[:, 4:8] & 15) | ((m[:, 4:8] & 15) << 4)
    qq = q.reshape(nb, 4, 2, 32)  # [c][hi][l]
    for c in range(4):
        for hi in range(2):
            out[:, 16:48] |= ((qq[:, c, hi, :] >> 4) & 1) << (2 * c + hi)
    out[:, 48:176] = ((qq[:, :, 0, :] & 15) | ((qq[:, :, 1, :] & 15) << 4)).reshape(nb, 128)
    return out.reshape(*lead, -1)


_IQ3S_GRID = None


def iq3s_grid() -> np.ndarray:
    """The IQ3_S codebook of the format as [512, 4] magnitudes (src/iq_tables.rs:4), from the packed
    constant table the library and its checker also include."""
    global _IQ3S_GRID
    if _IQ3S_GRID is None:
        import os
        import re
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "include", "pelica_iq3s_grid.inc")
        text = open(path).read()
        codes = np.array([int(w, 16) for w in re.findall(r"0x[0-9a-f]{3}\b", text[text.index("*/"):])], np.int32)
        assert codes.size == 512
        _IQ3S_GRID = np.stack([2 * ((codes >> (3 * j)) & 7) + 1 for j in range(4)], -1).astype(np.int32)
    return _IQ3S_GRID


def encode_iq3_s(x: np.ndarray) -> np.ndarray:
    """256 values -> 110 bytes: f16 d, 64 index bytes (8 per sub-block of 32: one per group of four
    values), 8 bytes of ninth index bits (byte ib, bit k), 32 bytes of sign bits (bit v % 8 of byte
    v / 8), 4 bytes of sub-block scale nibbles; value = d * (1 + 2 sc) * +-codebook[index][j]
    (src/q4x_cpu.rs:64-82). Each group of four takes the nearest codebook entry."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 8, 32)
    nb = xb.shape[0]
    grid = iq3s_grid().astype(np.float32)            # [512, 4]
    amax = np.abs(xb).max(-1)                        # [nb, 8]
    d = (amax.max(-1) / 15.0 / 31.0).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df[:, None] > 0, np.rint((amax / 15.0 / df[:, None] - 1.0) / 2.0), 0.0)
    sc = np.clip(sc, 0, 15).astype(np.int32)
    dl = df[:, None] * (1 + 2 * sc).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        t = np.where(dl[:, :, None] > 0, np.abs(xb) / dl[:, :, None], 0.0).reshape(-1, 4)  # groups of four
    idx = np.empty(t.shape[0], np.int32)
    for i in range(0, t.shape[0], 4096):
        c = t[i:i + 4096]
        idx[i:i + 4096] = ((c[:, None, :] - grid[None]) ** 2).sum(-1).argmin(-1)
    idx = idx.reshape(nb, 8, 8)
    neg = (xb < 0).reshape(nb, 32, 8)                # [byte][bit]
    out = np.zeros((nb, 110), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:66] = (idx & 0xFF).astype(np.uint8).reshape(nb, 64)
    for k in range(8):
        out[:, 66:74] |= (((idx[:, :, k] >> 8) & 1) << k).astype(np.uint8)
    for bit in range(8):
        out[:, 74:106] |= (neg[:, :, bit].astype(np.uint8) << bit)
    for ib in range(8):
        out[:, 106 + ib // 2] |= ((sc[:, ib] & 15) << (4 * (ib % 2))).astype(np.uint8)
    return out.reshape(*lead, -1)


def encode_glm_q4(x: np.ndarray) -> np.ndarray:
    """`quantize_q4` (src/quant.rs:179-201): groups of 64, step = max(amax / 7, 1e-8), levels
    round(v / step) (ties to even) clamped to [-8, 7] and stored + 8, value c in byte c / 2 (low
    nibble first). f32 [..., n] -> uint8 [..., n/2 + n/64*4]: each row's nibbles, then its scales
    (`encode_matrix` puts a whole matrix into the container's two regions)."""
    x = np.asarray(x, np.float32)
    lead = x.shape[:-1]
    xb = x.reshape(-1, 64)
    step = np.maximum(np.abs(xb).max(-1) / np.float32(7.0), np.float32(1e-8)).astype(np.float32)
    lv = np.clip(np.rint(xb / step[:, None]), -8, 7).astype(np.int32) + 8
    q = (lv[:, 0::2] | (lv[:, 1::2] << 4)).astype(np.uint8)                 # [groups, 32]
    n = x.shape[-1]
    rows = q.reshape(-1, n // 2)
    sc = step.view(np.uint8).reshape(-1, n // 64 * 4)
    return np.concatenate([rows, sc], -1).reshape(*lead, -1)


def encode_matrix(ty: int, m: np.ndarray) -> np.ndarray:
    """A [rows][cols] f32 matrix as the bytes `pm_layer_set_expert` takes for type `ty`: rows of
    whole blocks, except the int4 container, whose nibble rows all come before its scale rows."""
    enc = ENCODERS[ty](m)
    if ty == GLM_Q4:
        nq = m.shape[-1] // 2
        return np.concatenate([enc[:, :nq].ravel(), enc[:, nq:].ravel()])
    return enc.ravel()


ENCODERS = {Q4_K: encode_q4_k, Q6_K: encode_q6_k, MXFP4: encode_mxfp4, Q8_0: encode_q8_0, IQ4_NL: encode_iq4_nl,
            IQ4_XS: encode_iq4_xs, Q5_K: encode_q5_k, IQ3_S: encode_iq3_s, GLM_Q4: encode_glm_q4}


def bf16_round(x: np.ndarray) -> np.ndarray:
    """f32 -> nearest-even bf16 -> f32 (the reference loads bf16 biases as f32, src/oss.rs:255-260)."""
    b = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000
    return b.astype(np.uint32).view(np.float32)


# --------------------------------------------------------------------------
# configs
# --------------------------------------------------------------------------

@dataclasses.dataclass
class Config:
    """A layer shape; field names follow pm_layer_desc."""

    name: str
    d: int
    ff: int
    n_exp: int
    top_k: int
    gating: int = GATE_SOFTMAX_ALL
    norm_w: int = 0
    w_scale: float = 0.0
    n_group: int = 0
    topk_group: int = 0
    act: int = ACT_SILU
    act_limit: float = 0.0
    act_alpha: float = 0.0
    type_gate: int = Q4_K
    type_up: int = Q4_K
    type_down: int = Q4_K
    act_quant: int = AQ_Q8X_256
    weight_fold: int = FOLD_BEFORE_DOWN
    has_expert_bias: int = 0
    shared: int = SHARED_NONE
    shared_ff: int = 0
    first_local_expert: int = 0
    n_exp_local: int = 0
    n_layers: int = 1
    logit_bias: bool = False
    select_bias_sigma: float = 0.0
    sigma: float = 0.02

    def desc_fields(self) -> dict:
        names = ["d", "ff", "n_exp", "top_k", "gating", "norm_w", "w_scale", "n_group", "topk_group", "act",
                 "act_limit", "act_alpha", "type_gate", "type_up", "type_down", "act_quant", "weight_fold",
                 "has_expert_bias", "shared", "shared_ff", "first_local_expert", "n_exp_local"]
        return {n: getattr(self, n) for n in names}

    def expert_bytes(self) -> int:
        b = row_bytes(self.type_gate, self.d) * self.ff + row_bytes(self.type_up, self.d) * self.ff
        b += row_bytes(self.type_down, self.ff) * self.d
        if self.has_expert_bias:
            b += 4 * (2 * self.ff + self.d)
        return b

    def scaled(self, **kw) -> "Config":
        return dataclasses.replace(self, **kw)


# the five benchmark shapes
C1_OLMOE = Config("olmoe-1b-7b", d=2048, ff=1024, n_exp=64, top_k=8, gating=GATE_SOFTMAX_ALL, norm_w=0)
C2_QWEN3 = Config("qwen3-30b-a3b", d=2048, ff=768, n_exp=128, top_k=8, gating=GATE_SOFTMAX_ALL, norm_w=1,
                  type_down=Q6_K, n_layers=48)
C3_GPTOSS = Config("gpt-oss-20b", d=2880, ff=2880, n_exp=32, top_k=4, gating=GATE_SOFTMAX_SELECTED,
                   act=ACT_OSS_GLU, act_limit=7.0, act_alpha=1.702, type_gate=MXFP4, type_up=MXFP4,
                   type_down=MXFP4, act_quant=AQ_F32, weight_fold=FOLD_IN_COMBINE, has_expert_bias=1,
                   n_layers=24, logit_bias=True)
C4_DSV3 = Config("deepseek-v3-shaped", d=7168, ff=2048, n_exp=256, top_k=8, gating=GATE_SIGMOID, norm_w=1,
                 w_scale=2.5, n_group=8, topk_group=4, shared=SHARED_PLAIN, shared_ff=2048, n_layers=58,
                 select_bias_sigma=0.01)
C5_ZIPF = Config("qwen3-zipf", d=2048, ff=768, n_exp=128, top_k=8, gating=GATE_SOFTMAX_ALL, norm_w=1)
# the reference's second CPU expert path (src/q4x_cpu.rs): 32-block Q8 activations against
# Q8_0 weights, softmax over the selected logits (src/q4x.rs:2213-2231); its own test shape
# is 2560 x 640 (src/q4x_cpu.rs:544)
C6_Q8_0 = Config("q4x-q8_0", d=2560, ff=640, n_exp=32, top_k=8, gating=GATE_SOFTMAX_SELECTED, type_gate=Q8_0,
                 type_up=Q8_0, type_down=Q8_0, act_quant=AQ_Q8_32)
# the same path with the 4-bit non-linear type of the reference's Qwen3.8 down tensors
C7_IQ4NL = C6_Q8_0.scaled(name="q4x-iq4_nl", type_gate=IQ4_NL, type_up=IQ4_NL, type_down=IQ4_NL)
C8_IQ4XS = C6_Q8_0.scaled(name="q4x-iq4_xs", type_gate=IQ4_XS, type_up=IQ4_XS, type_down=IQ4_NL)
# ... with the 3-bit codebook type of the reference's Qwen3.8 gate / up tensors (src/q4x_cpu.rs:118-127)
C9_IQ3S = C6_Q8_0.scaled(name="q4x-iq3_s", type_gate=IQ3_S, type_up=IQ3_S, type_down=IQ4_NL)
# Q5_K has a decoder only in the reference (src/moe_kernels.rs:74): f32 activations
C10_Q5K = C2_QWEN3.scaled(name="qwen3-q5_k-f32", type_gate=Q5_K, type_up=Q5_K, type_down=Q5_K, act_quant=AQ_F32,
                          weight_fold=FOLD_IN_COMBINE)
# the reference's GLM tier (src/forward.rs:95-113,488-504): int4 container, f32 activations, sigmoid scores
# ranked with a bias, clamped SwiGLU, a shared expert, weights applied to the expert outputs
C11_GLM = Config("glm-int4-gs64", d=2048, ff=1536, n_exp=64, top_k=8, gating=GATE_SIGMOID, norm_w=1, w_scale=2.5,
                 act=ACT_SILU_CLAMP, act_limit=10.0, type_gate=GLM_Q4, type_up=GLM_Q4, type_down=GLM_Q4,
                 act_quant=AQ_F32, weight_fold=FOLD_IN_COMBINE, shared=SHARED_PLAIN, shared_ff=1536,
                 select_bias_sigma=0.01)
# the OLMoE shape with the activation format its benchmark description words literally: Q4_K weights
# against 32-value int8 blocks with an f16 scale. No reference code pairs them (the reference's Q4_K
# path is C1's Q8x); a labelled second mode.
C12_Q4K_Q8_0 = C1_OLMOE.scaled(name="olmoe-q4_k-q8_0-acts", act_quant=AQ_Q8_32_F16)
CONFIGS = {"c1": C1_OLMOE, "c2": C2_QWEN3, "c3": C3_GPTOSS, "c4": C4_DSV3, "c5": C5_ZIPF, "c6": C6_Q8_0,
           "c7": C7_IQ4NL, "c8": C8_IQ4XS, "c9": C9_IQ3S, "c10": C10_Q5K, "c11": C11_GLM, "c12": C12_Q4K_Q8_0}


def make_weights(cfg: Config, seed: int, experts=None) -> dict:
    """Seeded N(0, sigma) weights quantised to cfg's types (numpy; test sizes).

    Returns the dict oracle.Layer and pelica_b200.MoeLayer.load take.
    """
    rng = np.random.default_rng(seed)
    E, d, ff = cfg.n_exp, cfg.d, cfg.ff
    w = {"router": rng.normal(0, cfg.sigma, (E, d)).astype(np.float32)}
    if cfg.logit_bias:
        w["logit_bias"] = bf16_round(rng.normal(0, cfg.sigma, E).astype(np.float32))
    if cfg.select_bias_sigma > 0:
        w["select_bias"] = rng.normal(0, cfg.select_bias_sigma, E).astype(np.float32)
    gate = np.zeros((E, row_bytes(cfg.type_gate, d) * ff), np.uint8)
    up = np.zeros((E, row_bytes(cfg.type_up, d) * ff), np.uint8)
    down = np.zeros((E, row_bytes(cfg.type_down, ff) * d), np.uint8)
    for e in range(E):
        g = rng.normal(0, cfg.sigma, (ff, d)).astype(np.float32)
        u = rng.normal(0, cfg.sigma, (ff, d)).astype(np.float32)
        dn = rng.normal(0, cfg.sigma, (d, ff)).astype(np.float32)
        if experts is not None and e not in experts:
            continue
        gate[e] = encode_matrix(cfg.type_gate, g)
        up[e] = encode_matrix(cfg.type_up, u)
        down[e] = encode_matrix(cfg.type_down, dn)
    w.update(gate=gate, up=up, down=down)
    if cfg.has_expert_bias:
        w["bias_gate"] = bf16_round(rng.normal(0, cfg.sigma, (E, ff)).astype(np.float32))
        w["bias_up"] = bf16_round(rng.normal(0, cfg.sigma, (E, ff)).astype(np.float32))
        w["bias_down"] = bf16_round(rng.normal(0, cfg.sigma, (E, d)).astype(np.float32))
    if cfg.shared:
        sf = cfg.shared_ff
        w["shared_gate"] = encode_matrix(cfg.type_gate, rng.normal(0, cfg.sigma, (sf, d)).astype(np.float32))
        w["shared_up"] = encode_matrix(cfg.type_up, rng.normal(0, cfg.sigma, (sf, d)).astype(np.float32))
        w["shared_down"] = encode_matrix(cfg.type_down, rng.normal(0, cfg.sigma, (d, sf)).astype(np.float32))
        if cfg.shared == SHARED_SIGMOID_GATED:
            w["shared_gate_inp"] = rng.normal(0, cfg.sigma, d).astype(np.float32)
    return w


def make_activations(T: int, d: int, seed: int, eps: float = 1e-6) -> np.ndarray:
    """f32 N(0,1) [T,d], RMS-normalised with unit weight (src/moe.rs:758 eps)."""
    rng = np.random.default_rng(seed)
    x = rng.normal(0, 1, (T, d)).astype(np.float32)
    ms = (x.astype(np.float64) ** 2).mean(-1, keepdims=True)
    return (x / np.sqrt(ms + eps)).astype(np.float32)


def zipf_router_bias(n_exp: int, seed: int, s: float = 1.2, dead: int = 8, strength: float = 1.0) -> np.ndarray:
    """Logit offsets that make expert popularity follow rank^-s over a seeded
    permutation, with the `dead` least popular experts pushed to never win."""
    rng = np.random.default_rng(seed)
    perm = rng.permutation(n_exp)
    rank = np.empty(n_exp, np.int64)
    rank[perm] = np.arange(1, n_exp + 1)
    bias = (-s * np.log(rank.astype(np.float64)) * strength).astype(np.float32)
    if dead:
        bias[perm[-dead:]] = -1.0e4
    return bias
