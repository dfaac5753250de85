"""Pins of the CPU oracle: the reference's own relational tests re-run on the
restatement, exact known answers for the scalar helpers and block decoders,
and the committed golden fixtures."""
import os

import numpy as np
import pytest

from pelica_b200 import synth
from tests.helpers import bits_equal, lcg, ref_acts, ref_q4k_blocks

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_f16_round_trip(oracle):
    # src/q4x.rs:3411-3420
    for v in [0.0, 1.0, -2.5, 65504.0, 1e-5, -3.14159, 1e-8, 0.333333]:
        h = oracle.f32_to_f16(v)
        back = oracle.f16_to_f32(h)
        assert abs(back - np.float32(v)) <= abs(v) * 1e-3 + 6e-8
    assert oracle.f32_to_f16(1.0 + 1.0 / 2048.0) == 0x3C00  # ties go to even
    assert oracle.f32_to_f16(1.0 + 3.0 / 2048.0) == 0x3C02


def test_f16_matches_ieee(oracle):
    bits = np.arange(0, 65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(b)) for b in bits], np.float32)
    ok = np.isnan(want) | (want.view(np.uint32) == got.view(np.uint32))
    assert ok.all()
    rng = np.random.default_rng(0)
    xs = np.concatenate([rng.normal(0, 1, 2000), rng.normal(0, 1e-6, 500), rng.normal(0, 3e4, 500)]).astype(np.float32)
    with np.errstate(over="ignore"):
        want16 = xs.astype(np.float16).view(np.uint16)
    got16 = np.array([oracle.f32_to_f16(float(x)) for x in xs], np.uint16)
    assert np.array_equal(want16, got16)


def test_vnni_matches_scalar(oracle):
    # src/ds4_cpu.rs:446-474 (seed 1, 4 blocks)
    rnd = lcg(1)
    w = ref_q4k_blocks(rnd, 4)
    x = ref_acts(rnd, 4 * 256)
    q, d, bs = oracle.q8x(x)
    a = oracle.row_q4k(w, 1024, q, d, bs, "scalar")
    f = oracle.row_q4k(w, 1024, q, d, bs, "fast")
    assert np.float32(a).tobytes() == np.float32(f).tobytes()
    if oracle.lib().po_have_vnni():
        b = oracle.row_q4k(w, 1024, q, d, bs, "vnni")
        assert abs(a - b) <= 1e-3 * max(abs(a), 1.0)


def test_multi_matches_single(oracle):
    # src/ds4_cpu.rs:476-503 (seed 7; 4 blocks, 3 rows, 19 tokens): bit-equal
    rnd = lcg(7)
    blocks, rows, toks = 4, 3, 19
    w = ref_q4k_blocks(rnd, rows * blocks)
    qs = [oracle.q8x(ref_acts(rnd, blocks * 256)) for _ in range(toks)]
    for canonical in (False, True):
        multi = oracle.q4k_rows_multi(w, rows, blocks * 256, qs, canonical=canonical)
        for t, (q, d, bs) in enumerate(qs):
            for r in range(rows):
                kind = "fast" if canonical else ("vnni" if oracle.lib().po_have_vnni() else "scalar")
                one = oracle.row_q4k(w[r * blocks * 144:(r + 1) * blocks * 144], blocks * 256, q, d, bs, kind)
                assert np.float32(one).tobytes() == np.float32(multi[r, t]).tobytes(), (r, t)


def test_dot_bf16_matches_dot_f32_bitwise(oracle):
    # src/quant.rs:535-552
    rng = np.random.default_rng(3)
    for n in (32, 64, 2048, 2880, 104):
        a = rng.normal(0, 1, n).astype(np.float32)
        a_bits = (a.view(np.uint32) >> 16).astype(np.uint16)
        a_exact = (a_bits.astype(np.uint32) << 16).view(np.float32)
        b = rng.normal(0, 1, n).astype(np.float32)
        assert np.float32(oracle.dot_bf16(a_bits, b)).tobytes() == np.float32(oracle.dot_f32(a_exact, b)).tobytes()
        assert abs(oracle.dot_f32(a_exact, b) - float(a_exact.astype(np.float64) @ b.astype(np.float64))) < 1e-3


def test_rows_match_dequant(oracle):
    # the shape of src/q4x_cpu.rs:509-535: a quantised row equals dequantised
    # weights . dequantised activations within 1e-3*max(|want|,1)
    rng = np.random.default_rng(5)
    for ty, n in ((synth.Q4_K, 1024), (synth.Q6_K, 768), (synth.Q8_0, 512), (synth.IQ4_NL, 2560),
                  (synth.IQ4_XS, 2560), (synth.IQ3_S, 2560)):
        w = synth.ENCODERS[ty](rng.normal(0, 0.02, n).astype(np.float32))
        x = rng.normal(0, 1, n).astype(np.float32)
        wd = oracle.dequant(ty, w, n).astype(np.float64)
        if ty in (synth.Q8_0, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_S):
            q, d = oracle.q8_32(x)
            got = {synth.Q8_0: oracle.row_q8_0, synth.IQ4_NL: oracle.row_iq4nl, synth.IQ4_XS: oracle.row_iq4xs,
                   synth.IQ3_S: oracle.row_iq3s}[ty](w, n, q, d)
            xd = q.astype(np.float64) * np.repeat(d, 32)
        else:
            q, d, bs = oracle.q8x(x)
            got = oracle.row_q4k(w, n, q, d, bs) if ty == synth.Q4_K else oracle.row_q6k(w, n, q, d)
            xd = q.astype(np.float64) * np.repeat(d, 256)
        want = float(wd @ xd)
        assert abs(got - want) <= 1e-3 * max(abs(want), 1.0)


def test_q6k_fast_is_scalar(oracle):
    rng = np.random.default_rng(6)
    for _ in range(5):
        w = rng.integers(0, 256, 3 * 210, dtype=np.uint8)
        w[208::210] = 0x00
        w[209::210] = 0x2C
        q, d, _ = oracle.q8x(rng.normal(0, 1, 768).astype(np.float32))
        a, b = oracle.row_q6k(w, 768, q, d), oracle.row_q6k(w, 768, q, d, "fast")
        assert np.float32(a).tobytes() == np.float32(b).tobytes()


def test_block_known_answers(oracle):
    # Q4_K: d = 1.0 (0x3c00), dmin = 0.5 (0x3800); sub-block 0: sc 3, m 2;
    # sub-block 5: sc 33 (needs the high bits), m 17
    blk = np.zeros(144, np.uint8)
    blk[0:2] = [0x00, 0x3C]
    blk[2:4] = [0x00, 0x38]
    s = blk[4:16]
    s[0] = 3
    s[4] = 2
    s[1] = (33 >> 4) << 6          # high bits of sc[5]
    s[5] = (17 >> 4) << 6          # high bits of m[5]
    s[9] = (33 & 15) | ((17 & 15) << 4)
    blk[16 + 0] = 0x07             # value 0 = 7 (sub-block 0)
    blk[16 + 64 + 3] = 0xA0        # c=2, i=3, high nibble -> value 64*2+32+3 = 163 (sub-block 5) = 10
    out = oracle.dequant(synth.Q4_K, blk, 256)
    assert out[0] == 1.0 * 3 * 7 - 0.5 * 2
    assert out[1] == -0.5 * 2
    assert out[163] == 1.0 * 33 * 10 - 0.5 * 17
    # Q6_K: d = 0.25 (0x3400); value 200: n=1 r=72 qt=2 l=8 -> ql byte 64+8 high nibble,
    # qh byte 32+8 bits 4-5, scale 8+0+4 = 12
    blk = np.zeros(210, np.uint8)
    blk[208:210] = [0x00, 0x34]
    blk[64 + 8] = 0xB0
    blk[128 + 32 + 8] = 0b00100000
    blk[192 + 12] = np.uint8(np.int8(-5).view(np.uint8))
    out = oracle.dequant(synth.Q6_K, blk, 256)
    assert out[200] == 0.25 * -5 * ((0xB | (2 << 4)) - 32)
    assert out[0] == 0.0  # scale 0
    # MXFP4: e = 129 -> 2.0; e = 1 -> 2^-127 (denormal branch); codes
    blk = np.zeros(34, np.uint8)
    blk[0] = 129
    blk[1] = 0x5F  # value 0 = code 15 (-12), value 16 = code 5 (6)
    blk[17] = 1
    blk[18] = 0x02
    out = oracle.dequant(synth.MXFP4, blk, 64)
    assert out[0] == -24.0 and out[16] == 12.0
    assert out[32] == np.float32(2.0) * np.float32(2.0 ** -127)
    # Q8_0
    blk = np.zeros(34, np.uint8)
    blk[0:2] = [0x00, 0x34]
    blk[2] = np.int8(-100).view(np.uint8)
    out = oracle.dequant(synth.Q8_0, blk, 32)
    assert out[0] == -25.0
    # IQ4_NL: d = 0.25; byte 0 = index 0 (low: value 0) and 15 (high: value 16); byte 15 = 8 / 7
    blk = np.zeros(18, np.uint8)
    blk[0:2] = [0x00, 0x34]
    blk[2] = 0xF0
    blk[17] = 0x78
    out = oracle.dequant(synth.IQ4_NL, blk, 32)
    assert out[0] == -31.75 and out[16] == 28.25 and out[15] == 0.25 and out[31] == -2.5
    assert out[1] == -31.75  # index 0 everywhere else


def test_q8x_known_answers(oracle):
    x = np.zeros(512, np.float32)
    x[0], x[1], x[2], x[40] = 2.0, -1.0, 0.0078740157, 0.5
    q, d, bs = oracle.q8x(x)
    assert d[0] == np.float32(2.0) / np.float32(127.0) and d[1] == 0.0
    assert q[0] == 127 and q[1] == -64  # -63.5 rounds away from zero
    assert q[2] == 1                    # 0.5000000 -> 1 (half away)
    assert q[40] == 32
    assert bs[0] == 127 - 64 + 1 and bs[1] == 32 and not bs[2:].any()


def test_exp_and_log1p(oracle):
    xs = np.concatenate([np.linspace(-87, 88, 3001), np.array([0.0, -0.0, 1e-8, -1e-8])]).astype(np.float32)
    got = np.array([oracle.exp(float(x)) for x in xs], np.float64)
    want = np.exp(xs.astype(np.float64))
    assert np.all(np.abs(got - want) <= 3e-7 * want)
    assert oracle.exp(-100.0) == 0.0 and np.isinf(oracle.exp(89.0))
    xs = np.concatenate([np.logspace(-30, 9, 2000), [0.0]]).astype(np.float32)
    got = np.array([oracle.log1p(float(x)) for x in xs], np.float64)
    want = np.log1p(xs.astype(np.float64))
    assert np.all(np.abs(got - want) <= 3e-7 * np.maximum(want, 1e-30) + 1e-37)


def test_route_ties_go_low(oracle):
    cfg = synth.C2_QWEN3.scaled(d=64, ff=256, n_exp=40, top_k=4)
    L = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), {"router": np.zeros((40, 64), np.float32)})
    ids, w = L.route_logits(np.zeros((2, 40), np.float32))
    assert ids.tolist() == [[0, 1, 2, 3]] * 2
    assert np.allclose(w, 0.25)
    lg = np.zeros((1, 40), np.float32)
    lg[0, [37, 5, 33]] = 1.0
    ids, _ = L.route_logits(lg)
    assert ids.tolist() == [[5, 33, 37, 0]]


def test_plan_layout(oracle):
    ids = np.array([[3, 1], [1, 0], [3, 2], [1, 3]], np.uint32)
    p = oracle.plan(ids, 6)
    assert p["n_active"] == 4
    assert p["active"][:4].tolist() == [0, 1, 2, 3]
    assert p["count"][:4].tolist() == [1, 3, 1, 3]
    assert p["offset"][:4].tolist() == [0, 1, 4, 5]
    assert p["pair_token"].tolist() == [1, 0, 1, 3, 2, 0, 2, 3]
    assert p["pair_pos"].tolist() == [5, 1, 2, 0, 6, 4, 3, 7]


def test_fast_layer_matches_canonical(oracle):
    cfg = synth.C2_QWEN3.scaled(d=512, ff=256, n_exp=16)
    W = synth.make_weights(cfg, 11)
    L = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)
    x = synth.make_activations(9, cfg.d, 12)
    y = L.forward(x)
    yf = L.forward_fast(x)
    assert np.abs(y - yf).max() <= 1e-3 * np.abs(y).max()


@pytest.mark.parametrize("name", ["c1", "c2", "c3", "c4", "c6", "c9", "c10", "c11", "c12"])
def test_golden_layer_outputs(oracle, name):
    """The committed fixtures (tests/golden/make_golden.py) pin the oracle itself."""
    from tests.golden.make_golden import case

    path = os.path.join(GOLDEN, f"layer_{name}.npz")
    g = np.load(path)
    cfg, W, x = case(name)
    L = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)
    ids, w = L.route(x)
    assert np.array_equal(ids, g["ids"])
    assert bits_equal(w, g["w"])
    assert bits_equal(L.forward(x), g["y"])


def _rand_vec64(n, seed):
    """`rand_vec` of the reference's quant tests (src/quant.rs:481-490): a 64-bit LCG, values in
    [-0.5, 0.5)."""
    s, out = seed, np.empty(n, np.float32)
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(np.float32(s >> 33) / np.float32(1 << 31)) - np.float32(0.5)
    return out


def test_int4_container_rows(oracle):
    """`q4_kernel_matches_scalar` (src/quant.rs:492-507) on the restated quantiser and row: the row
    over the container's bytes equals the dequantised weights times x, and stays within the
    reference's bound of the unquantised product."""
    rows, cols = 5, 256
    w = _rand_vec64(rows * cols, 1).reshape(rows, cols)
    x = _rand_vec64(cols, 2)
    m = synth.encode_matrix(synth.GLM_Q4, w)
    assert m.size == rows * cols // 2 + rows * (cols // 64) * 4
    # the quantiser's own contract (src/quant.rs:179-201): step = amax / 7, level + 8 per nibble
    step = m[rows * cols // 2:].view(np.float32).reshape(rows, cols // 64)
    assert np.array_equal(step, np.abs(w.reshape(rows, -1, 64)).max(-1) / np.float32(7.0))
    deq = oracle.dequant(synth.GLM_Q4, m, rows * cols).reshape(rows, cols)
    assert np.abs(deq - w).max() <= step.max() / 2 * 1.0001
    for o in range(rows):
        one_row = np.concatenate([m[o * cols // 2:(o + 1) * cols // 2],
                                  m[rows * cols // 2 + o * 16:rows * cols // 2 + (o + 1) * 16]])
        got = oracle.row_f32(synth.GLM_Q4, one_row, cols, x)
        assert abs(got - float(deq[o].astype(np.float64) @ x.astype(np.float64))) < 1e-4
        assert abs(got - float(w[o] @ x)) < 0.2


def test_q5k_and_iq3s_known_answers(oracle):
    # Q5_K (src/moe_kernels.rs:74): d = 1.0, dmin = 0.5; sub-block 5 (c = 2, high nibbles): sc 33, m 17;
    # value 163 = 64*2 + 32 + 3: nibble 0xA of qs byte 32*2 + 3, fifth bit = bit 2*2+1 of qh byte 3
    blk = np.zeros(176, np.uint8)
    blk[0:2] = [0x00, 0x3C]
    blk[2:4] = [0x00, 0x38]
    s = blk[4:16]
    s[0], s[4] = 3, 2
    s[1] = (33 >> 4) << 6
    s[5] = (17 >> 4) << 6
    s[9] = (33 & 15) | ((17 & 15) << 4)
    blk[48 + 64 + 3] = 0xA0
    blk[16 + 3] = 1 << 5
    blk[48 + 0] = 0x07              # value 0: nibble 7, no fifth bit (sub-block 0: sc 3, m 2)
    blk[16 + 1] = 1 << 0            # value 1: fifth bit only -> 16
    out = oracle.dequant(synth.Q5_K, blk, 256)
    assert out[163] == 1.0 * 33 * (0xA | 16) - 0.5 * 17
    assert out[0] == 1.0 * 3 * 7 - 0.5 * 2
    assert out[1] == 1.0 * 3 * 16 - 0.5 * 2
    # IQ3_S (src/q4x_cpu.rs:64-82): d = 0.5; sub-block 3: scale nibble 6 -> 1 + 2*6 = 13; its group 2 (values
    # 8..11 of the sub-block) takes codebook entry 0x100 | 0x2A with the ninth bit from qh; signs byte 4*3 + 1
    grid = synth.iq3s_grid()
    blk = np.zeros(110, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    blk[2 + 8 * 3 + 2] = 0x2A
    blk[66 + 3] = 1 << 2
    blk[74 + 4 * 3 + 1] = 0b00000101   # values 8 and 10 of the sub-block negative
    blk[106 + 1] = 6 << 4              # sub-block 3 = high nibble of scales byte 1
    out = oracle.dequant(synth.IQ3_S, blk, 256)
    mags = grid[0x12A]
    want = [-mags[0], mags[1], -mags[2], mags[3]]
    assert [float(v) for v in out[96 + 8:96 + 12]] == [0.5 * 13 * m for m in want]
    # every other value of the block: entry 0 of the codebook, scale 1, positive
    assert float(out[0]) == 0.5 * 1 * grid[0][0] and float(out[255]) == 0.5 * 1 * grid[0][3]
    # and the row against 32-block activations follows the same decode (src/q4x_cpu.rs:118-127)
    rng = np.random.default_rng(9)
    w = rng.integers(0, 256, 3 * 110, dtype=np.uint8)
    w[0::110], w[1::110] = 0x00, 0x2C
    x = rng.normal(0, 1, 768).astype(np.float32)
    q, d = oracle.q8_32(x)
    deq = oracle.dequant(synth.IQ3_S, w, 768).astype(np.float64)
    want_row = float(deq @ (q.astype(np.float64) * np.repeat(d, 32)))
    assert abs(oracle.row_iq3s(w, 768, q, d) - want_row) <= 1e-3 * max(abs(want_row), 1.0)
    # the codebook itself: 512 distinct entries of odd magnitudes 1..15, first and last as the format has them
    assert grid.shape == (512, 4) and len({tuple(g) for g in grid}) == 512
    assert set(np.unique(grid)) <= set(range(1, 16, 2))
    assert tuple(grid[0]) == (1, 1, 1, 1) and tuple(grid[1]) == (3, 1, 1, 1)


def test_q4k_against_32_block_activations(oracle):
    """The second activation mode (Q4_K weights, 32-value int8 blocks with an f16 scale). No reference
    code pairs them, so the pins are hand-computed: one super-block whose sub-block j has scale
    j + 1, min 2 j, every nibble 3 in the even and 5 in the odd sub-blocks; d = 0.5, dmin = 0.25."""
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.5).tobytes(), np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.25).tobytes(), np.uint8)
    sc = [j + 1 for j in range(8)]
    mn = [2 * j for j in range(8)]
    s = blk[4:16]
    for j in range(4):  # the 12 packed bytes of scales and mins (src/ds4_cpu.rs:45-57)
        s[j] = sc[j] | ((sc[j + 4] >> 4) << 6)
        s[j + 4] = mn[j] | ((mn[j + 4] >> 4) << 6)
        s[j + 8] = (sc[j + 4] & 15) | ((mn[j + 4] & 15) << 4)
    blk[16:144] = 3 | (5 << 4)
    q = np.zeros(256, np.int8)
    d32 = np.zeros(8, np.float32)
    want = 0.0
    for j in range(8):
        q[32 * j:32 * j + 32] = np.arange(32) - 10 - j  # sum = 176 - 32 j
        d32[j] = np.float32(2.0 ** -(j % 3))
        nib = 5 if j & 1 else 3
        isum = nib * int(q[32 * j:32 * j + 32].sum())
        bsum = int(q[32 * j:32 * j + 32].sum())
        want += float(d32[j]) * ((0.5 * sc[j]) * isum - (0.25 * mn[j]) * bsum)  # every step exact in f32
    got = oracle.row_q4k_q8_32(blk, 256, q, d32)
    assert got == np.float32(want)
    # the quantiser: the values of Q8::new, the scale rounded through f16
    x = np.linspace(-3.7, 5.3, 64).astype(np.float32)
    q0, d0 = oracle.q8_32(x)
    q1, d1 = oracle.q8_32(x, f16_scale=True)
    assert np.array_equal(q0, q1)
    assert np.array_equal(d1, d0.astype(np.float16).astype(np.float32))
    assert not np.array_equal(d0, d1)  # 5.3 / 127 is not an f16
    # and a layer in this mode is the 32-block expert flow (src/q4x_cpu.rs:399-440) on Q4_K rows
    cfg = synth.C12_Q4K_Q8_0.scaled(d=256, ff=256, n_exp=4, top_k=2)
    W = synth.make_weights(cfg, 5)
    L = oracle.Layer(oracle.LayerDesc(**cfg.desc_fields()), W)
    xx = synth.make_activations(3, cfg.d, 6)
    y = L.forward(xx)
    ref = oracle.Layer(oracle.LayerDesc(**cfg.scaled(act_quant=synth.AQ_Q8X_256).desc_fields()), W).forward(xx)
    assert np.all(np.isfinite(y)) and np.abs(y - ref).max() <= 0.02 * np.abs(ref).max()
