"""Integer identities the tensor-core grouped kernel's operand planes rely on
(pelica_b200/csrc/prefill_tc.cu), checked exhaustively in numpy: they are what makes its
products exact, so that the float tail sees the very integers the reference's row_scalar
computes (src/ds4_cpu.rs:80-113)."""
import numpy as np


def test_q4k_planes_reproduce_scale_times_nibble():
    """Q4_K: sc (6 bits) x nibble (4 bits) does not fit a byte, so the operand is two u8 planes
    hi = nibble * (sc >> 3), lo = nibble * (sc & 7) and isum = 8 * (hi . xq) + (lo . xq)."""
    sc = np.arange(64)[:, None]
    nib = np.arange(16)[None, :]
    hi, lo = nib * (sc >> 3), nib * (sc & 7)
    assert hi.max() <= 255 and lo.max() <= 255
    assert np.array_equal(8 * hi + lo, sc * nib)
    # the products' int32 accumulators over a 256-value block cannot overflow
    assert 256 * 127 * int(hi.max()) * 8 < 2 ** 31


def test_q4k_mins_term_is_exact_in_f16_times_f16():
    """The mins' term sum_j m_j * bsum_j runs as one f16 product step: m_j (6 bits) against
    (64 * (bsum_j >> 6), bsum_j & 63). Both halves are integers an f16 holds exactly, every
    product and the whole sum stay below 2^24, so the f32 accumulator is exact."""
    bs = np.arange(-32 * 128, 32 * 127 + 1)  # a sub-block's sum of 32 int8 values
    hi, lo = 64 * (bs >> 6), bs & 63
    assert np.array_equal(hi + lo, bs)
    for v in (hi, lo):
        assert np.array_equal(v.astype(np.float16).astype(np.int64), v)
    assert 8 * 63 * (np.abs(hi).max() + lo.max()) < 2 ** 24


def test_q6k_planes_from_one_multiply_add():
    """Q6_K: v = sc * (q - 32) with v + 4128 = 64 * th + tl. The kernel computes
    z4 = 4 * sc * q + 4 * (4128 - 32 * sc) in a 16-bit lane: its high byte is th and its low
    byte 4 * tl, both u8, and 4 * isum = 256 * (th . xq) + (4 tl . xq) - 16512 * sum(xq)."""
    sc = np.arange(-128, 128)[:, None]
    q = np.arange(64)[None, :]
    v = sc * (q - 32)
    z4 = 4 * sc * q + 4 * (4128 - 32 * sc)
    assert z4.min() >= 0 and z4.max() < 2 ** 16  # a 16-bit lane never borrows from its neighbour
    th, tl4 = z4 >> 8, z4 & 0xFF
    assert np.array_equal(64 * th + tl4 // 4, v + 4128)
    assert np.all(tl4 % 4 == 0) and th.max() <= 255
    rng = np.random.default_rng(0)
    for _ in range(20):
        scs = rng.integers(-128, 128, 16)
        qs = rng.integers(0, 64, 256)
        xq = rng.integers(-127, 128, 256)
        s = np.repeat(scs, 16)
        isum = int((s * (qs - 32) * xq).sum())
        zz = 4 * s * qs + 4 * (4128 - 32 * s)
        got4 = 256 * int(((zz >> 8) * xq).sum()) + int(((zz & 0xFF) * xq).sum()) - 16512 * int(xq.sum())
        assert got4 == 4 * isum
        # (d / 4) * float(4 isum) rounds as d * float(isum): both scalings are by a power of two
        d = np.float32(rng.standard_normal() * 1e-3)
        a = np.float32(d * np.float32(0.25)) * np.float32(got4)
        b = d * np.float32(isum)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32)
    # the extreme accumulators stay inside int32
    assert 256 * (256 * 255 * 127) < 2 ** 31 and 16512 * 256 * 127 < 2 ** 31


def test_q6k_high_bits_rotation():
    """The two high bits of a 6-bit value sit at bit 2 * j (+ 4 for the second nibble half) of a
    qh byte; one rotation by (shift - 4) mod 32 brings them to bits 4, 5 of the same byte."""
    rng = np.random.default_rng(1)
    for _ in range(200):
        w = int(rng.integers(0, 2 ** 32))
        for shift in (0, 2, 4, 6):
            r = (shift - 4) & 31
            rot = ((w >> r) | (w << (32 - r))) & 0xFFFFFFFF if r else w
            want = ((w >> shift) & 0x03030303) << 4
            assert rot & 0x30303030 == want
