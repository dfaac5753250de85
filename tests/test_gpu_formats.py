"""Bit-exact checks of block decoding and activation quantisation on the GPU
(through the C ABI) against the oracle."""
import numpy as np
import pytest

from pelica_b200 import synth
from tests.helpers import bits_equal, lcg, ref_acts, ref_q4k_blocks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ty", [synth.Q4_K, synth.Q5_K, synth.Q6_K, synth.MXFP4, synth.Q8_0, synth.IQ4_NL,
                                synth.IQ4_XS, synth.IQ3_S, synth.GLM_Q4])
def test_dequant_random_bytes_bit_exact(ctx, oracle, ty):
    """Every bit pattern path: random block bytes, only the f16 scales kept finite."""
    v, b = synth.BLOCK[ty]
    rng = np.random.default_rng(ty)
    nb = 257
    raw = rng.integers(0, 256, nb * b, dtype=np.uint8).reshape(nb, b)
    half = rng.normal(0, 0.05, (nb, 2)).astype(np.float16).view(np.uint8).reshape(nb, 4)
    if ty in (synth.Q4_K, synth.Q5_K):
        raw[:, 0:4] = half
    elif ty == synth.Q6_K:
        raw[:, 208:210] = half[:, :2]
    elif ty in (synth.Q8_0, synth.IQ4_NL, synth.IQ4_XS, synth.IQ3_S):
        raw[:, 0:2] = half[:, :2]
    elif ty == synth.GLM_Q4:  # the nibble region, then finite f32 group scales
        raw.reshape(-1)[nb * 32:] = rng.normal(0, 0.05, nb).astype(np.float32).view(np.uint8)
    else:
        raw[:3, 0] = [0, 1, 2]  # the denormal branch of e8 (src/oss_kernels.rs:42-45)
        raw[3, 0] = 254
    want = oracle.dequant(ty, raw.ravel(), nb * v)
    got = ctx.dequant(ty, raw.ravel(), nb * v)
    assert bits_equal(got, want)


@pytest.mark.parametrize("ty", [synth.Q4_K, synth.Q5_K, synth.Q6_K, synth.MXFP4, synth.IQ4_NL, synth.IQ4_XS,
                                synth.IQ3_S, synth.GLM_Q4])
def test_dequant_encoded_weights(ctx, oracle, ty):
    rng = np.random.default_rng(1)
    x = rng.normal(0, 0.02, 4096).astype(np.float32)
    raw = synth.ENCODERS[ty](x)
    assert bits_equal(ctx.dequant(ty, raw, 4096), oracle.dequant(ty, raw, 4096))


def test_dequant_empty_and_ragged(ctx):
    import pelica_b200 as pb

    assert ctx.dequant(synth.Q4_K, np.zeros(0, np.uint8), 0).size == 0
    with pytest.raises(pb.PelicaError):
        ctx.dequant(synth.Q4_K, np.zeros(144, np.uint8), 100)
    with pytest.raises(pb.PelicaError):
        ctx.dequant(5, np.zeros(144, np.uint8), 256)


def test_quant_act_bit_exact(ctx, oracle):
    rng = np.random.default_rng(2)
    cases = [rng.normal(0, 1, 2048), rng.normal(0, 1e-3, 768), np.zeros(512), rng.normal(0, 50, 7168)]
    x = rng.normal(0, 1, 1024)
    x[256:512] = 0.0          # an all-zero block in the middle: d = 0, q = 0
    x[5] = 3.0
    x[6] = -1.5 * 3.0 / 127   # lands on a .5 boundary: rounds away from zero
    cases.append(x)
    cases.append(ref_acts(lcg(1), 1024))  # the reference's test activations (src/ds4_cpu.rs:463)
    for x in cases:
        x = x.astype(np.float32)
        q, d, bs = ctx.quant_act(x)
        oq, od, obs = oracle.q8x(x)
        assert np.array_equal(q, oq)
        assert bits_equal(d, od)
        assert np.array_equal(bs, obs)


def test_quant_act_32_bit_exact(ctx, oracle):
    """`Q8::new` (src/q4x_cpu.rs:23-37): values, scales; zero blocks, ties, clamping."""
    rng = np.random.default_rng(12)
    cases = [rng.standard_normal(2560).astype(np.float32), np.zeros(64, np.float32),
             np.concatenate([np.zeros(32), np.full(32, -3.5), np.arange(32) - 15.5]).astype(np.float32),
             (rng.standard_normal(640) * 1e-30).astype(np.float32), (rng.standard_normal(320) * 1e30).astype(np.float32)]
    half = np.zeros(32, np.float32)  # .5 ties round away from zero
    half[0], half[1], half[2], half[3] = 127.0, 0.5, -0.5, 1.5
    cases.append(half)
    for x in cases:
        q, d = ctx.quant_act_32(x)
        oq, od = oracle.q8_32(x)
        assert np.array_equal(q, oq)
        assert bits_equal(d, od)


def test_quant_act_rejects_ragged(ctx):
    import pelica_b200 as pb

    with pytest.raises(pb.PelicaError):
        ctx.quant_act(np.zeros(300, np.float32))
