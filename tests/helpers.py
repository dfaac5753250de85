"""Shared pieces of the parity tests."""
import numpy as np

from pelica_b200 import synth


def lcg(seed):
    """The generator every hot-path test of the reference uses
    (s = s*1664525 + 1013904223, src/ds4_cpu.rs:448-452)."""
    s = seed & 0xFFFFFFFF

    def rnd():
        nonlocal s
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        return s

    return rnd


def ref_q4k_blocks(rnd, n_blocks, d_bits=0x2C00, dmin_bits=0x2800):
    """Q4_K blocks as the reference's tests build them: fixed f16 d/dmin, every
    other byte random (src/ds4_cpu.rs:454-462)."""
    w = np.zeros(n_blocks * 144, np.uint8)
    for b in range(n_blocks):
        blk = w[b * 144:(b + 1) * 144]
        blk[0:2] = np.frombuffer(np.uint16(d_bits).tobytes(), np.uint8)
        blk[2:4] = np.frombuffer(np.uint16(dmin_bits).tobytes(), np.uint8)
        for i in range(4, 144):
            blk[i] = rnd() & 0xFF
    return w


def ref_acts(rnd, n):
    """(rnd() % 2000) / 1000 - 1 (src/ds4_cpu.rs:463)."""
    return np.array([np.float32(rnd() % 2000) / np.float32(1000.0) - np.float32(1.0) for _ in range(n)], np.float32)


def tol_ok(got, ref):
    """|got-ref| <= 1e-3*|ref| + 1e-4*RMS(ref): the layer-output tolerance
    (1e-3 relative / 1e-4 absolute-over-RMS, fp32 accumulation)."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    rms = np.sqrt((ref ** 2).mean()) if ref.size else 0.0
    return np.all(np.abs(got - ref) <= 1e-3 * np.abs(ref) + 1e-4 * rms)


def bits_equal(a, b):
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


# reduced forms of the five benchmark shapes: same arithmetic, sizes the CPU
# checker finishes in about a second
SMALL = {
    "c1": synth.C1_OLMOE.scaled(d=512, ff=256, n_exp=16),
    "c2": synth.C2_QWEN3.scaled(d=512, ff=256, n_exp=24),
    "c3": synth.C3_GPTOSS.scaled(d=320, ff=160, n_exp=8),
    "c4": synth.C4_DSV3.scaled(d=512, ff=256, n_exp=32, n_group=4, topk_group=2, shared_ff=256),
    "c5": synth.C5_ZIPF.scaled(d=512, ff=256, n_exp=32),
    "c6": synth.C6_Q8_0.scaled(d=320, ff=160, n_exp=16),
    "c7": synth.C7_IQ4NL.scaled(d=320, ff=160, n_exp=16, type_down=synth.Q8_0),  # mixed 32-block types
    "c8": synth.C8_IQ4XS.scaled(d=512, ff=160, n_exp=16),
    "c9": synth.C9_IQ3S.scaled(d=512, ff=160, n_exp=16),
    "c10": synth.C10_Q5K.scaled(d=512, ff=256, n_exp=16),
    "c11": synth.C11_GLM.scaled(d=512, ff=192, n_exp=16, shared_ff=192),
    "c12": synth.C12_Q4K_Q8_0.scaled(d=512, ff=256, n_exp=16),  # Q4_K against 32-block activations, f16 scale
}


def make_pair(po, pb, ctx, cfg, seed):
    """The same weights on both sides: (oracle layer, CUDA layer, weights)."""
    W = synth.make_weights(cfg, seed)
    ol = po.Layer(po.LayerDesc(**cfg.desc_fields()), W)
    gl = pb.MoeLayer(ctx, cfg).load(W)
    return ol, gl, W


def device_pair(po, pb, ctx, cfg, seed):
    """A layer whose weights are generated on the GPU (any size, seconds) and read back for
    the CPU checker: (oracle layer, CUDA layer). Only the experts the context holds are
    read back (cfg.n_exp_local), so a shard of a full-width layer stays a few hundred MB."""
    gl = pb.MoeLayer(ctx, cfg).fill_synthetic(seed, cfg.sigma, cfg.sigma if cfg.logit_bias else 0.0,
                                              cfg.select_bias_sigma)
    W = gl.get_weights(dense=False)
    ol = po.Layer(po.LayerDesc(**cfg.desc_fields()), W)
    return ol, gl
