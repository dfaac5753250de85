"""The C-ABI library loads and exports every symbol include/pelica_moe.h
declares (no compute calls: this runs without a GPU)."""
import ctypes
import os
import re

import numpy as np
import pytest

import pelica_b200 as pb
from pelica_b200 import build, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols(header="pelica_moe.h"):
    src = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"PM_API[^;(]*?\b(pm_\w+)\s*\(", src)))


def test_header_and_binding_agree():
    names = declared_symbols()
    assert len(names) >= 30
    assert set(names) == set(pb.ABI), set(names) ^ set(pb.ABI)
    diag = declared_symbols("pelica_moe_diag.h")
    assert set(diag) == set(pb.ABI_DIAG), set(diag) ^ set(pb.ABI_DIAG)
    assert not set(diag) & set(names)


def test_boundary_header_cites_the_reference():
    """Every entry point of the boundary header sits under a comment that names the reference
    code it replaces or serves (src/...), except the documented addition without a counterpart."""
    src = open(os.path.join(ROOT, "include", "pelica_moe.h")).read()
    assert "src/ds4_cpu.rs:297" in src and "src/moe.rs:1377-1437" in src
    assert "No counterpart in the reference" in src  # pm_route_noalloc


def test_library_exports_every_declared_symbol():
    build.build_library()
    lib = ctypes.CDLL(pb.LIB_PATH)
    for name in declared_symbols() + declared_symbols("pelica_moe_diag.h"):
        assert hasattr(lib, name), name
    pb.load_library()
    assert b"sm_100a" in pb.load_library().pm_version()


def test_block_sizes():
    lib = pb.load_library()
    for ty, (v, b) in synth.BLOCK.items():
        assert lib.pm_type_block_values(ty) == v and lib.pm_type_block_bytes(ty) == b
    assert lib.pm_type_block_bytes(99) == 0


def test_no_cpu_fallback_in_product():
    """The package never reaches for the oracle."""
    pkg = os.path.join(ROOT, "pelica_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "pelica_oracle" not in text and "oracle/" not in text, f


def test_encoders_round_trip(oracle):
    rng = np.random.default_rng(0)
    x = rng.normal(0, 0.02, (3, 1024)).astype(np.float32)
    bound = {synth.Q4_K: 0.08, synth.Q6_K: 0.03, synth.MXFP4: 0.3, synth.Q8_0: 0.01, synth.IQ4_NL: 0.12, synth.IQ4_XS: 0.14,
             synth.Q5_K: 0.04, synth.IQ3_S: 0.35, synth.GLM_Q4: 0.08}
    for ty, enc in synth.ENCODERS.items():
        b = enc(x)
        assert b.shape == (3, synth.row_bytes(ty, 1024))
        y = oracle.dequant(ty, synth.encode_matrix(ty, x), x.size).reshape(x.shape)
        assert np.abs(y - x).max() <= bound[ty] * np.abs(x).max()
    z = np.zeros(256, np.float32)
    for ty, enc in synth.ENCODERS.items():
        assert not oracle.dequant(ty, enc(z), 256).any()
