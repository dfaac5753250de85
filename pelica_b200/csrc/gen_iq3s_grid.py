"""Writes include/pelica_iq3s_grid.inc: the IQ3_S codebook of the GGUF format in packed form.

The codebook is a constant of the format (ggml-common.h of llama.cpp, MIT licence: `iq3s_grid`,
512 entries of four odd magnitudes 1..15). Each entry is stored here as 12 bits, three per
magnitude: code = (magnitude - 1) / 2, value j in bits 3j..3j+2. Usage:

    python pelica_b200/csrc/gen_iq3s_grid.py <file holding the 512 hexadecimal words>

Any text file that lists the 512 grid words as 0x........ literals in order works (the table of
src/iq_tables.rs of the reference engine, or ggml-common.h).
"""
import os
import re
import sys


def main(src: str) -> None:
    text = open(src).read()
    start = text.index("IQ3S_GRID") if "IQ3S_GRID" in text else text.index("iq3s_grid")
    words = [int(w, 16) for w in re.findall(r"0x[0-9a-fA-F]{8}", text[start:])][:512]
    assert len(words) == 512
    codes = []
    for w in words:
        c = 0
        for j in range(4):
            m = (w >> (8 * j)) & 0xff
            assert m % 2 == 1 and 1 <= m <= 15, hex(w)
            c |= ((m - 1) // 2) << (3 * j)
        codes.append(c)
    out = os.path.join(os.path.dirname(__file__), "..", "..", "include", "pelica_iq3s_grid.inc")
    with open(out, "w") as f:
        f.write("/* IQ3_S codebook of the GGUF format (llama.cpp ggml-common.h `iq3s_grid`, MIT), packed:\n"
                " * entry i = 12 bits, magnitude j of the entry = 2 * ((code >> 3j) & 7) + 1.\n"
                " * Written by pelica_b200/csrc/gen_iq3s_grid.py. */\n")
        for i in range(0, 512, 16):
            f.write(" ".join(f"0x{c:03x}," for c in codes[i:i + 16]) + "\n")


if __name__ == "__main__":
    main(sys.argv[1])
