"""Writes tests/golden/known_answer_blocks.json: hand-derivable known-answer blocks per GGUF type.

The reference holds no golden vectors for Q8_0 / Q4_K / Q5_K / Q6_K (its specs read a model
file), only a synthetic IQ4_NL block with d = 1.0 and a nibble ramp
(spec/iq4_nl_dequant_spec.cr:36-51).  This script builds blocks in the same style — half scales
that are powers of two, unit or small integer sub-block scales, ramps of quants — and computes
the expected f32 outputs with plain integer arithmetic written out below, independently of the
oracle (it never imports it).  Each expected value is exactly representable, so the comparison
in the tests is bit-exact.

Run from the repository root:  python tests/golden/make_known_answer_blocks.py
"""
import json
import struct
from pathlib import Path

HALF_ONE, HALF_HALF, HALF_TWO, HALF_QUARTER = 0x3C00, 0x3800, 0x4000, 0x3400


def le16(v):
    return [v & 0xFF, (v >> 8) & 0xFF]


def pack_k4(sc, mn):
    """12 bytes from eight 6-bit (scale, min) pairs; layout read back by get_scale_min_k4."""
    out = [0] * 12
    for j in range(4):
        out[j] = (sc[j] & 63) | ((sc[j + 4] >> 4) << 6)
        out[j + 4] = (mn[j] & 63) | ((mn[j + 4] >> 4) << 6)
        out[j + 8] = (sc[j + 4] & 0x0F) | ((mn[j + 4] & 0x0F) << 4)
    return out


def q8_0_case():
    # d = 0.5, quants -16..15  ->  w = 0.5 * q
    qs = list(range(-16, 16))
    raw = le16(HALF_HALF) + [q & 0xFF for q in qs]
    return {"type": 8, "n": 32, "raw": raw, "expected": [0.5 * q for q in qs]}


def q4_k_case():
    # d = 1, dmin = 0.5, scale of sub-block s = s + 1, min of sub-block s = 2 s (so 33..40 uses the
    # high 2 bits of the packing too when offset by 32): element l of sub-block s has quant
    # (l + s) % 16  ->  w = (s + 1 + 32 [s >= 4]) * q - 0.5 * m
    sc = [1, 2, 3, 4, 37, 38, 39, 40]
    mn = [0, 2, 4, 6, 40, 42, 44, 63]
    qs = [0] * 128
    q_of = lambda s, l: (l + s) % 16
    for pair in range(4):
        for l in range(32):
            qs[32 * pair + l] = q_of(2 * pair, l) | (q_of(2 * pair + 1, l) << 4)
    raw = le16(HALF_ONE) + le16(HALF_HALF) + pack_k4(sc, mn) + qs
    exp = []
    for s in range(8):
        for l in range(32):
            exp.append(1.0 * sc[s] * q_of(s, l) - 0.5 * mn[s])
    return {"type": 12, "n": 256, "raw": raw, "expected": exp}


def q5_k_case():
    # d = 2, dmin = 1; quant of element l in sub-block s is (3 l + 5 s) % 32 (five bits)
    sc = [1, 3, 5, 7, 33, 45, 50, 63]
    mn = [1, 0, 2, 0, 35, 0, 61, 17]
    q_of = lambda s, l: (3 * l + 5 * s) % 32
    ql = [0] * 128
    qh = [0] * 32
    for pair in range(4):
        for l in range(32):
            a, b = q_of(2 * pair, l), q_of(2 * pair + 1, l)
            ql[32 * pair + l] = (a & 15) | ((b & 15) << 4)
            qh[l] |= ((a >> 4) << (2 * pair)) | ((b >> 4) << (2 * pair + 1))
    raw = le16(HALF_TWO) + le16(HALF_ONE) + pack_k4(sc, mn) + qh + ql
    exp = []
    for s in range(8):
        for l in range(32):
            exp.append(2.0 * sc[s] * q_of(s, l) - 1.0 * mn[s])
    return {"type": 13, "n": 256, "raw": raw, "expected": exp}


def q6_k_case():
    # d = 0.25; scale of 16-element group j is j - 8 (signed); quant of element e is (7 e) % 64,
    # stored minus nothing: value = d * sc * (q - 32)
    q_of = lambda e: (7 * e) % 64
    ql = [0] * 128
    qh = [0] * 64
    for half in range(2):
        for l in range(32):
            e = [128 * half + l + 32 * k for k in range(4)]
            q = [q_of(x) for x in e]
            ql[64 * half + l] = (q[0] & 15) | ((q[2] & 15) << 4)
            ql[64 * half + 32 + l] = (q[1] & 15) | ((q[3] & 15) << 4)
            qh[32 * half + l] = (q[0] >> 4) | ((q[1] >> 4) << 2) | ((q[2] >> 4) << 4) | ((q[3] >> 4) << 6)
    scales = [j - 8 for j in range(16)]
    raw = ql + qh + [s & 0xFF for s in scales] + le16(HALF_QUARTER)
    exp = [0.25 * scales[e // 16] * (q_of(e) - 32) for e in range(256)]
    return {"type": 14, "n": 256, "raw": raw, "expected": exp}


def main():
    cases = [q8_0_case(), q4_k_case(), q5_k_case(), q6_k_case()]
    for c in cases:  # every expected value must survive a round trip through f32 unchanged
        for v in c["expected"]:
            assert struct.unpack("<f", struct.pack("<f", v))[0] == v
        assert all(0 <= b <= 255 for b in c["raw"])
    path = Path(__file__).resolve().parent / "known_answer_blocks.json"
    path.write_text(json.dumps(cases))
    print(path, [len(c["raw"]) for c in cases])


if __name__ == "__main__":
    main()
