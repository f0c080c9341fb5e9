"""The Crystal source of record (crystal/src/ml/cuda/cogni_qmm.cr) against the C headers.

No Crystal compiler exists where the engine is built, so the binding is checked as text, the way
the reference's source-shape specs check kernel sources (spec/gemm_mm_barrier_spec.cr:4-29): every
symbol the headers declare has a `fun` with the same name, the same number of parameters and a
return type of the same width; no `fun` names a symbol the headers do not have."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CR = (ROOT / "crystal" / "src" / "ml" / "cuda" / "cogni_qmm.cr").read_text()
HEADERS = (ROOT / "include" / "cogni_qmm.h").read_text() + (ROOT / "include" / "cogni_qmm_diag.h").read_text()

RET = {"int": "Int32", "unsigned": "UInt32", "size_t": "LibC::SizeT", "int64_t": "Int64",
       "const char *": "UInt8*"}


def c_prototypes():
    body = re.sub(r"/\*.*?\*/", "", HEADERS, flags=re.S)
    out = {}
    for m in re.finditer(r"^\s*((?:const\s+)?[a-z_0-9]+(?:\s*\*)?)\s*(cogni_qmm_\w+)\s*\(([^;{]*?)\)\s*;", body, re.M):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        n = 0 if params in ("", "void") else len([p for p in params.split(",") if p.strip()])
        out[name] = (re.sub(r"\s+", " ", ret), n)
    return out


def crystal_funs():
    lib = CR[CR.index("lib LibCogniQMM"):CR.index("\nend\n", CR.index("lib LibCogniQMM"))]
    out = {}
    for m in re.finditer(r"^\s*fun (cogni_qmm_\w+)(?:\(([^)]*)\))?\s*:\s*([\w:*]+)", lib, re.M | re.S):
        params = m.group(2)
        n = 0 if not params else len([p for p in params.split(",") if p.strip()])
        out[m.group(1)] = (m.group(3), n)
    return out


def test_binding_and_headers_agree():
    c, cr = c_prototypes(), crystal_funs()
    assert len(c) >= 30
    assert sorted(c) == sorted(cr), (sorted(set(c) - set(cr)), sorted(set(cr) - set(c)))
    for name, (ret, n) in c.items():
        assert cr[name][1] == n, f"{name}: {cr[name][1]} parameters in Crystal, {n} in C"
        assert cr[name][0] == RET[ret], f"{name}: returns {cr[name][0]} in Crystal, {ret} in C"


def test_exchange_struct_matches_the_header():
    body = HEADERS[HEADERS.index("typedef struct cogni_qmm_exchange"):HEADERS.index("} cogni_qmm_exchange;")]
    c_fields = re.findall(r"\b(world|rank|peer_offset|epoch|ticket)\b", body)
    cr = CR[CR.index("struct Exchange"):CR.index("end", CR.index("struct Exchange"))]
    assert c_fields == re.findall(r"\b(world|rank|peer_offset|epoch|ticket)\b", cr)
