"""The Rust binding shipped as source (no Rust toolchain exists where the library is built):
ffi.rs must be exactly what gen_ffi.py derives from the C header, must declare every exported
symbol, and every call in cuda_backend.rs must name a declared function with the declared number
of arguments."""
import re
import subprocess
import sys
from pathlib import Path

from agention_infer_b200 import _abi

ROOT = Path(__file__).resolve().parent.parent
RUST = ROOT / "agention_infer_b200" / "rust"


def _declared():
    out = {}
    for name, args in re.findall(r"pub fn (agn_\w+)\((.*?)\) ->", (RUST / "ffi.rs").read_text()):
        out[name] = 0 if not args.strip() else len(args.split(","))
    return out


def test_ffi_rs_is_up_to_date_with_the_header():
    assert subprocess.run([sys.executable, str(RUST / "gen_ffi.py"), "--check"]).returncode == 0


def test_ffi_rs_declares_every_entry_point_with_the_same_arity():
    decl = _declared()
    assert set(decl) == set(_abi.SIGNATURES)
    for name, (_, argtypes) in _abi.SIGNATURES.items():
        assert decl[name] == len(argtypes), name


def _call_args(text, start):
    """Top-level comma count of the call whose '(' is at text[start]."""
    depth, n, i, seen = 0, 0, start, False
    while True:
        c = text[i]
        if c in "([{":
            depth += 1
        elif c in ")]}":
            depth -= 1
            if depth == 0:
                return n + 1 if seen else 0
        elif c == "," and depth == 1:
            n += 1
        elif depth >= 1 and not c.isspace():
            seen = True
        i += 1


def test_cuda_backend_rs_calls_match_the_declarations():
    decl = _declared()
    text = re.sub(r"//.*", "", (RUST / "cuda_backend.rs").read_text())
    calls = [(m.group(1), _call_args(text, m.end() - 1)) for m in re.finditer(r"\b(agn_\w+)\(", text)]
    assert len(calls) > 20
    for name, n in calls:
        assert name in decl, name
        assert n == decl[name], (name, n, decl[name])
