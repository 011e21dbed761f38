"""Cross-checks the ctypes signatures of `native._SIGS` against the `extern "C"` prototypes in
`csrc/` (parsed as text), so an argument-type drift is caught on a CPU-only machine."""
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(os.path.dirname(_HERE), "csrc")


def _code(ctype):
    t = ctype.strip()
    if "*" in t or "cudaStream_t" in t:
        return "p"
    t = re.sub(r"\bconst\b", "", t).strip()
    t = " ".join(t.split()[:-1]) if len(t.split()) > 1 else t     # drop the parameter name
    return {"int": "i", "long long": "l", "float": "f", "unsigned long long": "u", "unsigned int": "I",
            "size_t": "z", "ssize_t": "l", "int64_t": "l", "double": "d"}[t]


def prototypes():
    out = {}
    for fn in sorted(os.listdir(_CSRC)):
        if not fn.endswith((".cu", ".cpp")):
            continue
        src = open(os.path.join(_CSRC, fn)).read()
        for m in re.finditer(r'extern "C" int (gb_\w+)\(([^)]*)\)', src):
            args = [a for a in m.group(2).replace("\n", " ").split(",") if a.strip()]
            out[m.group(1)] = "".join(_code(a) for a in args)
    return out


def mismatches():
    from . import native
    protos = prototypes()
    bad = []
    for name, sig in native._SIGS.items():
        if name not in protos:
            bad.append((name, sig, None))
        elif protos[name] != sig:
            bad.append((name, sig, protos[name]))
    return bad
