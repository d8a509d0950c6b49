"""The ctypes signature table must match the `extern "C"` declarations in the kernel sources.

A mismatch would not fail at import time -- it would corrupt arguments at the first launch -- so the table
is checked against the source text here, on CPU.
"""
import ctypes as C
import re
from pathlib import Path

from rembrandt_b200 import _native

CSRC = Path(_native.__file__).resolve().parent / "csrc"

_CTYPE = {
    "int": C.c_int, "long long": C.c_longlong, "float": C.c_float, "unsigned int": C.c_uint,
    "unsigned long long": C.c_ulonglong, "cudaStream_t": C.c_void_p,
}


def _parse_decls():
    decls = {}
    for src in sorted(CSRC.glob("*.cu")):
        text = src.read_text()
        for m in re.finditer(r'extern "C" \{(.*?)\n\}  // extern "C"', text, re.S):
            body = m.group(1)
            for f in re.finditer(r"\n(?:int|void) (rb_\w+)\(([^)]*)\)\s*\{", body):
                name, args = f.group(1), f.group(2).strip()
                types = []
                if args:
                    for a in args.split(","):
                        a = " ".join(a.split())
                        if "*" in a:
                            types.append(C.c_void_p)
                        else:
                            base = a.rsplit(" ", 1)[0].replace("const ", "")
                            types.append(_CTYPE[base])
                decls[name] = types
    return decls


def test_every_launcher_is_declared_with_matching_types():
    decls = _parse_decls()
    # the allocation-free entry point is bound by its own test straight from the C symbol
    decls = {k: v for k, v in decls.items() if not k.endswith("_noalloc")}
    table = dict(_native._CUDA_SIGS)
    # launchers bound by other modules through _native.register carry their own tables
    from rembrandt_b200.parallel import p2p_kernels
    table.update(p2p_kernels.SIGS)
    missing = sorted(set(decls) - set(table))
    assert not missing, f"launchers without a ctypes signature: {missing}"
    for name, sig in table.items():
        assert name in decls, f"{name} is in the table but not exported"
        assert len(sig) == len(decls[name]), f"{name}: {len(sig)} ctypes args vs {len(decls[name])} in source"
        for i, (a, b) in enumerate(zip(sig, decls[name])):
            assert a is b, f"{name} arg {i}: table {a.__name__} vs source {b.__name__}"
