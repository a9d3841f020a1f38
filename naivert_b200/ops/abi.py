"""ABI check between the kernels' C argument structs and their ctypes mirrors in ``ops/kernels.py``.

The library is driven through ~25 ``extern "C"`` entry points that take pointers to plain argument structs.  Their
Python mirrors are written by hand; this module reads the struct declarations from the CUDA sources (field names,
order, scalar / pointer / array / nested-struct kinds), computes the layout a 64-bit C compiler gives them and
compares names, offsets and total size with the ctypes classes - on the CPU, without building or loading the library
(at load time the sizes are checked once more against ``nrt_*_args_size`` of the built library).

    python -m naivert_b200.ops.abi                 # prints one line per struct, exit 1 on a mismatch
    python -m naivert_b200.ops.abi --emit FILE     # writes the ctypes classes generated from the CUDA sources

The same parse also generates bindings: ``generate(name)`` builds the ctypes class of a struct from its C
declaration, ``emit_module()`` writes all of them as Python source.  A binding for a new kernel starts from the
emitted class; the test suite checks that every hand-kept mirror equals its generated class field by field.

Reference counterpart: naivert/kernels/opgen.py generates entry and binding sources from op descriptors; here the
CUDA sources are the description, and bindings are generated from and checked against them.
"""
from __future__ import annotations

import ctypes as C
import os
import re
import sys
from typing import Dict, List, Optional, Tuple

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

# C struct -> (source file, ctypes class name in ops.kernels)
STRUCTS: Dict[str, Tuple[str, str]] = {
    "FabricArgs": ("gemm.cuh", "FabricArgs"), "AttnPostArgs": ("gemm.cuh", "AttnPostArgs"), "GemmArgs": ("gemm.cuh", "GemmArgs"),
    "RouterArgs": ("router.cuh", "RouterArgs"), "MoeArgs": ("moe_fused.cu", "MoeArgs"), "XchgArgs": ("fabric.cuh", "XchgArgs"),
    "AttnArgs": ("target_kernels.cu", "AttnArgs"), "IndexArgs": ("target_kernels.cu", "IndexArgs"),
    "PrologueArgs": ("target_kernels.cu", "PrologueArgs"), "SweepArgs": ("index_sweep.cu", "SweepArgs"),
    "ArgmaxArgs": ("argmax.cu", "ArgmaxArgs"), "SamplerArgs": ("sampler.cu", "SamplerArgs"), "TailArgs": ("sampler.cu", "TailArgs"),
    "RingRecord": ("sampler.cu", "RingRecord"), "MarkovArgs": ("draft.cu", "MarkovArgs"), "AgPushArgs": ("collectives.cu", "AgPushArgs"),
    "EpArgs": ("ep.cu", "EpArgs"), "EpCombineArgs": ("ep.cu", "EpCombineArgs"),
}
# structs that are declared in more than one translation unit must be identical there
DUPLICATES = {"AttnArgs": ["target_kernels.cu", "attn_decode.cu", "attn_group.cu"]}

SCALARS = {"int": 4, "unsigned": 4, "unsigned int": 4, "uint32_t": 4, "int32_t": 4, "float": 4, "double": 8, "long long": 8,
           "unsigned long long": 8, "uint64_t": 8, "int64_t": 8, "size_t": 8, "unsigned short": 2, "uint16_t": 2,
           "uint8_t": 1, "char": 1, "unsigned char": 1, "bool": 1}
CONSTANTS = {"kMaxPeers": 8, "kXchgPeers": 8}


CTYPES = {"int": "c_int", "unsigned": "c_uint", "unsigned int": "c_uint", "uint32_t": "c_uint32", "int32_t": "c_int32",
          "float": "c_float", "double": "c_double", "long long": "c_longlong", "unsigned long long": "c_ulonglong",
          "uint64_t": "c_uint64", "int64_t": "c_int64", "size_t": "c_size_t", "unsigned short": "c_ushort",
          "uint16_t": "c_uint16", "uint8_t": "c_uint8", "char": "c_char", "unsigned char": "c_ubyte", "bool": "c_bool"}


class Field:
    def __init__(self, name: str, size: int, align: int, kind: str, ctype: str = "", count: int = 1):
        self.name, self.size, self.align, self.kind = name, size, align, kind
        self.ctype, self.count = ctype, count           # C element type ("*" for any pointer) and array length


def _strip_comments(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def struct_body(path: str, name: str) -> Optional[str]:
    text = _strip_comments(open(path).read())
    m = re.search(r"\bstruct\s+" + re.escape(name) + r"\s*\{", text)
    if not m:
        return None
    depth, i = 1, m.end()
    while i < len(text) and depth:
        depth += {"{": 1, "}": -1}.get(text[i], 0)
        i += 1
    return text[m.end():i - 1]


def parse_fields(body: str, known: Dict[str, Tuple[int, int]]) -> List[Field]:
    """``known``: nested struct name -> (size, alignment)."""
    fields: List[Field] = []
    for decl in body.split(";"):
        decl = " ".join(decl.split())
        if not decl or "(" in decl:                     # no member functions in argument structs
            continue
        decl = re.sub(r"\b(const|volatile|struct)\b", " ", decl)
        decl = " ".join(decl.split())
        # split "type a, *b, c[4]" into type and declarators
        toks = decl.replace("*", " * ").split()
        n = 0
        while n < len(toks) and toks[n] in ("unsigned", "signed", "long", "short", "int", "char", "float", "double", "bool"):
            n += 1
        if n == 0:
            n = 1                                       # a typedef or struct name
        ctype, rest = " ".join(toks[:n]), " ".join(toks[n:])
        ctype = {"unsigned long long int": "unsigned long long", "long long int": "long long", "signed int": "int"}.get(ctype, ctype)
        for d in rest.split(","):
            d = d.strip()
            ptr = d.count("*")
            d = d.replace("*", "").strip()
            am = re.match(r"^([A-Za-z_][A-Za-z0-9_]*)\s*((?:\[[^\]]+\])*)$", d)
            if not am:
                raise ValueError(f"cannot parse declarator {d!r} in {decl!r}")
            name, dims = am.group(1), re.findall(r"\[([^\]]+)\]", am.group(2))
            count = 1
            for dim in dims:
                dim = dim.strip()
                count *= int(dim) if dim.isdigit() else CONSTANTS[dim]
            if ptr:
                size, align, kind = 8, 8, "pointer"
            elif ctype in SCALARS:
                size = align = SCALARS[ctype]
                kind = "scalar"
            elif ctype in known:
                size, align = known[ctype]
                kind = "struct"
            else:
                raise ValueError(f"unknown type {ctype!r} in {decl!r}")
            fields.append(Field(name, size * count, align, kind if count == 1 else kind + "[]", "*" if ptr else ctype, count))
    return fields


def layout(fields: List[Field]) -> Tuple[List[Tuple[str, int, int]], int, int]:
    """(name, offset, size) per field, total size, alignment - natural alignment rules of the C ABI."""
    off, out, amax = 0, [], 1
    for f in fields:
        off = (off + f.align - 1) // f.align * f.align
        out.append((f.name, off, f.size))
        off += f.size
        amax = max(amax, f.align)
    return out, (off + amax - 1) // amax * amax, amax


ORDER = ["FabricArgs", "AttnPostArgs", "XchgArgs", "GemmArgs", "RouterArgs", "MoeArgs"]


def _ordered() -> List[str]:
    return ORDER + [n for n in STRUCTS if n not in ORDER]


def parse_all() -> Dict[str, List[Field]]:
    """Fields of every argument struct, nested structs resolved in dependency order."""
    known: Dict[str, Tuple[int, int]] = {}
    out: Dict[str, List[Field]] = {}
    for name in _ordered():
        body = struct_body(os.path.join(CSRC, STRUCTS[name][0]), name)
        if body is None:
            raise ValueError(f"{name}: not found in {STRUCTS[name][0]}")
        out[name] = parse_fields(body, known)
        _, size, align = layout(out[name])
        known[name] = (size, align)
    return out


def generate(name: str, parsed: Optional[Dict[str, List[Field]]] = None, _cache: Optional[dict] = None):
    """The ctypes.Structure class of C struct ``name``, built from its declaration in the CUDA sources (pointers become
    ``c_void_p``, nested argument structs their generated classes)."""
    parsed = parsed or parse_all()
    cache = _cache if _cache is not None else {}
    if name in cache:
        return cache[name]
    fields = []
    for f in parsed[name]:
        if f.ctype == "*":
            t = C.c_void_p
        elif f.ctype in CTYPES:
            t = getattr(C, CTYPES[f.ctype])
        else:
            t = generate(f.ctype, parsed, cache)
        fields.append((f.name, t * f.count if f.count > 1 else t))
    cache[name] = type(name, (C.Structure,), {"_fields_": fields})
    return cache[name]


def emit_module() -> str:
    """Python source of all generated classes (the starting point of a new binding)."""
    parsed = parse_all()
    lines = ['"""ctypes mirrors of the kernels\' argument structs - generated by ``python -m naivert_b200.ops.abi --emit``."""',
             "import ctypes as C", ""]
    for name in _ordered():
        lines += ["", f"class {name}(C.Structure):      # {STRUCTS[name][0]}", "    _fields_ = ["]
        for f in parsed[name]:
            t = "C.c_void_p" if f.ctype == "*" else "C." + CTYPES[f.ctype] if f.ctype in CTYPES else f.ctype
            lines.append(f'        ("{f.name}", {t}{" * " + str(f.count) if f.count > 1 else ""}),')
        lines.append("    ]")
    return "\n".join(lines) + "\n"


def check_all() -> List[str]:
    from . import kernels as K
    problems: List[str] = []
    known: Dict[str, Tuple[int, int]] = {}
    order = ["FabricArgs", "AttnPostArgs", "XchgArgs", "GemmArgs", "RouterArgs", "MoeArgs"] + \
            [n for n in STRUCTS if n not in ("FabricArgs", "AttnPostArgs", "XchgArgs", "GemmArgs", "RouterArgs", "MoeArgs")]
    report = []
    for name in order:
        src, cls_name = STRUCTS[name]
        body = struct_body(os.path.join(CSRC, src), name)
        if body is None:
            problems.append(f"{name}: not found in {src}")
            continue
        fields = parse_fields(body, known)
        lay, size, align = layout(fields)
        known[name] = (size, align)
        cls = getattr(K, cls_name)
        py = [(n, getattr(cls, n).offset, getattr(cls, n).size) for n, _ in cls._fields_]
        if [x[0] for x in lay] != [x[0] for x in py]:
            problems.append(f"{name}: field names differ: C {[x[0] for x in lay]} vs ctypes {[x[0] for x in py]}")
        elif lay != py:
            bad = [(c, p) for c, p in zip(lay, py) if c != p]
            problems.append(f"{name}: layout differs (name, offset, size): first mismatch C {bad[0][0]} vs ctypes {bad[0][1]}")
        if size != C.sizeof(cls):
            problems.append(f"{name}: size {size} in C vs {C.sizeof(cls)} in ctypes")
        report.append(f"{name:16s} {len(fields):3d} fields {size:5d} bytes ({src})")
        for other in DUPLICATES.get(name, [])[1:]:
            b2 = struct_body(os.path.join(CSRC, other), name)
            if b2 is None or " ".join(b2.split()) != " ".join(body.split()):
                problems.append(f"{name}: declaration in {other} differs from the one in {src}")
    check_all.report = report
    return problems


def main() -> int:
    if len(sys.argv) >= 3 and sys.argv[1] == "--emit":
        with open(sys.argv[2], "w") as f:
            f.write(emit_module())
        return 0
    problems = check_all()
    print("\n".join(check_all.report))
    for p in problems:
        print("MISMATCH " + p)
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
