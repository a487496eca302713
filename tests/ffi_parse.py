"""A small reader of the C header's function declarations and of the Rust FFI crate's `extern "C"` block,
used to hold krea2-b200-sys/src/lib.rs to include/krea2_b200.h (names, arities, parameter types)."""
from __future__ import annotations

import re
from typing import List, Tuple

RUST_SCALARS = {"size_t": "usize", "int": "c_int", "float": "f32", "double": "f64", "uint32_t": "u32", "uint64_t": "u64",
                "uint16_t": "u16", "int32_t": "i32", "char": "c_char", "void": "c_void", "krea2_stream": "krea2_stream"}


def strip_comments(text: str) -> str:
    return re.sub(r"/\*.*?\*/", " ", text, flags=re.S)


def c_functions(header: str) -> List[Tuple[str, str, List[Tuple[str, str]]]]:
    """(name, return type, [(parameter type, parameter name)]) of every function the header declares."""
    text = strip_comments(header)
    text = re.sub(r"typedef\s+(struct|enum)\s+\w+\s*\{.*?\}\s*\w+\s*;", " ", text, flags=re.S)
    text = re.sub(r"\benum\s*\{.*?\}\s*;", " ", text, flags=re.S)
    out = []
    for match in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(krea2_\w+)\s*\(([^()]*)\)\s*;", text):
        ret, name, params = " ".join(match.group(1).split()), match.group(2), match.group(3).strip()
        if ret.startswith("typedef"):
            continue
        parsed = []
        if params and params != "void":
            for param in params.split(","):
                param = " ".join(param.split())
                m = re.fullmatch(r"(.*?)(\w+)", param)
                parsed.append((m.group(1).strip(), m.group(2)))
        out.append((name, ret, parsed))
    return out


def rust_type(c_type: str) -> str:
    """`const float *` -> `*const f32`, `krea2_weights **` -> `*mut *mut krea2_weights`, `size_t` -> `usize`."""
    tokens = c_type.replace("*", " * ").split()
    const = False
    base = None
    pointers = []  # constness of each pointer level, innermost first
    for token in tokens:
        if token == "const":
            const = True
        elif token == "*":
            pointers.append(const)
            const = False
        else:
            base = token
    result = RUST_SCALARS.get(base, base)
    for is_const in pointers:
        result = ("*const " if is_const else "*mut ") + result
    return result


def rust_functions(source: str) -> List[Tuple[str, str, List[Tuple[str, str]]]]:
    """(name, return type or "void", [(parameter type, parameter name)]) of every `pub fn` in the extern block."""
    block = re.search(r'extern\s+"C"\s*\{(.*?)\n\}', source, flags=re.S).group(1)
    block = re.sub(r"//[^\n]*", " ", block)
    out = []
    for match in re.finditer(r"pub\s+fn\s+(\w+)\s*\(([^()]*)\)\s*(->\s*([^;]+?))?\s*;", block, flags=re.S):
        name, params, ret = match.group(1), match.group(2).strip(), (match.group(4) or "void").strip()
        parsed = []
        for param in filter(None, (p.strip() for p in params.split(","))):
            pname, ptype = param.split(":", 1)
            parsed.append((" ".join(ptype.split()), pname.strip()))
        out.append((name, ret, parsed))
    return out
