"""The Rust FFI crate (krea2-b200-sys, uncompiled here: no Rust toolchain) against the C header: every function
include/krea2_b200.h declares must appear in the crate's `extern "C"` block under the same name, with the same
number of parameters and the Rust spelling of each C type, and nothing else may be declared there."""
import os

import ffi_parse

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def read(*parts):
    with open(os.path.join(ROOT, *parts)) as f:
        return f.read()


def test_extern_block_matches_the_header_name_by_name():
    header = ffi_parse.c_functions(read("include", "krea2_b200.h"))
    crate = ffi_parse.rust_functions(read("krea2-b200-sys", "src", "lib.rs"))
    assert len(header) > 70
    assert [name for name, _, _ in crate] == [name for name, _, _ in header], "same functions, in the header's order"
    for (name, c_ret, c_params), (_, r_ret, r_params) in zip(header, crate):
        assert (ffi_parse.rust_type(c_ret) if c_ret != "void" else "void") == r_ret, name
        assert [pname for _, pname in c_params] == [pname for _, pname in r_params], name
        assert [ffi_parse.rust_type(ptype) for ptype, _ in c_params] == [ptype for ptype, _ in r_params], name


def test_every_struct_of_the_header_has_a_repr_c_twin():
    import re
    header = ffi_parse.strip_comments(read("include", "krea2_b200.h"))
    crate = read("krea2-b200-sys", "src", "lib.rs")
    structs = re.findall(r"typedef\s+struct\s+(\w+)\s*\{(.*?)\}\s*\w+\s*;", header, flags=re.S)
    assert {name for name, _ in structs} == {"krea2_config_entry", "krea2_binding", "krea2_shard", "krea2_row_shard",
                                             "krea2_dims", "krea2_span_info"}
    for name, body in structs:
        fields = []
        for declaration in filter(None, (d.strip() for d in body.split(";"))):
            names = re.sub(r"\[[^\]]*\]", "", declaration.split(None, 1)[1] if " " in declaration else declaration)
            fields += [n.strip(" *") for n in names.replace("const", "").split(",")]
        fields = [f.split()[-1].lstrip("*") for f in fields]
        twin = re.search(r"#\[repr\(C\)\][^{]*pub struct " + name + r"\s*\{(.*?)\n\}", crate, flags=re.S)
        assert twin, name
        rust_fields = re.findall(r"pub (\w+):", twin.group(1))
        assert rust_fields == fields, (name, rust_fields, fields)
    for opaque in ("krea2_weights", "krea2_session", "krea2_checkpoint"):
        assert f"pub struct {opaque}" in crate


def test_build_script_compiles_every_source_of_the_library():
    from krea2_hrx_b200 import build
    script = read("krea2-b200-sys", "build.rs")
    for source in build.SOURCES:
        assert f'"{source}"' in script, source
    assert "arch=compute_100a,code=sm_100a" in script
