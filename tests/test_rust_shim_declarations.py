"""The Rust shim (bindings/rust) cannot be compiled where no Rust toolchain exists, but it can
at least not drift: every function its ``extern "C"`` block declares must exist in
``include/volta_b200.h`` with the same number of arguments, the same kind of each argument
(pointer or not) and matching scalar types, and the constants it repeats must have the header's
values."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "volta_b200.h")
SHIM = os.path.join(ROOT, "bindings", "rust", "src", "lib.rs")

C_TO_RUST = {"int": "c_int", "int64_t": "i64", "int32_t": "i32", "uint32_t": "u32", "uint64_t": "u64",
             "uint16_t": "u16", "float": "f32", "double": "f64", "size_t": "usize"}


def header_prototypes():
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    out = {}
    for ret, name, args in re.findall(r"\b(int|const char \*)\s*(vb_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text):
        args = " ".join(args.split())
        out[name] = [] if args in ("", "void") else [a.strip() for a in args.split(",")]
    return out


def rust_declarations():
    text = open(SHIM).read()
    block = text[text.index('unsafe extern "C" {'):]
    block = block[:block.index("\n    }\n")]
    block = re.sub(r"//[^\n]*", "", block)
    out = {}
    for name, args in re.findall(r"pub fn (vb_[a-z0-9_]+)\s*\(([^)]*)\)", block, flags=re.S):
        parts = [a.strip() for a in " ".join(args.split()).split(",") if a.strip()]
        out[name] = [p.split(":", 1)[1].strip() for p in parts]
    return out


def test_every_rust_declaration_matches_the_header():
    c = header_prototypes()
    r = rust_declarations()
    assert len(r) >= 30
    for name, rust_args in r.items():
        assert name in c, f"{name} is declared in the Rust shim but not in include/volta_b200.h"
        c_args = c[name]
        assert len(c_args) == len(rust_args), (name, c_args, rust_args)
        for ca, ra in zip(c_args, rust_args):
            c_is_ptr = "*" in ca
            assert c_is_ptr == ra.startswith("*"), (name, ca, ra)
            if not c_is_ptr:
                ctype = ca.replace("const ", "").rsplit(" ", 1)[0].strip()
                assert C_TO_RUST[ctype] == ra, (name, ca, ra)
            else:
                # constness of the pointee, and pointer-to-pointer depth
                assert ca.count("*") == ra.count("*"), (name, ca, ra)


def test_rust_constants_match_the_header():
    htext = open(HEADER).read()
    rtext = open(SHIM).read()
    defines = {k: int(v.rstrip("u"), 0) for k, v in re.findall(r"#define\s+(VB_[A-Z0-9_]+)\s+(\d+u?)\b", htext)}
    enums = {k: int(v) for k, v in re.findall(r"\b(VB_[A-Z0-9_]+)\s*=\s*(\d+)", htext)}
    rust = {k: int(v) for k, v in re.findall(r"pub const (VB_[A-Z0-9_]+):\s*\w+\s*=\s*(\d+);", rtext)}
    assert len(rust) >= 8
    for name, value in rust.items():
        want = defines.get(name, enums.get(name))
        assert want is not None, name
        assert want == value, (name, want, value)
