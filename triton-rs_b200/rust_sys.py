"""Generate the Rust `-sys` binding of libb200_kernels.so from include/b200_kernels.h.

The reference's consumer is Rust (cudarc buffers, `extern "C"` through a `-sys` crate, as
`crates/triton-sys` does for the MLIR C API).  This script writes
`rust/b200-kernels-sys/src/lib.rs` with one declaration per prototype of the header, the
`b200k_layer_config` struct with `#[repr(C)]`, the opaque handle types and the `B200K_*`
constants, so that the Rust side cannot drift from the header either:
`python triton-rs_b200/rust_sys.py` rewrites the file, `--check` exits 1 if it is stale.
"""
from __future__ import annotations

import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
HEADER = HERE.parent / "include" / "b200_kernels.h"
OUT = HERE / "rust" / "b200-kernels-sys" / "src" / "lib.rs"

_BASE = {
    "int": "c_int", "float": "f32", "size_t": "usize", "void": "c_void", "char": "c_char",
    "int8_t": "i8", "int32_t": "i32", "uint32_t": "u32", "int64_t": "i64", "uint64_t": "u64",
    "b200k_half": "b200k_half", "b200k_bf16": "b200k_bf16", "b200k_layer": "b200k_layer",
    "b200k_layer_config": "b200k_layer_config", "struct b200k_comm": "b200k_comm",
}
_KEYWORDS = {"type", "in", "ref", "mod", "fn", "loop", "match", "move", "box", "self", "where"}


def rust_type(ctype: str) -> str:
    """`const b200k_half *` -> `*const b200k_half`, `void **` -> `*mut *mut c_void`, `int` -> `c_int`."""
    ctype = " ".join(ctype.split())
    if ctype == "b200k_stream":
        return "b200k_stream"
    stars = ctype.count("*")
    base = ctype.replace("*", " ")
    const = bool(re.match(r"^const\b", base.strip()))
    base = " ".join(w for w in base.split() if w != "const")
    if base not in _BASE:
        raise ValueError(f"no Rust spelling for C type {ctype!r}")
    out = _BASE[base]
    for i in range(stars):
        out = ("*const " if (const and i == 0) else "*mut ") + out
    return out


def strip(text: str) -> str:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return re.sub(r"//[^\n]*", " ", text)


def prototypes(text: str):
    """-> [(name, rust return type or None, [(arg name, rust type)])] in header order."""
    text = re.sub(r"^\s*#.*$", " ", strip(text), flags=re.M)
    pat = re.compile(r"\b(const\s+char\s*\*\s*|int\s+|size_t\s+|void\s+)(\w+)\s*\(([^;{}]*?)\)\s*;", re.S)
    out = []
    for m in pat.finditer(text):
        ret, name, args = " ".join(m.group(1).split()), m.group(2), " ".join(m.group(3).split())
        rret = None if ret == "void" else ("*const c_char" if "char" in ret else rust_type(ret))
        parsed = []
        if args and args != "void":
            for a in args.split(","):
                am = re.match(r"^(.*?)(\w+)$", a.strip())
                an = am.group(2)
                parsed.append((an + "_" if an in _KEYWORDS else an, rust_type(am.group(1))))
        out.append((name, rret, parsed))
    return out


def constants(text: str):
    """The anonymous enum's status codes and the `#define B200K_X <integer expression>` lines
    -> [(name, rust expression, type)]."""
    out = []
    for em in re.finditer(r"\benum\s*\{(.*?)\}\s*;", strip(text), flags=re.S):
        for item in em.group(1).split(","):
            im = re.match(r"^\s*(B200K_\w+)\s*=\s*(-?\d+)\s*$", item)
            if im:
                out.append((im.group(1), im.group(2), "c_int"))
    for m in re.finditer(r"^\s*#define\s+(B200K_\w+)\s+(.+?)\s*$", strip(text), flags=re.M):
        name, val = m.group(1), m.group(2).strip()
        val = re.sub(r"\(\s*size_t\s*\)", "", val)
        val = re.sub(r"(\d)[uU]?[lL]{0,2}\b", r"\1", val)
        if not re.fullmatch(r"[-\d\s()<*+xXa-fA-F]+", val):
            continue
        big = "<<" in val or len(re.sub(r"\D", "", val)) > 9
        out.append((name, val, "usize" if big else "c_int"))
    return out


def config_struct(text: str):
    m = re.search(r"typedef\s+struct\s+b200k_layer_config\s*\{(.*?)\}\s*b200k_layer_config\s*;", strip(text), flags=re.S)
    fields = []
    for decl in m.group(1).split(";"):
        decl = " ".join(decl.split())
        if not decl:
            continue
        fm = re.match(r"^(\w+)\s+(\w+)(?:\[(\d+)\])?$", decl)
        ty = _BASE[fm.group(1)]
        fields.append((fm.group(2), f"[{ty}; {fm.group(3)}]" if fm.group(3) else ty))
    return fields


def generate(header: Path = HEADER) -> str:
    text = header.read_text()
    lines = [
        "// Generated from include/b200_kernels.h by triton-rs_b200/rust_sys.py; do not edit by hand.",
        "// One declaration per prototype of the header.  Device pointers are raw pointers into CUDA",
        "// memory (a cudarc `CudaSlice<T>`'s `device_ptr` cast to the pointer type); `b200k_stream` is",
        "// the `CUstream` of a cudarc `CudaStream`.",
        "#![allow(non_camel_case_types, non_upper_case_globals, clippy::too_many_arguments)]",
        "",
        "use std::os::raw::{c_char, c_int, c_void};",
        "",
        "/// IEEE binary16 bits (`half::f16::to_bits`).",
        "pub type b200k_half = u16;",
        "/// bfloat16 bits (`half::bf16::to_bits`).",
        "pub type b200k_bf16 = u16;",
        "/// `cudaStream_t` / `CUstream`; null is the legacy default stream.",
        "pub type b200k_stream = *mut c_void;",
        "",
        "#[repr(C)]",
        "pub struct b200k_layer {",
        "    _opaque: [u8; 0],",
        "}",
        "#[repr(C)]",
        "pub struct b200k_comm {",
        "    _opaque: [u8; 0],",
        "}",
        "",
        "#[repr(C)]",
        "#[derive(Clone, Copy, Debug, Default)]",
        "pub struct b200k_layer_config {",
    ]
    lines += [f"    pub {n}: {t}," for n, t in config_struct(text)]
    lines += ["}", ""]
    for name, val, ty in constants(text):
        lines.append(f"pub const {name}: {ty} = {val};")
    lines += ["", '#[link(name = "b200_kernels")]', 'extern "C" {']
    for name, ret, args in prototypes(text):
        head = f"    pub fn {name}("
        body = ", ".join(f"{n}: {t}" for n, t in args)
        tail = ")" + (f" -> {ret}" if ret else "") + ";"
        one = head + body + tail
        if len(one) <= 110:
            lines.append(one)
        else:
            lines.append(head)
            cur = "       "
            for i, (n, t) in enumerate(args):
                piece = f" {n}: {t}" + ("," if i + 1 < len(args) else "")
                if len(cur) + len(piece) > 110:
                    lines.append(cur)
                    cur = "       "
                cur += piece
            lines.append(cur)
            lines.append("    " + tail)
    lines += ["}", ""]
    return "\n".join(lines)


def main(argv):
    text = generate()
    if "--check" in argv:
        if not OUT.exists() or OUT.read_text() != text:
            print(f"{OUT} is stale: run python {Path(__file__).name}")
            return 1
        return 0
    OUT.parent.mkdir(parents=True, exist_ok=True)
    OUT.write_text(text)
    cargo = OUT.parent.parent / "Cargo.toml"
    cargo.write_text('[package]\nname = "b200-kernels-sys"\nversion = "0.1.0"\nedition = "2021"\nlinks = "b200_kernels"\n'
                     'build = "build.rs"\ndescription = "extern \\"C\\" declarations of libb200_kernels.so (sm_100a kernels behind the triton-kernels names)"\n\n[dependencies]\n')
    (OUT.parent.parent / "build.rs").write_text(
        '// Link against libb200_kernels.so; B200_KERNELS_LIB_DIR names the directory that holds it.\n'
        'fn main() {\n'
        '    if let Ok(dir) = std::env::var("B200_KERNELS_LIB_DIR") {\n'
        '        println!("cargo:rustc-link-search=native={dir}");\n'
        '        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");\n'
        '    }\n'
        '    println!("cargo:rerun-if-env-changed=B200_KERNELS_LIB_DIR");\n'
        '}\n')
    print(f"wrote {OUT} ({len(prototypes(HEADER.read_text()))} functions)")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
