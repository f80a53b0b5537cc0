#!/usr/bin/env python
"""Writes include/mcb_sys.rs, the Rust `extern "C"` mirror of include/mcb.h, from the header itself:

    python include/gen_rust_binding.py            # rewrite include/mcb_sys.rs
    python include/gen_rust_binding.py --check    # exit 1 if the committed file is not what the header gives

One declaration per C function, argument for argument, plus the status / dtype / enum constants.  The file is
what a maintainer drops into crates/modern-chainer-cuda/src/ (rustc is not needed to produce it, and none is
present where this library is built); tests/test_cabi_load.py runs the --check form, so the mirror cannot
drift from the header.  The hand-written forwarding of the `Ops<CudaBackend>` trait onto these functions is
include/mcb_ops.rs."""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "mcb.h")
OUT = os.path.join(HERE, "mcb_sys.rs")

OPAQUE = {"mcb_ctx": "McbCtx", "mcb_var": "McbVar", "mcb_adam": "McbAdam", "mcb_scaler": "McbScaler", "mcb_arena": "McbArena",
          "mcb_model": "McbModel", "mcb_static_step": "McbStaticStep", "mcb_dp_sim": "McbDpSim"}
SCALAR = {"int32_t": "i32", "int64_t": "i64", "uint32_t": "u32", "uint64_t": "u64", "double": "f64", "float": "f32", "size_t": "usize",
          "mcb_status": "Status", "char": "c_char", "void": "c_void"}


def strip_comments(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def rust_type(ctype):
    """'const float *' -> '*const f32', 'mcb_var **' -> '*mut *mut McbVar', 'const char *const *' -> '*const *const c_char'."""
    t = ctype.strip()
    stars = t.count("*")
    parts = [p.strip() for p in t.split("*")]
    base_tokens = parts[0].split()
    base_const = "const" in base_tokens
    base = [b for b in base_tokens if b != "const"][0]
    rs = OPAQUE.get(base) or SCALAR[base]
    # pointer levels, innermost first; a level is const when the pointee is const-qualified
    const_flags = [base_const] + ["const" in p.split() for p in parts[1:-1]]
    for lvl in range(stars):
        rs = ("*const " if const_flags[lvl] else "*mut ") + rs
    return rs


def parse(path=HEADER):
    text = strip_comments(open(path).read())
    funcs = []
    for m in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(mcb_\w+)\s*\(([^;{}]*?)\)\s*;", text):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        if ret.startswith("typedef"):
            continue
        params = []
        if args and args != "void":
            for a in args.split(","):
                a = " ".join(a.split())
                mm = re.match(r"(.*?)(\w+)$", a)
                ctype, pname = mm.group(1).strip(), mm.group(2)
                if pname in ("type", "ref", "fn", "in", "box", "move", "match", "loop", "impl", "use", "mod", "self"):
                    pname += "_"
                params.append((pname, rust_type(ctype)))
        rret = None if ret == "void" else rust_type(ret)
        funcs.append((name, params, rret))
    enums = []
    for m in re.finditer(r"enum\s*\{([^}]*)\}\s*;", text):
        value = -1
        for item in m.group(1).split(","):
            item = item.strip()
            if not item:
                continue
            if "=" in item:
                nm, v = [x.strip() for x in item.split("=")]
                value = int(v, 0)
            else:
                nm, value = item, value + 1
            enums.append((nm, value))
    return funcs, enums


def render():
    funcs, enums = parse()
    out = ["// GENERATED from include/mcb.h by include/gen_rust_binding.py -- do not edit by hand.",
           "// Raw FFI of libmcb.so: one declaration per function of the C ABI, argument for argument.",
           "// Place in crates/modern-chainer-cuda/src/ and link with `cargo:rustc-link-lib=dylib=mcb`.",
           "#![allow(non_camel_case_types, dead_code)]",
           "use core::ffi::{c_char, c_void};",
           "",
           "pub type Status = i32;"]
    for rs in sorted(set(OPAQUE.values())):
        out += ["#[repr(C)]", f"pub struct {rs} {{", "    _private: [u8; 0],", "}"]
    out.append("")
    for nm, v in enums:
        out.append(f"pub const {nm}: i32 = {v};")
    out += ["", '#[link(name = "mcb")]', 'unsafe extern "C" {']
    for name, params, ret in funcs:
        ps = ", ".join(f"{p}: {t}" for p, t in params)
        out.append(f"    pub fn {name}({ps})" + (f" -> {ret};" if ret else ";"))
    out += ["}", ""]
    return "\n".join(out)


def main():
    text = render()
    if "--check" in sys.argv:
        if not os.path.exists(OUT) or open(OUT).read() != text:
            sys.stderr.write("include/mcb_sys.rs is out of date: run python include/gen_rust_binding.py\n")
            sys.exit(1)
        return
    open(OUT, "w").write(text)


if __name__ == "__main__":
    main()
