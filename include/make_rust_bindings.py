"""Writes include/train_station_b200.rs from include/train_station_b200.h: the complete `extern "C"` block (every function
the header declares, with its argument names), the two opaque handle types, the statistics struct and the enum constants,
as the Rust side of the reference would import them (the reference binds its fifteen device symbols this way in
src/cuda/mod.rs:139-208).  No Rust toolchain is needed to run it; tests/test_abi.py checks that the committed file is what
this script produces and that it names every exported symbol.

    python include/make_rust_bindings.py            # rewrite the .rs file
    python include/make_rust_bindings.py --check    # exit 1 if the committed file is stale
"""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(HERE, "train_station_b200.h")
OUTPUT = os.path.join(HERE, "train_station_b200.rs")

SCALARS = {"bool": "bool", "int": "i32", "long long": "i64", "unsigned long long": "u64", "float": "f32", "double": "f64",
           "char": "c_char", "unsigned char": "u8", "void": "c_void"}
STRUCTS = {"ts_tensor": "TsTensor", "ts_adam": "TsAdam", "ts_allocator_stats": "TsAllocatorStats"}
RUST_KEYWORDS = {"ref", "type", "in", "match", "move", "fn", "mod", "loop", "impl", "use", "self", "box", "where", "as", "dyn"}


def strip_comments(text):
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.sub(r"//[^\n]*", "", text)


def rust_type(c_type):
    """`const float* const*` -> `*const *const f32`; array parameters decay to pointers."""
    c_type = " ".join(c_type.split())
    stars = c_type.count("*")
    tokens = [tok for tok in c_type.replace("*", " * ").split()]
    # split into the base type and the pointer levels with their constness, left to right
    base, levels, pending_const = [], [], False
    for tok in tokens:
        if tok == "const":
            pending_const = True
        elif tok == "*":
            levels.append(pending_const)      # constness of what THIS pointer points to, as gathered so far
            pending_const = False
        else:
            base.append(tok)
    name = " ".join(base)
    inner = STRUCTS.get(name) or SCALARS.get(name)
    if inner is None:
        raise ValueError(f"no Rust spelling for C type {c_type!r}")
    if stars == 0:
        return "()" if name == "void" else inner
    out = inner
    for is_const in levels:
        out = ("*const " if is_const else "*mut ") + out
    return out


def parse(header_text):
    text = strip_comments(header_text)
    consts = [(m.group(1), m.group(2)) for m in re.finditer(r"#define\s+(TS_[A-Z0-9_]+)\s+(-?\d+)\b", text)]
    enums = []
    for body in re.findall(r"enum\s+[a-z_0-9]+\s*\{(.*?)\}", text, flags=re.S):
        enums += [(m.group(1), m.group(2)) for m in re.finditer(r"(TS_[A-Z0-9_]+)\s*=\s*(-?\d+)", body)]
    structs = []
    for m in re.finditer(r"typedef\s+struct\s+([a-z_0-9]+)\s*\{(.*?)\}\s*\1\s*;", text, flags=re.S):
        fields = [(f.group(2), rust_type(f.group(1))) for f in re.finditer(r"([A-Za-z_][A-Za-z0-9_ \*]*?)\s+([a-z_0-9]+)\s*;", m.group(2))]
        structs.append((m.group(1), fields))
    text_no_structs = re.sub(r"typedef\s+struct\s+[a-z_0-9]+\s*\{.*?\}\s*[a-z_0-9]+\s*;", "", text, flags=re.S)
    functions = []
    for m in re.finditer(r"\n([A-Za-z_][A-Za-z0-9_ \*]*?)\b([a-z_][a-z_0-9]*)\s*\(([^;{}()]*)\)\s*;", text_no_structs):
        ret, name, args = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
        if ret.startswith("typedef") or not ret:
            continue
        params = []
        if args and args != "void":
            for index, arg in enumerate(a.strip() for a in args.split(",")):
                array = re.match(r"(.*?)\b([a-z_][a-z_0-9]*)\s*\[[^\]]*\]$", arg)
                if array:                                     # `unsigned char id_out[N]` is a pointer parameter
                    c_type, pname = array.group(1).strip() + "*", array.group(2)
                else:
                    named = re.match(r"(.*?[\s\*])([a-z_][a-z_0-9]*)$", arg)
                    c_type, pname = (named.group(1).strip(), named.group(2)) if named else (arg, f"arg{index}")
                if pname in RUST_KEYWORDS:
                    pname += "_"
                params.append((pname, rust_type(c_type)))
        functions.append((name, params, rust_type(ret)))
    return consts, enums, structs, functions


def render(consts, enums, structs, functions):
    out = ["// Generated from train_station_b200.h by make_rust_bindings.py: do not edit by hand.",
           "// The C ABI of libtrain_station_b200.so as a Rust `extern \"C\"` block.  Sizes are element counts, not bytes;",
           "// a null `stream` is the library's compute stream; `bool` results are success flags and ts_last_error() holds",
           "// the message of the last failure on the calling thread; handles are owned by the caller and released with",
           "// ts_tensor_free / ts_adam_free.",
           "#![allow(non_camel_case_types, dead_code)]",
           "use std::os::raw::{c_char, c_void};", ""]
    for name in ("TsTensor", "TsAdam"):
        out += ["#[repr(C)]", f"pub struct {name} {{ _private: [u8; 0] }}", ""]
    for cname, fields in structs:
        out += ["#[repr(C)]", "#[derive(Clone, Copy, Debug, Default)]", f"pub struct {STRUCTS[cname]} {{"]
        out += [f"    pub {fname}: {ftype}," for fname, ftype in fields]
        out += ["}", ""]
    for name, value in consts + enums:
        kind = "usize" if name.endswith("_BYTES") else "i32"
        out.append(f"pub const {name}: {kind} = {value};")
    out += ["", '#[link(name = "train_station_b200")]', 'extern "C" {']
    for name, params, ret in functions:
        args = ", ".join(f"{p}: {t}" for p, t in params)
        out.append(f"    pub fn {name}({args})" + ("" if ret == "()" else f" -> {ret}") + ";")
    out += ["}", ""]
    return "\n".join(out)


def generate():
    with open(HEADER) as f:
        return render(*parse(f.read()))


def main():
    text = generate()
    if "--check" in sys.argv[1:]:
        with open(OUTPUT) as f:
            sys.exit(0 if f.read() == text else 1)
    with open(OUTPUT, "w") as f:
        f.write(text)
    print(f"wrote {OUTPUT}")


if __name__ == "__main__":
    main()
