"""The Rust binding (bindings/rust/gemm.rs) must declare exactly what include/patina_gemm.h
declares: every exported function with the same number of arguments, every struct with the
same fields in the same order, the same error codes. The image has no Rust toolchain, so this
textual check is what keeps the two in step. Host-only."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def c_header():
    text = open(os.path.join(ROOT, "include", "patina_gemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    funcs = {}
    for _, name, args in re.findall(r"\n\s*((?:const\s+)?[\w ]+?\*?)\s*\b(patina_gemm_\w+)\s*\(([^;{]*?)\)\s*;",
                                    text, flags=re.S):
        args = " ".join(args.split())
        funcs[name] = 0 if args == "void" else len(args.split(","))
    structs = {}
    for name, body in re.findall(r"typedef struct (\w+) \{(.*?)\} \w+;", text, flags=re.S):
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = re.sub(r"^.*?[\s\*](?=[\w]+(\s*,\s*\w+)*$)", "", decl)
            fields += [n.strip() for n in names.split(",")]
        structs[name] = fields
    codes = dict(re.findall(r"(PATINA_GEMM_(?:OK|ERR_\w+))\s*=\s*(\d+)", text))
    return funcs, structs, codes


def rust_binding():
    text = open(os.path.join(ROOT, "bindings", "rust", "gemm.rs")).read()
    block = re.search(r'extern "C" \{(.*?)\n\}', text, flags=re.S).group(1)
    funcs = {}
    for name, args in re.findall(r"pub fn (patina_gemm_\w+)\((.*?)\)", block, flags=re.S):
        args = " ".join(args.split())
        funcs[name] = 0 if not args else len([a for a in args.split(",") if a.strip()])
    structs = {}
    for name, body in re.findall(r"#\[repr\(C\)\]\s*(?:#\[derive\([^)]*\)\]\s*)?pub struct (\w+) \{(.*?)\n\}", text, flags=re.S):
        structs[name] = re.findall(r"pub (\w+):", body)
    codes = dict(re.findall(r"pub const (PATINA_GEMM_(?:OK|ERR_\w+)): i32 = (\d+);", text))
    return funcs, structs, codes


def test_rust_binding_matches_the_header(built_lib):
    from patina_b200 import lib as L
    c_funcs, c_structs, c_codes = c_header()
    r_funcs, r_structs, r_codes = rust_binding()
    assert set(c_funcs) == set(L.SYMBOLS), "the ctypes symbol list and the header disagree"
    assert set(r_funcs) == set(c_funcs), (sorted(set(c_funcs) - set(r_funcs)), sorted(set(r_funcs) - set(c_funcs)))
    for name, n in c_funcs.items():
        assert r_funcs[name] == n, f"{name}: {n} arguments in the header, {r_funcs[name]} in the binding"
        assert hasattr(built_lib, name)
    for name, fields in c_structs.items():
        assert r_structs.get(name) == fields, f"struct {name}: {fields} vs {r_structs.get(name)}"
    assert r_codes == c_codes and len(c_codes) == 5
