"""The Rust half of the drop-in is source that no toolchain here compiles. What can be checked
without one: every function its `extern "C"` block declares exists in the C header with the same
number of parameters and matching pointer / integer / float kinds, the `#[repr(C)]` mirrors have the
header's fields in the header's order, and the library really exports each of those symbols."""
import os
import re

from velox_inferer_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RS = os.path.join(ROOT, "integration", "velox-variant", "src", "sm100.rs")
HDR = os.path.join(ROOT, "include", "velox_sm100.h")


def _strip_comments(text, line_prefix):
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    return "\n".join(l.split(line_prefix)[0] for l in text.splitlines())


def _rust_decls():
    src = _strip_comments(open(RS).read(), "//")
    block = src[src.index('extern "C"'):]
    block = block[: block.index("\n}")]
    out = {}
    for name, args, ret in re.findall(r"fn\s+(velox_sm100_\w+)\s*\((.*?)\)\s*->\s*(\w+)\s*;", block, flags=re.S):
        params = [a.strip() for a in args.split(",") if a.strip()]
        out[name] = ([p.split(":", 1)[1].strip() for p in params], ret)
    return out


def _c_decls():
    src = _strip_comments(open(HDR).read(), "//")
    out = {}
    for ret, name, args in re.findall(r"\b(int|long long)\s+(velox_sm100_\w+)\s*\((.*?)\)\s*;", src, flags=re.S):
        args = " ".join(args.split())
        params = [] if args in ("", "void") else [a.strip() for a in args.split(",")]
        out[name] = (params, ret)
    return out


def _kind_rust(t):
    if t.startswith("*"):
        return "ptr"
    return {"i32": "i32", "i64": "i64", "u32": "i32", "f32": "f32"}[t]


def _kind_c(p):
    if "*" in p:
        return "ptr"
    t = p.rsplit(" ", 1)[0].replace("const ", "").strip()
    return {"int": "i32", "int32_t": "i32", "unsigned int": "i32", "uint32_t": "i32", "long long": "i64", "int64_t": "i64",
            "float": "f32"}[t]


def test_extern_block_matches_the_header_and_the_library():
    rust, c = _rust_decls(), _c_decls()
    assert len(rust) >= 12, sorted(rust)
    lib = _lib.lib()
    for name, (rargs, rret) in rust.items():
        assert name in c, f"{name} is declared in sm100.rs but not in velox_sm100.h"
        cargs, cret = c[name]
        assert len(rargs) == len(cargs), (name, rargs, cargs)
        assert [_kind_rust(t) for t in rargs] == [_kind_c(p) for p in cargs], (name, rargs, cargs)
        assert (rret, cret) in (("i32", "int"), ("i64", "long long")), (name, rret, cret)
        assert hasattr(lib, name), f"libvelox_sm100.so does not export {name}"


def _struct_fields_c(name):
    src = _strip_comments(open(HDR).read(), "//")
    body = re.search(r"typedef struct " + name + r"\s*\{(.*?)\}\s*" + name + r"\s*;", src, flags=re.S).group(1)
    return [re.sub(r"\[.*\]", "", f.strip().rsplit(" ", 1)[1].lstrip("*")) for f in body.split(";") if f.strip()]


def _struct_fields_rust(name):
    src = _strip_comments(open(RS).read(), "//")
    m = re.search(r"#\[repr\(C\)\][^{]*struct\s+" + name + r"\s*\{(.*?)\}", src, flags=re.S)
    assert m, name
    return [f.split(":")[0].replace("pub", "").strip() for f in m.group(1).split(",") if f.strip()]


def test_repr_c_mirrors_follow_the_header_field_for_field():
    assert _struct_fields_rust("View") == _struct_fields_c("velox_sm100_view")
    assert _struct_fields_rust("Part") == _struct_fields_c("velox_sm100_part")
