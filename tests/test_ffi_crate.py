"""The Rust `-sys` crate under ffi/ cannot be compiled where this repository is built (no Rust
toolchain), so it is checked as text: its `extern "C"` block must declare exactly the functions of
include/bonsai_attn.h with the same number of arguments and the same kind of return value, its status
constants must equal the header's enum, and its two `repr(C)` structs must list the header's fields in
order."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "bonsai_attn.h")
LIB_RS = os.path.join(ROOT, "ffi", "bonsai-attn-sys", "src", "lib.rs")


def header_text(path=HEADER):
    return re.sub(r"/\*.*?\*/", "", open(path).read(), flags=re.S)


def header_functions(path=HEADER):
    out = {}
    for m in re.finditer(r"([a-zA-Z_][\w \*]*?)\b(bp_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", header_text(path)):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3)
        out[name] = (len([a for a in args.split(",") if a.strip() and a.strip() != "void"]), ret == "void")
    return out


MODEL_HEADER = os.path.join(ROOT, "include", "bonsai_model.h")
MODEL_RS = os.path.join(ROOT, "ffi", "bonsai-attn-sys", "src", "model.rs")


def rust_functions(path=LIB_RS):
    text = re.sub(r"//.*", "", open(path).read())
    block = re.search(r'extern "C" \{(.*?)\n\}', text, flags=re.S).group(1)
    out = {}
    for m in re.finditer(r"pub fn (bp_[a-z0-9_]+)\s*\((.*?)\)\s*(->\s*[^;]+)?;", block, flags=re.S):
        args = [a for a in m.group(2).split(",") if a.strip()]
        out[m.group(1)] = (len(args), m.group(3) is None)
    return out


def test_extern_block_matches_the_header():
    h, r = header_functions(), rust_functions()
    assert len(h) >= 35
    assert sorted(h) == sorted(r)
    for name in h:
        assert h[name] == r[name], (name, h[name], r[name])


def test_status_constants_match_the_header_enum():
    enum = dict((k, int(v)) for k, v in re.findall(r"\b(BP_[A-Z_]+)\s*=\s*(\d+)", header_text()))
    rust = dict((k, int(v)) for k, v in re.findall(r"pub const (BP_[A-Z_]+): c_int = (\d+);", open(LIB_RS).read()))
    assert enum == rust and len(enum) == 9
    # a timed-out device-side wait is sticky like a lost device: check() must not map it to Config
    check = re.search(r"pub unsafe fn check\(.*?\n\}", open(LIB_RS).read(), flags=re.S).group(0)
    arm = re.search(r"([A-Z_| ]+)=> AttnError::DeviceLost", check).group(1)
    assert "BP_ERR_TIMEOUT" in arm and "BP_ERR_DEVICE_LOST" in arm


def c_struct_fields(name):
    body = re.search(r"typedef struct %s \{(.*?)\}" % name, header_text(), flags=re.S).group(1)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        ctype, names = decl.split(None, 1)
        fields += [(n.strip(), ctype) for n in names.split(",")]
    return fields


def rust_struct_fields(name):
    body = re.search(r"pub struct %s \{(.*?)\n\}" % name, re.sub(r"//.*", "", open(LIB_RS).read()), flags=re.S).group(1)
    return [(n, t.strip()) for n, t in re.findall(r"pub (\w+):\s*([^,\n]+)", body)]


def test_repr_c_structs_match_the_header():
    ctype = {"u32": "uint32_t", "i32": "int32_t", "f32": "float"}
    for name in ("bp_attn_config", "bp_error_detail"):
        c, r = c_struct_fields(name), rust_struct_fields(name)
        assert [n for n, _ in c] == [n for n, _ in r], name
        assert [t for _, t in c] == [ctype[t] for _, t in r], name


def test_model_module_matches_the_model_header():
    """src/model.rs declares exactly the functions of include/bonsai_model.h, with the same number of
    arguments and the same kind of return value, and its two repr(C) structs list the header's fields."""
    h, r = header_functions(MODEL_HEADER), rust_functions(MODEL_RS)
    assert len(h) >= 40
    assert sorted(h) == sorted(r)
    for name in h:
        assert h[name] == r[name], (name, h[name], r[name])
    text = re.sub(r"//.*", "", open(MODEL_RS).read())
    cfg = re.search(r"pub struct bp_model_config \{(.*?)\n\}", text, flags=re.S).group(1)
    fields = [n for n, _ in re.findall(r"pub (\w+):\s*([^,\n]+)", cfg)]
    body = re.search(r"typedef struct bp_model_config \{(.*?)\}", header_text(MODEL_HEADER), flags=re.S).group(1)
    want = []
    for decl in body.split(";"):
        decl = decl.strip()
        if decl:
            want += [n.strip() for n in decl.split(None, 1)[1].split(",")]
    assert fields == want
    smp = re.search(r"pub struct bp_sampler \{(.*?)\n\}", text, flags=re.S).group(1)
    assert [n for n, _ in re.findall(r"pub (\w+):\s*([^,\n]+)", smp)] == ["temperature", "top_k", "top_p", "seed"]
    assert "pub mod model;" in open(LIB_RS).read()
