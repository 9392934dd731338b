"""The Rust binding under integration/ cannot be compiled where these tests run; what can be checked is that it
declares what the header declares: every `extern "C"` function of src/ffi.rs exists in include/sapient_cuda.h with the
same number of arguments and argument kinds, the status and dtype constants agree, and SpModelDesc has the header's
fields in the header's order (its size is pinned separately by the ABI test)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "sapient_cuda.h")
FFI = os.path.join(ROOT, "integration", "crates", "sapient-backends", "cuda", "src", "ffi.rs")


def _strip_c_comments(s):
    return re.sub(r"/\*.*?\*/", " ", s, flags=re.S)


C2R = {"int32_t": "i32", "int64_t": "i64", "uint32_t": "u32", "uint64_t": "u64", "size_t": "usize", "float": "f32", "double": "f64",
       "char": "c_char", "void": "c_void", "SpEngine": "SpEngine", "SpWeight": "SpWeight", "SpBatcher": "SpBatcher", "SpModelDesc": "SpModelDesc"}


def _header_functions():
    src = _strip_c_comments(open(HEADER).read())
    out = {}
    for m in re.finditer(r"\b(int32_t|void|const char\s*\*)\s+(sp_cuda_\w+)\s*\(([^)]*)\)\s*;", src):
        args = [a for a in (x.strip() for x in m.group(3).split(",")) if a and a != "void"]
        kinds = []
        for a in args:
            # drop the parameter name (last identifier) unless the declaration is a bare type
            mm = re.match(r"^(.*?)([A-Za-z_]\w*)$", a)
            ty = mm.group(1) if mm and mm.group(1).strip() else a
            ptr = ty.count("*")
            base = [w for w in ty.replace("*", " ").split() if w != "const"][0]
            kinds.append((C2R[base], ptr))
        out[m.group(2)] = kinds
    return out


def _rust_functions():
    src = re.sub(r"//.*", "", open(FFI).read())
    block = src[src.index('extern "C"'):]
    out = {}
    for m in re.finditer(r"pub fn (sp_cuda_\w+)\s*\((.*?)\)\s*(?:->\s*[^;]+)?;", block, flags=re.S):
        kinds = []
        for a in (x.strip() for x in m.group(2).split(",")):
            if not a:
                continue
            ty = a.split(":", 1)[1].strip()
            ptr = len(re.findall(r"\*(?:mut|const)", ty))
            base = re.sub(r"\*(?:mut|const)\s*", "", ty).strip()
            kinds.append((base, ptr))
        out[m.group(1)] = kinds
    return out


def test_every_bound_function_matches_the_header():
    hdr, rs = _header_functions(), _rust_functions()
    assert len(rs) >= 25
    for name, kinds in rs.items():
        assert name in hdr, f"{name} is bound but not declared by the header"
        assert kinds == hdr[name], (name, kinds, hdr[name])


def test_the_engine_surface_is_bound():
    rs = _rust_functions()
    for need in ["sp_cuda_engine_create", "sp_cuda_engine_set_tensor", "sp_cuda_engine_finalize", "sp_cuda_engine_destroy",
                 "sp_cuda_forward_logits", "sp_cuda_forward_all_logits", "sp_cuda_forward_all_logits_cached", "sp_cuda_reset_cache",
                 "sp_cuda_truncate_cache", "sp_cuda_decode_greedy", "sp_cuda_spec_greedy", "sp_cuda_engine_tp_handle",
                 "sp_cuda_engine_tp_connect", "sp_cuda_engine_from_gguf"]:
        assert need in rs, need


def test_constants_and_struct_fields_agree():
    hsrc = _strip_c_comments(open(HEADER).read())
    rsrc = open(FFI).read()
    for name, val in re.findall(r"\b(SP_(?:OK|ERR_\w+|F32|F16|BF16|Q\w+))\s*=\s*(\d+)", hsrc):
        m = re.search(rf"pub const {name}: i32 = (\d+);", rsrc)
        assert m and m.group(1) == val, name
    body = re.search(r"typedef struct SpModelDesc \{(.*?)\} SpModelDesc;", hsrc, flags=re.S).group(1)
    c_fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        ty, names = decl.split(None, 1)
        c_fields += [(n.strip(), C2R[ty]) for n in names.split(",")]
    rbody = re.search(r"pub struct SpModelDesc \{(.*?)\}", rsrc, flags=re.S).group(1)
    r_fields = re.findall(r"pub (\w+): (\w+),", rbody)
    assert r_fields == c_fields
