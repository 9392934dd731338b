"""CPU-side checks of the C-ABI library: it loads, exports every declared symbol, and
fails loudly (never falls back) when there is no CUDA device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from sapient_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "sapient_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sp_cuda_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 35
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/sapient_cuda.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_desc_struct_layout_matches_header():
    # 17 int32/float fields then an int64: 4*17 = 68 -> padded to 72, + 8
    assert C.sizeof(_lib.SpModelDesc) == 80


def test_host_side_validation_needs_no_gpu():
    L = _lib.lib()
    h = C.c_void_p()
    buf = np.zeros(144, np.uint8)
    # k % 256 != 0 for a K-quant is rejected before any CUDA call (kernels/matmul.rs:863-865)
    st = L.sp_cuda_upload_weight(0, 12, 1, 128, buf.ctypes.data_as(C.c_void_p), 72, C.byref(h))
    assert st == _lib.SP_ERR_SHAPE and b"256" in L.sp_cuda_last_error()
    st = L.sp_cuda_upload_weight(0, 8, 1, 48, buf.ctypes.data_as(C.c_void_p), 51, C.byref(h))
    assert st == _lib.SP_ERR_SHAPE
    st = L.sp_cuda_upload_weight(0, 99, 1, 256, buf.ctypes.data_as(C.c_void_p), 144, C.byref(h))
    assert st == _lib.SP_ERR_DTYPE
    st = L.sp_cuda_upload_weight(0, 12, 1, 256, buf.ctypes.data_as(C.c_void_p), 100, C.byref(h))
    assert st == _lib.SP_ERR_SHAPE
    assert L.sp_cuda_forward_logits(None, None, 0, 1, None) == _lib.SP_ERR_ARG


def test_gguf_errors_before_any_device_work(tmp_path):
    L = _lib.lib()
    h = C.c_void_p()
    assert L.sp_cuda_engine_from_gguf(str(tmp_path / "nope.gguf").encode(), 0, 0, 1, C.byref(h)) == _lib.SP_ERR_IO
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"NOPE" + b"\0" * 64)
    assert L.sp_cuda_engine_from_gguf(str(bad).encode(), 0, 0, 1, C.byref(h)) == _lib.SP_ERR_IO
    assert b"magic" in L.sp_cuda_last_error()
    import gguf

    p = tmp_path / "arch.gguf"
    w = gguf.GGUFWriter(str(p), "gpt2")
    w.add_uint32("gpt2.block_count", 1)
    w.add_tensor("token_embd.weight", np.zeros((2, 32), np.float32))
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    assert L.sp_cuda_engine_from_gguf(str(p).encode(), 0, 0, 1, C.byref(h)) == _lib.SP_ERR_DTYPE
    assert b"gpt2" in L.sp_cuda_last_error()


def _raw_gguf(tensors, alignment=None, arch=b"llama", data=b""):
    """A GGUF v3 file written by hand, so that fields the writer package would refuse can be set.
    tensors: [(name, dims, ggml_type, offset)]; layout as crates/sapient-io/src/gguf.rs:517-578 reads it."""
    import struct

    def s(b):
        return struct.pack("<Q", len(b)) + b

    kv = [s(b"general.architecture") + struct.pack("<I", 8) + s(arch)]
    if alignment is not None:
        kv.append(s(b"general.alignment") + struct.pack("<I", 4) + struct.pack("<I", alignment & 0xFFFFFFFF))
    out = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv)) + b"".join(kv)
    for name, dims, typ, off in tensors:
        out += s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d & 0xFFFFFFFFFFFFFFFF) for d in dims)
        out += struct.pack("<IQ", typ, off & 0xFFFFFFFFFFFFFFFF)
    return out + b"\0" * 64 + data


@pytest.mark.parametrize("tensors,alignment,status", [
    ([(b"token_embd.weight", [32, 2], 0, 2**64 - 64)], None, _lib.SP_ERR_IO),       # offset that wraps the bounds sum
    ([(b"token_embd.weight", [32, 2], 0, 2**40)], None, _lib.SP_ERR_IO),            # offset far past the file
    ([(b"token_embd.weight", [2**62, 4], 0, 0)], None, _lib.SP_ERR_SHAPE),          # element count overflows 64 bits
    ([(b"token_embd.weight", [32, -2], 0, 0)], None, _lib.SP_ERR_SHAPE),            # negative dim (as a u64: huge)
    ([(b"token_embd.weight", [32, 0], 0, 0)], None, _lib.SP_ERR_SHAPE),             # empty dim
    ([(b"token_embd.weight", [32, 2**40], 0, 0)], None, _lib.SP_ERR_IO),            # more blocks than the file holds
    ([(b"token_embd.weight", [32, 2], 0, 0)], 0, _lib.SP_ERR_IO),                   # zero alignment
    ([(b"token_embd.weight", [32, 2], 0, 0)], 48, _lib.SP_ERR_IO),                  # not a power of two
    ([(b"token_embd.weight", [32, 2], 0, 0)], 1 << 30, _lib.SP_ERR_IO),             # absurd alignment
])
def test_gguf_crafted_headers_are_rejected(tmp_path, tensors, alignment, status):
    """Offsets, dims and the alignment are raw words of a downloaded file; a header built to wrap the bounds arithmetic
    must end in a status code before any byte outside the file is touched (the reference panics on the slice instead,
    crates/sapient-io/src/gguf.rs:636-676)."""
    L = _lib.lib()
    h = C.c_void_p()
    p = tmp_path / "crafted.gguf"
    p.write_bytes(_raw_gguf(tensors, alignment, data=b"\0" * 256))
    assert L.sp_cuda_engine_from_gguf(str(p).encode(), 0, 0, 1, C.byref(h)) == status, L.sp_cuda_last_error()


def test_no_device_is_an_error_not_a_fallback():
    L = _lib.lib()
    if L.sp_cuda_device_count() > 0:
        pytest.skip("a CUDA device is present")
    d = _lib.SpModelDesc()
    h = C.c_void_p()
    assert L.sp_cuda_engine_create(C.byref(d), C.byref(h)) == _lib.SP_ERR_CUDA
    from sapient_b200 import ops

    with pytest.raises(_lib.SapientCudaError):
        ops.rms_norm(np.ones((1, 4), np.float32), None, 1e-5)


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "sapient_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen", "tiny_phi2", "tiny_phi3"])
def test_gguf_of_every_family_parses_up_to_the_first_device_call(name, tmp_path):
    """Header, metadata, name map, fused-tensor splits (Phi-2 q|k|v, Phi-3 q|k|v and gate|up) and every bounds check run
    on the host before any device work: without a GPU the load must get as far as the first CUDA call (SP_ERR_CUDA) and
    not stop at an IO / shape / dtype error. With a GPU it simply succeeds."""
    import torch

    from sapient_b200 import synth
    from sapient_b200.engine import ForwardEngine

    cfg, W = synth.build_model(synth.CONFIGS[name], seed=5, device="cpu", max_ctx=64)
    if cfg["arch"] == "phi2":
        W.pop("model.norm.bias")
    path = str(tmp_path / f"{name}.gguf")
    synth.write_gguf(path, cfg, W)
    if torch.cuda.is_available():
        ForwardEngine.from_gguf(path).close()
        return
    with pytest.raises(_lib.SapientCudaError) as e:
        ForwardEngine.from_gguf(path)
    assert e.value.status == _lib.SP_ERR_CUDA, (e.value.status, str(e.value))


def test_nccl_arm_reports_a_missing_library_instead_of_crashing():
    """The library all-reduce arm opens NCCL at run time from a caller-named path: a wrong path is a status code and a
    message, and an undersized id buffer is refused before anything is opened."""
    L = _lib.lib()
    buf = C.create_string_buffer(128)
    assert L.sp_cuda_nccl_unique_id(b"/nonexistent/libnccl.so.2", buf, 128) == _lib.SP_ERR_STATE
    assert b"NCCL" in L.sp_cuda_last_error()
    assert L.sp_cuda_nccl_unique_id(b"/nonexistent/libnccl.so.2", buf, 64) == _lib.SP_ERR_ARG
    assert L.sp_cuda_engine_tp_set_allreduce(None, 1) == _lib.SP_ERR_ARG


def test_gguf_loader_survives_corrupted_headers(tmp_path):
    """GGUF files are downloaded content: whatever bytes the header, metadata and tensor table hold, the loader must answer
    with a status code (an IO / shape / dtype / state error, or SP_ERR_CUDA once it reaches device work on a machine
    without a GPU) and never read outside the mapping. 400 seeded corruptions of a valid file: single bytes, 64-bit
    fields set to extreme values, truncations."""
    import torch

    from sapient_b200 import synth
    from sapient_b200.engine import ForwardEngine

    cfg, W = synth.build_model(synth.CONFIGS["tiny_llama"], seed=6, device="cpu", max_ctx=64)
    good = str(tmp_path / "good.gguf")
    synth.write_gguf(good, cfg, W)
    data = bytearray(open(good, "rb").read())
    # the header region: everything before the first tensor's bytes (found by parsing nothing: corrupt the first 6 KB)
    region = min(len(data), 6144)
    rng = np.random.default_rng(1234)
    bad = str(tmp_path / "bad.gguf")
    extreme = [0, 1, 0xFFFFFFFF, 0x7FFFFFFFFFFFFFFF, 0xFFFFFFFFFFFFFFFF, 0x8000000000000000, 1 << 40]
    ok_status = {_lib.SP_ERR_IO, _lib.SP_ERR_SHAPE, _lib.SP_ERR_DTYPE, _lib.SP_ERR_STATE, _lib.SP_ERR_ARG, _lib.SP_ERR_CUDA,
                 _lib.SP_ERR_OOM, _lib.SP_ERR_KV_FULL}
    for trial in range(400):
        buf = bytearray(data)
        kind = trial % 3
        if kind == 0:
            for _ in range(int(rng.integers(1, 4))):
                buf[int(rng.integers(4, region))] = int(rng.integers(0, 256))
        elif kind == 1:
            at = int(rng.integers(4, region - 8))
            buf[at:at + 8] = int(extreme[int(rng.integers(0, len(extreme)))]).to_bytes(8, "little")
        else:
            buf = buf[: int(rng.integers(5, len(buf)))]
        with open(bad, "wb") as f:
            f.write(buf)
        try:
            eng = ForwardEngine.from_gguf(bad)
        except _lib.SapientCudaError as e:
            assert e.status in ok_status, (trial, e.status, str(e))
        else:
            assert torch.cuda.is_available()  # a harmless corruption (an unused byte): only a GPU box gets this far
            eng.close()
