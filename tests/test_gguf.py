"""GGUF ingest (format/gguf_codec.cpp): the fixture tests/golden/tiny.gguf was written by the
reference's own GGUFWriter and tests/golden/gguf_expected.npz holds what its GGUFReader
returns for every tensor (tests/golden/make_golden.py gguf).

CPU part: the header / tensor-table parse behind the C ABI, the storage-kind policy, and the
oracle's quantisers against the bytes the reference's writer and reader produced.
GPU part: b200_gguf_load_tensor - the verbatim copy and the decode + quantise-on-load path -
bit for bit against the reader's bytes.
"""
import ctypes as C
import importlib
import os

import numpy as np
import pytest

import golden_gguf as gg
from oracle_lib import packed_bytes

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "golden", "tiny.gguf").encode()
EXPECT = np.load(os.path.join(HERE, "golden", "gguf_expected.npz"))
LABEL = {-2: "f32", 0: "q4_0", 1: "q4_1", 2: "q8_0"}


@pytest.fixture(scope="module")
def lib():
    return importlib.import_module("jdm-ghassan_v1_flach_b200").lib()


@pytest.fixture()
def gguf(lib):
    h = C.c_void_p()
    lib.b200_gguf_open(PATH, C.byref(h))
    yield h
    lib.b200_gguf_close(h)


def _info(lib, g, i):
    name = C.create_string_buffer(128)
    dims = (C.c_int64 * 4)()
    nd, ty, nb = C.c_int(), C.c_int(), C.c_uint64()
    lib.b200_gguf_tensor_info(g, i, name, 128, dims, C.byref(nd), C.byref(ty), C.byref(nb))
    return name.value.decode(), list(dims)[:nd.value], ty.value, nb.value


def _file_bytes(lib, g, i, nbytes):
    p = C.c_void_p()
    lib.b200_gguf_tensor_data(g, i, C.byref(p))
    return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), (nbytes,)).copy()


def test_tensor_table(lib, gguf):
    n = C.c_int()
    lib.b200_gguf_tensor_count(gguf, C.byref(n))
    assert n.value == len(gg.TENSORS)
    for i, (name, rows, cols, ty) in enumerate(gg.TENSORS):
        got_name, dims, got_ty, nb = _info(lib, gguf, i)
        assert got_name == name and got_ty == ty
        assert dims == ([rows, cols] if cols else [rows])
        kind = gg.KIND_OF_GGML[ty]
        elems = rows * max(cols, 1)
        assert nb == (elems * 4 if kind == -2 else elems * 2 if kind == -1 else packed_bytes(kind, elems))
        idx = C.c_int(-5)
        lib.b200_gguf_find_tensor(gguf, name.encode(), C.byref(idx))
        assert idx.value == i
    idx = C.c_int(0)
    lib.b200_gguf_find_tensor(gguf, b"layers.9.nothing", C.byref(idx))
    assert idx.value == -1


def test_metadata_and_errors(lib, gguf):
    v = C.c_double()
    lib.b200_gguf_metadata_number(gguf, b"b200.fixture.answer", C.byref(v))
    assert v.value == 42.0
    lib.b200_gguf_metadata_number(gguf, b"ghassan.embedding_length", C.byref(v))
    assert v.value == 64.0
    lib.b200_gguf_metadata_number(gguf, b"ghassan.block_count", C.byref(v))
    assert v.value == 1.0
    lib.b200_gguf_metadata_number(gguf, b"ghassan.attention.layer_norm_rms_epsilon", C.byref(v))
    assert v.value == float(np.float32(1e-5))
    assert lib.raw("b200_gguf_metadata_number", gguf, b"general.architecture", C.byref(v)) != 0   # a string
    assert lib.raw("b200_gguf_metadata_number", gguf, b"no.such.key", C.byref(v)) != 0
    h = C.c_void_p()
    assert lib.raw("b200_gguf_open", b"/nonexistent/file.gguf", C.byref(h)) != 0
    assert "nonexistent" in lib.last_error()


def test_rejects_a_file_that_is_not_gguf(lib, tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUX" + bytes(60))
    h = C.c_void_p()
    assert lib.raw("b200_gguf_open", str(p).encode(), C.byref(h)) != 0
    raw = open(PATH, "rb").read()
    p.write_bytes(raw[:200])                       # cut inside the tensor table
    assert lib.raw("b200_gguf_open", str(p).encode(), C.byref(h)) != 0
    # a tensor whose dimensions multiply past 2^64 (would wrap to a small element count)
    import struct
    name = b"tok_embeddings"
    at = raw.index(struct.pack("<Q", len(name)) + name) + 8 + len(name)       # its table entry: n_dims, dims ...
    nd = struct.unpack_from("<I", raw, at)[0]
    assert nd == 2
    bad = bytearray(raw)
    struct.pack_into("<QQ", bad, at + 4, 1 << 62, 1 << 62)
    p.write_bytes(bytes(bad))
    assert lib.raw("b200_gguf_open", str(p).encode(), C.byref(h)) != 0
    assert "shape" in lib.last_error()


def test_storage_kind_policy(lib):
    """Model::storage_dtype_for (model/model.cpp:959-986) for packed weights of kind 3."""
    want = {
        "tok_embeddings": -1, "lm_head": -1, "final_norm": -2,
        "layers.0.attn_norm": -2, "layers.3.ffn_norm": -2,
        "layers.0.mamba.in_proj": 3, "layers.0.mamba.out_proj": 3, "layers.0.mamba.conv1d": -2,
        "layers.0.mamba.conv1d_bias": -2, "layers.0.mamba.dt_bias": -2, "layers.0.mamba.A_log": -2,
        "layers.0.mamba.D": -2, "layers.0.mamba.norm": -2,
        "layers.5.wq": 3, "layers.5.wo": 3,
        "layers.0.moe_router": -2, "layers.0.moe_router_bias": -2, "layers.0.moe_gate": 3,
        "layers.0.moe_down": 3, "layers.0.moe_shared_up": 3,
    }
    for name, kind in want.items():
        k = C.c_int(99)
        lib.b200_gguf_storage_kind(name.encode(), 3, C.byref(k))
        assert k.value == kind, name


def test_oracle_quantisers_reproduce_the_writers_bytes(lib, gguf, oracle):
    """The bytes the reference's writer stored for the packed tensors: Q4_0 by the signed-extreme
    rule (oracle kind 4), Q8_0 and Q4_1 by the rules the oracle has as kinds 2 and 1."""
    seen = 0
    for i, (name, rows, cols, ty) in enumerate(gg.TENSORS):
        kind = gg.KIND_OF_GGML[ty]
        if kind < 0:
            continue
        stored = _file_bytes(lib, gguf, i, _info(lib, gguf, i)[3])
        want = oracle.quantize(gg.source(name), 4 if kind == 0 else kind)
        assert np.array_equal(stored, want), name
        # and the reader hands those bytes back unchanged when asked for the stored layout
        assert np.array_equal(EXPECT[f"{name}/{LABEL[kind]}"], stored)
        seen += 1
    assert seen == 4


def test_oracle_reproduces_the_readers_quantise_on_load(oracle):
    """GGUFReader::read_tensor_quant's slow path: decode to fp32, quantise with
    quantization/quantize.cpp - the oracle's dequantize_f32 + quantize on the same bytes."""
    for name, rows, cols, ty in gg.TENSORS:
        f32 = EXPECT[f"{name}/f32"].view(np.float32)
        kind = gg.KIND_OF_GGML[ty]
        if kind == -2:
            assert np.array_equal(f32, gg.source(name))
        elif kind == -1:
            assert np.array_equal(f32, gg.source(name).astype(np.float16).astype(np.float32))
        else:
            stored = EXPECT[f"{name}/{LABEL[kind]}"]
            assert np.array_equal(f32, oracle.dequantize_f32(stored, f32.size, kind))
        for k in (0, 1, 2):
            if k == kind or f"{name}/{LABEL[k]}" not in EXPECT.files:
                continue
            assert np.array_equal(EXPECT[f"{name}/{LABEL[k]}"], oracle.quantize(f32, k)), (name, k)


@pytest.mark.gpu
def test_load_tensor_matches_the_reader(lib, gguf):
    import torch
    from gpu_util import empty, host
    checked = 0
    for i, (name, rows, cols, ty) in enumerate(gg.TENSORS):
        for kind, label in LABEL.items():
            key = f"{name}/{label}"
            if key not in EXPECT.files:
                continue
            nb = C.c_uint64()
            lib.b200_gguf_tensor_bytes(gguf, i, kind, C.byref(nb))
            want = EXPECT[key]
            assert nb.value == want.size, key
            out = empty(nb.value + 16, torch.uint8)
            lib.b200_gguf_load_tensor(gguf, i, kind, out, nb.value)
            got = host(out)
            assert np.array_equal(got[:nb.value], want), key
            assert np.all(got[nb.value:] == np.uint8(-7 & 0xFF)), f"{key}: wrote past the tensor"
            checked += 1
    assert checked == 32


@pytest.mark.gpu
def test_load_tensor_to_fp16_and_q4k(lib, gguf, oracle):
    """Kinds the reference reader has no call for: fp16 storage (its tok_embeddings policy) and
    this library's Q4_K, against the oracle on the decoded values."""
    import torch
    from gpu_util import empty, host
    for i, (name, rows, cols, ty) in enumerate(gg.TENSORS):
        f32 = EXPECT[f"{name}/f32"].view(np.float32)
        out = empty(f32.size, torch.int16)
        lib.b200_gguf_load_tensor(gguf, i, -1, out, f32.size * 2)
        assert np.array_equal(host(out).view(np.float16), f32.astype(np.float16)), name
        if f32.size % 256 == 0:
            want = oracle.quantize(f32, 3)
            out = empty(want.size, torch.uint8)
            lib.b200_gguf_load_tensor(gguf, i, 3, out, want.size)
            assert np.array_equal(host(out), want), name
    small = empty(8, torch.uint8)
    assert lib.raw("b200_gguf_load_tensor", gguf, 0, -2, small, 8) != 0        # destination too small
