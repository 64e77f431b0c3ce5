"""GGUF container parsing (host only): the reference's own container tests (tests/gguf_parity.rs:78-105,
src/gguf.rs:633-640) and the header / metadata / tensor-info rules of GgufFile::parse (src/gguf.rs:411-482)."""
import struct

import numpy as np
import pytest

import _gguf_writer as W
from peregrine_b200.gguf_file import GGUF_MAGIC, GgufFile, GgufPanic


def test_magic_constant():
    """src/gguf.rs:633-640"""
    assert struct.unpack("<I", b"GGUF")[0] == GGUF_MAGIC


def test_invalid_magic():
    """tests/gguf_parity.rs:78-84"""
    with pytest.raises(ValueError, match="invalid GGUF magic"):
        GgufFile.parse(bytes(64))


def test_minimal_valid():
    """tests/gguf_parity.rs:86-105"""
    data = struct.pack("<IIQQ", 0x46554747, 3, 0, 0)
    data += bytes(64 - len(data))
    f = GgufFile.parse(data)
    assert f.metadata == {} and f.tensors == {}


@pytest.mark.parametrize("version,ok", [(1, False), (2, True), (3, True), (4, False)])
def test_versions(version, ok):
    data = W.build([], [], version=version)
    if ok:
        GgufFile.parse(data)
    else:
        with pytest.raises(ValueError, match=f"unsupported GGUF version: {version}"):
            GgufFile.parse(data)


def test_every_metadata_type_and_accessors():
    kvs = [("a.u8", W.U8, 200), ("a.i8", W.I8, -5), ("a.u16", W.U16, 65000), ("a.i16", W.I16, -300), ("a.u32", W.U32, 4000000000),
           ("a.i32", W.I32, -7), ("a.f32", W.F32, 1.5), ("a.bool", W.BOOL, 1), ("a.str", W.STR, "llama é"), ("a.u64", W.U64, 2 ** 40 + 3),
           ("a.i64", W.I64, -2), ("a.f64", W.F64, 0.1), ("a.strs", W.ARR, (W.STR, ["x", "yz", ""])), ("a.f32s", W.ARR, (W.F32, [0.5, -2.0])),
           ("a.nested", W.ARR, (W.ARR, [(W.U32, [1, 2]), (W.U32, [])]))]
    f = GgufFile.parse(W.build(kvs, []))
    m = f.metadata
    assert m["a.u8"] == 200 and m["a.i8"] == -5 and m["a.u16"] == 65000 and m["a.i16"] == -300 and m["a.u32"] == 4000000000
    assert m["a.i32"] == -7 and m["a.f32"] == np.float32(1.5) and m["a.bool"] is True and m["a.str"] == "llama é"
    assert m["a.u64"] == 2 ** 40 + 3 and m["a.i64"] == -2 and m["a.f64"] == 0.1
    assert m["a.strs"] == ["x", "yz", ""] and m["a.f32s"] == [np.float32(0.5), np.float32(-2.0)] and m["a.nested"] == [[1, 2], []]
    # as_u32 takes the four 32/64-bit integer types (truncating like `as u32`), as_f32 the two float types
    assert f.get_u32("a.u32") == 4000000000 and f.get_u32("a.i32") == 2 ** 32 - 7 and f.get_u32("a.u64") == 3 and f.get_u32("a.i64") == 2 ** 32 - 2
    assert f.get_u32("a.u8") is None and f.get_u32("a.f32") is None and f.get_u32("missing") is None
    assert f.get_f32("a.f32") == np.float32(1.5) and f.get_f32("a.f64") == np.float32(0.1) and f.get_f32("a.u32") is None
    assert f.get_metadata("a.str") == "llama é" and f.get_metadata("missing") is None


def test_unknown_metadata_type_and_tensor_type_panic():
    bad = struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1) + b"k" + struct.pack("<I", 13)
    with pytest.raises(GgufPanic, match="unknown GGUF metadata value type: 13"):
        GgufFile.parse(bad + bytes(32))
    with pytest.raises(GgufPanic, match="unsupported GGML type 7 for tensor 'w'"):
        GgufFile.parse(W.build([], [("w", [32], 7, bytes(34))]))
    with pytest.raises(GgufPanic):
        GgufFile.parse(struct.pack("<IIQQ", 0x46554747, 3, 5, 0))       # tensor infos missing: truncated header


@pytest.mark.parametrize("alignment", [None, 32, 64, 256])
def test_tensor_infos_offsets_alignment_and_shapes(alignment):
    g = np.random.Generator(np.random.PCG64(5))
    a = g.standard_normal(6).astype(np.float32)
    b = g.standard_normal((3, 5)).astype(np.float32)
    f = GgufFile.parse(W.build([("general.name", W.STR, "t")], [("a", [6], 0, a.tobytes()), ("b", [5, 3], 0, b.tobytes()),
                                                              ("q", [64, 2], 8, bytes(4 * 34))], alignment=alignment))
    al = alignment or 32
    assert f.data_start % al == 0 and sorted(f.tensor_names()) == ["a", "b", "q"]
    assert f.tensors["b"].shape == [5, 3] and f.tensor_shape("b") == [3, 5] and f.tensor_shape("a") == [6]
    assert f.tensors["a"].data_offset == 0 and f.tensors["b"].data_offset % al == 0 and f.tensors["q"].data_offset % al == 0
    assert f.tensors["q"].num_elements() == 128 and f.tensors["q"].data_size() == 4 * 34
    # F32 data is a reinterpretation of the file bytes: no GPU involved
    assert np.array_equal(f.load_tensor_f32("a"), a) and np.array_equal(f.load_tensor_f32("b"), b.reshape(-1))
    with pytest.raises(GgufPanic, match="tensor 'zz' not found"):
        f.load_tensor_f32("zz")
    with pytest.raises(GgufPanic, match="tensor 'zz' not found"):
        f.tensor_shape("zz")


def test_elements_not_divisible_by_block():
    f = GgufFile.parse(W.build([], [("w", [40], 2, bytes(36))]))
    with pytest.raises(GgufPanic, match="tensor elements 40 not divisible by block size 32"):
        f.tensors["w"].data_size()
