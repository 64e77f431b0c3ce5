"""The quantised serial format, host side: exact byte layout of write_quantized_tensor (src/serial.rs:124-157) and
the checks read_quantized_tensor makes before any data is touched (src/serial.rs:159-186)."""
import io
import struct

import numpy as np
import pytest

from peregrine_b200.quant import QuantizedTensor
from peregrine_b200.serial import SerialPanic, read_quantized_tensor, write_quantized_tensor


def _tensor(rows, cols, seed=1):
    g = np.random.Generator(np.random.PCG64(seed))
    q = g.integers(-127, 128, (rows, cols), dtype=np.int8)
    s = g.random(cols, dtype=np.float32) + np.float32(0.01)
    return QuantizedTensor(q, np.ascontiguousarray(q.T), s, rows, cols)


def test_written_bytes():
    qt = _tensor(3, 5)
    buf = io.BytesIO()
    write_quantized_tensor(buf, "layer.0.wéight", qt)
    name = "layer.0.wéight".encode("utf-8")
    want = struct.pack("<I", len(name)) + name + b"\x01" + struct.pack("<III", 2, 3, 5) + qt.data_i8.tobytes() + qt.scales.tobytes()
    assert buf.getvalue() == want


def test_reader_rejects_other_dtypes_ranks_and_short_files():
    head = struct.pack("<I", 1) + b"w"
    with pytest.raises(SerialPanic, match="expected dtype=1"):
        read_quantized_tensor(io.BytesIO(head + b"\x02" + struct.pack("<III", 2, 1, 1)))
    with pytest.raises(SerialPanic, match="quantized tensors must be 2D"):
        read_quantized_tensor(io.BytesIO(head + b"\x01" + struct.pack("<IIII", 3, 1, 1, 1)))
    with pytest.raises(ValueError, match="failed to fill whole buffer"):
        read_quantized_tensor(io.BytesIO(head + b"\x01" + struct.pack("<III", 2, 4, 4) + bytes(10)))
    with pytest.raises(ValueError, match="failed to fill whole buffer"):
        read_quantized_tensor(io.BytesIO(b"\x05\x00"))
    with pytest.raises(ValueError, match="utf-8"):
        read_quantized_tensor(io.BytesIO(struct.pack("<I", 2) + b"\xff\xfe" + b"\x01"))


def _f32_record(name, shape, typed):
    nb = name.encode("utf-8")
    g = np.random.Generator(np.random.PCG64(len(name)))
    n = int(np.prod(shape)) if shape else 1
    return (struct.pack("<I", len(nb)) + nb + (b"\x00" if typed else b"") + struct.pack("<I", len(shape)) +
            struct.pack(f"<{len(shape)}I", *shape) + g.standard_normal(n).astype("<f4").tobytes())


def test_file_kind_follows_the_whole_chain_of_records(tmp_path):
    """Typed and plain model files differ by one byte per record; the detection must not be fooled by a typed file whose
    first record is a scalar or a vector f32 tensor (second byte after the name zero in both layouts), nor by a plain
    file whose first tensor has a rank that looks like a dtype."""
    from peregrine_b200.serial import file_kind

    qt = _tensor(4, 6)
    qrec = io.BytesIO()
    write_quantized_tensor(qrec, "blk.weight", qt)
    cases = {
        "typed_scalar_first": (struct.pack("<I", 3) + _f32_record("step", [], True) + _f32_record("bias", [6], True) + qrec.getvalue(), "typed"),
        "typed_matrix_first": (struct.pack("<I", 2) + _f32_record("w", [3, 5], True) + qrec.getvalue(), "typed"),
        "typed_i8_only": (struct.pack("<I", 1) + qrec.getvalue(), "typed"),
        "plain_rank1_first": (struct.pack("<I", 2) + _f32_record("bias", [7], False) + _f32_record("w", [2, 3], False), "plain"),
        "plain_rank3_first": (struct.pack("<I", 1) + _f32_record("conv", [2, 3, 4], False), "plain"),
        "plain_scalar_only": (struct.pack("<I", 1) + _f32_record("lr", [], False), "plain"),
        "empty": (struct.pack("<I", 0), "plain"),
    }
    for name, (data, want) in cases.items():
        path = tmp_path / (name + ".bin")
        path.write_bytes(data)
        assert file_kind(str(path)) == want, name
    bad = tmp_path / "truncated.bin"
    bad.write_bytes(cases["typed_matrix_first"][0][:-3])
    with pytest.raises(SerialPanic, match="neither"):
        file_kind(str(bad))
