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
