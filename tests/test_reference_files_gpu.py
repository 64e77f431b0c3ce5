"""Model files written by the reference's own converters (tests/golden/reference_model_*.bin), through the GPU: the
package's converter reproduces the int8 file byte for byte, and both quantised files load into the tensors the
reference wrote."""
import numpy as np
import pytest

from _inputs import bits_equal, normal, rng
from test_reference_files_cpu import F32, HUFF, INT8, parse_int8_file

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pg():
    import peregrine_b200

    return peregrine_b200


def test_int8_converter_reproduces_the_reference_file(pg, gpu, tmp_path):
    """scripts/convert_weights_int8.py on the f32 fixture, with the quantiser on the GPU."""
    out = tmp_path / "int8.bin"
    pg.serial.convert_weights_int8(F32, str(out), gpu)
    assert open(out, "rb").read() == open(INT8, "rb").read()


def test_typed_file_loads_resident(pg, gpu, oracle):
    ref = parse_int8_file(INT8)
    records = pg.serial.load_typed_model(INT8, gpu)
    assert [n for n, _ in records] == list(ref)
    for name, item in records:
        if isinstance(item, tuple):
            assert item[0] == ref[name][0] and bits_equal(item[1], ref[name][1])
            continue
        rows, cols, q, s = ref[name]
        assert item.on_gpu and (item.rows, item.cols) == (rows, cols)
        assert np.array_equal(item.data_i8, q) and np.array_equal(item.data_i8_t, q.T) and bits_equal(item.scales, s)
        x = normal(rng(rows), (3, rows))
        want = oracle.matmul_quantized(x, 3, rows, oracle.quantize_weights((q * s[None, :]).astype(np.float32), rows, cols))
        assert bits_equal(pg.quant.matmul_quantized(x, 3, rows, item, gpu), want)


def test_huffman_file_decodes_to_the_reference_tensors(pg, gpu):
    ref = parse_int8_file(INT8)
    for name, ht in pg.serial.load_typed_model(HUFF, gpu):
        rows, cols, q, s = ref[name]
        qt = ht.decode_to_quantized(gpu)
        assert np.array_equal(qt.data_i8, q) and np.array_equal(qt.data_i8_t, q.T) and bits_equal(qt.scales, s), name


@pytest.mark.parametrize("source", ["int8", "f32"])
def test_huffman_converter(pg, gpu, tmp_path, source):
    """scripts/convert_huffman.py from either kind of input file: the records decode to the reference's tensors (the
    code itself may differ from the script's: other tie rules, same lengths in total)."""
    ref = parse_int8_file(INT8)
    out = tmp_path / "huff.bin"
    pg.serial.convert_huffman(INT8 if source == "int8" else F32, str(out), 4, gpu=gpu)
    mine = pg.serial.load_typed_model(str(out), gpu)
    theirs = dict(pg.serial.load_typed_model(HUFF, gpu))
    assert [n for n, _ in mine] == list(theirs)
    for name, ht in mine:
        rows, cols, q, s = ref[name]
        assert ht.stream_lengths == theirs[name].stream_lengths
        assert np.array_equal(ht.decode_to_quantized(gpu).data_i8, q) and bits_equal(ht.scales, s)
        # both codes are optimal: the same number of bits over the tensor, up to the padding of each stream's last byte
        assert abs(sum(len(x) for x in ht.streams) - sum(len(x) for x in theirs[name].streams)) <= 4
