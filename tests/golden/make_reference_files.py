"""Writes the model-file fixtures of this folder by running the reference's own conversion scripts.

    python tests/golden/make_reference_files.py <path of the reference checkout>

The reference ships its two weight converters as plain Python (scripts/convert_weights_int8.py,
scripts/convert_huffman.py).  This script imports them unchanged from the checkout and lets them convert one small
seeded model, so the three files it leaves here are OUTPUTS OF THE REFERENCE ITSELF:

    reference_model_f32.bin       the input, in the layout of serial::save_model (src/serial.rs:10-41)
    reference_model_int8.bin      convert_weights_int8.write_int8_model of it   (dtype 0 = f32 and dtype 1 = i8 records)
    reference_model_huffman.bin   convert_huffman.main of the int8 file         (dtype 3 records, 4 streams each)

The model: three 2-D ".weight" tensors of N(0, 0.05) values and two 1-D tensors, seeds below.  No value lands on a
rounding tie (checked here), because the scripts round half to even where src/quant.rs:62 rounds half away from zero.
"""
import importlib.util
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

TENSORS = [("layers.0.attn.weight", (24, 16), 101), ("layers.0.attn.bias", (16,), 102), ("layers.0.mlp.weight", (16, 40), 103),
           ("norm.scale", (16,), 104), ("head.weight", (40, 33), 105)]


def load_script(root, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(root, "scripts", name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def model():
    out = []
    for name, shape, seed in TENSORS:
        g = np.random.Generator(np.random.PCG64(seed))
        out.append((name, shape, (g.standard_normal(shape, dtype=np.float32) * np.float32(0.05)).astype(np.float32)))
    return out


def write_f32_model(path, tensors):
    with open(path, "wb") as f:
        f.write(struct.pack("<I", len(tensors)))
        for name, shape, data in tensors:
            nb = name.encode("utf-8")
            f.write(struct.pack("<I", len(nb)) + nb + struct.pack("<I", len(shape)) + struct.pack(f"<{len(shape)}I", *shape))
            f.write(data.astype("<f4").tobytes())


def main() -> None:
    root = sys.argv[1]
    int8 = load_script(root, "convert_weights_int8")
    huff = load_script(root, "convert_huffman")
    tensors = model()
    for name, shape, data in tensors:
        if len(shape) == 2:
            scales = np.abs(data).max(axis=0) / np.float32(127.0)
            frac = np.abs(data / scales[None, :]) % 1.0
            assert not np.any(frac == 0.5), f"{name}: a value lies on a rounding tie"
    f32_path = os.path.join(HERE, "reference_model_f32.bin")
    int8_path = os.path.join(HERE, "reference_model_int8.bin")
    huff_path = os.path.join(HERE, "reference_model_huffman.bin")
    write_f32_model(f32_path, tensors)
    loaded = int8.read_peregrine_model(f32_path)
    int8.write_int8_model(loaded, int8_path)
    # convert_huffman reads its arguments from sys.argv; its reader tells typed records from plain f32 ones by peeking
    # at the dtype byte, so it is given a file of the 2-D tensors only (an f32 record's dtype byte 0 would be misread)
    only2d = os.path.join(HERE, "_only2d_int8.bin")
    int8.write_int8_model([t for t in loaded if len(t[1]) == 2], only2d)
    argv = sys.argv
    try:
        sys.argv = ["convert_huffman.py", only2d, huff_path, "--streams", "4"]
        huff.main()
    finally:
        sys.argv = argv
        os.remove(only2d)
    for p in (f32_path, int8_path, huff_path):
        print(p, os.path.getsize(p), "bytes")


if __name__ == "__main__":
    main()
