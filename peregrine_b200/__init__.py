"""peregrine_b200: the quantized-inference path of etam103/peregrine on NVIDIA B200 (sm_100a).

    quant     mirror of peregrine::quant  (src/quant.rs)
    gguf      mirror of the block codecs of peregrine::gguf  (src/gguf.rs:284-401)
    gguf_file the GGUF container, mirror of GgufFile  (src/gguf.rs:140-283, 403-567)
    llama     the Llama decode step on the int8 path  (src/models/llama)
    llama_gguf  Llama::from_gguf for that step: config keys, tensor names, transposition, Q|K|V and gate|up fusion
    serial    the quantised serial formats  (src/serial.rs:124-222, 315-443)
    huffman   Huffman-coded int8 weights, mirror of HuffmanTable / HuffmanTensor  (src/huffman.rs:19-476)
    runtime   GpuContext / GpuBuffer / init_gpu / with_gpu  (the reference's `metal` seam)
    build     compiles libperegrine_b200.so with nvcc

Everything computes in hand-written CUDA behind the C ABI of include/peregrine_b200.h.
"""
from . import _lib
from ._lib import InvalidArgument, PeregrineError
from .runtime import GpuBuffer, GpuContext, current_gpu, init_gpu, with_gpu
from . import quant, gguf, gguf_file, serial, huffman
from .gguf_file import GgufFile

__all__ = ["quant", "gguf", "gguf_file", "GgufFile", "serial", "huffman", "GpuContext", "GpuBuffer", "init_gpu", "with_gpu", "current_gpu", "PeregrineError", "InvalidArgument"]
