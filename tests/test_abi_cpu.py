"""CPU-side checks of the boundary: the shared library builds, loads, and exports exactly the
symbols include/peregrine_b200.h declares.  No compute call is made (no GPU here)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols(name="peregrine_b200.h"):
    text = open(os.path.join(ROOT, "include", name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"PG_API\s+[\w\s\*]+?\b(pg_\w+)\s*\(", text)))


def test_header_declares_the_path():
    syms = _header_symbols()
    for must in ("pg_quantize_activations", "pg_quantize_weights", "pg_dequantize", "pg_matmul_quantized",
                 "pg_matmul_quantized_host", "pg_gemm_i8", "pg_dequant_blocks", "pg_f16_to_f32", "pg_matmul_gguf",
                 "pg_qtensor_upload", "pg_qtensor_download", "pg_ctx_create", "pg_ctx_sync"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    from peregrine_b200 import _lib
    from peregrine_b200.build import ensure_built

    ensure_built()
    lib = C.CDLL(_lib.LIB_PATH)
    declared = _header_symbols()
    assert declared, "no declarations parsed"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    # and the ctypes table covers every declaration
    assert sorted(_lib.SIGNATURES) == declared
    # the tuning knobs have a header of their own; nothing named pg_* is exported without a declaration in one of the two
    knobs = _header_symbols("peregrine_b200_tune.h")
    assert sorted(_lib.TUNE_SIGNATURES) == knobs
    for name in knobs:
        assert hasattr(lib, name), f"{name} is declared in the tuning header but not exported"
    import subprocess

    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = sorted({line.split()[-1] for line in out.splitlines() if line.split() and line.split()[-1].startswith("pg_")})
    assert exported == sorted(declared + knobs), sorted(set(exported) ^ set(declared + knobs))


def test_rust_binding_covers_the_header():
    """rust/peregrine-b200-sys/src/lib.rs (generated, uncompiled) names every function of both headers with as many
    parameters as the C declaration has, and regenerating it changes nothing."""
    import importlib.util

    path = os.path.join(ROOT, "rust", "peregrine-b200-sys")
    rs = open(os.path.join(path, "src", "lib.rs")).read()
    rust = {m.group(1): m.group(2) for m in re.finditer(r"pub fn (pg_\w+)\(([^)]*)\)", rs, flags=re.S)}
    spec = importlib.util.spec_from_file_location("gen_bindings", os.path.join(path, "gen_bindings.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    for header in ("peregrine_b200.h", "peregrine_b200_tune.h"):
        funcs, _ = gen.parse(os.path.join(ROOT, "include", header))
        assert sorted(f[0] for f in funcs) == _header_symbols(header)
        for name, params, _ret in funcs:
            assert name in rust, f"{name} missing from the Rust binding"
            n_rust = len([a for a in rust[name].split(",") if a.strip()])
            assert n_rust == len(params), f"{name}: {n_rust} parameters in Rust, {len(params)} in C"


def test_errors_are_reported_not_thrown():
    from peregrine_b200 import _lib

    lib = _lib.load()
    assert lib.pg_version() >= 100
    # null context -> PG_ERR_INVALID with a message, no crash
    rc = lib.pg_ctx_sync(None)
    assert rc == _lib.PG_ERR_INVALID
    assert b"null context" in lib.pg_last_error()
    out = C.c_void_p()
    rc = lib.pg_ctx_create(0, None, C.byref(out))
    import torch

    if not torch.cuda.is_available():
        # no GPU: creation must fail loudly, there is no CPU path to fall back to
        assert rc == _lib.PG_ERR_UNSUPPORTED and not out.value
        with pytest.raises(_lib.PeregrineError):
            _lib.check(rc)
    else:
        assert rc == 0
        lib.pg_ctx_destroy(out)


def test_product_does_not_import_the_oracle():
    """The package must never reach into oracle/ (it is test infrastructure)."""
    pkg = os.path.join(ROOT, "peregrine_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "pgoracle" not in src and "oracle/" not in src and "import oracle" not in src, f
