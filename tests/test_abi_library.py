"""The shared library loads on a machine without a GPU and exports every symbol the header
declares; compute entry points refuse to run without a device instead of falling back."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "pcb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pcb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from lvd_pg_b200 import _lib, build
    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    syms = declared_symbols()
    assert len(syms) >= 35
    for s in syms:
        assert hasattr(lib, s), s
    assert lib.pcb_version() >= 100
    assert set(_lib.SIGNATURES) <= set(syms)


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from lvd_pg_b200 import api
    from lvd_pg_b200._lib import PcbError
    from tests.helpers import simple3
    with pytest.raises(PcbError):
        api.CuMetaBitsProbCircuit(simple3())


def test_product_code_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "lvd_pg_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".jl")):
                assert "oracle" not in open(os.path.join(dirpath, f)).read().replace("the oracle", ""), f


def test_both_host_wrappers_bind_every_entry_point():
    """The Python mirror declares a signature for, and the shipped Julia wrapper `ccall`s, every entry point
    of the header (the two %globaltimer trace readers of diagnostic builds aside)."""
    from lvd_pg_b200 import _lib
    syms = [s for s in declared_symbols() if not s.startswith("pcb_debug_")]
    jl = open(os.path.join(ROOT, "lvd_pg_b200", "julia", "PCB200.jl")).read()
    missing_jl = [s for s in syms if f"(:{s}," not in jl]
    assert not missing_jl, missing_jl
    no_signature = [s for s in syms if s not in _lib.SIGNATURES and s not in ("pcb_last_error", "pcb_profile_class_name")]
    assert not no_signature, no_signature
