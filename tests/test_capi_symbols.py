"""CPU: the C-ABI library builds, loads, and exports every symbol the public header declares."""

import ctypes
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _declared():
    names = set()
    for header in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"\b(infiniops_b200_\w+)\s*\(", header.read_text()))
    return names


def test_library_exports_every_declared_symbol():
    from infiniops_b200 import build, capi

    build.build_kernels()
    lib = ctypes.CDLL(str(build.LIB))
    declared = _declared()
    assert len(declared) >= 14
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert declared == set(capi.PROTOTYPES), "ctypes prototypes and header disagree"
    assert b"sm_100a" in capi.lib().infiniops_b200_version()


def test_argument_validation_without_gpu():
    """Validation runs before any CUDA call, so it can be exercised on a CPU-only host."""
    from infiniops_b200 import capi

    lib = capi.lib()
    rc = lib.infiniops_b200_gptq_marlin_repack(ctypes.c_void_p(16), None, 100, 64, 4, 0, ctypes.c_void_p(16), None)
    assert rc == 1 and b"divisible by 16" in lib.infiniops_b200_last_error()
    rc = lib.infiniops_b200_gptq_marlin_repack(ctypes.c_void_p(16), None, 128, 64, 3, 0, ctypes.c_void_p(16), None)
    assert rc == 1 and b"`num_bits` must be 4 or 8" in lib.infiniops_b200_last_error()
    rc = lib.infiniops_b200_grouped_topk(ctypes.c_void_p(16), 0, ctypes.c_void_p(16), 0, 1, 2, 2, 1, 1, 0, 1.0, 0,
                                         ctypes.c_void_p(16), ctypes.c_void_p(16), None)
    assert rc == 1 and b"at least two experts per group" in lib.infiniops_b200_last_error()
    rc = lib.infiniops_b200_moe_align_block_size(None, None, 0, 2000, 4, None, 0, None, 0, None, None, 0, None)
    assert rc == 1 and b"[1, 1023]" in lib.infiniops_b200_last_error()
