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


def test_ctypes_structs_match_the_header(tmp_path):
    """Every struct of the C ABI as a C compiler lays it out (size and field offsets) against its ctypes
    mirror in `capi`: a field added on one side only would otherwise shift every later argument silently."""
    import subprocess

    from infiniops_b200 import capi

    mirrors = {
        "iob_gemm_problem": (capi.GemmProblem, ("a", "b_q_weight", "b_bias", "b_scales", "b_zeros", "out", "size_m", "size_n",
                                                "size_k", "num_groups", "out_ld", "out_col0", "n_peers", "peer_out",
                                                "scale_layout", "g_idx", "perm")),
        "iob_peer_signal": (capi.PeerSignal, ("done_counter", "epoch", "n_peers", "peer_flags", "flag_slot")),
        "iob_routed_options": (capi.RoutedOptions, ("scale_layout", "a_sorted", "out_sorted", "fuse_silu", "g_idx", "perm",
                                                    "route_position", "block_rows", "row_dest", "dest_base", "n_dest",
                                                    "signal")),
        "iob_ep_context": (capi.EpContext, ("world", "rank", "top_k", "hidden", "inter", "experts_per_rank", "capacity",
                                            "moe_block_size", "a_dtype", "b_type_id", "arena", "flags", "ctrl")),
        "iob_expert_weights": (capi.ExpertWeightsC, ("w13", "s13", "z13", "groups13", "w2", "s2", "z2", "groups2",
                                                     "w13_interleaved")),
        "iob_peer_copy": (capi.PeerCopy, ("src", "dst", "rows", "row_bytes", "pitch_bytes")),
    }
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "infiniops_b200.h"', "int main(void) {"]
    for name, (_, fields) in mirrors.items():
        lines.append(f'  printf("{name} %zu", sizeof({name}));')
        for f in fields:
            lines.append(f'  printf(" %zu", offsetof({name}, {f}));')
        lines.append('  printf("\\n");')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip().splitlines()
    for line in out:
        name, size, *offsets = line.split()
        mirror, fields = mirrors[name]
        assert ctypes.sizeof(mirror) == int(size), f"{name}: size {ctypes.sizeof(mirror)} != {size}"
        assert [f for f, _ in mirror._fields_] == list(fields), f"{name}: field list differs"
        for f, off in zip(fields, offsets):
            assert getattr(mirror, f).offset == int(off), f"{name}.{f}: offset {getattr(mirror, f).offset} != {off}"


def test_weight_type_ids_agree_between_header_bindings_and_operator_layer():
    """The vLLM scalar-type ids appear three times (C header, ctypes constants, C++ operator layer): one
    list, compared number by number."""
    import re

    from infiniops_b200 import capi

    header = (ROOT / "include" / "infiniops_b200.h").read_text()
    in_header = {name: int(value) for name, value in re.findall(r"#define IOB_QTYPE_(\w+) (\d+)LL", header)}
    assert set(in_header) == {"UINT4B8", "UINT4", "UINT8B128", "UINT8", "FLOAT8_E4M3FN"}
    for name, value in in_header.items():
        assert getattr(capi, "QTYPE_" + name) == value, name
    base = (ROOT / "include" / "base" / "moe_wna16_marlin_gemm.h").read_text()
    in_base = {name: int(value) for name, value in re.findall(r"k(\w+) = (\d+)", base)}
    spelled = {"UINT4B8": "Uint4B8", "UINT4": "Uint4", "UINT8B128": "Uint8B128", "UINT8": "Uint8",
               "FLOAT8_E4M3FN": "Float8E4M3Fn"}
    for name, value in in_header.items():
        assert in_base[spelled[name]] == value, name
