"""A compiled C++ consumer of `#include <infini/ops.h>` (tests/cpp/consumer.cc): built on any
machine, run on the GPU and checked against the oracle.

The program drives the operators the way a C++ application does -- `Op::Call(handle, config, ...)`,
`Op::Make(...)` + `(*op)(handle, ...)`, `SiluAndMul::MakeReturnValue` with an owning tensor type of
its own -- through ONE Handle whose workspace is filled with 0xFF beforehand and is shared by the
token sort (which writes its histograms there) and the GEMMs (which count split-K arrivals there):
the reference gives a workspace no zeroing contract (src/handle.h:10-41 of the reference).  Modelled
on the compiled smoke programs of tests/test_cpp_api.py:10-33,74-124 of the reference."""

import pathlib
import subprocess

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import quant as oq

ROOT = pathlib.Path(__file__).resolve().parent.parent
TOKENS, EXPERTS, TOP_K, HIDDEN, INTER, BLOCK = 700, 8, 2, 256, 128, 16   # kept in step with consumer.cc


def _build(tmp_path) -> pathlib.Path:
    from infiniops_b200 import build

    build.build_kernels()
    binary = tmp_path / "consumer"
    lib_dir = ROOT / "infiniops_b200" / "lib"
    cmd = ["g++", "-std=c++17", "-Werror", "-Wall", f"-I{ROOT / 'include'}", "-I/usr/local/cuda/include",
           str(ROOT / "tests" / "cpp" / "consumer.cc"), f"-L{lib_dir}", "-linfiniops_b200", "-L/usr/local/cuda/lib64",
           "-lcudart", f"-Wl,-rpath,{lib_dir}", "-Wl,-rpath,/usr/local/cuda/lib64", "-o", str(binary)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return binary


def test_consumer_compiles_against_the_shipped_headers(tmp_path):
    assert _build(tmp_path).exists()


@pytest.mark.gpu
def test_consumer_runs_and_matches_the_oracle(tmp_path):
    binary = _build(tmp_path)
    gen = torch.Generator().manual_seed(77)

    def experts(k, n):
        q = torch.randint(0, 16, (EXPERTS, k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
        s = (torch.randn((EXPERTS, k // 128, n), generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        return q, s, np.stack([oq.gptq_pack(q[e], 4) for e in range(EXPERTS)])

    q13, s13, g13 = experts(HIDDEN, 2 * INTER)
    q2, s2, g2 = experts(INTER, HIDDEN)
    x = torch.randn((TOKENS, HIDDEN), generator=gen).bfloat16()
    logits = torch.randn((TOKENS, EXPERTS), generator=gen)
    tw, ids, _ = omoe.topk_softmax(logits, None, None, TOP_K, True)
    m, k, n = 16, 8192, 128
    dq = torch.randint(0, 16, (k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
    ds = (torch.randn((k // 128, n), generator=gen).abs() * 0.01 + 1e-3).half()
    da = torch.randn((m, k), generator=gen).half()

    def dump(name, array):
        (tmp_path / name).write_bytes(np.ascontiguousarray(array).tobytes())

    dump("w13_gptq.bin", g13), dump("w2_gptq.bin", g2)
    dump("s13.bin", s13.view(torch.int16).numpy()), dump("s2.bin", s2.view(torch.int16).numpy())
    dump("x.bin", x.view(torch.int16).numpy()), dump("topk_ids.bin", ids.to(torch.int32).numpy())
    dump("topk_weights.bin", tw.flatten().numpy())
    dump("dense_a.bin", da.view(torch.int16).numpy()), dump("dense_w.bin", oq.marlin_pack(dq, 4, False))
    dump("dense_s.bin", ds.view(torch.int16).numpy())

    proc = subprocess.run([str(binary), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr + proc.stdout
    assert "active slots: 1" in proc.stdout

    def load(name, dtype, shape):
        raw = np.frombuffer((tmp_path / name).read_bytes(), dtype=np.int16 if dtype in (torch.bfloat16, torch.float16) else dtype)
        t = torch.from_numpy(raw.copy())
        return (t.view(dtype) if dtype in (torch.bfloat16, torch.float16) else t).reshape(shape)

    marlin13 = load("w13_marlin.bin", np.int32, (EXPERTS, HIDDEN // 16, 4 * INTER)).numpy()
    assert all(np.array_equal(marlin13[e], oq.marlin_pack(q13[e], 4, False)) for e in range(EXPERTS))
    rs, re, rn = omoe.moe_align_block_size(ids.to(torch.int32), None, EXPERTS, BLOCK)
    assert np.array_equal(load("sorted.bin", np.int32, (-1,)).numpy(), rs)

    def close(got, ref, tol=1e-2):
        return float((got.float() - ref.float()).abs().max() / ref.float().abs().max()) <= tol

    g = load("g.bin", torch.bfloat16, (TOKENS * TOP_K, 2 * INTER))
    assert close(g, omoe.moe_w4a16_gemm(x, q13, s13, None, rs, re, rn, None, BLOCK, TOP_K, False))
    h = load("h.bin", torch.bfloat16, (TOKENS * TOP_K, INTER))
    torch.testing.assert_close(h, omoe.silu_and_mul(g), rtol=1e-2, atol=5e-3)
    y = load("y.bin", torch.bfloat16, (TOKENS * TOP_K, HIDDEN))
    assert close(y, omoe.moe_w4a16_gemm(h, q2, s2, None, rs, re, rn, tw.flatten(), BLOCK, 1, True))
    out = load("out.bin", torch.bfloat16, (TOKENS, HIDDEN))
    torch.testing.assert_close(out, omoe.moe_sum(y.view(TOKENS, TOP_K, HIDDEN)), rtol=1e-2, atol=1e-2)
    dense = load("dense_out.bin", torch.float16, (m, n))
    assert close(dense, oq.w4a16_gemm(da, dq, ds, None))
