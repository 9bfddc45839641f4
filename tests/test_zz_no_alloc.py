"""GPU: the allocation-free GEMM entry point against the ordinary one.

`infiniops_b200_marlin_gemm_static_scratch` exists for hosts that cannot give the GEMM a scratch
buffer -- an engine whose memory arena already owns the device, or a caller that runs only while
work is being recorded and may not call cudaMalloc.  It keeps its split-K scratch in an array
inside the library.  Called through the C ABI twice in a row (the second call finds what the
first left in the shared array), it must give what the caller-scratch entry point gives; both
sum their partials in a fixed order, so the comparison is exact, within the GEMM tests' 1e-2
tolerance a fortiori.  This file sorts last so a run that stops at the first failure has
already run everything else; it also passes on its own in a fresh process.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(m, k, n, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    marlin = torch.randint(-2**31, 2**31 - 1, (k // 16, 2 * n), dtype=torch.int32, device="cuda", generator=gen)
    scales = (torch.randn((k // 128, n), device="cuda", generator=gen).abs() * 0.01 + 1e-3).bfloat16()
    zeros = torch.randint(-2**31, 2**31 - 1, (k // 128, n // 8), dtype=torch.int32, device="cuda", generator=gen)
    a = torch.randn((m, k), device="cuda", generator=gen).bfloat16()
    return a, marlin, scales, zeros


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    from infiniops_b200 import capi

    for call, (m, k, n) in enumerate(((16, 4096, 4096), (64, 2048, 6144))):
        a, marlin, scales, zeros = _problem(m, k, n, 11 + call)
        expect = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        capi.marlin_gemm(a, marlin, None, scales, zeros, capi.QTYPE_UINT4, m, n, k, expect)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]   # the driver's view: sees a cudaMalloc torch would not
        capi.marlin_gemm_static_scratch(a, marlin, None, scales, zeros, capi.QTYPE_UINT4, m, n, k, got)
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        # (the first call on a device may load the kernel's module lazily; later calls may not move it)
        if call > 0:
            assert torch.cuda.mem_get_info()[0] == free_before
        assert capi.lib().infiniops_b200_static_scratch_status(None) == 0
        assert not torch.isnan(got.float()).any()
        scale = float(expect.float().abs().max())
        assert float((got.float() - expect.float()).abs().max()) <= 1e-2 * scale
        assert torch.equal(got, expect), f"call {call}: results differ from the caller-scratch entry point"


def test_static_scratch_rejects_problems_beyond_its_capacity():
    from infiniops_b200 import capi

    # the limit itself on a 148-SM GPU: 64 rows fit, 65 do not
    lib = capi.lib()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if sms == 148:
        assert lib.infiniops_b200_marlin_gemm_scratch_bytes(64, 128, 256) <= (10 << 20)
        assert lib.infiniops_b200_marlin_gemm_scratch_bytes(65, 128, 256) > (10 << 20)
        a, marlin, scales, zeros = _problem(65, 256, 128, 4)
        with pytest.raises(capi.Error, match="built-in buffer holds"):
            capi.marlin_gemm_static_scratch(a, marlin, None, scales, zeros, capi.QTYPE_UINT4, 65, 128, 256,
                                            torch.empty((65, 128), dtype=torch.bfloat16, device="cuda"))
    m, k, n = 4096, 256, 128
    a, marlin, scales, zeros = _problem(m, k, n, 3)
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    assert capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n, k) > (10 << 20)
    with pytest.raises(capi.Error, match="built-in buffer holds"):
        capi.marlin_gemm_static_scratch(a, marlin, None, scales, zeros, capi.QTYPE_UINT4, m, n, k, out)
