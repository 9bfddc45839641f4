"""GPU: dense W4A16 GEMM through the C ABI against the dequantise-then-matmul oracle.

Tolerance (stated by the benchmark definition): max |got - ref| <= 1e-2 * max |ref|, with
`ref` accumulated in fp32 from the fp32-dequantised weights."""

import numpy as np
import pytest
import torch

from oracle import quant as oq
from tests.helpers import make_quantized, rel_max_err, to_device_weights

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _gemm(a, q, scales, zeros, source, bias=None):
    from infiniops_b200 import capi

    k, n = q.shape
    packed, scales_d, zeros_d = to_device_weights(q, scales, zeros, source)
    marlin = torch.empty((k // 16, 2 * n), dtype=torch.int32, device="cuda")
    if source == "gptq":
        capi.gptq_marlin_repack(packed, None, k, n, 4, False, marlin)
    else:
        capi.awq_marlin_repack(packed, k, n, 4, False, marlin)
    assert np.array_equal(marlin.cpu().numpy(), oq.marlin_pack(q, 4, False))
    out = torch.full((a.shape[0], n), float("nan"), dtype=a.dtype, device="cuda")
    qtype = capi.QTYPE_UINT4 if zeros is not None else capi.QTYPE_UINT4B8
    capi.marlin_gemm(a.cuda(), marlin, None if bias is None else bias.cuda(), scales_d, zeros_d, qtype,
                     a.shape[0], n, k, out)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    return out


def test_config1_gptq_fp16_m16():
    """Dense GPTQ W4A16, fp16 activations [16, 4096], weights [4096, 4096], group 128, zero point 8."""
    q, scales, _ = make_quantized(4096, 4096, 128, torch.float16, False, 20260728)
    a = torch.randn((16, 4096), generator=torch.Generator().manual_seed(1)).half()
    out = _gemm(a, q, scales, None, "gptq")
    assert rel_max_err(out, oq.w4a16_gemm(a, q, scales, None)) <= TOL


@pytest.mark.parametrize("m", (1, 4, 16, 64))
@pytest.mark.parametrize("k,n", ((4096, 6144), (4096, 4096), (14336, 4096)))
def test_config2_awq_bf16_decode(m, k, n):
    q, scales, zeros = make_quantized(k, n, 128, torch.bfloat16, True, k + n + m)
    a = torch.randn((m, k)).bfloat16()
    out = _gemm(a, q, scales, zeros, "awq")
    assert rel_max_err(out, oq.w4a16_gemm(a, q, scales, zeros)) <= TOL


def test_config2_gate_up_shape():
    q, scales, zeros = make_quantized(4096, 28672, 128, torch.bfloat16, True, 5)
    a = torch.randn((16, 4096)).bfloat16()
    out = _gemm(a, q, scales, zeros, "awq")
    assert rel_max_err(out, oq.w4a16_gemm(a, q, scales, zeros)) <= TOL


@pytest.mark.parametrize("m,k,n,group,dtype,zeros", (
    (3, 128, 64, 64, torch.float16, False),     # one k stage, half-width tile, two groups in it
    (17, 128, 192, 128, torch.bfloat16, True),  # ragged tile in n, token tile 32
    (100, 256, 320, 64, torch.float16, True),   # token tile 128, group size 64
    (130, 512, 128, -1, torch.bfloat16, False), # per-channel scales, token tile 256, ragged rows
    (300, 1024, 256, 128, torch.bfloat16, True),  # two token tiles
    (513, 640, 768, 128, torch.float16, True),   # three 256-column tile pairs, ragged rows in the last token tile
    (257, 256, 384, 128, torch.bfloat16, False), # 256-token tiles whose columns do not pair up
    (48, 256, 9728, 128, torch.float16, True),   # 64-row late-scale tiles (too many column tiles for two 32-row ones), float16
    (40, 384, 192, 128, torch.bfloat16, True),   # 33..64 rows as two 32-row tiles
    (64, 256, 9728, 64, torch.bfloat16, True),   # 64-row tiles, group 64: scaled-weight path
    (700, 384, 512, 64, torch.float16, False),   # paired blocks, group 64, three token tiles (last ragged)
    (64, 8192, 64, 128, torch.float16, False),  # one tile shared by many blocks along k
))
def test_edge_shapes(m, k, n, group, dtype, zeros):
    q, scales, z = make_quantized(k, n, group, dtype, zeros, m * 13 + k)
    a = torch.randn((m, k)).to(dtype)
    bias = torch.randn(n).to(dtype)
    out = _gemm(a, q, scales, z, "awq" if zeros else "gptq", bias=bias)
    assert rel_max_err(out, oq.w4a16_gemm(a, q, scales, z, bias=bias)) <= TOL


def test_prefill_tile_and_linearity():
    """M = 4096 (the compute-bound regime) on one Llama-shaped matrix, checked against the oracle on
    a slice of rows and through linearity, C(a1 + a2) = C(a1) + C(a2), on all of them."""
    k, n, m = 4096, 4096, 4096
    q, scales, _ = make_quantized(k, n, 128, torch.bfloat16, False, 99)
    a1 = torch.randn((m, k)).bfloat16()
    out1 = _gemm(a1, q, scales, None, "gptq")
    ref = oq.w4a16_gemm(a1[:256], q, scales, None)
    assert rel_max_err(out1[:256], ref) <= TOL
    ref_tail = oq.w4a16_gemm(a1[-64:], q, scales, None)
    assert rel_max_err(out1[-64:], ref_tail) <= TOL
    # exact linearity in the activations: scaling by 2 is exact in bf16 and fp32
    out2 = _gemm(a1 * 2, q, scales, None, "gptq")
    assert torch.equal(out2.float(), out1.float() * 2)


def test_repeatable_and_scratch_left_clean():
    from infiniops_b200 import capi

    q, scales, zeros = make_quantized(4096, 4096, 128, torch.bfloat16, True, 3)
    a = torch.randn((16, 4096)).bfloat16()
    first = _gemm(a, q, scales, zeros, "awq")
    for _ in range(3):
        assert torch.equal(_gemm(a, q, scales, zeros, "awq"), first)
    buf = capi.scratch("cuda", 0)
    need = capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(16, 4096, 4096)
    header = buf[:256 + 4 * 4 * 1024].view(torch.int32)  # status word and arrival counters
    assert int(header.abs().sum()) == 0 and need <= buf.numel()


def test_rejects_unsupported():
    from infiniops_b200 import capi

    a = torch.zeros((4, 128), dtype=torch.float16, device="cuda")
    w = torch.zeros((8, 128), dtype=torch.int32, device="cuda")
    s = torch.zeros((1, 64), dtype=torch.float16, device="cuda")
    out = torch.zeros((4, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(capi.Error, match="only the weight types"):
        capi.marlin_gemm(a, w, None, s, None, 1125899906908928, 4, 64, 128, out)   # int4 (signed)
    with pytest.raises(capi.Error, match="zero points are required"):
        capi.marlin_gemm(a, w, None, s, None, capi.QTYPE_UINT4, 4, 64, 128, out)


def test_bounded_wait_gives_up_and_reports():
    """The bounded device-side wait in isolation: a stand-alone kernel (no copies, no tensor cores)
    whose one waiting thread polls a barrier nobody arrives at.  It must give up after its poll
    limit, leave (code 7, block 0, thread 0, detail 42) in the status header, end normally and
    leave the context usable."""
    from infiniops_b200 import capi

    scratch = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    result = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    rc = capi.lib().infiniops_b200_selftest_bounded_wait(scratch.data_ptr(), scratch.numel(), result.data_ptr(), None)
    assert rc == 0, capi.lib().infiniops_b200_last_error()
    torch.cuda.synchronize()
    assert result.tolist() == [0, 1]
    assert capi.scratch_status(scratch) == 7
    assert scratch[:16].view(torch.int32).tolist() == [7, 0, 0, 42]
    # memory of unknown content becomes usable scratch again through the prepare call
    scratch.fill_(0xFF)
    assert capi.lib().infiniops_b200_gemm_scratch_prepare(scratch.data_ptr(), scratch.numel(), None) == 0
    assert capi.scratch_status(scratch) == 0
    q, scales, zeros = make_quantized(512, 256, 128, torch.bfloat16, True, 21)
    a = torch.randn((16, 512)).bfloat16()
    assert rel_max_err(_gemm(a, q, scales, zeros, "awq"), oq.w4a16_gemm(a, q, scales, zeros)) <= TOL


def test_scratch_of_unknown_content_after_prepare():
    """A split-K problem (one column tile, 64 k-stages over many blocks) on a scratch buffer that
    was filled with 0xFF and then prepared: the arrival counters must work from the first call."""
    from infiniops_b200 import capi

    m, k, n = 16, 8192, 128
    q, scales, _ = make_quantized(k, n, 128, torch.float16, False, 31)
    a = torch.randn((m, k)).half()
    marlin = torch.from_numpy(oq.marlin_pack(q, 4, False)).cuda()
    need = capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n, k)
    scratch = torch.full((need,), 0xFF, dtype=torch.uint8, device="cuda")
    assert capi.lib().infiniops_b200_gemm_scratch_prepare(scratch.data_ptr(), scratch.numel(), None) == 0
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    capi.marlin_gemm(a.cuda(), marlin, None, scales.cuda(), None, capi.QTYPE_UINT4B8, m, n, k, out, scratch_buf=scratch)
    torch.cuda.synchronize()
    assert capi.scratch_status(scratch) == 0
    assert rel_max_err(out, oq.w4a16_gemm(a, q, scales, None)) <= TOL
