"""GPU: 8-bit weights (`uint8b128`, w = (q - 128) * s) in the dense and the routed Marlin GEMM.

The weights go the reference's way -- GPTQ-packed [K/4, N] words through `gptq_marlin_repack`
(num_bits = 8), bit-exact against the oracle's Marlin packing -- and the products are compared with the
oracle's dequantise-then-matmul.  Tolerance as for the 4-bit GEMMs: max |got - ref| <= 1e-2 max |ref|.
"""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import quant as oq
from tests.helpers import rel_max_err

pytestmark = pytest.mark.gpu
TOL = 1e-2
UINT8B128 = 1125899923621888
UINT8 = 1125899906844672


def _pack_zeros8(zeros: np.ndarray) -> np.ndarray:
    """[G, N] bytes -> int32 [G, N/4]: byte n % 4 of word n / 4 (little endian), the 8-bit form of the
    reference's zero-point packing (pack factor 4, src/base/moe_wna16_marlin_gemm.h:231-240)."""
    return np.ascontiguousarray(zeros.astype(np.uint8)).view(np.int32)


def _weights(k, n, group, dtype, seed):
    from infiniops_b200 import capi

    gen = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 256, (k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
    groups = 1 if group in (-1, k) else k // group
    scales = (torch.randn((groups, n), generator=gen).abs() * 0.002 + 2e-4).to(dtype)
    packed = torch.from_numpy(oq.gptq_pack(q, 8)).cuda()
    marlin = torch.empty((k // 16, 4 * n), dtype=torch.int32, device="cuda")
    capi.gptq_marlin_repack(packed, None, k, n, 8, False, marlin)
    assert np.array_equal(marlin.cpu().numpy(), oq.marlin_pack(q, 8, False))
    return q, scales, marlin


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("m,k,n,group", ((1, 512, 256, 128), (16, 1024, 320, 128), (48, 512, 128, 64), (100, 768, 256, 128),
                                         (300, 512, 384, 256), (7, 256, 64, -1)))
def test_dense_gemm_with_8bit_weights(dtype, m, k, n, group):
    from infiniops_b200 import capi

    q, scales, marlin = _weights(k, n, group, dtype, 8000 + m + n)
    a = torch.randn((m, k), generator=torch.Generator().manual_seed(m)).to(dtype)
    bias = (torch.randn(n, generator=torch.Generator().manual_seed(n)) * 0.1).to(dtype)
    out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    capi.marlin_gemm(a.cuda(), marlin, bias.cuda(), scales.cuda(), None, UINT8B128, m, n, k, out)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    ref = a.float() @ oq.dequantize(q, scales, None, 8) + bias.float()
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, ref) <= TOL


@pytest.mark.parametrize("block,top_k,mul", ((16, 2, True), (64, 2, False), (128, 1, True)))
def test_routed_gemm_with_8bit_weights(block, top_k, mul):
    from infiniops_b200 import capi

    tokens, experts, k, n, dtype = 90, 4, 512, 256, torch.bfloat16
    qs, ss, ws = zip(*[_weights(k, n, 128, dtype, 8100 + e) for e in range(experts)])
    words, scales = torch.stack(ws), torch.stack(ss).cuda()
    gen = torch.Generator().manual_seed(block)
    ids = torch.randint(0, experts, (tokens, top_k), generator=gen, dtype=torch.int32)
    x = torch.randn((tokens, k), generator=gen).to(dtype)
    tw = torch.rand(tokens * top_k, generator=gen)
    rows = tokens * top_k
    size, blocks = omoe.padded_sizes(rows, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids.cuda(), None, experts, block, sorted_ids, expert_ids, npost)
    out = torch.full((rows, n), float("nan"), dtype=dtype, device="cuda")
    capi.moe_wna16_marlin_gemm(x.cuda(), words, None, scales, None, sorted_ids, expert_ids, npost, tw.cuda(), block, top_k,
                               mul, UINT8B128, tokens, n, k, out)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    ref = torch.zeros((rows, n))
    for t in range(tokens):
        for j in range(top_k):
            e = int(ids[t, j])
            r = x[t].float() @ oq.dequantize(qs[e], ss[e], None, 8)
            ref[t * top_k + j] = r * tw[t * top_k + j] if mul else r
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, ref) <= TOL


def test_8bit_weights_refuse_what_is_not_built():
    from infiniops_b200 import capi

    k, n, m = 256, 128, 4
    q, scales, marlin = _weights(k, n, 128, torch.bfloat16, 1)
    a = torch.randn((m, k), device="cuda").bfloat16()
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    zeros = torch.zeros((k // 128, n // 8), dtype=torch.int32, device="cuda")
    with pytest.raises(capi.Error, match="zero points"):
        capi.marlin_gemm(a, marlin, None, scales.cuda(), zeros, UINT8B128, m, n, k, out)
    g = capi.gemm_problem(a, marlin, None, scales.cuda(), None, out, m, n, k)
    buf = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes(), dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.Error, match="4-bit weights only"):
        capi.marlin_gemm_batch(capi.problem_array([g]), torch.bfloat16, UINT8B128, buf)


def test_8bit_weights_through_the_operator_api():
    """`infini.ops.moe_wna16_marlin_gemm` and `infini.ops.marlin_gemm` with `b_type_id` uint8b128."""
    import infini.ops

    tokens, experts, top_k, k, n, block, dtype = 40, 4, 2, 256, 128, 16, torch.float16
    qs, ss, ws = zip(*[_weights(k, n, 128, dtype, 8200 + e) for e in range(experts)])
    words, scales = torch.stack(ws), torch.stack(ss).cuda()
    gen = torch.Generator().manual_seed(9)
    ids = torch.randint(0, experts, (tokens, top_k), generator=gen, dtype=torch.int32).cuda()
    x = torch.randn((tokens, k), generator=gen).to(dtype)
    rows = tokens * top_k
    size, blocks = omoe.padded_sizes(rows, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    infini.ops.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost, stream=stream)
    tw = torch.ones(rows, dtype=torch.float32, device="cuda")
    out = torch.full((rows, n), float("nan"), dtype=dtype, device="cuda")
    workspace = torch.zeros(432, dtype=torch.int32, device="cuda")
    infini.ops.moe_wna16_marlin_gemm(x.cuda(), words, None, scales, None, None, None, None, None, workspace, sorted_ids,
                                     expert_ids, npost, tw, block, top_k, False, UINT8B128, tokens, n, k, True, False, True,
                                     False, -1, -1, -1, out, stream=stream)
    torch.cuda.synchronize()
    ids_cpu = ids.cpu()
    ref = torch.stack([x[t].float() @ oq.dequantize(qs[int(ids_cpu[t, j])], ss[int(ids_cpu[t, j])], None, 8)
                       for t in range(tokens) for j in range(top_k)])
    assert rel_max_err(out, ref) <= TOL

    dense_out = torch.full((tokens, n), float("nan"), dtype=dtype, device="cuda")
    infini.ops.marlin_gemm(x.cuda(), words[0], None, scales[0], None, None, None, None, None, workspace, UINT8B128,
                           tokens, n, k, True, False, True, False, dense_out, stream=stream)
    torch.cuda.synchronize()
    assert rel_max_err(dense_out, x.float() @ oq.dequantize(qs[0], ss[0], None, 8)) <= TOL


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("m,k,n,group", ((3, 512, 256, 128), (40, 1024, 320, 128), (100, 512, 128, 64)))
def test_dense_gemm_with_8bit_weights_and_zero_points(dtype, m, k, n, group):
    from infiniops_b200 import capi

    q, scales, marlin = _weights(k, n, group, dtype, 8300 + m)
    zeros = torch.randint(0, 256, (k // group, n), generator=torch.Generator().manual_seed(m + 1), dtype=torch.int32) \
        .numpy().astype(np.uint8)
    a = torch.randn((m, k), generator=torch.Generator().manual_seed(m)).to(dtype)
    out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    capi.marlin_gemm(a.cuda(), marlin, None, scales.cuda(), torch.from_numpy(_pack_zeros8(zeros)).cuda(), UINT8, m, n, k, out)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    ref = a.float() @ oq.dequantize(q, scales, zeros, 8)
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, ref) <= TOL


def test_routed_gemm_with_8bit_weights_and_zero_points():
    from infiniops_b200 import capi

    tokens, experts, top_k, k, n, block, dtype = 70, 4, 2, 512, 256, 32, torch.bfloat16
    qs, ss, ws = zip(*[_weights(k, n, 128, dtype, 8400 + e) for e in range(experts)])
    gen = torch.Generator().manual_seed(12)
    zs = [torch.randint(0, 256, (k // 128, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8) for _ in range(experts)]
    words, scales = torch.stack(ws), torch.stack(ss).cuda()
    zp = torch.stack([torch.from_numpy(_pack_zeros8(z)) for z in zs]).cuda()
    ids = torch.randint(0, experts, (tokens, top_k), generator=gen, dtype=torch.int32)
    x = torch.randn((tokens, k), generator=gen).to(dtype)
    tw = torch.rand(tokens * top_k, generator=gen)
    rows = tokens * top_k
    size, blocks = omoe.padded_sizes(rows, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids.cuda(), None, experts, block, sorted_ids, expert_ids, npost)
    out = torch.full((rows, n), float("nan"), dtype=dtype, device="cuda")
    capi.moe_wna16_marlin_gemm(x.cuda(), words, None, scales, zp, sorted_ids, expert_ids, npost, tw.cuda(), block, top_k,
                               True, UINT8, tokens, n, k, out)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    ref = torch.zeros((rows, n))
    for t in range(tokens):
        for j in range(top_k):
            e = int(ids[t, j])
            ref[t * top_k + j] = (x[t].float() @ oq.dequantize(qs[e], ss[e], zs[e], 8)) * tw[t * top_k + j]
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, ref) <= TOL
