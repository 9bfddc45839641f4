"""GPU: float8_e4m3fn weights (w = float8(byte) * s) in the dense and the routed Marlin GEMM.

The bytes travel as 8-bit weights do -- GPTQ-packed [K/4, N] words through `gptq_marlin_repack`
(num_bits = 8) -- and the products are compared with dequantise-then-matmul, the bytes read as
`torch.float8_e4m3fn` on the CPU.  Every byte value except the type's two NaN patterns is used, the
subnormal ones included.  Tolerance as for the other GEMMs: max |got - ref| <= 1e-2 max |ref|.
"""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import quant as oq
from tests.helpers import rel_max_err

pytestmark = pytest.mark.gpu
TOL = 1e-2
FLOAT8_E4M3FN = 2814749767172868


def _weights(k, n, group, dtype, seed):
    from infiniops_b200 import capi

    gen = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 256, (k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
    q[(q & 0x7F) == 0x7F] = 0x38   # the two NaN bytes become 1.0
    groups = 1 if group in (-1, k) else k // group
    scales = (torch.randn((groups, n), generator=gen).abs() * 0.02 + 2e-3).to(dtype)
    packed = torch.from_numpy(oq.gptq_pack(q, 8)).cuda()
    marlin = torch.empty((k // 16, 4 * n), dtype=torch.int32, device="cuda")
    capi.gptq_marlin_repack(packed, None, k, n, 8, False, marlin)
    return oq.dequantize_float8(q, scales), scales, marlin


def test_every_byte_value_converts_exactly():
    """K = 256 rows hold the 254 finite byte values once per column block; unit scale and a one-hot
    activation row read each weight back alone, so the comparison is exact."""
    from infiniops_b200 import capi

    k, n = 256, 64
    for dtype in (torch.float16, torch.bfloat16):
        q = np.repeat(np.arange(256, dtype=np.uint8)[:, None], n, axis=1)
        q[(q & 0x7F) == 0x7F] = 0
        packed = torch.from_numpy(oq.gptq_pack(q, 8)).cuda()
        marlin = torch.empty((k // 16, 4 * n), dtype=torch.int32, device="cuda")
        capi.gptq_marlin_repack(packed, None, k, n, 8, False, marlin)
        scales = torch.ones((2, n), dtype=dtype, device="cuda")
        a = torch.eye(k, dtype=dtype, device="cuda")
        out = torch.full((k, n), float("nan"), dtype=dtype, device="cuda")
        capi.marlin_gemm(a, marlin, None, scales, None, FLOAT8_E4M3FN, k, n, k, out)
        torch.cuda.synchronize()
        want = oq.dequantize_float8(q, torch.ones((1, n)))
        assert torch.equal(out.float().cpu(), want.to(dtype).float())


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("m,k,n,group", ((1, 512, 256, 128), (16, 1024, 320, 128), (48, 512, 128, 64), (100, 768, 256, 128),
                                         (300, 512, 384, 256), (7, 256, 64, -1)))
def test_dense_gemm_with_float8_weights(dtype, m, k, n, group):
    from infiniops_b200 import capi

    dense, scales, marlin = _weights(k, n, group, dtype, 9000 + m + n)
    a = torch.randn((m, k), generator=torch.Generator().manual_seed(m)).to(dtype)
    out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    capi.marlin_gemm(a.cuda(), marlin, None, scales.cuda(), None, FLOAT8_E4M3FN, m, n, k, out)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, a.float() @ dense) <= TOL


@pytest.mark.parametrize("block,top_k,mul", ((16, 2, True), (64, 2, False), (128, 1, True)))
def test_routed_gemm_with_float8_weights(block, top_k, mul):
    from infiniops_b200 import capi

    tokens, experts, k, n, dtype = 90, 4, 512, 256, torch.bfloat16
    ds, ss, ws = zip(*[_weights(k, n, 128, dtype, 9100 + e) for e in range(experts)])
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
                               mul, FLOAT8_E4M3FN, tokens, n, k, out)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    ref = torch.zeros((rows, n))
    for t in range(tokens):
        for j in range(top_k):
            r = x[t].float() @ ds[int(ids[t, j])]
            ref[t * top_k + j] = r * tw[t * top_k + j] if mul else r
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, ref) <= TOL


def test_float8_weights_through_the_operator_api_and_refusals():
    import infini.ops

    from infiniops_b200 import capi

    m, k, n, dtype = 24, 512, 256, torch.float16
    dense, scales, marlin = _weights(k, n, 128, dtype, 9300)
    a = torch.randn((m, k), generator=torch.Generator().manual_seed(4)).to(dtype)
    out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    workspace = torch.zeros(432, dtype=torch.int32, device="cuda")
    infini.ops.marlin_gemm(a.cuda(), marlin, None, scales.cuda(), None, None, None, None, None, workspace, FLOAT8_E4M3FN,
                           m, n, k, True, False, True, False, out, stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rel_max_err(out, a.float() @ dense) <= TOL
    zeros = torch.zeros((k // 128, n // 4), dtype=torch.int32, device="cuda")
    with pytest.raises(capi.Error, match="zero points"):
        capi.marlin_gemm(a.cuda(), marlin, None, scales.cuda(), zeros, FLOAT8_E4M3FN, m, n, k, out)
    g = capi.gemm_problem(a.cuda(), marlin, None, scales.cuda(), None, out, m, n, k, scale_layout=1)
    buf = capi.scratch("cuda", capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n, k))
    with pytest.raises(capi.Error, match="plain layout only"):
        capi.marlin_gemm_placed(g, dtype, FLOAT8_E4M3FN, buf)
