"""GPU: scales and zero points in the layouts vLLM's Marlin kernels take (what a checkpoint prepared
for the reference's linked provider holds), dense and routed, through the C ABI (`scale_layout = 1`)
and through `infini.ops` at the provider slot (`implementation_index = 16`).

The provider layouts are produced by the installed vLLM's own helpers (`marlin_permute_scales`,
`marlin_zero_points`), imported here and not restated; the result must equal, bit for bit, what the
plain layouts give, and match the oracle."""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import quant as oq
from tests.helpers import make_quantized, rel_max_err

pytestmark = pytest.mark.gpu
UINT4B8, UINT4 = 1125899907892224, 1125899906843648


def _vllm_layouts():
    utils = pytest.importorskip("vllm.model_executor.layers.quantization.utils.marlin_utils")
    return utils.marlin_permute_scales, utils.marlin_zero_points


def _provider(scales, zeros, k, n, group):
    permute_scales, marlin_zeros = _vllm_layouts()
    s = permute_scales(scales.clone(), k, n, group)
    z = None if zeros is None else marlin_zeros(torch.from_numpy(zeros.astype(np.int32)), zeros.shape[0], n, 4)
    return s.contiguous(), None if z is None else z.contiguous()


@pytest.mark.parametrize("m,k,n,group,dtype,zeros", (
    (16, 1024, 512, 128, torch.bfloat16, True),    # late-scale tiles
    (1, 512, 192, 128, torch.float16, False),      # ragged last tile (64 columns)
    (64, 256, 9728, 64, torch.bfloat16, True),     # group 64: scales applied to the weights, two rows per stage
    (100, 512, 320, 128, torch.float16, True),     # 128-token tiles
    (300, 512, 512, 128, torch.bfloat16, True),    # paired blocks
    (16, 1024, 256, -1, torch.float16, False),     # one group: the 32-column permutation
))
def test_dense_provider_layout_equals_plain(m, k, n, group, dtype, zeros):
    from infiniops_b200 import capi

    q, scales, z = make_quantized(k, n, group, dtype, zeros, m + k + n)
    a = torch.randn((m, k)).to(dtype).cuda()
    marlin = torch.from_numpy(oq.marlin_pack(q, 4, False)).cuda()
    ps, pz = _provider(scales, z, k, n, group)
    scratch = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n, k), dtype=torch.uint8, device="cuda")
    qtype = UINT4 if zeros else UINT4B8
    outs = []
    for layout, s_t, z_t in ((0, scales, None if z is None else torch.from_numpy(oq.pack_zeros(z))), (1, ps, pz)):
        out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        g = capi.gemm_problem(a, marlin, None, s_t.cuda(), None if z_t is None else z_t.cuda(), out, m, n, k,
                              scale_layout=layout)
        capi.marlin_gemm_placed(g, dtype, qtype, scratch)
        torch.cuda.synchronize()
        assert capi.scratch_status(scratch) == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    assert rel_max_err(outs[1], oq.w4a16_gemm(a.cpu(), q, scales, z)) <= 1e-2


@pytest.mark.parametrize("zeros", (False, True))
def test_routed_provider_layout_through_the_provider_slot(zeros):
    import infini.ops

    assert list(infini.ops.MoeWna16MarlinGemm.active_implementation_indices("cuda")) == [0, 16]
    assert list(infini.ops.MarlinGemm.active_implementation_indices("cuda")) == [0, 16]
    assert list(infini.ops.MoeSum.active_implementation_indices("cuda")) == [0]
    tokens, experts, top_k, k, n, block = 90, 8, 2, 512, 384, 16
    dtype = torch.bfloat16
    q = np.empty((experts, k, n), dtype=np.uint8)
    scales = torch.empty((experts, k // 128, n), dtype=dtype)
    z = np.empty((experts, k // 128, n), dtype=np.uint8) if zeros else None
    ps = torch.empty_like(scales)
    pz = torch.empty((experts, k // 128, n // 8), dtype=torch.int32) if zeros else None
    packed = torch.empty((experts, k // 16, 2 * n), dtype=torch.int32)
    for e in range(experts):
        qe, se, ze = make_quantized(k, n, 128, dtype, zeros, 300 + e)
        q[e], scales[e], packed[e] = qe, se, torch.from_numpy(oq.marlin_pack(qe, 4, False))
        pse, pze = _provider(se, ze, k, n, 128)
        ps[e] = pse
        if zeros:
            z[e], pz[e] = ze, pze
    x = torch.randn((tokens, k)).to(dtype)
    ids = torch.randint(0, experts, (tokens, top_k), dtype=torch.int32)
    tw = torch.rand(tokens * top_k)
    rs, re, rn = omoe.moe_align_block_size(ids, None, experts, block)
    out = torch.full((tokens * top_k, n), float("nan"), dtype=dtype, device="cuda")
    workspace = torch.zeros(432, dtype=torch.int32, device="cuda")
    infini.ops.moe_wna16_marlin_gemm(x.cuda(), packed.cuda(), None, ps.cuda(), None, None, None if pz is None else pz.cuda(),
                                     None, None, workspace, torch.from_numpy(rs).cuda(), torch.from_numpy(re).cuda(),
                                     torch.from_numpy(rn).cuda(), tw.cuda(), block, top_k, True, UINT4 if zeros else UINT4B8,
                                     tokens, n, k, True, False, True, False, -1, -1, -1, out,
                                     stream=torch.cuda.current_stream().cuda_stream, implementation_index=16)
    ref = omoe.moe_w4a16_gemm(x, q, scales, z, rs, re, rn, tw, block, top_k, True)
    assert rel_max_err(out, ref) <= 1e-2
