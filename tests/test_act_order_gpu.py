"""GPU: activation order (`g_idx` / `perm`) in the routed and the dense Marlin GEMM.

A GPTQ act-order checkpoint stores, per expert, weights [K, N] whose row k belongs to scale group
g_idx[k] (groups scattered over the rows).  The provider's preparation sorts the rows by group --
`perm = argsort(g_idx)`, weights repacked in that row order (gptq_marlin_repack's `perm`), `g_idx`
sorted -- and the GEMM reads activation column perm[k] against weight row k.  The oracle is the plain
definition on the UNSORTED tensors: out = a @ ((q - 8) * scales[g_idx]).
"""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import quant as oq
from tests.helpers import rel_max_err

pytestmark = pytest.mark.gpu
TOL = 1e-2
GROUP = 128


def _act_order_experts(experts, k, n, seed):
    """Per expert: unsorted q [K, N], scattered g_idx [K], scales [G, N]; and what the device takes:
    Marlin words of the rows in sorted order, perm, sorted g_idx."""
    from infiniops_b200 import capi

    gen = torch.Generator().manual_seed(seed)
    groups = k // GROUP
    qs, gs, ss, words, perms, sorted_g = [], [], [], [], [], []
    for _ in range(experts):
        q = torch.randint(0, 16, (k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
        g_idx = (torch.arange(k) // GROUP)[torch.randperm(k, generator=gen)].to(torch.int32)
        scales = (torch.randn((groups, n), generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        perm = torch.argsort(g_idx.long(), stable=True).to(torch.int32)
        packed = torch.from_numpy(oq.gptq_pack(q, 4)).cuda()
        marlin = torch.empty((k // 16, 2 * n), dtype=torch.int32, device="cuda")
        capi.gptq_marlin_repack(packed, perm.cuda(), k, n, 4, False, marlin)
        qs.append(q), gs.append(g_idx), ss.append(scales), words.append(marlin), perms.append(perm)
        sorted_g.append(g_idx[perm.long()])
    return (qs, gs, ss, torch.stack(words), torch.stack(ss).cuda(), torch.stack(perms).cuda(),
            torch.stack(sorted_g).cuda().contiguous())


def _dequant_scattered(q, g_idx, scales):
    return (torch.from_numpy(q.astype(np.float32)) - 8.0) * scales.float()[g_idx.long()]


@pytest.mark.parametrize("block,a_sorted", ((16, False), (64, False), (128, False), (64, True)))
def test_routed_gemm_with_activation_order(block, a_sorted):
    from infiniops_b200 import capi

    tokens, experts, top_k, k, n = 70, 4, 2, 512, 256
    qs, gs, ss, words, scales, perm, g_sorted = _act_order_experts(experts, k, n, 900 + block)
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, experts, (tokens, top_k), generator=gen, dtype=torch.int32)
    x = torch.randn((tokens, k), generator=gen).bfloat16()
    tw = torch.rand((tokens, top_k), generator=gen).reshape(-1)
    rows = tokens * top_k
    size, blocks = omoe.padded_sizes(rows, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids.cuda(), None, experts, block, sorted_ids, expert_ids, npost)

    ref = torch.zeros((rows, n))
    for t in range(tokens):
        for j in range(top_k):
            e = int(ids[t, j])
            ref[t * top_k + j] = (x[t].float() @ _dequant_scattered(qs[e], gs[e], ss[e])) * tw[t * top_k + j]
    out = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    if a_sorted:
        # the activations given in sorted order, one row per entry of `sorted_ids` (top_k = 1 form)
        srt = sorted_ids.cpu().long()
        a_rows = torch.zeros((size, k), dtype=torch.bfloat16)
        live = srt < rows
        a_rows[live] = x[srt[live] // top_k]
        capi.moe_wna16_marlin_gemm(a_rows.cuda(), words, None, scales, None, sorted_ids, expert_ids, npost, tw.cuda(),
                                   block, 1, True, capi.QTYPE_UINT4B8, rows, n, k, out, a_sorted=True, g_idx=g_sorted,
                                   perm=perm)
    else:
        capi.moe_wna16_marlin_gemm(x.cuda(), words, None, scales, None, sorted_ids, expert_ids, npost, tw.cuda(), block,
                                   top_k, True, capi.QTYPE_UINT4B8, tokens, n, k, out, g_idx=g_sorted, perm=perm)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, ref) <= TOL


def test_unsorted_g_idx_is_reported_not_misread():
    from infiniops_b200 import capi

    tokens, experts, k, n, block = 8, 2, 256, 128, 16
    qs, gs, ss, words, scales, perm, g_sorted = _act_order_experts(experts, k, n, 5)
    ids = torch.zeros((tokens, 1), dtype=torch.int32, device="cuda")
    size, blocks = omoe.padded_sizes(tokens, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, k), device="cuda").bfloat16()
    tw = torch.ones(tokens, device="cuda")
    out = torch.empty((tokens, n), dtype=torch.bfloat16, device="cuda")
    scattered = torch.stack(gs).cuda().contiguous()   # the checkpoint's own table, not the sorted one
    capi.moe_wna16_marlin_gemm(x, words, None, scales, None, sorted_ids, expert_ids, npost, tw, block, 1, False,
                               capi.QTYPE_UINT4B8, tokens, n, k, out, g_idx=scattered, perm=perm)
    torch.cuda.synchronize()
    buf = capi.scratch("cuda", 0)
    assert capi.scratch_status(buf) == 9
    capi.lib().infiniops_b200_gemm_scratch_prepare(buf.data_ptr(), buf.numel(), None)
    torch.cuda.synchronize()
    assert capi.scratch_status(buf) == 0
    with pytest.raises(capi.Error, match="together"):
        capi.moe_wna16_marlin_gemm(x, words, None, scales, None, sorted_ids, expert_ids, npost, tw, block, 1, False,
                                   capi.QTYPE_UINT4B8, tokens, n, k, out, perm=perm)


def test_operator_api_takes_activation_order():
    """The reference's own act-order case (tests/test_moe_wna16_marlin_gemm.py:64-79 of the reference):
    identity `perm`, sorted `g_idx`, zero scales -- through `infini.ops`."""
    import infini.ops

    experts, k, n, block, tokens, top_k, groups = 4, 128 * 8, 256, 16, 2, 2, 8
    dev = "cuda"
    a = torch.randn((tokens, k), dtype=torch.float16, device=dev)
    wq = torch.zeros((experts, k // 16, 2 * n), dtype=torch.int32, device=dev)
    scales = torch.full((experts, groups, n), 0.25, dtype=torch.float16, device=dev)
    g_idx = torch.arange(groups, dtype=torch.int32, device=dev).repeat_interleave(k // groups).repeat(experts, 1)
    perm = torch.arange(k, dtype=torch.int32, device=dev).repeat(experts, 1)
    routes = tokens * top_k
    ids = (torch.arange(routes, dtype=torch.int32, device=dev) % experts).view(tokens, top_k)
    size, blocks = omoe.padded_sizes(routes, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(blocks, dtype=torch.int32, device=dev)
    npost = torch.empty(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    infini.ops.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost, stream=stream)
    tw = torch.ones(routes, dtype=torch.float32, device=dev)
    out = torch.full((routes, n), float("nan"), dtype=torch.float16, device=dev)
    workspace = torch.zeros(432, dtype=torch.int32, device=dev)
    infini.ops.moe_wna16_marlin_gemm(a, wq, None, scales, None, None, None, g_idx, perm, workspace, sorted_ids,
                                     expert_ids, npost, tw, block, top_k, True, 1125899907892224, tokens, n, k, True,
                                     False, True, False, -1, -1, -1, out, stream=stream)
    torch.cuda.synchronize()
    # all-zero words are q = 0, i.e. the weight -8 * 0.25 = -2 everywhere
    want = (a.float().sum(dim=1, keepdim=True) * -2.0).repeat_interleave(top_k, dim=0).expand(routes, n)
    assert rel_max_err(out, want) <= 2e-2


@pytest.mark.parametrize("m,k,n,dtype", ((1, 512, 256, torch.bfloat16), (48, 1024, 384, torch.float16),
                                         (200, 512, 512, torch.bfloat16), (300, 2048, 256, torch.bfloat16)))
def test_dense_gemm_with_activation_order(m, k, n, dtype):
    """All token tiles (16 .. 256 rows, the paired kernel at n % 256 == 0 included) read the permuted copy."""
    from infiniops_b200 import capi

    qs, gs, ss, words, scales, perm, g_sorted = _act_order_experts(1, k, n, 40 + m)
    x = torch.randn((m, k), generator=torch.Generator().manual_seed(m)).to(dtype)
    ref = x.float() @ _dequant_scattered(qs[0], gs[0], ss[0].to(dtype))
    out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    capi.marlin_gemm(x.cuda(), words[0], None, scales[0].to(dtype).contiguous(), None, capi.QTYPE_UINT4B8, m, n, k, out,
                     g_idx=g_sorted[0].contiguous(), perm=perm[0].contiguous())
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    assert not torch.isnan(out.float()).any()
    assert rel_max_err(out, ref) <= TOL
    # identical to the plain GEMM on activations permuted by hand
    plain = torch.empty_like(out)
    capi.marlin_gemm(x[:, perm[0].cpu().long()].contiguous().cuda(), words[0], None, scales[0].to(dtype).contiguous(), None,
                     capi.QTYPE_UINT4B8, m, n, k, plain)
    torch.cuda.synchronize()
    assert torch.equal(out, plain)


def test_dense_gemm_reports_an_unsorted_g_idx_and_refuses_half_a_pair():
    from infiniops_b200 import capi

    m, k, n = 8, 256, 128
    qs, gs, ss, words, scales, perm, g_sorted = _act_order_experts(1, k, n, 6)
    x = torch.randn((m, k), device="cuda").bfloat16()
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    capi.marlin_gemm(x, words[0], None, scales[0].contiguous(), None, capi.QTYPE_UINT4B8, m, n, k, out,
                     g_idx=gs[0].cuda(), perm=perm[0].contiguous())
    torch.cuda.synchronize()
    buf = capi.scratch("cuda", 0)
    assert capi.scratch_status(buf) == 9
    capi.lib().infiniops_b200_gemm_scratch_prepare(buf.data_ptr(), buf.numel(), None)
    torch.cuda.synchronize()
    assert capi.scratch_status(buf) == 0
    with pytest.raises(capi.Error, match="together"):
        capi.marlin_gemm(x, words[0], None, scales[0].contiguous(), None, capi.QTYPE_UINT4B8, m, n, k, out,
                         perm=perm[0].contiguous())


def test_dense_operator_api_takes_activation_order():
    import infini.ops

    m, k, n = 24, 512, 256
    qs, gs, ss, words, scales, perm, g_sorted = _act_order_experts(1, k, n, 8)
    x = torch.randn((m, k), generator=torch.Generator().manual_seed(2)).bfloat16()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    workspace = torch.zeros(432, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    infini.ops.marlin_gemm(x.cuda(), words[0], None, scales[0].contiguous(), None, None, None, g_sorted[0].contiguous(),
                           perm[0].contiguous(), workspace, 1125899907892224, m, n, k, True, False, True, False, out,
                           stream=stream)
    torch.cuda.synchronize()
    ref = x.float() @ _dequant_scattered(qs[0], gs[0], ss[0])
    assert rel_max_err(out, ref) <= TOL
