"""GPU: `silu_and_mul` applied inside the epilogue of the first routed GEMM (gate and up columns
interleaved in runs of 16) against the unfused chain and against the oracle.

Two kinds of check:

* bit identity -- on the SAME interleaved weights, the fused call must equal the unfused sorted-order
  call followed by a de-interleave and the library's own `silu_and_mul` (same tiles, same split of
  the k range, same rounding points);
* oracle parity -- a small layer whose w13 is prepared from a plain [gate | up] matrix with
  `gate_up_interleave`, run through the whole chain with and without the fused epilogue, both within
  the GEMM tolerance of the oracle's dequantise -> matmul -> silu_and_mul -> matmul -> sum.
"""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import quant as oq
from tests.helpers import make_quantized, rel_max_err

pytestmark = pytest.mark.gpu
TOL = 1e-2
GROUP = 128


def _random_experts(e, k, n, zeros, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randint(-2**31, 2**31 - 1, (e, k // 16, 2 * n), dtype=torch.int32, device="cuda", generator=gen)
    s = (torch.randn((e, k // GROUP, n), device="cuda", generator=gen).abs() * 0.01 + 1e-3).bfloat16()
    z = torch.randint(-2**31, 2**31 - 1, (e, k // GROUP, n // 8), dtype=torch.int32, device="cuda", generator=gen) \
        if zeros else None
    return w, s, z


def test_interleave_index_convention():
    from infiniops_b200 import moe_layer

    inter = 48
    idx = moe_layer.gate_up_interleave(inter).numpy()
    assert sorted(idx.tolist()) == list(range(2 * inter))
    for p, src in enumerate(idx):
        feature = (p // 32) * 16 + p % 16
        assert src == (feature if p % 32 < 16 else inter + feature)


@pytest.mark.parametrize("block,zeros,with_bias", ((16, False, False), (64, True, True), (128, False, True),
                                                   (256, True, False)))
def test_fused_epilogue_equals_gemm_then_silu(block, zeros, with_bias):
    from infiniops_b200 import capi

    tokens, experts, top_k, hidden, inter = 600, 8, 2, 512, 256
    qtype = capi.QTYPE_UINT4 if zeros else capi.QTYPE_UINT4B8
    ids = torch.randint(0, experts, (tokens, top_k), dtype=torch.int32, device="cuda")
    tw = torch.rand((tokens, top_k), device="cuda").reshape(-1)
    w13, s13, z13 = _random_experts(experts, hidden, 2 * inter, zeros, 300 + block)
    bias = (torch.randn((experts, 2 * inter), device="cuda") * 0.2).bfloat16() if with_bias else None
    size, blocks = omoe.padded_sizes(tokens * top_k, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()

    gs = torch.zeros((size, 2 * inter), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w13, bias, s13, z13, sorted_ids, expert_ids, npost, tw, block, top_k, False, qtype,
                               tokens, 2 * inter, hidden, gs, out_sorted=True)
    # columns 32b..32b+15 are gate features 16b.., 32b+16..32b+31 the matching up features
    feature = torch.arange(inter, device="cuda")
    gate_col = (feature // 16) * 32 + feature % 16
    plain = torch.cat([gs[:, gate_col], gs[:, gate_col + 16]], dim=1).contiguous()
    want = torch.empty((size, inter), dtype=torch.bfloat16, device="cuda")
    capi.silu_and_mul(plain, want)

    got = torch.full((size, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w13, bias, s13, z13, sorted_ids, expert_ids, npost, tw, block, top_k, False, qtype,
                               tokens, 2 * inter, hidden, got, out_sorted=True, fuse_silu=True)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    live = torch.nonzero(sorted_ids[: int(npost.cpu()[0])].long() < tokens * top_k).flatten()
    assert live.numel() == tokens * top_k
    assert not torch.isnan(got[live].float()).any()
    assert torch.equal(got[live], want[live])


def test_fused_epilogue_refuses_what_it_cannot_do():
    from infiniops_b200 import capi

    experts, hidden, inter, block, tokens = 2, 256, 96, 16, 8     # 2 * inter = 192: not a multiple of 128
    w13, s13, _ = _random_experts(experts, hidden, 2 * inter, False, 5)
    ids = torch.zeros((tokens, 1), dtype=torch.int32, device="cuda")
    size, blocks = omoe.padded_sizes(tokens, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()
    tw = torch.ones(tokens, device="cuda")
    out = torch.empty((size, inter), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.Error, match="fused silu"):
        capi.moe_wna16_marlin_gemm(x, w13, None, s13, None, sorted_ids, expert_ids, npost, tw, block, 1, False,
                                   capi.QTYPE_UINT4B8, tokens, 2 * inter, hidden, out, out_sorted=True, fuse_silu=True)
    with pytest.raises(capi.Error, match="fused silu"):
        capi.moe_wna16_marlin_gemm(x, w13[:, :, :512], None, s13[:, :, :256].contiguous(), None, sorted_ids, expert_ids,
                                   npost, tw, block, 1, False, capi.QTYPE_UINT4B8, tokens, 256, hidden, out,
                                   out_sorted=False, fuse_silu=True)


@pytest.mark.parametrize("zeros", (False, True))
def test_layer_with_interleaved_w13_matches_the_oracle(zeros):
    """w13 given as [gate | up] is reordered with `gate_up_interleave`, packed, and the layer run with the
    fused epilogue; the plain packing runs the unfused chain.  Both against the oracle layer."""
    from infiniops_b200 import capi, moe_layer

    tokens, experts, top_k, hidden, inter, block = 96, 4, 2, 256, 128, 32
    q13, s13, z13 = [], [], []
    q2, s2, z2 = [], [], []
    for e in range(experts):
        q, s, z = make_quantized(hidden, 2 * inter, GROUP, torch.bfloat16, zeros, 400 + e)
        q13.append(q), s13.append(s), z13.append(z)
        q, s, z = make_quantized(inter, hidden, GROUP, torch.bfloat16, zeros, 500 + e)
        q2.append(q), s2.append(s), z2.append(z)

    def pack(qs, ss, zs, order=None):
        words, scales, zps = [], [], []
        for q, s, z in zip(qs, ss, zs):
            if order is not None:
                q, s = q[:, order], s[:, order]
                z = None if z is None else z[:, order]
            words.append(torch.from_numpy(oq.marlin_pack(q, 4)))
            scales.append(s)
            zps.append(None if z is None else torch.from_numpy(oq.pack_zeros(z, 4)))
        return (torch.stack(words).cuda(), torch.stack(scales).cuda(),
                None if zps[0] is None else torch.stack(zps).cuda())

    order = moe_layer.gate_up_interleave(inter).numpy()
    w2_dev = pack(q2, s2, z2)
    plain = moe_layer.ExpertWeights(*pack(q13, s13, z13), *w2_dev, hidden, inter)
    fused = moe_layer.ExpertWeights(*pack(q13, s13, z13, order), *w2_dev, hidden, inter, interleaved=True)

    gen = torch.Generator().manual_seed(77)
    x = torch.randn((tokens, hidden), generator=gen).bfloat16()
    logits = torch.randn((tokens, experts), generator=gen)
    tw, ids, _ = omoe.topk_softmax(logits, None, None, top_k, True)
    tw, ids = torch.as_tensor(tw), torch.as_tensor(ids).to(torch.int32)

    # oracle layer: per route, dequantised expert matmuls in fp32 with the intermediates rounded to bf16
    ref = torch.zeros((tokens, hidden))
    for t in range(tokens):
        for j in range(top_k):
            e = int(ids[t, j])
            g = (x[t].float() @ oq.dequantize(q13[e], s13[e], z13[e], 4)).bfloat16()
            h = omoe.silu_and_mul(g[None])[0]
            y = ((h.float() @ oq.dequantize(q2[e], s2[e], z2[e], 4)) * tw[t, j]).bfloat16()
            ref[t] += y.float()
    ref = ref.bfloat16()

    outs = {}
    for name, weights in (("plain", plain), ("fused", fused)):
        runner = moe_layer.RoutedExperts(weights, block)
        outs[name] = moe_layer.single_gpu_layer(x.cuda(), tw.cuda().float(), ids.cuda(), runner).clone()
        torch.cuda.synchronize()
        assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
        assert rel_max_err(outs[name], ref) <= TOL, name
    # the two chains round at the same points; they differ only by the order of a few fp32 additions
    assert rel_max_err(outs["fused"], outs["plain"]) <= 2e-2


# ---- router + token sort in one launch -----------------------------------------------------------------
def _sort_outputs(numel, experts, block):
    size, blocks = omoe.padded_sizes(numel, experts, block)
    return (torch.full((size,), -7, dtype=torch.int32, device="cuda"),
            torch.full((blocks,), -7, dtype=torch.int32, device="cuda"), torch.full((1,), -7, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("tokens,experts,top_k,block,dtype,sigmoid", (
    (1, 8, 2, 16, torch.float32, False), (64, 8, 2, 64, torch.float32, False), (512, 8, 2, 32, torch.bfloat16, False),
    (37, 60, 4, 16, torch.float16, False), (128, 256, 8, 16, torch.float32, True), (600, 8, 2, 64, torch.float32, False)))
def test_softmax_router_and_sort_in_one_call(tokens, experts, top_k, block, dtype, sigmoid):
    """Same bits as the two operators called one after the other (600 x 2 ids exceed one block: the
    call then issues the separate launches itself)."""
    from infiniops_b200 import capi

    gen = torch.Generator(device="cuda").manual_seed(tokens * 31 + experts)
    logits = torch.randn((tokens, experts), device="cuda", generator=gen).to(dtype)
    bias = torch.randn(experts, device="cuda", generator=gen) * 0.1 if sigmoid else None
    pad = torch.zeros(tokens, dtype=torch.bool, device="cuda")
    pad[tokens // 2] = tokens > 2

    w0 = torch.empty((tokens, top_k), device="cuda")
    i0 = torch.empty((tokens, top_k), dtype=torch.int32, device="cuda")
    t0 = torch.empty_like(i0)
    if sigmoid:
        capi.topk_sigmoid(logits, bias, pad, True, 2.5, w0, i0, t0)
    else:
        capi.topk_softmax(logits, bias, pad, True, w0, i0, t0)
    s0, e0, n0 = _sort_outputs(tokens * top_k, experts, block)
    capi.moe_align_block_size(i0, None, experts, block, s0, e0, n0)

    w1, i1, t1 = torch.empty_like(w0), torch.empty_like(i0), torch.empty_like(t0)
    s1, e1, n1 = _sort_outputs(tokens * top_k, experts, block)
    capi.topk_softmax_align(logits, bias, pad, True, w1, i1, t1, None, block, s1, e1, n1, sigmoid=sigmoid,
                            routed_scaling_factor=2.5)
    torch.cuda.synchronize()
    for a, b in ((w0, w1), (i0, i1), (t0, t1), (s0, s1), (e0, e1), (n0, n1)):
        assert torch.equal(a, b)
    # and the sort itself against the oracle
    rs, re, rn = omoe.moe_align_block_size(i1.cpu().numpy(), None, experts, block)
    assert np.array_equal(s1.cpu().numpy(), rs) and np.array_equal(e1.cpu().numpy(), re) and int(n1.cpu()[0]) == int(rn[0])


@pytest.mark.parametrize("tokens,block,dtype", ((16, 16, torch.float32), (128, 16, torch.float32), (64, 32, torch.bfloat16),
                                                (512, 64, torch.float32)))
def test_grouped_router_and_sort_in_one_call(tokens, block, dtype):
    from infiniops_b200 import capi

    experts, top_k = 256, 8
    gen = torch.Generator(device="cuda").manual_seed(tokens + 5)
    scores = torch.randn((tokens, experts), device="cuda", generator=gen).to(dtype)
    bias = torch.randn(experts, device="cuda", generator=gen) * 0.01
    w0 = torch.empty((tokens, top_k), device="cuda")
    i0 = torch.empty((tokens, top_k), dtype=torch.int32, device="cuda")
    capi.grouped_topk(scores, bias, 8, 4, top_k, True, 2.5, 1, w0, i0)
    s0, e0, n0 = _sort_outputs(tokens * top_k, experts, block)
    capi.moe_align_block_size(i0, None, experts, block, s0, e0, n0)

    w1, i1 = torch.empty_like(w0), torch.empty_like(i0)
    s1, e1, n1 = _sort_outputs(tokens * top_k, experts, block)
    capi.grouped_topk_align(scores, bias, 8, 4, top_k, True, 2.5, 1, w1, i1, None, block, s1, e1, n1)
    torch.cuda.synchronize()
    for a, b in ((w0, w1), (i0, i1), (s0, s1), (e0, e1), (n0, n1)):
        assert torch.equal(a, b)


def test_layer_from_logits_equals_the_chain():
    from infiniops_b200 import moe_layer

    tokens, experts, top_k, hidden, inter, block = 48, 8, 2, 256, 128, 16
    w13, s13, _ = _random_experts(experts, hidden, 2 * inter, False, 11)
    w2, s2, _ = _random_experts(experts, inter, hidden, False, 12)
    weights = moe_layer.ExpertWeights(w13, s13, None, w2, s2, None, hidden, inter)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()
    logits = torch.randn((tokens, experts), device="cuda")
    runner = moe_layer.RoutedExperts(weights, block)
    tw, ids = moe_layer.route_softmax(logits, top_k)
    want = moe_layer.single_gpu_layer(x, tw, ids, runner).clone()
    got = moe_layer.layer_from_logits(x, logits, {"kind": "softmax", "top_k": top_k}, runner)
    torch.cuda.synchronize()
    assert torch.equal(got, want)


# ---- second GEMM with tile stores + sum by position --------------------------------------------------------
@pytest.mark.parametrize("block,zeros,with_bias", ((128, False, False), (256, True, True), (256, False, False)))
def test_tile_store_chain_equals_the_scattered_chain(block, zeros, with_bias):
    """w2 with `a_sorted` + `out_sorted` + routing weights, then moe_gather_sum by the positions the first
    GEMM's gather wrote, against w2 scattering rows to their routes followed by moe_sum: same bits.  One
    token carries an expert id outside the table (its route occurs nowhere in the sort)."""
    from infiniops_b200 import capi

    tokens, experts, top_k, hidden, inter = 700, 8, 2, 512, 256
    qtype = capi.QTYPE_UINT4 if zeros else capi.QTYPE_UINT4B8
    ids = torch.randint(0, experts, (tokens, top_k), dtype=torch.int32, device="cuda")
    ids[5, 1] = experts + 2
    tw = torch.rand((tokens, top_k), device="cuda").reshape(-1)
    w13, s13, z13 = _random_experts(experts, hidden, 2 * inter, zeros, 600 + block)
    w2, s2, z2 = _random_experts(experts, inter, hidden, zeros, 601 + block)
    b2 = (torch.randn((experts, hidden), device="cuda") * 0.2).bfloat16() if with_bias else None
    rows = tokens * top_k
    size, blocks = omoe.padded_sizes(rows, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()

    position = torch.full((tokens, top_k), 12345, dtype=torch.int32, device="cuda")
    g = torch.zeros((size, 2 * inter), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w13, None, s13, z13, sorted_ids, expert_ids, npost, tw, block, top_k, False, qtype,
                               tokens, 2 * inter, hidden, g, out_sorted=True, route_position=position)
    h = torch.empty((size, inter), dtype=torch.bfloat16, device="cuda")
    capi.silu_and_mul(g, h)

    y = torch.zeros((rows, hidden), dtype=torch.bfloat16, device="cuda")    # the dropped route's row stays zero
    capi.moe_wna16_marlin_gemm(h, w2, b2, s2, z2, sorted_ids, expert_ids, npost, tw, block, 1, True, qtype, rows, hidden,
                               inter, y, a_sorted=True)
    want = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    capi.moe_sum(y.view(tokens, top_k, hidden), want)

    ys = torch.full((size, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(h, w2, b2, s2, z2, sorted_ids, expert_ids, npost, tw, block, 1, True, qtype, rows, hidden,
                               inter, ys, a_sorted=True, out_sorted=True)
    got = torch.empty_like(want)
    capi.moe_gather_sum(ys, position, got)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    # positions: the inverse of the sort, -1 for the route that was dropped
    pos = position.cpu().flatten()
    srt = sorted_ids.cpu().long()
    assert int(pos[5 * top_k + 1]) == -1 and int((pos < 0).sum()) == 1
    live = pos >= 0
    assert torch.equal(srt[pos[live].long()], torch.nonzero(live).flatten())
    assert not torch.isnan(got.float()).any()
    assert torch.equal(got, want)


def test_sorted_output_with_weights_needs_large_blocks():
    from infiniops_b200 import capi

    experts, hidden, n, block, tokens = 2, 256, 128, 64, 8
    w, s, _ = _random_experts(experts, hidden, n, False, 7)
    ids = torch.zeros((tokens, 1), dtype=torch.int32, device="cuda")
    size, blocks = omoe.padded_sizes(tokens, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()
    out = torch.empty((size, n), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.Error, match="128- or 256-row"):
        capi.moe_wna16_marlin_gemm(x, w, None, s, None, sorted_ids, expert_ids, npost, torch.ones(tokens, device="cuda"),
                                   block, 1, True, capi.QTYPE_UINT4B8, tokens, n, hidden, out, out_sorted=True)


# ---- MMAs and epilogue restricted to the live rows of a routing block ---------------------------------------
@pytest.mark.parametrize("block,zeros,tokens", ((32, False, 37), (64, True, 150), (128, False, 700), (256, True, 700),
                                                (256, False, 90)))
def test_live_row_extent_changes_no_bit(block, zeros, tokens):
    """With `block_rows` the GEMMs issue their MMAs over a block's live rows (rounded up to 16) instead of
    the whole block; every live row must come out bit for bit as without it -- scattered and sorted form --
    and the table itself must hold the number of live rows of every block."""
    from infiniops_b200 import capi

    experts, top_k, hidden, n = 8, 2, 512, 256
    qtype = capi.QTYPE_UINT4 if zeros else capi.QTYPE_UINT4B8
    ids = torch.randint(0, experts, (tokens, top_k), dtype=torch.int32, device="cuda")
    tw = torch.rand((tokens, top_k), device="cuda").reshape(-1)
    w, s, z = _random_experts(experts, hidden, n, zeros, 700 + block)
    rows = tokens * top_k
    size, blocks = omoe.padded_sizes(rows, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()

    plain = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w, None, s, z, sorted_ids, expert_ids, npost, tw, block, top_k, True, qtype, tokens, n,
                               hidden, plain)
    live = torch.full((blocks + 1,), -5, dtype=torch.int32, device="cuda")
    shrunk = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w, None, s, z, sorted_ids, expert_ids, npost, tw, block, top_k, True, qtype, tokens, n,
                               hidden, shrunk, block_rows=live)
    sorted_plain = torch.zeros((size, n), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w, None, s, z, sorted_ids, expert_ids, npost, tw, block, top_k, False, qtype, tokens, n,
                               hidden, sorted_plain, out_sorted=True)
    sorted_shrunk = torch.zeros((size, n), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w, None, s, z, sorted_ids, expert_ids, npost, tw, block, top_k, False, qtype, tokens, n,
                               hidden, sorted_shrunk, out_sorted=True, block_rows=live)
    # a second GEMM reading the sorted rows in place, given the same table
    w2, s2, z2 = _random_experts(experts, n, hidden, zeros, 701 + block)
    y_plain = torch.full((rows, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(sorted_plain, w2, None, s2, z2, sorted_ids, expert_ids, npost, tw, block, 1, True, qtype, rows,
                               hidden, n, y_plain, a_sorted=True)
    y_shrunk = torch.full((rows, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(sorted_shrunk, w2, None, s2, z2, sorted_ids, expert_ids, npost, tw, block, 1, True, qtype, rows,
                               hidden, n, y_shrunk, a_sorted=True, block_rows=live)
    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0
    total = int(npost.cpu()[0])
    srt = sorted_ids.cpu().long()[:total].view(-1, block)
    want_live = (srt < rows).sum(dim=1).to(torch.int32)
    assert torch.equal(live.cpu()[: total // block], want_live)
    assert not torch.isnan(shrunk.float()).any() and torch.equal(shrunk, plain)
    keep = torch.nonzero(sorted_ids[:total].long() < rows).flatten()
    assert torch.equal(sorted_shrunk[keep], sorted_plain[keep])
    assert not torch.isnan(y_shrunk.float()).any() and torch.equal(y_shrunk, y_plain)
