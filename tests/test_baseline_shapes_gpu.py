"""GPU: the GEMMs at the full sizes of the benchmark configurations, against the oracle.

Dense prefill (M = 4096) on the three Llama-shaped matrices the small-shape tests do not reach,
the gate_up matrix at every decode M, and the routed GEMM pair at the Mixtral (E=8, top-2,
H=4096, I=14336) and DeepSeek (E=256, top-8 grouped, H=7168, I=2048, AWQ zero points) layer sizes.

To keep the CPU side to seconds the expert weights are random Marlin words generated on the
device (the repack has its own bit-exact tests); the oracle unpacks only what a check needs:

* every routed row is compared on a SAMPLE OF COLUMNS -- the 64-column blocks that hold the first,
  the last and two middle columns of the matrix (a block of 64 columns is a self-contained slice
  of the Marlin layout);
* the rows of the first and of the last routing block are compared on ALL columns.

Tolerance as stated by the benchmark definition: max |got - ref| <= 1e-2 * max |ref|.
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


def _scratch_ok():
    from infiniops_b200 import capi

    torch.cuda.synchronize()
    assert capi.scratch_status(capi.scratch("cuda", 0)) == 0, "a GEMM kernel gave up on a wait"


# ---- dense ---------------------------------------------------------------------------------------------
def _dense_problem(k, n, zeros, seed):
    """Random Marlin words + scales (+ zero points) on the device, and an oracle view of them."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    marlin = torch.randint(-2**31, 2**31 - 1, (k // 16, 2 * n), dtype=torch.int32, device="cuda", generator=gen)
    scales = (torch.randn((k // GROUP, n), device="cuda", generator=gen).abs() * 0.01 + 1e-3).bfloat16()
    zp = torch.randint(-2**31, 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, device="cuda", generator=gen) \
        if zeros else None
    return marlin, scales, zp


def _unpack_zeros(zp_words: np.ndarray) -> np.ndarray:
    """int32 [..., N/8] -> uint8 [..., N]; field j of a word is column 8 * (n / 8) + j."""
    w = zp_words.view(np.uint32)
    fields = (w[..., None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF
    return fields.reshape(*w.shape[:-1], -1).astype(np.uint8)


def _dequant_columns(marlin, scales, zp, k, col_blocks):
    """fp32 [K, 64 * len(col_blocks)] of the given 64-column blocks."""
    parts = []
    for nb in col_blocks:
        words = marlin[:, 128 * nb:128 * (nb + 1)].cpu().numpy()
        q = oq.marlin_unpack_w4(words, k, 64)
        s = scales[:, 64 * nb:64 * (nb + 1)].cpu()
        z = None if zp is None else _unpack_zeros(zp[:, 8 * nb:8 * (nb + 1)].cpu().numpy())
        parts.append(oq.dequantize(q, s, z, 4))
    return torch.cat(parts, dim=1)


def _columns_of(col_blocks):
    return torch.cat([torch.arange(64 * nb, 64 * (nb + 1)) for nb in col_blocks])


@pytest.mark.parametrize("k,n", ((4096, 6144), (4096, 28672), (14336, 4096)))
def test_config3_prefill_m4096(k, n):
    """GPTQ-symmetric, bf16, M = 4096 (paired-block kernel: 24 / 112 / 16 tile pairs, 32 / 32 / 112
    k-stages).  Oracle on three row slices (first, a middle and the last token tile) over all columns
    of four column blocks and over ALL columns for 16 rows; exact linearity on everything."""
    from infiniops_b200 import capi

    m = 4096
    marlin, scales, _ = _dense_problem(k, n, False, k + n)
    a = torch.randn((m, k), device="cuda").bfloat16()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.marlin_gemm(a, marlin, None, scales, None, capi.QTYPE_UINT4B8, m, n, k, out)
    _scratch_ok()
    assert not torch.isnan(out.float()).any()
    nb_total = n // 64
    blocks = sorted({0, 1, nb_total // 2, nb_total - 1})
    w = _dequant_columns(marlin, scales, None, k, blocks)
    cols = _columns_of(blocks)
    for lo in (0, 1792, m - 256):   # token tiles 0, 7 and 15 of 16
        ref = a[lo:lo + 256].float().cpu() @ w
        assert rel_max_err(out[lo:lo + 256][:, cols.cuda()], ref) <= TOL
    # all columns for a few rows spread over the token tiles
    rows = torch.tensor([0, 255, 256, 1000, 2047, 2048, 3000, 4095])
    q_full = oq.marlin_unpack_w4(marlin.cpu().numpy(), k, n)
    ref = a[rows.cuda()].float().cpu() @ oq.dequantize(q_full, scales.cpu(), None, 4)
    assert rel_max_err(out[rows.cuda()], ref) <= TOL
    out2 = torch.empty_like(out)
    capi.marlin_gemm(a * 2, marlin, None, scales, None, capi.QTYPE_UINT4B8, m, n, k, out2)
    _scratch_ok()
    assert torch.equal(out2.float(), out.float() * 2)


@pytest.mark.parametrize("m", (1, 4, 64))
def test_config2_gate_up_every_decode_m(m):
    """AWQ bf16 gate_up (4096 x 28672) at the decode sizes the small-shape file leaves out."""
    from infiniops_b200 import capi

    k, n = 4096, 28672
    marlin, scales, zp = _dense_problem(k, n, True, 7 + m)
    a = torch.randn((m, k), device="cuda").bfloat16()
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.marlin_gemm(a, marlin, None, scales, zp, capi.QTYPE_UINT4, m, n, k, out)
    _scratch_ok()
    q = oq.marlin_unpack_w4(marlin.cpu().numpy(), k, n)
    ref = a.float().cpu() @ oq.dequantize(q, scales.cpu(), _unpack_zeros(zp.cpu().numpy()), 4)
    assert rel_max_err(out, ref) <= TOL


# ---- routed ---------------------------------------------------------------------------------------------
def _experts(e, k, n, zeros, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.empty((e, k // 16, 2 * n), dtype=torch.int32, device="cuda")
    for i in range(e):   # one expert at a time: torch.randint materialises int64 first
        w[i] = torch.randint(-2**31, 2**31 - 1, (k // 16, 2 * n), dtype=torch.int32, device="cuda", generator=gen)
    s = (torch.randn((e, k // GROUP, n), device="cuda", generator=gen).abs() * 0.01 + 1e-3).bfloat16()
    z = torch.randint(-2**31, 2**31 - 1, (e, k // GROUP, n // 8), dtype=torch.int32, device="cuda", generator=gen) \
        if zeros else None
    return w, s, z


def _check_routed(a, w, s, z, bias, sorted_ids, expert_ids, npost, tw, block, top_k, mul, out):
    """`out` [M * top_k, N] against the oracle: all routed rows on sampled column blocks, the first
    and the last routing block on all columns."""
    e, _, n2 = w.shape
    n, k = n2 // 2, a.shape[1]
    rows_total = a.shape[0] * top_k
    sorted_np, experts_np = sorted_ids.cpu().numpy(), expert_ids.cpu().numpy()
    cutoff = int(npost.cpu()[0])
    a_cpu = a.float().cpu()
    tw_cpu = None if tw is None else tw.float().cpu()
    bias_cpu = None if bias is None else bias.float().cpu()
    nb_total = n // 64
    blocks = sorted({0, nb_total // 3, (2 * nb_total) // 3, nb_total - 1})
    cols = _columns_of(blocks)
    live = [b for b in range(cutoff // block) if experts_np[b] >= 0]
    assert live, "no routed block"
    by_expert: dict[int, list[int]] = {}
    for b in live:
        by_expert.setdefault(int(experts_np[b]), []).append(b)

    def rows_of(b):
        r = sorted_np[b * block:(b + 1) * block]
        return torch.from_numpy(r[r < rows_total].astype(np.int64))

    def expected(rows, ex, weight, col_index):
        val = a_cpu[rows // top_k] @ weight
        if bias_cpu is not None:
            val = val + bias_cpu[ex][col_index]
        if mul:
            val = val * tw_cpu[rows].unsqueeze(-1)
        return val

    worst, scale = 0.0, 0.0
    got_cols = out[:, cols.cuda()].float().cpu()
    seen = torch.zeros(rows_total, dtype=torch.bool)
    for ex, blks in by_expert.items():
        weight = _dequant_columns(w[ex], s[ex], None if z is None else z[ex], k, blocks)
        rows = torch.cat([rows_of(b) for b in blks])
        seen[rows] = True
        ref = expected(rows, ex, weight, cols)
        worst = max(worst, float((got_cols[rows] - ref).abs().max()))
        scale = max(scale, float(ref.abs().max()))
    assert worst <= TOL * scale, f"sampled columns: {worst} vs scale {scale}"
    for b in {live[0], live[-1]}:
        ex = int(experts_np[b])
        q = oq.marlin_unpack_w4(w[ex].cpu().numpy(), k, n)
        weight = oq.dequantize(q, s[ex].cpu(), None if z is None else _unpack_zeros(z[ex].cpu().numpy()), 4)
        rows = rows_of(b)
        ref = expected(rows, ex, weight, slice(None))
        assert rel_max_err(out[rows.cuda()], ref) <= TOL
    return seen


def _layer(tokens, experts, top_k, hidden, inter, block, zeros, ids, weights, seed, with_bias=False,
           topk_weight_dtype=torch.float32):
    """w13 GEMM and w2 GEMM of one layer at full size, each checked on its own inputs."""
    from infiniops_b200 import capi

    w13, s13, z13 = _experts(experts, hidden, 2 * inter, zeros, seed)
    w2, s2, z2 = _experts(experts, inter, hidden, zeros, seed + 1)
    qtype = capi.QTYPE_UINT4 if zeros else capi.QTYPE_UINT4B8
    size, blocks = omoe.padded_sizes(tokens * top_k, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    rs, re, rn = omoe.moe_align_block_size(ids.cpu(), None, experts, block)
    assert np.array_equal(sorted_ids.cpu().numpy(), rs) and np.array_equal(expert_ids.cpu().numpy(), re)
    assert int(npost.cpu()[0]) == int(rn[0])
    gen = torch.Generator(device="cuda").manual_seed(seed + 2)
    x = torch.randn((tokens, hidden), device="cuda", generator=gen).bfloat16()
    b13 = torch.randn((experts, 2 * inter), device="cuda", generator=gen).bfloat16() if with_bias else None
    b2 = torch.randn((experts, hidden), device="cuda", generator=gen).bfloat16() if with_bias else None
    flat_w = weights.reshape(-1).contiguous()
    g = torch.full((tokens * top_k, 2 * inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w13, b13, s13, z13, sorted_ids, expert_ids, npost, flat_w, block, top_k, False,
                               qtype, tokens, 2 * inter, hidden, g)
    _scratch_ok()
    seen = _check_routed(x, w13, s13, z13, b13, sorted_ids, expert_ids, npost, None, block, top_k, False, g)
    assert bool(seen.all()) and not torch.isnan(g.float()).any()
    h = torch.empty((tokens * top_k, inter), dtype=torch.bfloat16, device="cuda")
    capi.silu_and_mul(g, h)
    y = torch.full((tokens * top_k, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(h, w2, b2, s2, z2, sorted_ids, expert_ids, npost, flat_w, block, 1, True, qtype,
                               tokens * top_k, hidden, inter, y)
    _scratch_ok()
    seen = _check_routed(h, w2, s2, z2, b2, sorted_ids, expert_ids, npost, flat_w, block, 1, True, y)
    assert bool(seen.all()) and not torch.isnan(y.float()).any()


@pytest.mark.parametrize("tokens,with_bias", ((1, False), (64, True), (1024, False)))
def test_config4_mixtral_layer_gemms(tokens, with_bias):
    """E=8, top-2 (topk_softmax), H=4096, I=14336, GPTQ-symmetric, block 64."""
    from infiniops_b200 import capi

    experts, top_k = 8, 2
    logits = torch.randn((tokens, experts), device="cuda")
    w = torch.empty((tokens, top_k), dtype=torch.float32, device="cuda")
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device="cuda")
    tei = torch.empty((tokens, top_k), dtype=torch.int32, device="cuda")
    capi.topk_softmax(logits, None, None, True, w, ids, tei)
    _, rids, _ = omoe.topk_softmax(logits.cpu(), None, None, top_k, True)
    assert torch.equal(ids.cpu().long(), rids)
    _layer(tokens, experts, top_k, 4096, 14336, 64, False, ids, w, 4000 + tokens, with_bias)


@pytest.mark.parametrize("tokens", (16, 512))
def test_config5_deepseek_layer_gemms(tokens):
    """E=256, top-8 via grouped_topk (8 groups, 4 kept, sigmoid + fp32 bias), H=7168, I=2048, AWQ zero
    points, block 64: 1276-block-class routing tables, 114 688-row weight tensor map."""
    from infiniops_b200 import capi

    experts, top_k = 256, 8
    scores = torch.randn((tokens, experts), device="cuda")
    bias = torch.randn(experts, device="cuda") * 0.1
    w = torch.empty((tokens, top_k), dtype=torch.float32, device="cuda")
    ids = torch.empty((tokens, top_k), dtype=torch.int32, device="cuda")
    capi.grouped_topk(scores, bias, 8, 4, top_k, True, 2.5, 1, w, ids)
    assert int(ids.min()) >= 0 and int(ids.max()) < experts
    _layer(tokens, experts, top_k, 7168, 2048, 64, True, ids, w, 5000 + tokens, with_bias=(tokens == 16))


@pytest.mark.parametrize("block", (8, 16, 32, 48, 64))
def test_every_accepted_block_size(block):
    """The reference accepts moe_block_size in {8, 16, 32, 48, 64}
    (src/base/moe_wna16_marlin_gemm.h:165-168 of the reference)."""
    from infiniops_b200 import capi

    tokens, experts, top_k, hidden, n = 77, 8, 2, 512, 384
    ids = torch.randint(0, experts, (tokens, top_k), dtype=torch.int32, device="cuda")
    tw = torch.rand((tokens, top_k), device="cuda")
    w, s, _ = _experts(experts, hidden, n, False, 60 + block)
    size, blocks = omoe.padded_sizes(tokens * top_k, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()
    out = torch.full((tokens * top_k, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w, None, s, None, sorted_ids, expert_ids, npost, tw.reshape(-1), block, top_k, True,
                               capi.QTYPE_UINT4B8, tokens, n, hidden, out)
    _scratch_ok()
    seen = _check_routed(x, w, s, None, None, sorted_ids, expert_ids, npost, tw.reshape(-1), block, top_k, True, out)
    assert bool(seen.all()) and not torch.isnan(out.float()).any()


@pytest.mark.parametrize("block,n,zeros,mul", ((128, 384, False, True), (256, 512, True, True), (256, 384, False, False),
                                               (256, 2048, True, False)))
def test_large_routing_blocks(block, n, zeros, mul):
    """Routing blocks of 128 and 256 rows (beyond the reference's set; the sort accepts any block size):
    the 128-token kernel, the 256-token kernel, and -- when the columns pair up -- the paired-block
    kernel in its routed form, with whole and K-split tiles."""
    from infiniops_b200 import capi

    tokens, experts, top_k, hidden = 700, 8, 2, 1024
    ids = torch.randint(0, experts, (tokens, top_k), dtype=torch.int32, device="cuda")
    tw = torch.rand((tokens, top_k), device="cuda")
    w, s, z = _experts(experts, hidden, n, zeros, 70 + block + n)
    size, blocks = omoe.padded_sizes(tokens * top_k, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    rs, re, rn = omoe.moe_align_block_size(ids.cpu(), None, experts, block)
    assert np.array_equal(sorted_ids.cpu().numpy(), rs) and np.array_equal(expert_ids.cpu().numpy(), re)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()
    out = torch.full((tokens * top_k, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w, None, s, z, sorted_ids, expert_ids, npost, tw.reshape(-1), block, top_k, mul,
                               capi.QTYPE_UINT4 if zeros else capi.QTYPE_UINT4B8, tokens, n, hidden, out)
    _scratch_ok()
    seen = _check_routed(x, w, s, z, None, sorted_ids, expert_ids, npost, tw.reshape(-1), block, top_k, mul, out)
    assert bool(seen.all()) and not torch.isnan(out.float()).any()


@pytest.mark.parametrize("block,zeros", ((16, False), (64, True), (128, False), (256, True)))
def test_sorted_order_chain_equals_the_scattered_chain(block, zeros):
    """w13 with `out_sorted` (dense tile stores, rows in sorted order) -> silu_and_mul -> w2 with `a_sorted`
    (reads the sorted rows in place) must give, row for row, what the chain through route-ordered
    intermediates gives: the arithmetic per row is the same, only where the rows live differs."""
    from infiniops_b200 import capi

    tokens, experts, top_k, hidden, inter = 600, 8, 2, 512, 256
    qtype = capi.QTYPE_UINT4 if zeros else capi.QTYPE_UINT4B8
    ids = torch.randint(0, experts, (tokens, top_k), dtype=torch.int32, device="cuda")
    tw = torch.rand((tokens, top_k), device="cuda").reshape(-1)
    w13, s13, z13 = _experts(experts, hidden, 2 * inter, zeros, 80 + block)
    w2, s2, z2 = _experts(experts, inter, hidden, zeros, 81 + block)
    size, blocks = omoe.padded_sizes(tokens * top_k, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    x = torch.randn((tokens, hidden), device="cuda").bfloat16()
    rows = tokens * top_k

    g = torch.full((rows, 2 * inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w13, None, s13, z13, sorted_ids, expert_ids, npost, tw, block, top_k, False, qtype,
                               tokens, 2 * inter, hidden, g)
    h = torch.empty((rows, inter), dtype=torch.bfloat16, device="cuda")
    capi.silu_and_mul(g, h)
    y = torch.full((rows, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(h, w2, None, s2, z2, sorted_ids, expert_ids, npost, tw, block, 1, True, qtype, rows, hidden,
                               inter, y)

    gs = torch.full((size, 2 * inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(x, w13, None, s13, z13, sorted_ids, expert_ids, npost, tw, block, top_k, False, qtype,
                               tokens, 2 * inter, hidden, gs, out_sorted=True)
    hs = torch.empty((size, inter), dtype=torch.bfloat16, device="cuda")
    capi.silu_and_mul(gs, hs)
    ys = torch.full((rows, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.moe_wna16_marlin_gemm(hs, w2, None, s2, z2, sorted_ids, expert_ids, npost, tw, block, 1, True, qtype, rows, hidden,
                               inter, ys, a_sorted=True)
    _scratch_ok()
    sorted_cpu = sorted_ids.cpu().long()
    live = torch.nonzero(sorted_cpu[: int(npost.cpu()[0])] < rows).flatten()
    assert torch.equal(gs[live.cuda()], g[sorted_cpu[live].cuda()])
    assert not torch.isnan(ys.float()).any() and torch.equal(ys, y)
