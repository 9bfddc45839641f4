"""GPU: the operators through the `infini.ops` module (the reference's Python entry points)."""

import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import quant as oq
from tests.helpers import make_quantized, rel_max_err

pytestmark = pytest.mark.gpu
UINT4B8, UINT4 = 1125899907892224, 1125899906843648


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_repack_function_class_and_stream():
    import infini.ops

    k, n = 256, 128
    q = np.random.default_rng(1).integers(0, 16, size=(k, n), dtype=np.uint8)
    expect = oq.marlin_pack(q, 4, False)
    src = torch.from_numpy(oq.gptq_pack(q, 4)).cuda()
    perm = torch.empty(0, dtype=torch.int32, device="cuda")
    out = torch.empty(expect.shape, dtype=torch.int32, device="cuda")
    assert infini.ops.gptq_marlin_repack(src, perm, k, n, 4, False, out, stream=_stream()) is None
    assert np.array_equal(out.cpu().numpy(), expect)
    op = infini.ops.AwqMarlinRepack(torch.from_numpy(oq.awq_pack(q, 4)).cuda(), k, n, 4, False, out)
    q2 = np.random.default_rng(2).integers(0, 16, size=(k, n), dtype=np.uint8)
    out2 = torch.empty_like(out)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        op(torch.from_numpy(oq.awq_pack(q2, 4)).cuda(), k, n, 4, False, out2, stream=side.cuda_stream)
    side.synchronize()
    assert np.array_equal(out2.cpu().numpy(), oq.marlin_pack(q2, 4, False))
    infini.ops.AwqMarlinRepack.clear_cache()


def test_router_and_align_through_module():
    import infini.ops

    gen = torch.Generator().manual_seed(4711)   # fixed inputs: the checks below must not depend on test order
    gate = torch.randn((7, 13), generator=gen).bfloat16()
    w = torch.full((7, 4), torch.nan, device="cuda")
    idx = torch.full((7, 4), 2**31 - 1, dtype=torch.int32, device="cuda")
    tei = torch.full((7, 4), -1, dtype=torch.int32, device="cuda")
    infini.ops.topk_softmax(gate.cuda(), None, None, True, w, idx, tei, stream=_stream())
    rw, ridx, rtei = omoe.topk_softmax(gate, None, None, 4, True)
    assert torch.equal(idx.cpu().long(), ridx) and torch.equal(tei.cpu(), rtei)
    torch.testing.assert_close(w.cpu(), rw, rtol=1e-5, atol=1e-6)

    scores = torch.randn((16, 256), generator=gen)
    bias = torch.randn(256, generator=gen) * 0.1
    v = torch.empty((16, 8), device="cuda")
    gi = torch.empty((16, 8), dtype=torch.int32, device="cuda")
    infini.ops.grouped_topk(scores.cuda(), bias.cuda(), 8, 4, 8, True, 2.5, 1, v, gi)
    rv, rgi = omoe.grouped_topk(scores, bias, 8, 4, 8, True, 2.5, 1)
    assert torch.equal(gi.cpu(), rgi)
    # the values against the oracle's float32 evaluation and, independently of how any float32 tanh
    # rounds, against the same formula in float64
    exact = torch.sigmoid(scores.double()).gather(1, rgi.long())
    exact = (exact / exact.sum(dim=-1, keepdim=True) * 2.5).float()
    torch.testing.assert_close(v.cpu(), exact, rtol=1e-5, atol=1e-5)   # (the tolerance of the layer-size router test)
    torch.testing.assert_close(rv, exact, rtol=1e-4, atol=1e-6)

    ids = torch.randint(0, 256, (512, 8), dtype=torch.int32, generator=gen)
    size, blocks = omoe.padded_sizes(ids.numel(), 256, 64)
    s = torch.full((size,), -2, dtype=torch.int32, device="cuda")
    e = torch.full((blocks,), -2, dtype=torch.int32, device="cuda")
    npost = torch.full((1,), -2, dtype=torch.int32, device="cuda")
    infini.ops.moe_align_block_size(ids.cuda(), None, 256, 64, s, e, npost)
    rs, re, rn = omoe.moe_align_block_size(ids, None, 256, 64)
    assert np.array_equal(s.cpu().numpy(), rs) and np.array_equal(e.cpu().numpy(), re)
    assert np.array_equal(npost.cpu().numpy(), rn)


def test_descriptor_reuse_and_moe_sum_overloads():
    import infini.ops

    x = torch.randn((3, 4, 17), dtype=torch.float16, device="cuda")
    ids = torch.tensor(((0, 1, -1, 2), (2, -1, 1, 0), (1, 2, 0, -1)), dtype=torch.int32, device="cuda")
    emap = torch.tensor((0, -1, 1), dtype=torch.int32, device="cuda")
    out = torch.full((3, 17), torch.nan, dtype=torch.float16, device="cuda")
    infini.ops.moe_sum(x, out)
    torch.testing.assert_close(out.cpu(), omoe.moe_sum(x), rtol=1e-3, atol=1e-3)
    op = infini.ops.MoeSum(x, ids, emap, out)
    x2 = torch.randn_like(x)
    out2 = torch.empty_like(out)
    op(x2, ids.clone(), emap.clone(), out2)
    torch.testing.assert_close(out2.cpu(), omoe.moe_sum(x2, ids, emap), rtol=1e-3, atol=1e-3)
    g = torch.randn((16, 2 * 5632), dtype=torch.bfloat16, device="cuda")
    h = torch.empty((16, 5632), dtype=torch.bfloat16, device="cuda")
    infini.ops.silu_and_mul(g, h, stream=_stream())
    torch.testing.assert_close(h.cpu(), omoe.silu_and_mul(g), rtol=1e-2, atol=5e-3)


def _expert_weights(experts, k, n, dtype, zeros, seed):
    import infini.ops

    q = np.empty((experts, k, n), dtype=np.uint8)
    scales = torch.empty((experts, k // 128, n), dtype=dtype)
    z = np.empty((experts, k // 128, n), dtype=np.uint8) if zeros else None
    packed = torch.empty((experts, k // 16, 2 * n), dtype=torch.int32, device="cuda")
    zp = torch.empty((experts, k // 128, n // 8), dtype=torch.int32, device="cuda") if zeros else None
    for e in range(experts):
        qe, se, ze = make_quantized(k, n, 128, dtype, zeros, seed + e)
        q[e], scales[e] = qe, se
        if zeros:
            z[e] = ze
            zp[e] = torch.from_numpy(oq.pack_zeros(ze)).cuda()
            infini.ops.awq_marlin_repack(torch.from_numpy(oq.awq_pack(qe, 4)).cuda(), k, n, 4, False, packed[e])
        else:
            infini.ops.gptq_marlin_repack(torch.from_numpy(oq.gptq_pack(qe, 4)).cuda(),
                                          torch.empty(0, dtype=torch.int32, device="cuda"), k, n, 4, False, packed[e])
    return q, scales, z, packed, zp


def _moe_gemm(a, packed, scales, zp, sorted_ids, expert_ids, npost, tw, block, top_k, mul, size_m, n, k, out):
    import infini.ops

    workspace = torch.zeros(432, dtype=torch.int32, device="cuda")
    infini.ops.moe_wna16_marlin_gemm(a, packed, None, scales, None, None, zp, None, None, workspace, sorted_ids,
                                     expert_ids, npost, tw, block, top_k, mul, UINT4 if zp is not None else UINT4B8,
                                     size_m, n, k, True, False, True, False, -1, -1, -1, out, stream=_stream())


@pytest.mark.parametrize("tokens,experts,topk,hidden,inter,block,zeros", (
    (1, 8, 2, 512, 256, 64, False),      # Mixtral-shaped routing, one token
    (64, 8, 2, 512, 384, 64, False),
    (300, 8, 2, 256, 256, 16, False),
    (16, 32, 8, 512, 128, 64, True),     # DeepSeek-shaped routing (grouped, AWQ zeros), fewer experts
    (200, 32, 8, 256, 128, 32, True),
    (1000, 8, 2, 256, 256, 64, False),   # enough rows per expert for merged 256-row tiles
    (900, 8, 2, 384, 512, 64, False),    # merged tiles, ragged runs of blocks
))
def test_moe_layer_against_oracle(tokens, experts, topk, hidden, inter, block, zeros):
    """router -> sort -> w13 GEMM -> silu_and_mul -> w2 GEMM (x routing weight) -> moe_sum, every stage
    compared with the oracle on the stage's own inputs (so errors do not accumulate across stages)."""
    import infini.ops

    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(tokens * 31 + experts)
    x = torch.randn((tokens, hidden), generator=gen).to(dtype)
    w = torch.empty((tokens, topk), device="cuda")
    ids = torch.empty((tokens, topk), dtype=torch.int32, device="cuda")
    if zeros:
        scores = torch.randn((tokens, experts), generator=gen)
        bias = torch.randn(experts, generator=gen) * 0.1
        infini.ops.grouped_topk(scores.cuda(), bias.cuda(), 8, 4, topk, True, 2.5, 1, w, ids)
        rw, rids = omoe.grouped_topk(scores, bias, 8, 4, topk, True, 2.5, 1)
    else:
        logits = torch.randn((tokens, experts), generator=gen)
        tei = torch.empty((tokens, topk), dtype=torch.int32, device="cuda")
        infini.ops.topk_softmax(logits.cuda(), None, None, True, w, ids, tei)
        rw, rids, _ = omoe.topk_softmax(logits, None, None, topk, True)
    assert torch.equal(ids.cpu().long(), rids.long())
    size, blocks = omoe.padded_sizes(tokens * topk, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    infini.ops.moe_align_block_size(ids, None, experts, block, sorted_ids, expert_ids, npost)
    rs, re, rn = omoe.moe_align_block_size(ids.cpu(), None, experts, block)
    assert np.array_equal(sorted_ids.cpu().numpy(), rs) and np.array_equal(expert_ids.cpu().numpy(), re)

    q13, s13, z13, w13, zp13 = _expert_weights(experts, hidden, 2 * inter, dtype, zeros, 100)
    q2, s2, z2, w2, zp2 = _expert_weights(experts, inter, hidden, dtype, zeros, 500)
    g = torch.full((tokens * topk, 2 * inter), float("nan"), dtype=dtype, device="cuda")
    _moe_gemm(x.cuda(), w13, s13.cuda(), zp13, sorted_ids, expert_ids, npost, w.flatten(), block, topk, False, tokens,
              2 * inter, hidden, g)
    rg = omoe.moe_w4a16_gemm(x, q13, s13, z13, rs, re, rn, None, block, topk, False)
    assert rel_max_err(g, rg) <= 1e-2
    h = torch.empty((tokens * topk, inter), dtype=dtype, device="cuda")
    infini.ops.silu_and_mul(g, h)
    torch.testing.assert_close(h.cpu(), omoe.silu_and_mul(g.cpu()), rtol=1e-2, atol=5e-3)
    y = torch.full((tokens * topk, hidden), float("nan"), dtype=dtype, device="cuda")
    _moe_gemm(h, w2, s2.cuda(), zp2, sorted_ids, expert_ids, npost, w.flatten(), block, 1, True, tokens * topk, hidden,
              inter, y)
    ry = omoe.moe_w4a16_gemm(h.cpu(), q2, s2, z2, rs, re, rn, w.flatten().cpu(), block, 1, True)
    assert rel_max_err(y, ry) <= 1e-2
    out = torch.empty((tokens, hidden), dtype=dtype, device="cuda")
    infini.ops.moe_sum(y.view(tokens, topk, hidden), out)
    torch.testing.assert_close(out.cpu(), omoe.moe_sum(y.view(tokens, topk, hidden).cpu()), rtol=1e-2, atol=1e-2)


def test_moe_gemm_expert_map_skips_blocks_and_leaves_rows_untouched():
    """Blocks whose expert id is -1 (expert not on this rank) are skipped; their rows keep their content."""
    import infini.ops

    tokens, experts, topk, hidden, n, block = 40, 8, 2, 256, 128, 16
    x = torch.randn((tokens, hidden)).bfloat16()
    ids = torch.randint(0, experts, (tokens, topk), dtype=torch.int32)
    emap = torch.tensor([0, 1, 2, 3, -1, -1, -1, -1], dtype=torch.int32)   # this rank owns experts 0..3
    size, blocks = omoe.padded_sizes(tokens * topk, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    infini.ops.moe_align_block_size(ids.cuda(), emap.cuda(), experts, block, sorted_ids, expert_ids, npost)
    rs, re, rn = omoe.moe_align_block_size(ids, emap, experts, block)
    assert np.array_equal(sorted_ids.cpu().numpy(), rs)
    q, s, _, packed, _ = _expert_weights(4, hidden, n, torch.bfloat16, False, 9)
    out = torch.full((tokens * topk, n), 7.0, dtype=torch.bfloat16, device="cuda")
    tw = torch.rand(tokens * topk, device="cuda")
    _moe_gemm(x.cuda(), packed, s.cuda(), None, sorted_ids, expert_ids, npost, tw, block, topk, True, tokens, n, hidden, out)
    ref = omoe.moe_w4a16_gemm(x, q, s, None, rs, re, rn, tw.cpu(), block, topk, True)
    routed = torch.zeros(tokens * topk, dtype=torch.bool)
    routed[torch.from_numpy(rs[: int(rn[0])][rs[: int(rn[0])] < tokens * topk].astype(np.int64))] = True
    assert rel_max_err(out[routed.cuda()], ref[routed]) <= 1e-2
    assert bool((out[~routed.cuda()] == 7.0).all())


def test_dense_marlin_gemm_through_module_and_trace_line():
    import infini.ops

    m, k, n = 16, 1024, 512
    q, scales, zeros = make_quantized(k, n, 128, torch.float16, True, 77)
    a = torch.randn((m, k)).half()
    packed = torch.empty((k // 16, 2 * n), dtype=torch.int32, device="cuda")
    infini.ops.awq_marlin_repack(torch.from_numpy(oq.awq_pack(q, 4)).cuda(), k, n, 4, False, packed)
    out = torch.empty((m, n), dtype=torch.float16, device="cuda")
    workspace = torch.zeros(432, dtype=torch.int32, device="cuda")
    infini.ops.marlin_gemm(a.cuda(), packed, None, scales.cuda(), None, None,
                           torch.from_numpy(oq.pack_zeros(zeros)).cuda(), None, None, workspace, UINT4, m, n, k, True,
                           False, True, False, out, stream=_stream())
    assert rel_max_err(out, oq.w4a16_gemm(a, q, scales, zeros)) <= 1e-2
    assert int(workspace.abs().sum()) == 0
    script = textwrap.dedent("""
        import torch, infini.ops
        x = torch.randn((4, 16), device="cuda"); out = torch.empty((4, 8), device="cuda")
        infini.ops.silu_and_mul(x, out); torch.cuda.synchronize()
    """)
    env = dict(os.environ, INFINI_OPS_TRACE_CALLS="1")
    r = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stderr
    assert '[INFINI_OPS_TRACE_CALLS] {"operator_name": "SiluAndMul", "device_type": "nvidia", "implementation": 0}' in r.stderr


def test_device_guard_runs_on_the_tensors_device_and_restores_the_callers():
    """Tensors on cuda:1 while cuda:0 is current: the operators launch on the tensors' device and leave
    the caller's current device alone (tests/test_topk_softmax.py:258-288 of the reference).  Needs two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import infini.ops

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 1)
    logits = torch.randn((33, 8))
    w = torch.empty((33, 2), device=dev)
    ids = torch.empty((33, 2), dtype=torch.int32, device=dev)
    tei = torch.empty((33, 2), dtype=torch.int32, device=dev)
    with torch.cuda.device(1):
        stream = torch.cuda.current_stream(dev).cuda_stream
    infini.ops.topk_softmax(logits.to(dev), None, None, True, w, ids, tei, stream=stream)
    assert torch.cuda.current_device() == 0
    rw, rids, _ = omoe.topk_softmax(logits, None, None, 2, True)
    assert torch.equal(ids.cpu().long(), rids)
    # a GEMM too: its tensor maps and scratch belong to device 1
    m, k, n = 16, 512, 256
    q, scales, zeros = make_quantized(k, n, 128, torch.float16, True, 5)
    a = torch.randn((m, k)).half()
    packed = torch.from_numpy(oq.marlin_pack(q, 4, False)).to(dev)
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    workspace = torch.zeros(432, dtype=torch.int32, device=dev)
    infini.ops.marlin_gemm(a.to(dev), packed, None, scales.to(dev), None, None, torch.from_numpy(oq.pack_zeros(zeros)).to(dev),
                           None, None, workspace, UINT4, m, n, k, True, False, True, False, out, stream=stream)
    assert torch.cuda.current_device() == 0
    assert rel_max_err(out, oq.w4a16_gemm(a, q, scales, zeros)) <= 1e-2
