"""GPU: the sibling MoE operators -- topk_sigmoid, moe_wna16_gemm (plain weight layout, 4 and 8 bit)
and get_cutlass_moe_mm_data -- through `infini.ops`, against golden vectors made with the
reference's own test helpers and against the oracle at layer sizes."""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from tests.test_oracle_golden import _unpack_plain

pytestmark = pytest.mark.gpu
_DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _sigmoid(gate, bias, pad, topk, renorm, scale, index_dtype=torch.int32):
    import infini.ops

    shape = (gate.shape[0], topk)
    w = torch.full(shape, torch.nan, dtype=torch.float32, device="cuda")
    ids = torch.full(shape, 2**31 - 1, dtype=index_dtype, device="cuda")
    tei = torch.full(shape, -1, dtype=torch.int32, device="cuda")
    infini.ops.topk_sigmoid(gate, bias, pad, renorm, scale, w, ids, tei, stream=_stream())
    return w.cpu(), ids.cpu(), tei.cpu()


def test_topk_sigmoid_golden(golden):
    g = golden["topk_sigmoid"]
    bias = torch.from_numpy(g["bias"]).cuda()
    for i in range(int(g["n_cases"][0])):
        dt, has_bias, renorm = (int(v) for v in g[f"c{i}_meta"])
        gate = torch.from_numpy(g[f"c{i}_gate"]).to(_DT[dt]).cuda()
        for index_dtype in (torch.int32, torch.int64, torch.uint32):
            w, ids, tei = _sigmoid(gate, bias if has_bias else None, None, 2, bool(renorm), 0.75, index_dtype)
            assert np.array_equal(ids.numpy().astype(np.int64), g[f"c{i}_ids"]) and np.array_equal(tei.numpy(), g[f"c{i}_tei"])
            np.testing.assert_allclose(w.numpy(), g[f"c{i}_w"], rtol=1e-6, atol=1e-6)
    pad = torch.from_numpy(g["pad_mask"]).cuda()
    w, ids, tei = _sigmoid(torch.from_numpy(g["pad_gate"]).half().cuda(), None, pad, 3, True, 1.0)
    assert np.array_equal(ids.numpy(), g["pad_ids"]) and np.array_equal(tei.numpy(), g["pad_tei"])
    np.testing.assert_allclose(w.numpy(), g["pad_w"], rtol=1e-6, atol=1e-6)


def test_topk_sigmoid_known_answers():
    # the correction bias changes the selection only; the weight stays the un-biased score
    gate = torch.tensor(((3.0, 2.0, 1.0),), device="cuda")
    w, ids, _ = _sigmoid(gate, torch.tensor((0.0, 0.0, 1.0), device="cuda"), None, 1, False, 1.0)
    assert ids.tolist() == [[2]]
    torch.testing.assert_close(w, torch.sigmoid(gate.cpu())[:, 2:3])
    # all-NaN row: every score counts as 0, ties go to the lower ids
    w, ids, _ = _sigmoid(torch.full((1, 4), torch.nan, device="cuda"), None, None, 2, False, 1.0)
    assert ids.tolist() == [[0, 1]] and w.tolist() == [[0.0, 0.0]]
    # empty input: nothing launched, nothing touched
    infini_empty = _sigmoid(torch.empty((0, 4), device="cuda"), None, None, 2, True, 1.0)
    assert infini_empty[0].shape == (0, 2)


@pytest.mark.parametrize("tokens,experts,topk,dtype", ((4096, 8, 2, torch.float32), (8192, 256, 8, torch.bfloat16),
                                                      (513, 160, 6, torch.float16)))
def test_topk_sigmoid_layer_sizes(tokens, experts, topk, dtype):
    gate = torch.randn((tokens, experts)).to(dtype)
    bias = torch.randn(experts) * 0.1
    w, ids, tei = _sigmoid(gate.cuda(), bias.cuda(), None, topk, True, 2.5)
    rw, rids, rtei = omoe.topk_sigmoid(gate, bias, None, topk, True, 2.5)
    # expf on the device and torch.sigmoid on the host may differ in the last bit: a row whose
    # selection differs must be a tie at that precision
    same = (ids.long() == rids).all(dim=1)
    assert same.float().mean() > 0.999
    sel = torch.sigmoid(gate.float()) + bias
    for row in torch.nonzero(~same).flatten().tolist():
        got = torch.sort(sel[row][ids[row].long()], descending=True).values
        ref = torch.sort(sel[row][rids[row]], descending=True).values
        assert float((got - ref).abs().max()) <= 2.4e-7
    torch.testing.assert_close(w[same], rw[same], rtol=1e-5, atol=1e-6)
    assert torch.equal(tei, rtei)


def test_moe_wna16_gemm_golden(golden):
    import infini.ops

    g = golden["moe_wna16_gemm"]
    for i in range(int(g["n_cases"][0])):
        bit, has_zp, mul, dt, group_size, k = (int(v) for v in g[f"c{i}_meta"])
        dtype = _DT[dt]
        x = torch.from_numpy(g[f"c{i}_x"]).to(dtype).cuda()
        s = torch.from_numpy(g[f"c{i}_s"]).to(dtype).cuda()
        qw = torch.from_numpy(g[f"c{i}_qw"]).cuda()
        qz = torch.from_numpy(g[f"c{i}_qz"]).cuda() if has_zp else None
        tw = torch.from_numpy(g[f"c{i}_tw"]).cuda() if mul else None
        out = torch.full((2, 2, qw.shape[1]), torch.nan, dtype=dtype, device="cuda")
        infini.ops.moe_wna16_gemm(x, qw, s, qz, tw, torch.from_numpy(g[f"c{i}_sorted"]).cuda(),
                                  torch.from_numpy(g[f"c{i}_experts"]).cuda(), torch.from_numpy(g[f"c{i}_npost"]).cuda(),
                                  2, 2, 16, k, bit, out, stream=_stream())
        tol = 2e-2 if dt == 1 else 5e-2
        torch.testing.assert_close(out.float().cpu(), torch.from_numpy(g[f"c{i}_out"]), rtol=tol, atol=tol)


@pytest.mark.parametrize("bit,zeros", ((4, True), (4, False), (8, True)))
def test_moe_wna16_gemm_layer_shape(bit, zeros):
    """E=8, top-2, H=1024 -> N=768, group 128, block 16, 300 tokens: the routing comes from the
    library's own sort; blocks of absent experts (-1) are skipped and their rows read zero."""
    import infini.ops

    tokens, experts, top_k, k, n, group, block = 300, 8, 2, 1024, 768, 128, 16
    dtype = torch.bfloat16
    gen = torch.Generator().manual_seed(bit * 10 + zeros)
    q = torch.randint(0, 1 << bit, (experts, n, k), generator=gen)
    z = torch.randint(1 << (bit - 2), 3 << (bit - 2), (experts, n, k // group), generator=gen) if zeros else None
    s = (torch.rand((experts, n, k // group), generator=gen) * 0.05 + 0.01).to(dtype)
    x = torch.randn((tokens, k), generator=gen).to(dtype)
    ids = torch.randint(0, experts, (tokens, top_k), generator=gen, dtype=torch.int32)
    emap = torch.tensor([0, 1, 2, -1, 4, 5, 6, 7], dtype=torch.int32)
    size, blocks = omoe.padded_sizes(tokens * top_k, experts, block)
    sorted_ids = torch.empty(size, dtype=torch.int32, device="cuda")
    expert_ids = torch.empty(blocks, dtype=torch.int32, device="cuda")
    npost = torch.empty(1, dtype=torch.int32, device="cuda")
    infini.ops.moe_align_block_size(ids.cuda(), emap.cuda(), experts, block, sorted_ids, expert_ids, npost)

    def pack(values, axis):
        if bit == 8:
            return values.to(torch.uint8).contiguous()
        lo = values.index_select(axis, torch.arange(0, values.shape[axis], 2))
        hi = values.index_select(axis, torch.arange(1, values.shape[axis], 2))
        return (lo | (hi << 4)).to(torch.uint8).contiguous()

    tw = torch.rand((tokens, top_k), generator=gen)
    out = torch.full((tokens, top_k, n), torch.nan, dtype=dtype, device="cuda")
    infini.ops.moe_wna16_gemm(x.cuda(), pack(q, 2).cuda(), s.cuda(), None if z is None else pack(z, 1).cuda(), tw.cuda(),
                              sorted_ids, expert_ids, npost, top_k, block, 128, 128, bit, out, stream=_stream())
    ref = omoe.moe_wna16_gemm(x, q.numpy(), s, None if z is None else z.numpy(), bit, tw, sorted_ids.cpu(), expert_ids.cpu(),
                              npost.cpu(), block, top_k)
    err = float((out.float().cpu() - ref).abs().max() / ref.abs().max())
    assert err <= 1e-2, err
    absent = (ids == 3)
    assert bool((out.cpu()[absent] == 0).all())


def _mm_data(ids, experts, n, k, gated, blockscale):
    import infini.ops

    numel = ids.numel()
    outs = [torch.full((experts + 1,), -7, dtype=torch.int32, device="cuda"),
            torch.full((experts, 3), -7, dtype=torch.int32, device="cuda"),
            torch.full((experts, 3), -7, dtype=torch.int32, device="cuda"),
            torch.full((numel,), -7, dtype=torch.int32, device="cuda"),
            torch.full((numel,), -7, dtype=torch.int32, device="cuda")]
    scale = torch.full((experts + 1,), -7, dtype=torch.int32, device="cuda") if blockscale else None
    if gated is None:
        infini.ops.get_cutlass_moe_mm_data(ids, experts, n, k, *outs, scale, stream=_stream())
    else:
        infini.ops.get_cutlass_moe_mm_data(ids, experts, n, k, gated, *outs, scale, stream=_stream())
    return [o.cpu().numpy() for o in outs] + [None if scale is None else scale.cpu().numpy()]


def test_get_cutlass_moe_mm_data_golden_tables(golden):
    g = golden["moe_mm_data"]
    for i in range(int(g["n_cases"][0])):
        experts, blockscale = (int(v) for v in g[f"c{i}_meta"])
        ids = torch.from_numpy(g[f"c{i}_ids"]).cuda()
        for gated in (True, False, None):
            got = _mm_data(ids, experts, 64, 128, gated, bool(blockscale))
            ref = omoe.get_cutlass_moe_mm_data(ids.cpu(), experts, 64, 128, gated is not False, bool(blockscale))
            for a, b in zip(got, ref):
                assert (a is None and b is None) or np.array_equal(a, b), (i, gated)


def test_get_cutlass_moe_mm_data_layer_size_and_determinism():
    ids = torch.randint(0, 256, (8192, 8), dtype=torch.int32)
    ids[5, 3] = -1
    first = _mm_data(ids.cuda(), 256, 2048, 7168, True, False)
    ref = omoe.get_cutlass_moe_mm_data(ids, 256, 2048, 7168, True, False)
    for a, b in zip(first, ref):
        assert (a is None and b is None) or np.array_equal(a, b)
    again = _mm_data(ids.cuda(), 256, 2048, 7168, True, False)
    assert all((a is None and b is None) or np.array_equal(a, b) for a, b in zip(first, again))
