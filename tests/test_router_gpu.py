"""GPU: topk_softmax and grouped_topk through the C ABI against golden vectors and the oracle."""

import numpy as np
import pytest
import torch

from oracle import moe as omoe

pytestmark = pytest.mark.gpu
_DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def _capi():
    from infiniops_b200 import capi
    return capi


def _run_topk_softmax(gate, bias, pad, topk, renorm, index_dtype=torch.int32, stream=None):
    capi = _capi()
    shape = (gate.shape[0], topk)
    w = torch.full(shape, torch.nan, dtype=torch.float32, device="cuda")
    idx = torch.full(shape, 2**31 - 1, dtype=index_dtype, device="cuda")
    tei = torch.full(shape, -1, dtype=torch.int32, device="cuda")
    capi.topk_softmax(gate, bias, pad, renorm, w, idx, tei, stream=stream)
    return w, idx, tei


def test_topk_softmax_golden(golden):
    g = golden["topk_softmax"]
    bias = torch.from_numpy(g["bias"]).cuda()
    for i in range(int(g["n_cases"][0])):
        dt, has_bias, renorm, topk = (int(v) for v in g[f"c{i}_meta"])
        gate = torch.from_numpy(g[f"c{i}_gate"]).to(_DT[dt]).cuda()
        for index_dtype in (torch.int32, torch.int64, torch.uint32):
            w, idx, tei = _run_topk_softmax(gate, bias if has_bias else None, None, topk, bool(renorm), index_dtype)
            assert np.array_equal(idx.cpu().numpy().astype(np.int64), g[f"c{i}_idx"])
            assert np.array_equal(tei.cpu().numpy(), g[f"c{i}_tei"])
            np.testing.assert_allclose(w.cpu().numpy(), g[f"c{i}_w"], rtol=1e-6, atol=1e-6)


def test_topk_softmax_padding_ties_bias_empty(golden):
    g = golden["topk_softmax"]
    pad = torch.from_numpy(g["pad_mask"]).to(torch.uint8).cuda()
    w, idx, tei = _run_topk_softmax(torch.from_numpy(g["pad_gate"]).half().cuda(), None, pad, 3, False, torch.int64)
    assert np.array_equal(idx.cpu().numpy(), g["pad_idx"]) and np.array_equal(tei.cpu().numpy(), g["pad_tei"])
    np.testing.assert_allclose(w.cpu().numpy(), g["pad_w"], rtol=1e-5, atol=1e-6)
    # uint32 padding sentinel
    _, idx, _ = _run_topk_softmax(torch.tensor([[1.0, 2.0, 3.0]], device="cuda"),
                                  None, torch.tensor([1], dtype=torch.uint8, device="cuda"), 2, False, torch.uint32)
    assert idx.cpu().numpy().tolist() == [[2**32 - 1, 2**32 - 1]]
    # ties go to the smaller index
    _, idx, _ = _run_topk_softmax(torch.zeros((1, 4), device="cuda"), None, None, 3, False)
    assert idx.cpu().tolist() == [[0, 1, 2]]
    # the bias changes the selection only
    gate = torch.tensor([[3.0, 2.0, 1.0]], device="cuda")
    w, idx, _ = _run_topk_softmax(gate, torch.tensor([-4.0, 0.0, 3.0], device="cuda"), None, 1, False)
    assert idx.item() == 2
    torch.testing.assert_close(w.cpu(), torch.softmax(gate.cpu(), -1)[:, 2:3])
    # non-finite bias still yields valid distinct experts, deterministically
    for bad in (float("nan"), float("-inf")):
        bias = torch.full((4,), bad, device="cuda")
        gate = torch.tensor([[1.0, 2.0, 3.0, 4.0]], device="cuda")
        a = _run_topk_softmax(gate, bias, None, 3, False)[1].cpu()
        b = _run_topk_softmax(gate, bias, None, 3, False)[1].cpu()
        assert torch.equal(a, b) and a.min() >= 0 and a.max() < 4 and a.unique().numel() == 3
    # empty
    capi = _capi()
    capi.topk_softmax(torch.empty((0, 4), dtype=torch.float16, device="cuda"), None, None, False,
                      torch.empty((0, 2), device="cuda"), torch.empty((0, 2), dtype=torch.int64, device="cuda"),
                      torch.empty((0, 2), dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("tokens,experts,topk,dtype", ((1, 8, 2, torch.float32), (64, 8, 2, torch.float32),
                                                        (4096, 8, 2, torch.float32), (1024, 8, 2, torch.bfloat16),
                                                        (777, 60, 4, torch.float16), (33, 1500, 6, torch.float32)))
def test_topk_softmax_matches_oracle(tokens, experts, topk, dtype):
    gate = torch.randn((tokens, experts)).to(dtype)
    w, idx, tei = _run_topk_softmax(gate.cuda(), None, None, topk, True)
    rw, ridx, rtei = omoe.topk_softmax(gate, None, None, topk, True)
    assert torch.equal(idx.cpu().long(), ridx)
    assert torch.equal(tei.cpu(), rtei)
    torch.testing.assert_close(w.cpu(), rw, rtol=1e-5, atol=1e-6)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    w2, idx2, _ = _run_topk_softmax(gate.cuda(), None, None, topk, True, stream=stream.cuda_stream)
    stream.synchronize()
    assert torch.equal(idx2, idx) and torch.equal(w2, w)


def _run_grouped(scores, bias, neg, tg, k, renorm, rsf, sf):
    capi = _capi()
    v = torch.full((scores.shape[0], k), torch.nan, dtype=torch.float32, device="cuda")
    idx = torch.full((scores.shape[0], k), -1, dtype=torch.int32, device="cuda")
    before = scores.clone()
    capi.grouped_topk(scores, bias, neg, tg, k, renorm, rsf, sf, v, idx)
    assert torch.equal(scores, before) or bool(torch.isnan(before).any())
    return v.cpu(), idx.cpu()


def test_grouped_topk_golden(golden):
    g = golden["grouped_topk"]
    for i in range(int(g["n_cases"][0])):
        sd, bd, neg, tg, k, renorm, sf = (int(v) for v in g[f"c{i}_meta"])
        scores = torch.from_numpy(g[f"c{i}_scores"]).to(_DT[sd]).cuda()
        bias = torch.from_numpy(g[f"c{i}_bias"]).to(_DT[bd]).cuda()
        v, idx = _run_grouped(scores, bias, neg, tg, k, bool(renorm), float(g[f"c{i}_rsf"][0]), sf)
        assert np.array_equal(idx.numpy(), g[f"c{i}_idx"]), i
        tol = 1e-6 if sd == 0 else 3e-3
        np.testing.assert_allclose(v.numpy(), g[f"c{i}_v"], rtol=tol, atol=tol)
    scores = torch.from_numpy(g["nonfinite_scores"]).cuda()
    for sf in (0, 1):
        v, idx = _run_grouped(scores, torch.zeros(8, device="cuda"), 2, 2, 4, False, 1.0, sf)
        assert torch.isfinite(v).all()
        assert np.array_equal(idx.numpy(), g[f"nonfinite{sf}_idx"])
        np.testing.assert_allclose(v.numpy(), g[f"nonfinite{sf}_v"], rtol=1e-6, atol=1e-6)


def test_grouped_topk_tie_kats():
    v, idx = _run_grouped(torch.full((1, 8), 0.5, device="cuda"), torch.zeros(8, device="cuda"), 2, 2, 4, False, 1.0, 0)
    assert idx.tolist() == [[0, 1, 2, 3]] and torch.equal(v, torch.full((1, 4), 0.5))
    scores = torch.tensor([[0.9, 0.8, 0.9, 0.8, 0.9, 0.8, 0.9, 0.8]], device="cuda")
    v, idx = _run_grouped(scores, torch.zeros(8, device="cuda"), 4, 2, 2, False, 1.0, 0)
    assert idx.tolist() == [[0, 2]] and torch.equal(v, torch.full((1, 2), 0.9))


@pytest.mark.parametrize("tokens", (16, 512, 8192))
@pytest.mark.parametrize("dtype", (torch.float32, torch.bfloat16))
def test_grouped_topk_deepseek_shape(tokens, dtype):
    """E=256, 8 groups, top-4 groups, top-8, sigmoid scores + fp32 bias ~N(0, 0.01)."""
    scores = torch.randn((tokens, 256)).to(dtype)
    bias = torch.randn(256) * 0.1
    v, idx = _run_grouped(scores.cuda(), bias.cuda(), 8, 4, 8, True, 2.5, 1)
    rv, ridx = omoe.grouped_topk(scores, bias, 8, 4, 8, True, 2.5, 1)
    # tanhf on the device and on the host may differ in the last bit (and so may the value
    # rounded to bf16).  Rows whose indices differ are therefore not failed outright, but each one
    # must PROVE it is such a near-tie: see _assert_near_tie.  Everything else must match exactly.
    same = (idx == ridx).all(dim=1)
    assert same.float().mean() > 0.999
    for row in torch.nonzero(~same).flatten().tolist():
        _assert_near_tie(scores[row], bias, idx[row], ridx[row], 8, 4, dtype)
    tol = 1e-5 if dtype == torch.float32 else 3e-3
    torch.testing.assert_close(v[same], rv[same], rtol=tol, atol=tol)


def _assert_near_tie(scores_row, bias, got_idx, ref_idx, groups, topk_group, dtype):
    """A row whose selection differs from the oracle's is accepted only if the difference is a
    rank boundary closer than one unit in the last place of the score type:

    * every group the device took experts from has an oracle group score within 1 ulp of the
      oracle's weakest kept group (or is one of the oracle's kept groups);
    * the oracle selection scores of the device's experts, sorted, are within 1 ulp of those of
      the oracle's experts, sorted (the device picked experts just as good, up to the last bit);
    * the experts both agree on are the same apart from the disputed ones: the symmetric
      difference only holds experts whose scores lie within 1 ulp of the boundary score."""
    ulp = 2.0 ** -23 * 2 if dtype == torch.float32 else 2.0 ** -7   # of values in [1, 2)
    routed = (0.5 * torch.tanh(0.5 * scores_row.float()) + 0.5).to(dtype)
    selection = (routed + bias.to(dtype)).to(dtype).double()
    per = selection.numel() // groups
    group_scores = torch.topk(selection.view(groups, per).float(), 2, dim=-1).values.sum(-1).to(dtype).double()
    kept = torch.topk(group_scores, topk_group).values
    got_groups = set((got_idx // per).tolist())
    for g in got_groups:
        assert float(group_scores[g]) >= float(kept[-1]) - 2 * ulp, f"group {g} is not a near-tie with the kept groups"
    got_sel = torch.sort(selection[got_idx.long()], descending=True).values
    ref_sel = torch.sort(selection[ref_idx.long()], descending=True).values
    group_dispute = got_groups != set((ref_idx // per).tolist())
    if not group_dispute:
        assert float((got_sel - ref_sel).abs().max()) <= ulp, (got_sel, ref_sel)
        disputed = set(got_idx.tolist()) ^ set(ref_idx.tolist())
        boundary = float(ref_sel[-1])
        for e in disputed:
            assert abs(float(selection[e]) - boundary) <= ulp, f"expert {e} is not at the rank boundary"
