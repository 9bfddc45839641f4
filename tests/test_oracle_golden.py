"""CPU: the oracle reproduces every golden vector generated from the reference's test helpers."""

import numpy as np
import torch

from oracle import moe as omoe
from oracle import quant as oq

_DT = {0: torch.float32, 1: torch.float16, 2: torch.bfloat16}


def test_repack_golden(golden):
    g = golden["repack"]
    keys = [k[:-3] for k in g.files if k.endswith("_in")]
    assert len(keys) == 24
    for key in keys:
        parts = key.split("_")
        if parts[0] == "gptq":
            _, k, n, bits, a8, _perm = parts
            got = oq.gptq_marlin_repack(g[key + "_in"], g[key + "_perm"], int(k), int(n), int(bits), bool(int(a8)))
        else:
            _, k, n, bits, a8 = parts
            got = oq.awq_marlin_repack(g[key + "_in"], int(k), int(n), int(bits), bool(int(a8)))
        assert np.array_equal(got, g[key + "_out"]), key


def test_marlin_pack_roundtrip():
    rng = np.random.default_rng(0)
    for bits, a8 in ((4, False), (8, False), (4, True), (8, True)):
        w = rng.integers(0, 1 << bits, size=(64, 128), dtype=np.uint8)
        packed = oq.marlin_pack(w, bits, a8)
        assert packed.shape == (4, 128 * 16 * bits // 32)
        assert np.array_equal(oq.marlin_unpack(packed, 64, 128, bits, a8), w)


def test_fast_w4_unpack_matches_the_index_map():
    rng = np.random.default_rng(1)
    for k, n in ((16, 64), (128, 192), (512, 256)):
        words = rng.integers(-2**31, 2**31 - 1, size=(k // 16, 2 * n), dtype=np.int64).astype(np.int32)
        assert np.array_equal(oq.marlin_unpack_w4(words, k, n), oq.marlin_unpack(words, k, n, 4, False))


def test_topk_softmax_golden(golden):
    g = golden["topk_softmax"]
    bias = torch.from_numpy(g["bias"])
    for i in range(int(g["n_cases"][0])):
        dt, has_bias, renorm, topk = (int(v) for v in g[f"c{i}_meta"])
        gate = torch.from_numpy(g[f"c{i}_gate"]).to(_DT[dt])
        w, idx, tei = omoe.topk_softmax(gate, bias if has_bias else None, None, topk, bool(renorm))
        assert np.array_equal(idx.numpy(), g[f"c{i}_idx"])
        assert np.array_equal(tei.numpy(), g[f"c{i}_tei"])
        np.testing.assert_allclose(w.numpy(), g[f"c{i}_w"], rtol=1e-6, atol=1e-6)
    w, idx, tei = omoe.topk_softmax(torch.from_numpy(g["pad_gate"]).half(), None, torch.from_numpy(g["pad_mask"]), 3, False)
    assert np.array_equal(idx.numpy(), g["pad_idx"]) and np.array_equal(tei.numpy(), g["pad_tei"])


def test_topk_softmax_ties_and_bias():
    # tests/test_topk_softmax.py:169-187 and :61-80 of the reference
    _, idx, _ = omoe.topk_softmax(torch.zeros((1, 4)), None, None, 3, False)
    assert idx.tolist() == [[0, 1, 2]]
    w, idx, _ = omoe.topk_softmax(torch.tensor([[3.0, 2.0, 1.0]]), torch.tensor([-4.0, 0.0, 3.0]), None, 1, False)
    assert idx.item() == 2
    torch.testing.assert_close(w, torch.softmax(torch.tensor([[3.0, 2.0, 1.0]]), -1)[:, 2:3])


def test_grouped_topk_golden(golden):
    g = golden["grouped_topk"]
    for i in range(int(g["n_cases"][0])):
        sd, bd, neg, tg, k, renorm, sf = (int(v) for v in g[f"c{i}_meta"])
        scores = torch.from_numpy(g[f"c{i}_scores"]).to(_DT[sd])
        bias = torch.from_numpy(g[f"c{i}_bias"]).to(_DT[bd])
        v, idx = omoe.grouped_topk(scores, bias, neg, tg, k, bool(renorm), float(g[f"c{i}_rsf"][0]), sf)
        assert np.array_equal(idx.numpy(), g[f"c{i}_idx"]), i
        np.testing.assert_allclose(v.numpy(), g[f"c{i}_v"], rtol=1e-6, atol=1e-6)
    scores = torch.from_numpy(g["nonfinite_scores"])
    for sf in (0, 1):
        v, idx = omoe.grouped_topk(scores, torch.zeros(8), 2, 2, 4, False, 1.0, sf)
        assert np.array_equal(idx.numpy(), g[f"nonfinite{sf}_idx"])


def test_grouped_topk_tie_kats():
    # tests/test_grouped_topk.py:206-263 of the reference
    _, idx = omoe.grouped_topk(torch.full((1, 8), 0.5), torch.zeros(8), 2, 2, 4, False, 1.0, 0)
    assert idx.tolist() == [[0, 1, 2, 3]]
    scores = torch.tensor([[0.9, 0.8, 0.9, 0.8, 0.9, 0.8, 0.9, 0.8]])
    v, idx = omoe.grouped_topk(scores, torch.zeros(8), 4, 2, 2, False, 1.0, 0)
    assert idx.tolist() == [[0, 2]]


def test_moe_align_golden(golden):
    g = golden["moe_align"]
    for i in range(int(g["n_cases"][0])):
        ne, bs = (int(v) for v in g[f"c{i}_meta"])
        emap = g[f"c{i}_emap"]
        s, e, npost = omoe.moe_align_block_size(g[f"c{i}_ids"], emap if emap.size else None, ne, bs)
        assert np.array_equal(s, g[f"c{i}_sorted"]) and np.array_equal(e, g[f"c{i}_experts"])
        assert np.array_equal(npost, g[f"c{i}_npost"])


def test_dequant_matmul_golden(golden):
    g = golden["moe_dequant_matmul"]
    for i in range(int(g["n_cases"][0])):
        has_zp, mul, dt = (int(v) for v in g[f"c{i}_meta"])
        x = torch.from_numpy(g[f"c{i}_x"]).to(_DT[dt])
        s = torch.from_numpy(g[f"c{i}_s"]).to(_DT[dt])
        out = omoe.moe_w4a16_gemm(x, g[f"c{i}_q"], s, g[f"c{i}_z"] if has_zp else None, g[f"c{i}_sorted"],
                                  g[f"c{i}_experts"], g[f"c{i}_npost"], g[f"c{i}_tw"] if mul else None, 2, 2, bool(mul))
        ref = torch.from_numpy(g[f"c{i}_out"]).reshape(out.shape)
        torch.testing.assert_close(out.to(_DT[dt]).float(), ref, rtol=0, atol=0)


def test_silu_and_moe_sum_oracle():
    x = torch.randn(5, 12)
    torch.testing.assert_close(omoe.silu_and_mul(x), torch.nn.functional.silu(x[:, :6]) * x[:, 6:])
    y = torch.randn(3, 4, 17)
    ids = torch.tensor(((0, 1, -1, 2), (2, -1, 1, 0), (1, 2, 0, -1)))
    emap = torch.tensor((0, -1, 1), dtype=torch.int32)
    active = (ids >= 0) & (emap[ids.clamp_min(0)] >= 0)
    torch.testing.assert_close(omoe.moe_sum(y, ids, emap), (y * active.unsqueeze(-1)).sum(1))
