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


def test_topk_sigmoid_golden(golden):
    g = golden["topk_sigmoid"]
    bias = torch.from_numpy(g["bias"])
    for i in range(int(g["n_cases"][0])):
        dt, has_bias, renorm = (int(v) for v in g[f"c{i}_meta"])
        gate = torch.from_numpy(g[f"c{i}_gate"]).to(_DT[dt])
        w, ids, tei = omoe.topk_sigmoid(gate, bias if has_bias else None, None, 2, bool(renorm), 0.75)
        assert np.array_equal(ids.numpy(), g[f"c{i}_ids"]) and np.array_equal(tei.numpy(), g[f"c{i}_tei"])
        np.testing.assert_allclose(w.numpy(), g[f"c{i}_w"], rtol=0, atol=0)
    w, ids, tei = omoe.topk_sigmoid(torch.from_numpy(g["pad_gate"]).half(), None, torch.from_numpy(g["pad_mask"]), 3, True, 1.0)
    assert np.array_equal(ids.numpy(), g["pad_ids"]) and np.array_equal(tei.numpy(), g["pad_tei"])
    w, ids, _ = omoe.topk_sigmoid(torch.full((1, 4), float("nan")), None, None, 2, False, 1.0)
    assert ids.tolist() == [[0, 1]] and w.tolist() == [[0.0, 0.0]]


def test_moe_wna16_gemm_golden(golden):
    g = golden["moe_wna16_gemm"]
    for i in range(int(g["n_cases"][0])):
        bit, has_zp, mul, dt, group_size, k = (int(v) for v in g[f"c{i}_meta"])
        q, z = _unpack_plain(g[f"c{i}_qw"], g[f"c{i}_qz"] if has_zp else None, bit)
        x = torch.from_numpy(g[f"c{i}_x"]).to(_DT[dt])
        s = torch.from_numpy(g[f"c{i}_s"]).to(_DT[dt])
        out = omoe.moe_wna16_gemm(x, q, s, z, bit, torch.from_numpy(g[f"c{i}_tw"]) if mul else None, g[f"c{i}_sorted"],
                                  g[f"c{i}_experts"], g[f"c{i}_npost"], 2, 2)
        tol = 2e-2 if dt == 1 else 5e-2
        torch.testing.assert_close(out.to(_DT[dt]).float(), torch.from_numpy(g[f"c{i}_out"]), rtol=tol, atol=tol)


def _unpack_plain(qw, qz, bit):
    """uint8-packed weight [E, N, K / (8 / bit)] and zero points [E, N / (8 / bit), G] -> integers."""
    if bit == 8:
        return qw.astype(np.int64), None if qz is None else qz.astype(np.int64)
    q = np.stack((qw & 0xF, qw >> 4), axis=-1).reshape(qw.shape[0], qw.shape[1], -1).astype(np.int64)
    z = None
    if qz is not None:
        z = np.stack((qz & 0xF, qz >> 4), axis=2).reshape(qz.shape[0], -1, qz.shape[2]).astype(np.int64)
    return q, z


def test_moe_mm_data_oracle_shapes(golden):
    g = golden["moe_mm_data"]
    for i in range(int(g["n_cases"][0])):
        experts, blockscale = (int(v) for v in g[f"c{i}_meta"])
        ids = g[f"c{i}_ids"]
        offsets, ps1, ps2, in_perm, out_perm, scale = omoe.get_cutlass_moe_mm_data(ids, experts, 64, 128, True, bool(blockscale))
        valid = int(((ids >= 0) & (ids < experts)).sum())
        assert offsets[-1] == valid and sorted(out_perm[(ids.reshape(-1) >= 0) & (ids.reshape(-1) < experts)].tolist()) == list(range(valid))
        assert (scale is not None) == bool(blockscale)


def test_float8_dequantisation_known_values():
    """float8_e4m3fn bytes by the type's definition: bias 7, three mantissa bits, subnormals below 2**-6,
    largest finite value 448."""
    import numpy as np
    import torch

    from oracle import quant as oq

    q = np.array([[0x38, 0x40, 0x7E, 0x01, 0xB8, 0x08, 0x07, 0x00]], dtype=np.uint8).T.repeat(2, axis=1)
    got = oq.dequantize_float8(q, torch.tensor([[1.0, 0.5]]))
    want = torch.tensor([1.0, 2.0, 448.0, 2.0**-9, -1.0, 2.0**-6, 7 * 2.0**-9, 0.0])
    assert torch.equal(got[:, 0], want) and torch.equal(got[:, 1], want * 0.5)
