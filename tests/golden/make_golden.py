"""Generate the golden fixtures in this folder from the reference's own test helpers.

Run in a container where the reference checkout is available (its path is a required argument):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's test modules (pure torch helpers; `infini.ops` itself
is replaced by an empty stub because the compiled reference library is not
needed for the helpers), evaluates them on CPU, checks that this repository's
oracle reproduces every result, and stores inputs + expected outputs as small
`.npz` files.  The GPU and CPU tests read only the `.npz` files.
"""

from __future__ import annotations

import importlib
import pathlib
import sys
import types

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
REPO = HERE.parent.parent


def _load_reference_tests(ref_root: str):
    stub = types.ModuleType("infini")
    ops = types.ModuleType("infini.ops")
    for name in ("GptqMarlinRepack", "AwqMarlinRepack", "MoeWna16MarlinGemm", "TopkSoftmax",
                 "GroupedTopk", "MoeAlignBlockSize", "SiluAndMul", "MoeSum", "MoeWna16Gemm", "TopkSigmoid",
                 "GetCutlassMoeMmData"):
        setattr(ops, name, type(name, (), {"active_implementation_indices": staticmethod(lambda d: ())}))
    stub.ops = ops
    sys.modules["infini"] = stub
    sys.modules["infini.ops"] = ops
    sys.path.insert(0, ref_root)
    names = ("test_gptq_marlin_repack", "test_awq_marlin_repack", "test_topk_softmax",
             "test_grouped_topk", "test_moe_align_block_size", "test_moe_wna16_gemm", "test_topk_sigmoid",
             "test_get_cutlass_moe_mm_data")
    return {n: importlib.import_module(f"tests.{n}") for n in names}


def main(ref_root: str) -> None:
    sys.path.insert(0, str(REPO))
    from oracle import moe as omoe
    from oracle import quant as oq

    ref = _load_reference_tests(ref_root)
    out: dict[str, np.ndarray] = {}

    # ---- repack -------------------------------------------------------------------------------
    g = ref["test_gptq_marlin_repack"]
    n_cases = 0
    for size_k, size_n in ((128, 64), (256, 128)):
        for bits, a8, has_perm in ((4, False, False), (4, False, True), (8, False, False),
                                   (8, False, True), (4, True, False), (8, True, False)):
            unpacked = g._make_unpacked_weight(size_k, size_n, bits, "cpu")
            packed = g._gptq_pack(unpacked, bits)
            perm = g._make_perm(size_k, "cpu") if has_perm else g._empty_perm("cpu")
            expect = g._marlin_pack(unpacked[perm.long()] if has_perm else unpacked, bits, a8)
            assert np.array_equal(oq.gptq_pack(unpacked.numpy(), bits), packed.numpy())
            mine = oq.gptq_marlin_repack(packed.numpy(), perm.numpy(), size_k, size_n, bits, a8)
            assert np.array_equal(mine, expect.numpy()), ("gptq", size_k, size_n, bits, a8, has_perm)
            assert np.array_equal(oq.marlin_unpack(mine, size_k, size_n, bits, a8),
                                  (unpacked[perm.long()] if has_perm else unpacked).numpy())
            key = f"gptq_{size_k}_{size_n}_{bits}_{int(a8)}_{int(has_perm)}"
            out[key + "_in"] = packed.numpy()
            out[key + "_perm"] = perm.numpy()
            out[key + "_out"] = expect.numpy()
            n_cases += 1
    a = ref["test_awq_marlin_repack"]
    for size_k, size_n in ((128, 64), (256, 128), (128, 832)):
        for bits in (4, 8):
            for a8 in (False, True):
                unpacked = a._make_unpacked_weight(size_k, size_n, bits, "cpu")
                packed = a._awq_pack(unpacked, bits)
                expect = a._marlin_pack(unpacked, bits, a8)
                assert np.array_equal(oq.awq_pack(unpacked.numpy(), bits), packed.numpy())
                mine = oq.awq_marlin_repack(packed.numpy(), size_k, size_n, bits, a8)
                assert np.array_equal(mine, expect.numpy()), ("awq", size_k, size_n, bits, a8)
                key = f"awq_{size_k}_{size_n}_{bits}_{int(a8)}"
                out[key + "_in"] = packed.numpy()
                out[key + "_out"] = expect.numpy()
                n_cases += 1
    np.savez_compressed(HERE / "repack.npz", **out)
    print(f"repack: {n_cases} cases pinned")

    # ---- topk_softmax -------------------------------------------------------------------------
    t = ref["test_topk_softmax"]
    out = {}
    logits = torch.tensor(((1.25, -0.5, 0.75, 2.0, -1.0), (-0.25, 1.5, 0.5, -1.25, 2.25),
                           (0.125, 0.75, 2.5, 1.0, -0.75)))
    bias = torch.tensor((0.0, 0.75, -0.5, -1.0, 1.25))
    i = 0
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        for has_bias in (False, True):
            for renorm in (False, True):
                gate = logits.to(dtype)
                w, idx, tei = t._reference(gate, bias if has_bias else None, None, 2, renorm)
                mw, midx, mtei = omoe.topk_softmax(gate, bias if has_bias else None, None, 2, renorm)
                assert torch.equal(idx, midx) and torch.equal(tei, mtei)
                torch.testing.assert_close(w, mw, rtol=0, atol=0)
                out[f"c{i}_gate"] = gate.float().numpy()
                out[f"c{i}_meta"] = np.array([{torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype],
                                              int(has_bias), int(renorm), 2])
                out[f"c{i}_w"], out[f"c{i}_idx"], out[f"c{i}_tei"] = w.numpy(), idx.numpy(), tei.numpy()
                i += 1
    out["bias"] = bias.numpy()
    # padding case (tests/test_topk_softmax.py:111-140)
    gate = torch.tensor(((0.25, 2.0, -0.5, 1.0), (1.5, -0.25, 0.75, 0.0), (-1.0, 0.5, 2.25, 1.25)),
                        dtype=torch.float16)
    pad = torch.tensor((False, True, False))
    w, idx, tei = t._reference(gate, None, pad, 3, False)
    mw, midx, mtei = omoe.topk_softmax(gate, None, pad, 3, False)
    assert torch.equal(idx, midx) and torch.equal(tei, mtei)
    out["pad_gate"], out["pad_mask"] = gate.float().numpy(), pad.numpy()
    out["pad_w"], out["pad_idx"], out["pad_tei"] = w.numpy(), idx.numpy(), tei.numpy()
    out["n_cases"] = np.array([i])
    np.savez_compressed(HERE / "topk_softmax.npz", **out)
    print(f"topk_softmax: {i + 1} cases pinned")

    # ---- grouped_topk -------------------------------------------------------------------------
    gt = ref["test_grouped_topk"]
    out = {}
    rows = ((torch.float16, torch.float32, (1, 16), 8, 2, 2, False, 1.0, 0),
            (torch.bfloat16, torch.float32, (5, 128), 8, 2, 4, True, 1.0, 0),
            (torch.float32, torch.float16, (3, 256), 8, 4, 8, False, 2.5, 0),
            (torch.float16, torch.bfloat16, (7, 128), 8, 4, 8, True, 2.5, 1),
            (torch.bfloat16, torch.float16, (2, 384), 1, 1, 8, False, 1.0, 1),
            (torch.float32, torch.bfloat16, (4, 512), 1, 1, 22, True, 2.5, 1))
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}
    for i, (sd, bd, shape, neg, tg, k, renorm, rsf, sf) in enumerate(rows):
        scores, b = gt._make_inputs(shape, sd, bd, sf, "cpu")
        v, idx = gt._reference(scores, b, neg, tg, k, renorm, rsf, sf)
        mv, midx = omoe.grouped_topk(scores, b, neg, tg, k, renorm, rsf, sf)
        assert torch.equal(idx, midx), i
        torch.testing.assert_close(v, mv, rtol=0, atol=0)
        out[f"c{i}_scores"], out[f"c{i}_bias"] = scores.float().numpy(), b.float().numpy()
        out[f"c{i}_meta"] = np.array([code[sd], code[bd], neg, tg, k, int(renorm), sf])
        out[f"c{i}_rsf"] = np.array([rsf])
        out[f"c{i}_v"], out[f"c{i}_idx"] = v.numpy(), idx.numpy()
    # non-finite exclusion KAT (tests/test_grouped_topk.py:266-298)
    scores = torch.tensor(((torch.nan, torch.inf, -torch.inf, 0.8, 0.9, 0.7, -0.1, 0.3),))
    for sf in (0, 1):
        v, idx = gt._reference(scores, torch.zeros(8), 2, 2, 4, False, 1.0, sf)
        mv, midx = omoe.grouped_topk(scores, torch.zeros(8), 2, 2, 4, False, 1.0, sf)
        assert torch.equal(idx, midx)
        out[f"nonfinite{sf}_v"], out[f"nonfinite{sf}_idx"] = v.numpy(), idx.numpy()
    out["nonfinite_scores"] = scores.numpy()
    out["n_cases"] = np.array([len(rows)])
    np.savez_compressed(HERE / "grouped_topk.npz", **out)
    print(f"grouped_topk: {len(rows) + 2} cases pinned")

    # ---- moe_align_block_size ---------------------------------------------------------------------
    al = ref["test_moe_align_block_size"]
    out = {}
    tables = [(((0, 2), (0, 2), (2, 0)), None, 4, 2), (((1, 1), (3, 0), (3, 3)), None, 5, 4),
              (((4, 1), (0, 4), (2, 1), (4, 2)), None, 5, 8),
              (((-1, 4), (2**31 - 1, 0), (2, -(2**31))), None, 4, 4),
              (((0, 1), (2, 3), (0, 2), (3, 1)), (0, -1, 1, -1), 4, 4),
              (((-1, 0), (1, 2), (3, 4), (2**31 - 1, 1)), (0, 5, -1, 2), 4, 4)]
    sparse = torch.arange(390, dtype=torch.int32) % 3
    sparse[0] = 256
    tables.append((sparse.reshape(130, 3).tolist(), None, 257, 128))
    tables.append(((torch.arange(2048, dtype=torch.int32) % 7).reshape(512, 4).tolist(), None, 7, 32))
    for i, (ids, emap, ne, bs) in enumerate(tables):
        ids_t = torch.tensor(ids, dtype=torch.int32)
        emap_t = None if emap is None else torch.tensor(emap, dtype=torch.int32)
        s, e, npost = omoe.moe_align_block_size(ids_t, emap_t, ne, bs)
        # the reference's checker asserts on mismatch
        al._assert_matches_reference(ids_t, emap_t, ne, bs, torch.from_numpy(s), torch.from_numpy(e),
                                     torch.from_numpy(npost))
        out[f"c{i}_ids"] = ids_t.numpy()
        out[f"c{i}_emap"] = np.zeros(0, np.int32) if emap is None else emap_t.numpy()
        out[f"c{i}_meta"] = np.array([ne, bs])
        out[f"c{i}_sorted"], out[f"c{i}_experts"], out[f"c{i}_npost"] = s, e, npost
    out["n_cases"] = np.array([len(tables)])
    np.savez_compressed(HERE / "moe_align.npz", **out)
    print(f"moe_align_block_size: {len(tables)} cases pinned")

    # ---- routed dequantise-then-matmul --------------------------------------------------------
    mg = ref["test_moe_wna16_gemm"]
    out = {}
    i = 0
    for has_zp in (False, True):
        for mul in (False, True):
            for dtype in (torch.float16, torch.bfloat16):
                (x, _qw, scales, _qz, tw, sorted_ids, expert_ids, npost, _o, qweight, zps) = mg._make_case(
                    4, has_zp, mul, dtype, "cpu")
                expect = mg._reference(x, qweight, scales, zps, 4, tw, sorted_ids, expert_ids, npost,
                                       block_size_m=2)
                q_kn = qweight.permute(0, 2, 1).contiguous().numpy()
                s_gn = scales.permute(0, 2, 1).contiguous()
                z_gn = None if zps is None else zps.permute(0, 2, 1).contiguous().numpy()
                mine = omoe.moe_w4a16_gemm(x, q_kn, s_gn, z_gn, sorted_ids, expert_ids, npost, tw, 2, 2, mul)
                torch.testing.assert_close(mine.reshape(expect.shape).to(dtype), expect, rtol=0, atol=0)
                out[f"c{i}_x"], out[f"c{i}_q"], out[f"c{i}_s"] = x.float().numpy(), q_kn, s_gn.float().numpy()
                out[f"c{i}_z"] = np.zeros(0) if z_gn is None else z_gn
                out[f"c{i}_tw"] = np.zeros(0, np.float32) if tw is None else tw.numpy()
                out[f"c{i}_sorted"], out[f"c{i}_experts"] = sorted_ids.numpy(), expert_ids.numpy()
                out[f"c{i}_npost"] = npost.numpy()
                out[f"c{i}_meta"] = np.array([int(has_zp), int(mul), code[dtype]])
                out[f"c{i}_out"] = expect.float().numpy()
                i += 1
    out["n_cases"] = np.array([i])
    np.savez_compressed(HERE / "moe_dequant_matmul.npz", **out)
    print(f"dequantise-then-matmul: {i} cases pinned")

    # ---- sibling operators: topk_sigmoid, moe_wna16_gemm (4- and 8-bit), get_cutlass_moe_mm_data ---------
    ts = ref["test_topk_sigmoid"]
    out = {}
    gate = torch.tensor(((1.25, -0.5, 0.75, 2.0, -1.0), (-0.25, 1.5, 0.5, -1.25, 2.25), (0.125, 0.75, 2.5, 1.0, -0.75)))
    bias = torch.tensor((0.0, 0.75, -0.5, -1.0, 1.25))
    i = 0
    for dtype in (torch.float32, torch.float16, torch.bfloat16):
        for has_bias in (False, True):
            for renorm in (False, True):
                g_in = gate.to(dtype)
                expect = ts._reference(g_in, bias if has_bias else None, None, 2, renorm, 0.75)
                mine = omoe.topk_sigmoid(g_in, bias if has_bias else None, None, 2, renorm, 0.75)
                torch.testing.assert_close(mine[0], expect[0], rtol=0, atol=0)
                assert torch.equal(mine[1], expect[1]) and torch.equal(mine[2], expect[2])
                out[f"c{i}_gate"] = g_in.float().numpy()
                out[f"c{i}_meta"] = np.array([code[dtype], int(has_bias), int(renorm)])
                out[f"c{i}_w"], out[f"c{i}_ids"], out[f"c{i}_tei"] = (v.numpy() for v in expect)
                i += 1
    out["bias"], out["n_cases"] = bias.numpy(), np.array([i])
    pad_gate = torch.tensor(((0.25, 2.0, -0.5, 1.0), (1.5, -0.25, 0.75, 0.0), (-1.0, 0.5, 2.25, 1.25)), dtype=torch.float16)
    pad = torch.tensor((False, True, False))
    expect = ts._reference(pad_gate, None, pad, 3, True, 1.0)
    mine = omoe.topk_sigmoid(pad_gate, None, pad, 3, True, 1.0)
    assert torch.equal(mine[1], expect[1]) and torch.equal(mine[2], expect[2])
    out["pad_gate"], out["pad_mask"] = pad_gate.float().numpy(), pad.numpy()
    out["pad_w"], out["pad_ids"], out["pad_tei"] = (v.numpy() for v in expect)
    np.savez_compressed(HERE / "topk_sigmoid.npz", **out)
    print(f"topk_sigmoid: {i + 1} cases pinned")

    out = {}
    i = 0
    for bit, group_size, k in ((4, 16, 32), (4, 32, 64), (8, 4, 32), (8, 16, 32)):
        for has_zp in (False, True):
            for mul in (False, True):
                for dtype in (torch.float16, torch.bfloat16):
                    (x, qw, scales, qz, tw, sorted_ids, expert_ids, npost, _o, qweight, zps) = mg._make_case(
                        bit, has_zp, mul, dtype, "cpu", group_size=group_size, k=k)
                    expect = mg._reference(x, qweight, scales, zps, bit, tw, sorted_ids, expert_ids, npost, block_size_m=2)
                    mine = omoe.moe_wna16_gemm(x, qweight, scales, zps, bit, tw, sorted_ids, expert_ids, npost, 2, 2)
                    tol = 2e-2 if dtype == torch.float16 else 5e-2
                    torch.testing.assert_close(mine.to(dtype), expect, rtol=tol, atol=tol)
                    out[f"c{i}_x"], out[f"c{i}_qw"], out[f"c{i}_s"] = x.float().numpy(), qw.numpy(), scales.float().numpy()
                    out[f"c{i}_qz"] = np.zeros(0, np.uint8) if qz is None else qz.numpy()
                    out[f"c{i}_tw"] = np.zeros(0, np.float32) if tw is None else tw.numpy()
                    out[f"c{i}_sorted"], out[f"c{i}_experts"], out[f"c{i}_npost"] = (
                        sorted_ids.numpy(), expert_ids.numpy(), npost.numpy())
                    out[f"c{i}_meta"] = np.array([bit, int(has_zp), int(mul), code[dtype], group_size, k])
                    out[f"c{i}_out"] = expect.float().numpy()
                    i += 1
    out["n_cases"] = np.array([i])
    np.savez_compressed(HERE / "moe_wna16_gemm.npz", **out)
    print(f"moe_wna16_gemm: {i} cases pinned")

    md = ref["test_get_cutlass_moe_mm_data"]
    out = {}
    tables = [(((2, 0), (1, 2), (0, 3), (3, 1)), 4, False), (((0, 1), (2, 3), (0, 3), (2, 1)), 4, True),
              (tuple((0, 1) for _ in range(130)), 4, True), (((0, -1), (2, 1), (-1, 2)), 4, False),
              ((torch.arange(513, dtype=torch.int32) % 4).reshape(513, 1).tolist(), 4, False),
              ((torch.arange(2600, dtype=torch.int32) * 7 % 61).reshape(650, 4).tolist(), 61, False)]
    for i, (ids, experts, blockscale) in enumerate(tables):
        ids_t = torch.tensor(ids, dtype=torch.int32)
        for gated in (True, False):
            res = omoe.get_cutlass_moe_mm_data(ids_t, experts, 64, 128, gated, blockscale)
            tensors = [None if r is None else torch.from_numpy(r) for r in res]
            md._assert_matches_reference(ids_t, experts, 64, 128, gated, *tensors[:5], tensors[5])
        out[f"c{i}_ids"], out[f"c{i}_meta"] = ids_t.numpy(), np.array([experts, int(blockscale)])
    out["n_cases"] = np.array([len(tables)])
    np.savez_compressed(HERE / "moe_mm_data.npz", **out)
    print(f"get_cutlass_moe_mm_data: {len(tables)} routing tables checked by the reference's checker")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference-checkout")
    main(sys.argv[1])
