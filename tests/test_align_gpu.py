"""GPU: moe_align_block_size through the C ABI, bit-exact against golden vectors and the oracle."""

import numpy as np
import pytest
import torch

from oracle import moe as omoe

pytestmark = pytest.mark.gpu


def _run(ids, emap, ne, bs, extra=0):
    from infiniops_b200 import capi

    ids_d = torch.as_tensor(ids, dtype=torch.int32).cuda()
    emap_d = None if emap is None else torch.as_tensor(emap, dtype=torch.int32).cuda()
    size, blocks = omoe.padded_sizes(ids_d.numel(), ne, bs)
    sorted_ids = torch.full((size + extra,), -2, dtype=torch.int32, device="cuda")
    experts = torch.full((blocks + extra,), -2, dtype=torch.int32, device="cuda")
    npost = torch.full((1,), -2, dtype=torch.int32, device="cuda")
    capi.moe_align_block_size(ids_d, emap_d, ne, bs, sorted_ids, experts, npost)
    return sorted_ids.cpu().numpy(), experts.cpu().numpy(), npost.cpu().numpy()


def test_align_golden(golden):
    g = golden["moe_align"]
    for i in range(int(g["n_cases"][0])):
        ne, bs = (int(v) for v in g[f"c{i}_meta"])
        emap = g[f"c{i}_emap"]
        s, e, npost = _run(g[f"c{i}_ids"], emap if emap.size else None, ne, bs)
        assert np.array_equal(s, g[f"c{i}_sorted"]), i
        assert np.array_equal(e, g[f"c{i}_experts"]), i
        assert np.array_equal(npost, g[f"c{i}_npost"]), i


@pytest.mark.parametrize("tokens,topk,experts,block", ((1, 2, 8, 64), (64, 2, 8, 64), (1024, 2, 8, 64),
                                                        (4096, 2, 8, 64), (16, 8, 256, 64), (512, 8, 256, 64),
                                                        (8192, 8, 256, 64), (3000, 3, 1023, 16), (700, 5, 61, 48)))
def test_align_matches_oracle(tokens, topk, experts, block):
    gen = torch.Generator().manual_seed(tokens * 7 + experts)
    ids = torch.randint(0, experts, (tokens, topk), generator=gen, dtype=torch.int32)
    for emap in (None, torch.where(torch.arange(experts) % 4 == 1, -1, torch.arange(experts) // 2).int()):
        s, e, npost = _run(ids, emap, experts, block, extra=5)
        rs, re, rn = omoe.moe_align_block_size(ids, emap, experts, block, s.size, e.size)
        assert np.array_equal(npost, rn)
        assert np.array_equal(e, re)
        assert np.array_equal(s, rs)


def test_align_properties_at_full_size():
    """Sortedness / stability / padding properties at the largest benchmark size."""
    tokens, topk, experts, block = 8192, 8, 256, 64
    ids = torch.randint(0, experts, (tokens, topk), dtype=torch.int32)
    s, e, npost = _run(ids, None, experts, block)
    total = int(npost[0])
    flat = ids.flatten().numpy()
    assert total % block == 0 and (s[total:] == flat.size).all() and (e[total // block:] == -1).all()
    real = s[:total][s[:total] < flat.size]
    assert np.array_equal(np.sort(real), np.arange(flat.size))          # every id exactly once
    owner = np.repeat(e[: total // block], block)
    valid = s[:total] < flat.size
    assert np.array_equal(flat[s[:total][valid]], owner[valid])          # rows sit in their expert's blocks
    assert (np.diff(e[: total // block]) >= 0).all()                      # experts ascending
    run = s[:total].astype(np.int64)
    same_expert = owner[1:] == owner[:-1]
    assert (np.diff(run)[same_expert & valid[1:] & valid[:-1]] > 0).all()  # ascending inside an expert


def test_align_is_deterministic_and_honours_stream():
    from infiniops_b200 import capi

    ids = (torch.arange(8192, dtype=torch.int32) % 7).reshape(2048, 4).cuda()
    size, blocks = omoe.padded_sizes(8192, 7, 32)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    results = []
    for _ in range(5):
        outs = (torch.full((size,), -2, dtype=torch.int32, device="cuda"),
                torch.full((blocks,), -2, dtype=torch.int32, device="cuda"),
                torch.full((1,), -2, dtype=torch.int32, device="cuda"))
        with torch.cuda.stream(stream):
            capi.moe_align_block_size(ids, None, 7, 32, *outs, stream=stream.cuda_stream)
        results.append(outs)
    stream.synchronize()
    for outs in results[1:]:
        assert all(torch.equal(a, b) for a, b in zip(outs, results[0]))


def test_align_rejects_small_outputs():
    from infiniops_b200 import capi

    ids = torch.zeros((4, 2), dtype=torch.int32, device="cuda")
    with pytest.raises(capi.Error, match="output tensors are too small"):
        capi.moe_align_block_size(ids, None, 4, 4, torch.empty(3, dtype=torch.int32, device="cuda"),
                                  torch.empty(8, dtype=torch.int32, device="cuda"),
                                  torch.empty(1, dtype=torch.int32, device="cuda"))
