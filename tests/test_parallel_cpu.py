"""CPU, world size 2 over gloo: the sharding / dispatch / combine plumbing of `infiniops_b200.parallel`,
with the oracle standing in for the CUDA operators."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe as omoe
from oracle import quant as oq

WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _spawn(fn, *args):
    port = _free_port()
    mp.spawn(_entry, args=(fn, port, args), nprocs=WORLD, join=True)


def _entry(rank, fn, port, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        fn(rank, *args)
    finally:
        dist.destroy_process_group()


def _column_parallel(rank, source):
    from infiniops_b200 import parallel

    k, n, m = 256, 256, 5
    rng = np.random.default_rng(3)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    zeros = rng.integers(0, 16, size=(k // 128, n), dtype=np.uint8)
    gen = torch.Generator().manual_seed(4)
    scales = (torch.randn((k // 128, n), generator=gen).abs() * 0.01 + 1e-3)
    a = torch.randn((m, k), generator=gen)
    packed = torch.from_numpy(oq.gptq_pack(q, 4) if source == "gptq" else oq.awq_pack(q, 4))
    zp = torch.from_numpy(oq.pack_zeros(zeros))
    w, s, z = parallel.shard_columns(packed, scales, zp, n, rank, WORLD, source)
    q_local = oq.gptq_unpack(w.numpy(), 4) if source == "gptq" else oq.awq_unpack(w.numpy(), 4)
    lo, hi = parallel.column_range(n, rank, WORLD)
    assert np.array_equal(q_local, q[:, lo:hi])
    z_local = ((z.numpy().view(np.uint32)[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 0xF).reshape(z.shape[0], -1)
    assert np.array_equal(z_local, zeros[:, lo:hi])
    out_local = oq.w4a16_gemm(a, q_local, s, z_local)
    full = parallel.as_matrix(parallel.gather_columns(out_local))
    torch.testing.assert_close(full, oq.w4a16_gemm(a, q, scales, zeros), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("source", ("gptq", "awq"))
def test_column_parallel_matches_unsharded(source):
    _spawn(_column_parallel, source)


def test_column_range_rejects_ragged_shards():
    from infiniops_b200 import parallel

    assert parallel.column_range(4096, 3, 8) == (1536, 2048)
    with pytest.raises(ValueError):
        parallel.column_range(4096 + 64, 0, 8)
    with pytest.raises(ValueError):
        parallel.experts_per_rank(10, 4)


def _expert_parallel(rank, tokens_per_rank, experts, top_k):
    from infiniops_b200 import parallel

    hidden, inter = 16, 8
    gen = torch.Generator().manual_seed(11)
    w13 = torch.randn((experts, hidden, 2 * inter), generator=gen) * 0.3
    w2 = torch.randn((experts, inter, hidden), generator=gen) * 0.3
    x_all = torch.randn((WORLD * tokens_per_rank, hidden), generator=gen)
    logits_all = torch.randn((WORLD * tokens_per_rank, experts), generator=gen)
    mine = slice(rank * tokens_per_rank, (rank + 1) * tokens_per_rank)
    weights, ids, _ = omoe.topk_softmax(logits_all[mine], None, None, top_k, True)
    per_rank = experts // WORLD

    def local_experts_forward(rows, local_expert, row_weights):
        out = torch.empty((rows.shape[0], hidden))
        for i in range(rows.shape[0]):
            e = rank * per_rank + int(local_expert[i])
            g = rows[i] @ w13[e]
            out[i] = (omoe.silu_and_mul(g) @ w2[e]) * row_weights[i]
        return out

    got = parallel.expert_parallel_layer(x_all[mine], ids.to(torch.int32), weights, experts, top_k,
                                         local_experts_forward, omoe.moe_sum)
    w_all, ids_all, _ = omoe.topk_softmax(logits_all, None, None, top_k, True)
    expect = torch.zeros_like(x_all)
    for t in range(x_all.shape[0]):
        for s in range(top_k):
            e = int(ids_all[t, s])
            expect[t] += (omoe.silu_and_mul(x_all[t] @ w13[e]) @ w2[e]) * w_all[t, s]
    torch.testing.assert_close(got, expect[mine], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("tokens_per_rank,experts,top_k", ((5, 8, 2), (1, 8, 2), (9, 4, 3)))
def test_expert_parallel_dispatch_and_combine(tokens_per_rank, experts, top_k):
    _spawn(_expert_parallel, tokens_per_rank, experts, top_k)


def _all_to_one_rank(rank):
    """Every route goes to rank 0: rank 1 receives nothing and must still take part."""
    from infiniops_b200 import parallel

    ids = torch.tensor([[0, 1], [1, 2]], dtype=torch.int32)       # experts 0..3 live on rank 0 (E = 8)
    w = torch.full((2, 2), 0.5)
    for dtype in (torch.float32, torch.bfloat16):     # 32-bit metadata rides in 1 or 2 spare columns
        _one_rank_case(parallel, rank, ids, w, dtype)


def _one_rank_case(parallel, rank, ids, w, dtype):
    x = (torch.arange(8, dtype=torch.float32).reshape(2, 4) + 10 * rank).to(dtype)
    plan = parallel.plan_dispatch(ids, 8)
    rows = parallel.dispatch(x, ids, w, 8, plan)
    assert rows.shape[0] == (8 if rank == 0 else 0)
    if rank == 0:
        assert plan.local_expert.tolist() == [0, 1, 1, 2, 0, 1, 1, 2] and bool((plan.weights == 0.5).all())
    back = parallel.combine(rows * 2, plan)
    torch.testing.assert_close(back, x.repeat_interleave(2, dim=0) * 2)


def test_dispatch_with_an_idle_rank():
    _spawn(_all_to_one_rank)


def _late_rank(rank, result_path):
    """Rank 1 never enters the collective (it sits out the step on the host, as a crashed or stuck
    rank would); rank 0 must get an exception at its deadline instead of blocking, and a later
    collective that both ranks do enter -- on a fresh group -- must still work."""
    import time

    from infiniops_b200 import parallel

    import json

    x = torch.full((3, 4), float(rank))
    if rank == 0:
        result = {}
        t0 = time.monotonic()
        try:
            parallel.gather_columns(x, deadline_s=0.5)
            result["outcome"] = "returned"
        except parallel.CollectiveTimeout as e:
            result["outcome"] = "timeout"
            result["message"] = str(e)
        result["seconds"] = time.monotonic() - t0
        with open(result_path, "w") as f:
            json.dump(result, f)
    else:
        time.sleep(1.5)   # does not join
    # the ranks learn of the failure on the host (here: simply by both getting past the step) and
    # continue on a new group; the old communicator is abandoned
    fresh = dist.new_group(ranks=[0, 1], backend="gloo")
    got = parallel.as_matrix(parallel.gather_columns(x, group=fresh, deadline_s=20.0))
    assert torch.equal(got, torch.cat([torch.zeros(3, 4), torch.ones(3, 4)], dim=1))


def test_collective_gives_up_at_the_host_deadline(tmp_path):
    import json

    path = tmp_path / "rank0.json"
    _spawn(_late_rank, str(path))
    result = json.loads(path.read_text())
    assert result["outcome"] == "timeout", result
    assert "gather_columns" in result["message"] and 0.4 < result["seconds"] < 1.4
