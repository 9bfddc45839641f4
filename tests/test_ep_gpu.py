"""GPU: the expert-parallel MoE layer and the column-parallel linear against the single-GPU result.

* one GPU: the device-side expert-parallel layer with a world of one (same kernels: placement,
  dispatch into the arena, unpack, routed GEMM pair with the scattered epilogue, sum) against the
  oracle chain;
* two ranks (needs two GPUs, skipped otherwise): the same layer across two GPUs over peer-mapped
  arenas, the NCCL all-to-all formulation of it, the column-parallel linear whose epilogue stores
  its slice into both ranks' result matrices, and the NCCL all-gather formulation of that."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    import numpy as np
    import torch.distributed as dist

    from infiniops_b200 import capi, moe_layer, parallel

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        experts, top_k, hidden, inter, block, tokens = 8, 2, 512, 256, 64, 96
        gen = torch.Generator().manual_seed(5)

        def packed(k, n):
            src = torch.randint(-2**31, 2**31 - 1, (experts, k // 8, n), dtype=torch.int32, generator=gen).to(dev)
            out = torch.empty((experts, k // 16, 2 * n), dtype=torch.int32, device=dev)
            for e in range(experts):
                capi.gptq_marlin_repack(src[e], None, k, n, 4, False, out[e])
            scales = (torch.randn((experts, k // 128, n), generator=gen).abs() * 0.01 + 1e-3).bfloat16().to(dev)
            return out, scales

        w13, s13 = packed(hidden, 2 * inter)
        w2, s2 = packed(inter, hidden)
        x = torch.randn((tokens, hidden), generator=gen).bfloat16().to(dev)
        logits = torch.randn((tokens, experts), generator=gen).to(dev)
        weights, ids = moe_layer.route_softmax(logits, top_k)
        full = moe_layer.RoutedExperts(moe_layer.ExpertWeights(w13, s13, None, w2, s2, None, hidden, inter), block)
        expect = moe_layer.single_gpu_layer(x, weights, ids, full).clone()

        per = experts // world
        mine = slice(rank * per, (rank + 1) * per)
        local = moe_layer.RoutedExperts(
            moe_layer.ExpertWeights(w13[mine].contiguous(), s13[mine].contiguous(), None, w2[mine].contiguous(),
                                    s2[mine].contiguous(), None, hidden, inter), block)
        t0, t1 = rank * tokens // world, (rank + 1) * tokens // world

        def moe_sum(routed):
            out = torch.empty((routed.shape[0], routed.shape[2]), dtype=routed.dtype, device=dev)
            capi.moe_sum(routed, out)
            return out

        got = parallel.expert_parallel_layer(x[t0:t1].contiguous(), ids[t0:t1].contiguous(),
                                             weights[t0:t1].contiguous(), experts, top_k, local, moe_sum)
        torch.cuda.synchronize()
        # same kernels, same fp32 accumulation per row; only the bf16 product with the routing weight is shared
        err = float((got.float() - expect[t0:t1].float()).abs().max() / expect.float().abs().max())
        assert err <= 1e-2, err

        # the same layer on the device-side path: peer-mapped arenas, flags, no host read-back; twice,
        # so that the second call meets the buffers and epochs the first one left
        ep = parallel.DeviceExpertParallel(local.w, top_k, tokens // world + 8, dev, block)
        for _ in range(2):
            got2 = ep(x[t0:t1].contiguous(), ids[t0:t1].contiguous(), weights[t0:t1].contiguous())
            torch.cuda.synchronize()
            assert ep.status() == (0, 0, 0), ep.status()
            err = float((got2.float() - expect[t0:t1].float()).abs().max() / expect.float().abs().max())
            assert err <= 1e-2, err
        ep.close()
        # ... and with the columns of w13 read as gate/up interleaved (silu_and_mul in the GEMM epilogue),
        # against the single-GPU layer reading them the same way
        full.w.interleaved = local.w.interleaved = True
        expect_fused = moe_layer.single_gpu_layer(x, weights, ids, full).clone()
        ep_fused = parallel.DeviceExpertParallel(local.w, top_k, tokens // world + 8, dev, block)
        got3 = ep_fused(x[t0:t1].contiguous(), ids[t0:t1].contiguous(), weights[t0:t1].contiguous())
        torch.cuda.synchronize()
        assert ep_fused.status() == (0, 0, 0), ep_fused.status()
        err3 = float((got3.float() - expect_fused[t0:t1].float()).abs().max() / expect_fused.float().abs().max())
        assert err3 <= 1e-2, err3
        ep_fused.close()
        # ... and with 128-row routing blocks: the second GEMM stores tiles, a copy kernel sends the rows home
        full.w.interleaved = local.w.interleaved = False
        ep_tiles = parallel.DeviceExpertParallel(local.w, top_k, tokens // world + 8, dev, 128)
        for _ in range(2):
            got4 = ep_tiles(x[t0:t1].contiguous(), ids[t0:t1].contiguous(), weights[t0:t1].contiguous())
            torch.cuda.synchronize()
            assert ep_tiles.status() == (0, 0, 0), ep_tiles.status()
            err4 = float((got4.float() - expect[t0:t1].float()).abs().max() / expect.float().abs().max())
            assert err4 <= 1e-2, err4
        ep_tiles.close()

        # column-parallel dense linear
        k, n, m = 1024, 1024, 16
        awq = torch.randint(-2**31, 2**31 - 1, (k, n // 8), dtype=torch.int32, generator=gen).to(dev)
        scales = (torch.randn((k // 128, n), generator=gen).abs() * 0.01 + 1e-3).bfloat16().to(dev)
        zeros = torch.randint(-2**31, 2**31 - 1, (k // 128, n // 8), dtype=torch.int32, generator=gen).to(dev)
        a = torch.randn((m, k), generator=gen).bfloat16().to(dev)

        def gemm(w, s, z, width):
            marlin = torch.empty((k // 16, 2 * width), dtype=torch.int32, device=dev)
            capi.awq_marlin_repack(w, k, width, 4, False, marlin)
            out = torch.empty((m, width), dtype=torch.bfloat16, device=dev)
            capi.marlin_gemm(a, marlin, None, s, z, capi.QTYPE_UINT4, m, width, k, out)
            return out

        whole = gemm(awq, scales, zeros, n)
        w, s, z = parallel.shard_columns(awq, scales, zeros, n, rank, world, "awq")
        sharded = parallel.as_matrix(parallel.gather_columns(gemm(w, s, z, n // world)))
        torch.cuda.synchronize()
        assert torch.equal(sharded, whole)
        assert capi.scratch_status(capi.scratch(dev, 0)) == 0

        # the same shard, its slice stored by the GEMM epilogue into both ranks' [m, n] matrices
        from infiniops_b200 import peer

        group = peer.PeerGroup(m * n * 2, dev)
        off = group.carve(m * n * 2)
        full_out = group.local(off, (m, n), torch.bfloat16)
        marlin = torch.empty((k // 16, 2 * (n // world)), dtype=torch.int32, device=dev)
        capi.awq_marlin_repack(w, k, n // world, 4, False, marlin)
        g = capi.gemm_problem(a, marlin, None, s, z, full_out, m, n // world, k, out_ld=n, out_col0=rank * (n // world),
                              peer_out=[group.address(r, off) for r in group.others()])
        scratch = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes(), dtype=torch.uint8, device=dev)
        for _ in range(2):
            capi.marlin_gemm_batch(capi.problem_array([g]), torch.bfloat16, capi.QTYPE_UINT4, scratch,
                                   signal=group.signal())
            group.wait()
            torch.cuda.synchronize()
            assert group.wait_status() == (0, 0) and capi.scratch_status(scratch) == 0
            # each rank's slice equals what the all-gather formulation delivered
            assert torch.equal(full_out, sharded)
            dist.barrier()
        # the same again with the slices sent by one copy launch behind the GEMM (local placement only)
        full_out.zero_()
        dist.barrier()
        g_local = capi.gemm_problem(a, marlin, None, s, z, full_out, m, n // world, k, out_ld=n, out_col0=rank * (n // world))
        col_bytes = rank * (n // world) * 2
        copies = (capi.PeerCopy * 1)(capi.peer_copy(full_out.data_ptr() + col_bytes,
                                                    [group.address(r, off) + col_bytes for r in group.others()], m,
                                                    (n // world) * 2, n * 2))
        for _ in range(2):
            capi.marlin_gemm_batch(capi.problem_array([g_local]), torch.bfloat16, capi.QTYPE_UINT4, scratch)
            capi.peer_broadcast(copies, world - 1, signal=group.signal())
            group.wait()
            torch.cuda.synchronize()
            assert group.wait_status() == (0, 0) and capi.scratch_status(scratch) == 0
            assert torch.equal(full_out, sharded)
            dist.barrier()
        group.close()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_and_column_parallel_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)


@pytest.mark.parametrize("interleaved,block", ((False, 16), (True, 16), (False, 128), (True, 256)))
def test_device_expert_parallel_world_of_one_against_oracle(interleaved, block):
    """The device-side expert-parallel layer with this GPU as the only rank, against the oracle chain
    router -> sort -> w13 -> silu_and_mul -> w2 (x weight) -> sum.  One token carries an expert id
    outside the table: its route must contribute nothing.  `interleaved`: w13 is packed with gate and
    up interleaved and the layer applies silu_and_mul in the first GEMM's epilogue."""
    import numpy as np

    from infiniops_b200 import capi, moe_layer, parallel
    from oracle import moe as omoe
    from oracle import quant as oq

    experts, top_k, hidden, inter, tokens = 8, 2, 256, 128, 50   # (128- / 256-row blocks: tile stores + combine copy)
    dev = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(11)

    def packed(k, n, order=None):
        q = torch.randint(0, 16, (experts, k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
        s = (torch.randn((experts, k // 128, n), generator=gen).abs() * 0.01 + 1e-3).bfloat16()
        qd, sd = (q, s) if order is None else (q[:, :, order], s[:, :, order])
        w = torch.stack([torch.from_numpy(oq.marlin_pack(qd[e], 4, False)) for e in range(experts)]).to(dev)
        return q, s, w, sd

    order = moe_layer.gate_up_interleave(inter).numpy() if interleaved else None
    q13, s13, w13, s13_dev = packed(hidden, 2 * inter, order)
    q2, s2, w2, _ = packed(inter, hidden)
    x = torch.randn((tokens, hidden), generator=gen).bfloat16()
    logits = torch.randn((tokens, experts), generator=gen)
    rw, rids, _ = omoe.topk_softmax(logits, None, None, top_k, True)
    ids = rids.to(torch.int32)
    ids[7, 1] = experts + 3   # a route to nowhere
    weights = moe_layer.ExpertWeights(w13, s13_dev.to(dev).contiguous(), None, w2, s2.to(dev), None, hidden, inter,
                                      interleaved=interleaved)
    ep = parallel.DeviceExpertParallel(weights, top_k, tokens, dev, block, world=1)
    for _ in range(2):
        got = ep(x.to(dev), ids.to(dev), rw.to(dev))
        torch.cuda.synchronize()
    rs, re, rn = omoe.moe_align_block_size(ids, None, experts, block)
    g = omoe.moe_w4a16_gemm(x, q13, s13, None, rs, re, rn, None, block, top_k, False).bfloat16()
    h = omoe.silu_and_mul(g)
    y = omoe.moe_w4a16_gemm(h, q2, s2, None, rs, re, rn, rw.flatten(), block, 1, True).bfloat16()
    ref = omoe.moe_sum(y.view(tokens, top_k, hidden))
    err = float((got.float().cpu() - ref.float()).abs().max() / ref.float().abs().max())
    assert err <= 3e-2, err
