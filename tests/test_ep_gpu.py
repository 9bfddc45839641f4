"""GPU, two ranks over NCCL: expert-parallel MoE layer and column-parallel linear against the
single-GPU result.  Needs two GPUs; skipped otherwise."""

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
    finally:
        dist.destroy_process_group()


def test_expert_parallel_and_column_parallel_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
