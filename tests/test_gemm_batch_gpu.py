"""GPU: the batched dense GEMM (a list of decode-sized problems in one or two persistent launches),
output placement inside a wider matrix, the epilogue's extra stores into "peer" matrices and the
completion signal with its bounded wait -- all through the C ABI, against the oracle.

On one GPU the peer matrices and flag words are ordinary local buffers: the data path (plain stores
from the epilogue, release of the epoch by the last block, acquire by the waiting kernel) is the same
one that runs across GPUs, and the waiting kernel is enqueued BEHIND the launch that signals, so no
kernel ever waits for one that is not already complete.
"""

import ctypes

import pytest
import torch

from oracle import quant as oq
from tests.helpers import make_quantized, rel_max_err

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _device_problem(m, k, n, dtype, zeros, seed, bias=False):
    q, scales, z = make_quantized(k, n, 128, dtype, zeros, seed)
    a = torch.randn((m, k), generator=torch.Generator().manual_seed(seed + 1)).to(dtype)
    b = torch.randn(n, generator=torch.Generator().manual_seed(seed + 2)).to(dtype) if bias else None
    dev = {
        "a": a.cuda(), "w": torch.from_numpy(oq.marlin_pack(q, 4, False)).cuda(), "s": scales.cuda(),
        "z": None if z is None else torch.from_numpy(oq.pack_zeros(z)).cuda(), "b": None if b is None else b.cuda(),
    }
    ref = oq.w4a16_gemm(a, q, scales, z, bias=b)
    return dev, ref


SHAPES = ((1, 512, 256), (4, 1024, 192), (16, 256, 640), (16, 2048, 128), (40, 384, 320), (64, 1024, 256),
          (7, 128, 64), (33, 256, 128))


@pytest.mark.parametrize("dtype,zeros", ((torch.bfloat16, True), (torch.float16, False)))
def test_batch_matches_oracle(dtype, zeros):
    from infiniops_b200 import capi

    devs, refs, outs, problems = [], [], [], []
    for i, (m, k, n) in enumerate(SHAPES):
        dev, ref = _device_problem(m, k, n, dtype, zeros, 100 * i + 7, bias=(i % 2 == 0))
        out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        devs.append(dev), refs.append(ref), outs.append(out)
        problems.append(capi.gemm_problem(dev["a"], dev["w"], dev["b"], dev["s"], dev["z"], out, m, n, k))
    scratch = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes(), dtype=torch.uint8, device="cuda")
    table = capi.problem_array(problems)
    qtype = capi.QTYPE_UINT4 if zeros else capi.QTYPE_UINT4B8
    for _ in range(2):   # the second call finds the scratch as the first left it
        for out in outs:
            out.fill_(float("nan"))
        capi.marlin_gemm_batch(table, dtype, qtype, scratch)
        torch.cuda.synchronize()
        assert capi.scratch_status(scratch) == 0
        for (m, k, n), out, ref in zip(SHAPES, outs, refs):
            assert rel_max_err(out, ref) <= TOL, (m, k, n)
    assert int(scratch[:256 + 16 * 1024].view(torch.int32).abs().sum()) == 0   # header and counters left zero


def test_batch_many_problems_and_split_tiles():
    """Twenty problems (more than one table holds) whose tiles are shared by several blocks."""
    from infiniops_b200 import capi

    dtype = torch.bfloat16
    devs, refs, outs, problems = [], [], [], []
    for i in range(20):
        m, k, n = (1, 4, 16, 8)[i % 4], 4096 if i % 5 == 0 else 512, 128 if i % 3 == 0 else 384
        dev, ref = _device_problem(m, k, n, dtype, True, 900 + i)
        out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        devs.append(dev), refs.append(ref), outs.append(out)
        problems.append(capi.gemm_problem(dev["a"], dev["w"], None, dev["s"], dev["z"], out, m, n, k))
    scratch = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes(), dtype=torch.uint8, device="cuda")
    capi.marlin_gemm_batch(capi.problem_array(problems), dtype, capi.QTYPE_UINT4, scratch)
    torch.cuda.synchronize()
    assert capi.scratch_status(scratch) == 0
    for out, ref in zip(outs, refs):
        assert rel_max_err(out, ref) <= TOL


def test_batch_rejects_large_rows():
    from infiniops_b200 import capi

    dev, _ = _device_problem(65, 256, 128, torch.bfloat16, False, 5)
    out = torch.empty((65, 128), dtype=torch.bfloat16, device="cuda")
    scratch = torch.zeros(capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes(), dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.Error, match="at most 64 rows"):
        capi.marlin_gemm_batch(capi.problem_array([capi.gemm_problem(dev["a"], dev["w"], None, dev["s"], None, out,
                                                                      65, 128, 256)]),
                               torch.bfloat16, capi.QTYPE_UINT4B8, scratch)


@pytest.mark.parametrize("m,k,n", ((16, 512, 256), (16, 8192, 128), (64, 256, 9728), (300, 512, 512)))
def test_placement_peer_stores_and_signal(m, k, n):
    """A column shard writes columns [n, 2n) of a 3n-wide matrix, here and in two stand-in peer
    matrices; the launch then raises the epoch in the flag arrays, which the bounded wait sees.
    Whole tiles, split tiles, 64-row tiles and the paired-block prefill kernel."""
    from infiniops_b200 import capi

    dtype = torch.bfloat16
    dev, ref = _device_problem(m, k, n, dtype, True, m + k + n)
    wide = [torch.full((m, 3 * n), 7.0, dtype=dtype, device="cuda") for _ in range(3)]
    g = capi.gemm_problem(dev["a"], dev["w"], None, dev["s"], dev["z"], wide[0], m, n, k, out_ld=3 * n, out_col0=n,
                          peer_out=[wide[1].data_ptr(), wide[2].data_ptr()])
    ctrl = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags = [torch.zeros(4, dtype=torch.int32, device="cuda") for _ in range(2)]
    sig = capi.PeerSignal()
    sig.done_counter, sig.epoch, sig.n_peers, sig.flag_slot = ctrl[0:].data_ptr(), ctrl[1:].data_ptr(), 2, 1
    sig.peer_flags[0], sig.peer_flags[1] = flags[0].data_ptr(), flags[1].data_ptr()
    need = max(capi.lib().infiniops_b200_marlin_gemm_scratch_bytes(m, n, k),
               capi.lib().infiniops_b200_marlin_gemm_batch_scratch_bytes())
    scratch = torch.zeros(need, dtype=torch.uint8, device="cuda")
    for epoch in (1, 2):
        if m <= 64:
            capi.marlin_gemm_batch(capi.problem_array([g]), dtype, capi.QTYPE_UINT4, scratch, signal=sig)
        else:
            capi.marlin_gemm_placed(g, dtype, capi.QTYPE_UINT4, scratch, signal=sig)
        # the receiving side: wait for slot 1 of flag array 0 to reach the next epoch
        capi._check(capi.lib().infiniops_b200_peer_wait(flags[0].data_ptr(), 2, 0, ctrl[2:].data_ptr(),
                                                        ctrl[3:].data_ptr(), None))
        torch.cuda.synchronize()
        assert capi.scratch_status(scratch) == 0
        assert ctrl.tolist()[:5] == [0, epoch, epoch, 0, 0]
        assert flags[0].tolist() == [0, epoch, 0, 0] and flags[1].tolist() == [0, epoch, 0, 0]
    for w in wide:
        assert rel_max_err(w[:, n:2 * n], ref) <= TOL
        assert bool((w[:, :n] == 7.0).all()) and bool((w[:, 2 * n:] == 7.0).all())
    assert torch.equal(wide[0], wide[1]) and torch.equal(wide[0], wide[2])


def test_peer_wait_runs_out_and_reports():
    """A flag that nothing sets: the wait gives up after its poll limit (about a second), records
    (8, slot) and the stream carries on."""
    from infiniops_b200 import capi

    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    flags[0] = 1    # slot 0 is there, slot 2 never comes, slot 1 is the waiter's own
    ctrl = torch.zeros(4, dtype=torch.int32, device="cuda")
    capi._check(capi.lib().infiniops_b200_peer_wait(flags.data_ptr(), 3, 1, ctrl[0:].data_ptr(), ctrl[1:].data_ptr(),
                                                    None))
    after = torch.ones(4, device="cuda") * 2   # work behind the wait still runs
    torch.cuda.synchronize()
    assert ctrl.tolist()[:3] == [1, 8, 2]
    assert after.tolist() == [2.0] * 4
