"""GPU: gptq/awq_marlin_repack through the C ABI, bit-exact against the golden vectors and the oracle."""

import numpy as np
import pytest
import torch

from oracle import quant as oq

pytestmark = pytest.mark.gpu


def _capi():
    from infiniops_b200 import capi
    return capi


def test_repack_matches_reference_golden(golden):
    capi = _capi()
    g = golden["repack"]
    keys = [k[:-3] for k in g.files if k.endswith("_in")]
    for key in keys:
        parts = key.split("_")
        src = torch.from_numpy(g[key + "_in"]).cuda()
        expect = g[key + "_out"]
        out = torch.full(expect.shape, -1, dtype=torch.int32, device="cuda")
        if parts[0] == "gptq":
            _, k, n, bits, a8, _p = parts
            perm = torch.from_numpy(g[key + "_perm"]).cuda()
            capi.gptq_marlin_repack(src, perm, int(k), int(n), int(bits), bool(int(a8)), out)
        else:
            _, k, n, bits, a8 = parts
            capi.awq_marlin_repack(src, int(k), int(n), int(bits), bool(int(a8)), out)
        assert np.array_equal(out.cpu().numpy(), expect), key


@pytest.mark.parametrize("k,n", ((4096, 4096), (1024, 28672), (14336, 512), (64, 320)))
@pytest.mark.parametrize("source", ("gptq", "awq"))
def test_repack_full_size_matches_oracle(k, n, source):
    capi = _capi()
    rng = np.random.default_rng(k * 31 + n)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    expect = oq.marlin_pack(q, 4, False)
    out = torch.empty(expect.shape, dtype=torch.int32, device="cuda")
    if source == "gptq":
        capi.gptq_marlin_repack(torch.from_numpy(oq.gptq_pack(q, 4)).cuda(), None, k, n, 4, False, out)
    else:
        capi.awq_marlin_repack(torch.from_numpy(oq.awq_pack(q, 4)).cuda(), k, n, 4, False, out)
    assert np.array_equal(out.cpu().numpy(), expect)


def test_repack_act_order_and_stream():
    capi = _capi()
    k, n = 512, 256
    rng = np.random.default_rng(7)
    q = rng.integers(0, 16, size=(k, n), dtype=np.uint8)
    perm = torch.randperm(k, generator=torch.Generator().manual_seed(20260728), dtype=torch.int32)
    expect = oq.marlin_pack(q[perm.numpy().astype(np.int64)], 4, False)
    out = torch.empty(expect.shape, dtype=torch.int32, device="cuda")
    src = torch.from_numpy(oq.gptq_pack(q, 4)).cuda()
    perm_d = perm.cuda()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        capi.gptq_marlin_repack(src, perm_d, k, n, 4, False, out, stream=stream.cuda_stream)
    stream.synchronize()
    assert np.array_equal(out.cpu().numpy(), expect)


def test_repack_is_a_permutation_of_nibbles():
    """Size-independent property at a full benchmark size: unpacking the GPU result with the
    inverse index map returns the original matrix."""
    capi = _capi()
    k, n = 4096, 6144
    q = np.random.default_rng(3).integers(0, 16, size=(k, n), dtype=np.uint8)
    out = torch.empty((k // 16, 2 * n), dtype=torch.int32, device="cuda")
    capi.awq_marlin_repack(torch.from_numpy(oq.awq_pack(q, 4)).cuda(), k, n, 4, False, out)
    assert np.array_equal(oq.marlin_unpack(out.cpu().numpy(), k, n, 4, False), q)


def test_repack_rejects_bad_arguments():
    capi = _capi()
    src = torch.zeros((16, 64), dtype=torch.int32, device="cuda")
    out = torch.zeros((8, 128), dtype=torch.int32, device="cuda")
    with pytest.raises(capi.Error, match="divisible by 16"):
        capi.gptq_marlin_repack(src, None, 100, 64, 4, False, out)
    with pytest.raises(capi.Error, match="not supported for 8-bit-activation"):
        capi.gptq_marlin_repack(src, torch.zeros(128, dtype=torch.int32, device="cuda"), 128, 64, 4, True, out)
