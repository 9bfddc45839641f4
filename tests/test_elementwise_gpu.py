"""GPU: silu_and_mul and moe_sum through the C ABI against the oracle."""

import pytest
import torch

from oracle import moe as omoe

pytestmark = pytest.mark.gpu

_SHAPES = (((13, 4), None, None), ((13, 4), (12, 1), (6, 1)), ((13, 4, 4), None, None),
           ((13, 4, 4), (48, 10, 1), (24, 6, 1)), ((16, 5632), None, None), ((16, 5632), (13312, 1), (6656, 1)),
           ((4, 4, 5632), None, None), ((4, 4, 5632), (53248, 13312, 1), (26624, 6656, 1)),
           ((7, 6), (24, 2), (12, 2)))


def _strided(shape, strides, dtype):
    if strides is None:
        return torch.empty(shape, dtype=dtype, device="cuda")
    return torch.empty_strided(shape, strides, dtype=dtype, device="cuda")


@pytest.mark.parametrize("out_shape,in_strides,out_strides", _SHAPES)
@pytest.mark.parametrize("dtype,rtol,atol", ((torch.float32, 1e-6, 1e-7), (torch.float16, 1e-3, 1e-3),
                                             (torch.bfloat16, 1e-2, 5e-3)))
def test_silu_and_mul(out_shape, in_strides, out_strides, dtype, rtol, atol):
    from infiniops_b200 import capi

    in_shape = (*out_shape[:-1], out_shape[-1] * 2)
    x = _strided(in_shape, in_strides, dtype)
    x.copy_(torch.randn(in_shape, dtype=dtype))
    out = _strided(out_shape, out_strides, dtype)
    out.fill_(float("nan"))
    capi.silu_and_mul(x, out)
    torch.testing.assert_close(out.cpu(), omoe.silu_and_mul(x), rtol=rtol, atol=atol)


def test_silu_and_mul_stream_and_large():
    from infiniops_b200 import capi

    x = torch.randn((8192, 2 * 14336), dtype=torch.bfloat16, device="cuda")
    out = torch.empty((8192, 14336), dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        capi.silu_and_mul(x, out, stream=stream.cuda_stream)
    stream.synchronize()
    ref = (torch.nn.functional.silu(x[:, :14336].float()) * x[:, 14336:].float()).bfloat16()
    torch.testing.assert_close(out, ref, rtol=1e-2, atol=5e-3)


@pytest.mark.parametrize("dtype,rtol,atol", ((torch.float32, 1e-6, 1e-6), (torch.float16, 1e-3, 1e-3),
                                             (torch.bfloat16, 1e-2, 1e-2)))
def test_moe_sum(dtype, rtol, atol):
    from infiniops_b200 import capi

    for shape in ((3, 4, 17), (5, 2, 4096), (64, 8, 7168), (2, 1, 8)):
        x = torch.randn(shape, dtype=dtype, device="cuda")
        out = torch.full((shape[0], shape[2]), torch.nan, dtype=dtype, device="cuda")
        capi.moe_sum(x, out)
        torch.testing.assert_close(out.cpu(), omoe.moe_sum(x), rtol=rtol, atol=atol)
    x = torch.randn((3, 4, 17), dtype=dtype, device="cuda")
    emap = torch.tensor((0, -1, 1), dtype=torch.int32, device="cuda")
    for ids_dtype in (torch.int32, torch.int64):
        ids = torch.tensor(((0, 1, -1, 2), (2, -1, 1, 0), (1, 2, 0, -1)), dtype=ids_dtype, device="cuda")
        for m in (None, emap):
            out = torch.full((3, 17), torch.nan, dtype=dtype, device="cuda")
            capi.moe_sum(x, out, ids, m)
            torch.testing.assert_close(out.cpu(), omoe.moe_sum(x, ids, m), rtol=rtol, atol=atol)


def test_moe_sum_strided_input():
    from infiniops_b200 import capi

    x = torch.empty_strided((3, 4, 17), (167, 40, 2), dtype=torch.float32, device="cuda")
    x.normal_()
    ids = torch.empty_strided((3, 4), (11, 2), dtype=torch.int64, device="cuda")
    ids.copy_(torch.tensor(((0, 1, -1, 2), (2, -1, 1, 0), (1, 2, 0, -1))))
    out = torch.full((3, 17), torch.nan, device="cuda")
    capi.moe_sum(x, out, ids, None)
    torch.testing.assert_close(out.cpu(), (x.cpu() * (ids.cpu() >= 0).unsqueeze(-1)).sum(1))
