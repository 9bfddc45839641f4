"""CPU: the `infini.ops` module builds, exposes the reference's names, and validates like it."""

import subprocess
import sys
import textwrap

import pytest

NAMES = ("gptq_marlin_repack", "awq_marlin_repack", "marlin_gemm", "moe_wna16_marlin_gemm", "topk_softmax",
         "grouped_topk", "moe_align_block_size", "silu_and_mul", "moe_sum", "topk_sigmoid", "moe_wna16_gemm",
         "get_cutlass_moe_mm_data")


@pytest.fixture(scope="module")
def ops():
    from infiniops_b200 import build

    build.build_all()
    import infini.ops

    return infini.ops


def test_module_surface(ops):
    for name in NAMES:
        assert callable(getattr(ops, name))
        cls = getattr(ops, "".join(part.capitalize() for part in name.split("_")))
        # slot 0 everywhere; the two Marlin GEMMs also answer at the provider slot (vLLM's scale layouts)
        slots = [0, 16] if name in ("marlin_gemm", "moe_wna16_marlin_gemm") else [0]
        assert cls.active_implementation_indices("cuda") == slots
        assert cls.active_implementation_indices("nvidia") == slots
        assert cls.active_implementation_indices("cpu") == []
        cls.clear_cache()
    with pytest.raises(ValueError):
        ops.MoeSum.active_implementation_indices("tpu")


_FAKE = textwrap.dedent("""
    import infini.ops, torch

    class Fake:
        # a CPU tensor dressed as a CUDA one: validation runs before any launch
        def __init__(self, t):
            self.t, self.shape, self.dtype = t, tuple(t.shape), t.dtype
        def data_ptr(self): return self.t.data_ptr()
        def stride(self): return self.t.stride()
        @property
        def device(self):
            class D: type = "cuda"; index = 0
            return D()
    i32 = lambda *s: Fake(torch.zeros(s, dtype=torch.int32))
""")

_CASES = {
    "at least two experts per group": """
        infini.ops.GroupedTopk(Fake(torch.ones((1, 2))), Fake(torch.zeros(2)), 2, 1, 1, False, 1.0, 0,
                               Fake(torch.empty((1, 1))), i32(1, 1))""",
    "output tensors are too small": """
        infini.ops.MoeAlignBlockSize(i32(4, 2), None, 4, 4, i32(3), i32(8), i32(1))""",
    "requires `num_experts` in [1, 1023]": """
        infini.ops.MoeAlignBlockSize(i32(4, 2), None, 1024, 4, i32(5000), i32(2000), i32(1))""",
    "requires `num_bits` to be 4 or 8": """
        infini.ops.GptqMarlinRepack(i32(16, 64), i32(0), 128, 64, 3, False, i32(8, 128))""",
    "does not support `perm` for A8 layouts": """
        infini.ops.GptqMarlinRepack(i32(16, 64), i32(128), 128, 64, 4, True, i32(8, 128))""",
    "output shape is incorrect": """
        infini.ops.AwqMarlinRepack(i32(128, 8), 128, 64, 4, False, i32(8, 64))""",
    "`MoeSum` expert_map requires topk_ids": """
        infini.ops.MoeSum(Fake(torch.zeros((2, 2, 4))), None, i32(3), Fake(torch.zeros((2, 4))))""",
    "input last dimension to be twice output last dimension": """
        infini.ops.SiluAndMul(Fake(torch.zeros((2, 6))), Fake(torch.zeros((2, 4))))""",
    "requires `topk` in `[1, num_experts]`": """
        infini.ops.TopkSoftmax(Fake(torch.zeros((2, 4))), None, None, False, Fake(torch.zeros((2, 5))),
                               i32(2, 5), i32(2, 5))""",
    "received an unsupported `moe_block_size`": """
        h = lambda *s: Fake(torch.zeros(s, dtype=torch.float16))
        infini.ops.MoeWna16MarlinGemm(h(2, 128), i32(2, 8, 128), None, h(2, 1, 64), None, None, None, None, None,
                                      i32(16), i32(64), i32(4), i32(1), Fake(torch.zeros(4)), 24, 2, False,
                                      1125899907892224, 2, 64, 128, True, False, True, False, -1, -1, -1, h(4, 64))""",
    "requires contiguous int32 `g_idx` and `perm` of `size_k` entries": """
        h = lambda *s: Fake(torch.zeros(s, dtype=torch.float16))
        infini.ops.MarlinGemm(h(2, 256), i32(16, 128), None, h(2, 64), None, None, None, i32(256), i32(128), i32(16),
                              1125899907892224, 2, 64, 256, True, False, True, False, h(2, 64))""",
    "act-order needs grouped scales": """
        h = lambda *s: Fake(torch.zeros(s, dtype=torch.float16))
        infini.ops.MarlinGemm(h(2, 256), i32(16, 128), None, h(1, 64), None, None, None, i32(256), i32(256), i32(16),
                              1125899907892224, 2, 64, 256, True, False, True, False, h(2, 64))""",
    "has no implementation 16": """
        infini.ops.SiluAndMul(Fake(torch.zeros((2, 8))), Fake(torch.zeros((2, 4))), implementation_index=16)""",
}


@pytest.mark.parametrize("message", sorted(_CASES))
def test_validation_aborts_with_the_reference_message(ops, message):
    """Validation failures abort the process with the reference's assertion text, so they are run
    in a child (as tests/test_moe_align_block_size.py:201-228 of the reference does)."""
    script = _FAKE + textwrap.dedent(_CASES[message])
    result = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True)
    assert result.returncode != 0
    assert message in result.stderr, result.stderr[-400:]


def test_routing_block_rule_and_gate_up_interleave():
    """Host-side helpers of the MoE layer: the routing block chosen from the rows per expert, and the
    column order for the fused silu epilogue."""
    from infiniops_b200 import moe_layer

    mixtral, deepseek = 4096 * 14336, 7168 * 2048
    picks = [moe_layer.routing_block(t * 2, 8, mixtral) for t in (1, 16, 64, 128, 256, 1024, 4096)]
    assert picks == [16, 16, 32, 64, 128, 128, 256]
    picks = [moe_layer.routing_block(t * 8, 256, deepseek) for t in (16, 64, 256, 512, 1024, 8192)]
    assert picks == [16, 16, 32, 64, 128, 128]
    assert moe_layer.routing_block(0, 8) == 16 and moe_layer.routing_block(10**6, 1) == 256

    idx = moe_layer.gate_up_interleave(64)
    assert sorted(idx.tolist()) == list(range(128))
    assert idx[:16].tolist() == list(range(16)) and idx[16:32].tolist() == list(range(64, 80))
    assert idx[32:48].tolist() == list(range(16, 32))
    with pytest.raises(ValueError):
        moe_layer.gate_up_interleave(40)
