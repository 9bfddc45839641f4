"""The MoE operator chain as a caller strings it together (the reference ships the operators,
not this caller): router -> moe_align_block_size -> moe_wna16_marlin_gemm (w13) -> silu_and_mul
-> moe_wna16_marlin_gemm (w2, x routing weight) -> moe_sum.  Used by the tests, the smoke check
and the MoE benchmark; every step is a call into the CUDA library through `capi`.
"""

from __future__ import annotations

import dataclasses

import torch

from . import capi


def padded_sizes(numel: int, num_experts: int, block: int) -> tuple[int, int]:
    size = numel + num_experts * (block - 1)
    if numel < num_experts:
        size = min(numel * block, size)
    return size, (size + block - 1) // block


@dataclasses.dataclass
class ExpertWeights:
    """Marlin-packed experts of one rank: w13 [E, H/16, 2*2I], w2 [E, I/16, 2H], scales, optional zeros.
    `interleaved`: the columns of w13 / s13 / z13 were reordered with `gate_up_interleave` before
    packing, so the first GEMM can apply silu_and_mul in its epilogue."""
    w13: torch.Tensor
    s13: torch.Tensor
    z13: torch.Tensor | None
    w2: torch.Tensor
    s2: torch.Tensor
    z2: torch.Tensor | None
    hidden: int
    inter: int
    interleaved: bool = False

    @property
    def num_experts(self) -> int:
        return self.w13.shape[0]

    @property
    def qtype(self) -> int:
        return capi.QTYPE_UINT4 if self.z13 is not None else capi.QTYPE_UINT4B8


def gate_up_interleave(inter: int, device=None) -> torch.Tensor:
    """Column order of a gate/up projection for the fused silu epilogue: index tensor `idx` [2 * inter]
    such that `w13[..., idx]` holds, in every run of 32 columns, 16 gate features followed by the
    same 16 up features (`w13` being [gate | up] along its last axis, as `silu_and_mul` reads it).
    Apply it to the unpacked weights, the scales and the unpacked zero points before packing."""
    if inter % 16:
        raise ValueError("the fused silu epilogue needs an intermediate size that is a multiple of 16")
    p = torch.arange(2 * inter, device=device)
    return (p // 32) * 16 + p % 16 + (p % 32 >= 16) * inter


class RoutedExperts:
    """Runs a set of experts on rows that each name ONE expert (top-1 form).  A token with k experts
    appears as k rows; this is also exactly what an expert-parallel rank receives."""

    def __init__(self, weights: ExpertWeights, block: int = 64):
        self.w, self.block = weights, block
        self._buffers: dict = {}

    def _buf(self, name, shape, dtype, device):
        key = (name, tuple(shape), dtype)
        t = self._buffers.get(key)
        if t is None:
            t = torch.empty(shape, dtype=dtype, device=device)
            self._buffers[key] = t
        return t

    def __call__(self, rows: torch.Tensor, expert: torch.Tensor, weights: torch.Tensor, stream=None) -> torch.Tensor:
        w, block, dev = self.w, self.block, rows.device
        r = rows.shape[0]
        out = self._buf("y", (r, w.hidden), rows.dtype, dev)
        if r == 0:
            return out
        size, blocks = padded_sizes(r, w.num_experts, block)
        sorted_ids = self._buf("sorted", (size,), torch.int32, dev)
        expert_ids = self._buf("eids", (blocks,), torch.int32, dev)
        npost = self._buf("npost", (1,), torch.int32, dev)
        capi.moe_align_block_size(expert.view(r, 1), None, w.num_experts, block, sorted_ids, expert_ids, npost,
                                  stream=stream)
        g = self._buf("g", (r, 2 * w.inter), rows.dtype, dev)
        capi.moe_wna16_marlin_gemm(rows, w.w13, None, w.s13, w.z13, sorted_ids, expert_ids, npost, weights, block, 1,
                                   False, w.qtype, r, 2 * w.inter, w.hidden, g, stream=stream)
        h = self._buf("h", (r, w.inter), rows.dtype, dev)
        capi.silu_and_mul(g, h, stream=stream)
        capi.moe_wna16_marlin_gemm(h, w.w2, None, w.s2, w.z2, sorted_ids, expert_ids, npost, weights, block, 1, True,
                                   w.qtype, r, w.hidden, w.inter, out, stream=stream)
        return out


def routing_block(routes: int, num_experts: int, expert_elems: int | None = None) -> int:
    """Rows per routing block for a layer with `routes` routed rows over `num_experts` experts
    (`expert_elems`: hidden x intermediate size of one expert, if known).  The reference's operators
    take 8..64; the sort and the GEMMs of this library also take 128 and 256, and the GEMM converts
    each weight once per block of rows -- so with many rows per expert larger blocks do a quarter of
    the conversion work (and 256-row blocks run on paired thread blocks).  The padding (at most
    block - 1 rows per expert) must stay small against the rows themselves."""
    per_expert = routes / max(1, num_experts)
    # Small experts (DeepSeek shape: 7168 x 2048 against Mixtral's 4096 x 14336) have short tiles, whose
    # fixed cost a larger block amortises: their best block sits one step higher at every point measured
    # below 640 rows per expert (T = 512: 64 rows beat 32 by 7 %, T = 1024: 128 beat 64 by 10 %).
    if expert_elems is not None and expert_elems < (32 << 20) and per_expert < 320:
        per_expert *= 2
    # Measured on a B200 with Mixtral- and DeepSeek-shaped layers.  With 128- and 256-row blocks both
    # GEMMs store tiles and each weight is converted once per block of rows: 128-row blocks beat
    # 64-row ones from about 64 rows per expert on (DeepSeek shape +25 % at 64 rows per expert, +47 %
    # at 128; Mixtral shape -2 % at 64, +12 % at 128, +30 % at 256), and 256-row blocks (paired
    # thread blocks) beat 128-row ones from about 640 rows per expert on (+12 % at 768, +11 % at 1024;
    # -3 % at 512, where they pad too much).  Few rows per expert: a block is mostly padding, and the
    # GEMM's token tile follows the block, so 16-row blocks win below about 8 rows per expert (by
    # 25-50 %) and 32-row blocks up to about 32.
    if per_expert >= 640:
        return 256
    if per_expert >= 64:
        return 128
    if per_expert >= 32:
        return 64
    return 32 if per_expert >= 8 else 16


def route_softmax(logits: torch.Tensor, top_k: int, renormalize: bool = True, stream=None):
    t = logits.shape[0]
    w = torch.empty((t, top_k), dtype=torch.float32, device=logits.device)
    ids = torch.empty((t, top_k), dtype=torch.int32, device=logits.device)
    tei = torch.empty((t, top_k), dtype=torch.int32, device=logits.device)
    capi.topk_softmax(logits, None, None, renormalize, w, ids, tei, stream=stream)
    return w, ids


def route_grouped(scores, bias, groups, topk_group, top_k, scaling, stream=None):
    t = scores.shape[0]
    w = torch.empty((t, top_k), dtype=torch.float32, device=scores.device)
    ids = torch.empty((t, top_k), dtype=torch.int32, device=scores.device)
    capi.grouped_topk(scores, bias, groups, topk_group, top_k, True, scaling, 1, w, ids, stream=stream)
    return w, ids


def _sort_buffers(experts: RoutedExperts, routes: int, dev):
    size, blocks = padded_sizes(routes, experts.w.num_experts, experts.block)
    return (experts._buf("L_sorted", (size,), torch.int32, dev), experts._buf("L_eids", (blocks,), torch.int32, dev),
            experts._buf("L_npost", (1,), torch.int32, dev))


def layer_from_logits(x, logits, router: dict, experts: RoutedExperts, stream=None) -> torch.Tensor:
    """The whole layer from the router's input, with router and token sort issued as one call (one
    launch while tokens x top_k <= 1024).  `router`: {"kind": "softmax", "top_k": k, "renormalize": bool}
    or {"kind": "grouped", "top_k": k, "bias": tensor, "groups": g, "topk_group": n, "scaling": f}."""
    t, dev, k = logits.shape[0], logits.device, router["top_k"]
    w = experts._buf("L_tw", (t, k), torch.float32, dev)
    ids = experts._buf("L_ids", (t, k), torch.int32, dev)
    sorted_ids, expert_ids, npost = _sort_buffers(experts, t * k, dev)
    if router["kind"] == "softmax":
        tei = experts._buf("L_tei", (t, k), torch.int32, dev)
        capi.topk_softmax_align(logits, None, None, router.get("renormalize", True), w, ids, tei, None, experts.block,
                                sorted_ids, expert_ids, npost, stream=stream)
    else:
        capi.grouped_topk_align(logits, router["bias"], router["groups"], router["topk_group"], k, True,
                                router["scaling"], 1, w, ids, None, experts.block, sorted_ids, expert_ids, npost,
                                stream=stream)
    return single_gpu_layer(x, w, ids, experts, stream=stream, presorted=True)


def single_gpu_layer(x, topk_weights, topk_ids, experts: RoutedExperts, stream=None, presorted=False) -> torch.Tensor:
    """The layer on one GPU in the reference's chaining: the sort runs on the [T, k] ids and the first
    GEMM reads token `route // k` directly (no row duplication).  `presorted`: the sort's outputs for
    these ids are already in the runner's buffers (see `layer_from_logits`)."""
    w, block, dev = experts.w, experts.block, x.device
    t, k = topk_ids.shape
    size, _ = padded_sizes(t * k, w.num_experts, block)
    sorted_ids, expert_ids, npost = _sort_buffers(experts, t * k, dev)
    if not presorted:
        capi.moe_align_block_size(topk_ids, None, w.num_experts, block, sorted_ids, expert_ids, npost, stream=stream)
    flat_w = topk_weights.reshape(-1)
    # The intermediates stay in sorted (expert) order -- one row per entry of `sorted_ids` -- so the
    # first GEMM stores dense tiles and the second reads them in place.
    tiles_only = block >= 128
    position = None
    if tiles_only:
        # 128- / 256-row blocks: the second GEMM stores tiles in sorted order too (rows already
        # multiplied by their routing weight) and the final sum picks each token's rows by position,
        # so no GEMM epilogue scatters single rows.  The first GEMM's gather notes the positions.
        position = experts._buf("L_pos", (t, k), torch.int32, dev)
    # live rows per routing block, noted by the first GEMM's gather: both GEMMs then spend tensor-core
    # time on a partly filled block in proportion to its rows, not to the block size
    live = experts._buf("L_rows", (sorted_ids.numel() // block + 1,), torch.int32, dev) if block >= 32 else None
    h = experts._buf("L_h", (size, w.inter), x.dtype, dev)
    if w.interleaved and (2 * w.inter) % 128 == 0:
        # gate and up meet in the epilogue: the [size, 2I] product is never stored
        capi.moe_wna16_marlin_gemm(x, w.w13, None, w.s13, w.z13, sorted_ids, expert_ids, npost, flat_w, block, k,
                                   False, w.qtype, t, 2 * w.inter, w.hidden, h, stream=stream, out_sorted=True,
                                   fuse_silu=True, route_position=position, block_rows=live)
    else:
        g = experts._buf("L_g", (size, 2 * w.inter), x.dtype, dev)
        capi.moe_wna16_marlin_gemm(x, w.w13, None, w.s13, w.z13, sorted_ids, expert_ids, npost, flat_w, block, k,
                                   False, w.qtype, t, 2 * w.inter, w.hidden, g, stream=stream, out_sorted=True,
                                   route_position=position, block_rows=live)
        capi.silu_and_mul(g, h, stream=stream)
    out = experts._buf("L_out", (t, w.hidden), x.dtype, dev)
    if tiles_only:
        y = experts._buf("L_ys", (size, w.hidden), x.dtype, dev)
        capi.moe_wna16_marlin_gemm(h, w.w2, None, w.s2, w.z2, sorted_ids, expert_ids, npost, flat_w, block, 1, True,
                                   w.qtype, t * k, w.hidden, w.inter, y, stream=stream, a_sorted=True, out_sorted=True,
                                   block_rows=live)
        capi.moe_gather_sum(y, position, out, stream=stream)
        return out
    y = experts._buf("L_y", (t * k, w.hidden), x.dtype, dev)
    capi.moe_wna16_marlin_gemm(h, w.w2, None, w.s2, w.z2, sorted_ids, expert_ids, npost, flat_w, block, 1, True,
                               w.qtype, t * k, w.hidden, w.inter, y, stream=stream, a_sorted=True, block_rows=live)
    capi.moe_sum(y.view(t, k, w.hidden), out, stream=stream)
    return out

