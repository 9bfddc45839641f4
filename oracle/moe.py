"""CPU oracle for the mixture-of-experts chain (TEST INFRASTRUCTURE ONLY).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may
import this module; the product path never does.  Each function restates the
torch reference the reference's own test file uses for that operator:

* topk_softmax           -- tests/test_topk_softmax.py:306-324
* grouped_topk           -- tests/test_grouped_topk.py:443-486
* moe_align_block_size   -- tests/test_moe_align_block_size.py:342-381 and the kernel's
                            id mapping src/native/cuda/nvidia/ops/moe_align_block_size/kernel.cuh:10-21
* routed W4A16 GEMM      -- tests/test_moe_wna16_gemm.py:384-442 (dequantise-then-matmul per
                            routed row), output row = flat routing id
* silu_and_mul           -- tests/test_silu_and_mul.py:108-113
* moe_sum                -- tests/test_moe_sum.py:50,95-99
* topk_sigmoid           -- tests/test_topk_sigmoid.py:352-381
* moe_wna16_gemm         -- tests/test_moe_wna16_gemm.py:384-442 (plain [E, N, K] layout)
* get_cutlass_moe_mm_data -- tests/test_get_cutlass_moe_mm_data.py:412-491
"""

from __future__ import annotations

import numpy as np
import torch

from . import quant


def topk_softmax(gating_output, bias, is_padding, topk: int, renormalize: bool):
    """Returns (weights f32 [T,k], indices i64 [T,k], token_expert_indices i32 [T,k])."""
    g = torch.as_tensor(gating_output).cpu()
    scores = torch.softmax(g, dim=-1, dtype=torch.float32)
    selection = scores if bias is None else scores + torch.as_tensor(bias).cpu()
    # torch.topk does not promise an order among equal values; the reference kernel
    # (src/native/cuda/ops/topk_softmax/kernel.cuh:55-64) breaks ties towards the
    # smaller expert index, which a stable descending sort reproduces.
    indices = torch.argsort(selection, dim=-1, descending=True, stable=True)[:, :topk]
    weights = scores.gather(1, indices)
    if renormalize:
        weights = weights / weights.sum(dim=-1, keepdim=True)
    if is_padding is not None:
        pad = torch.as_tensor(is_padding).cpu().bool().unsqueeze(-1)
        indices = indices.masked_fill(pad, -1)
    t = g.shape[0]
    tei = (torch.arange(topk, dtype=torch.int32).unsqueeze(0).expand(t, -1) * t
           + torch.arange(t, dtype=torch.int32).unsqueeze(-1))
    return weights, indices, tei


def grouped_topk(scores, bias, num_expert_group: int, topk_group: int, topk: int,
                 renormalize: bool, routed_scaling_factor: float, scoring_func: int):
    """Returns (values f32 [T,k], indices i32 [T,k])."""
    scores = torch.as_tensor(scores).cpu()
    bias = torch.as_tensor(bias).cpu()
    if scoring_func == 0:
        routed = scores
    else:
        routed = (0.5 * torch.tanh(0.5 * scores.float()) + 0.5).to(scores.dtype)
    selection = (routed + bias.to(scores.dtype).unsqueeze(0)).to(scores.dtype)
    per_group = scores.size(1) // num_expert_group
    grouped = selection.reshape(scores.size(0), num_expert_group, per_group)
    grouped = grouped.masked_fill(torch.isnan(grouped), -torch.inf)
    group_scores = torch.topk(grouped.float(), 2, dim=-1).values.sum(dim=-1).to(scores.dtype)
    chosen = torch.argsort(group_scores.float(), dim=-1, descending=True, stable=True)[:, :topk_group]
    group_mask = torch.zeros_like(group_scores, dtype=torch.bool)
    group_mask.scatter_(1, chosen, True)
    expert_mask = group_mask.repeat_interleave(per_group, dim=-1)
    selected = selection.float().masked_fill(~expert_mask | ~torch.isfinite(scores.float()), -torch.inf)
    indices = torch.argsort(selected, dim=-1, descending=True, stable=True)[:, :topk].to(torch.int32)
    values = routed.gather(1, indices.to(torch.int64)).float()
    if renormalize:
        values = values / (values.sum(dim=-1, keepdim=True) + 1e-20)
    values = values * routed_scaling_factor
    return values, indices


def padded_sizes(numel: int, num_experts: int, block_size: int):
    """Output sizes the reference requires (src/base/moe_align_block_size.h:119-131)."""
    size = numel + num_experts * (block_size - 1)
    if numel < num_experts:
        size = min(numel * block_size, size)
    return size, (size + block_size - 1) // block_size


def moe_align_block_size(topk_ids, expert_map, num_experts: int, block_size: int,
                         sorted_size: int | None = None, blocks_size: int | None = None):
    """Returns (sorted_token_ids, expert_ids, num_tokens_post_pad) as int32 numpy arrays,
    fully materialised the way the reference kernel leaves its buffers: padding
    entries hold `numel`, unused blocks hold -1."""
    ids = quant._as_np(topk_ids).reshape(-1).astype(np.int64)
    numel = ids.size
    valid = (ids >= 0) & (ids < num_experts)
    mapped = np.full(numel, -1, dtype=np.int64)
    if expert_map is not None:
        emap = quant._as_np(expert_map).astype(np.int64)
        mapped[valid] = emap[ids[valid]]
        mapped[(mapped < 0) | (mapped >= num_experts)] = -1
    else:
        mapped[valid] = ids[valid]
    need_sorted, need_blocks = padded_sizes(numel, num_experts, block_size)
    sorted_size = need_sorted if sorted_size is None else sorted_size
    blocks_size = need_blocks if blocks_size is None else blocks_size
    sorted_ids = np.full(sorted_size, numel, dtype=np.int32)
    expert_ids = np.full(blocks_size, -1, dtype=np.int32)
    pos = 0
    for e in range(num_experts):
        rows = np.nonzero(mapped == e)[0]
        if rows.size == 0:
            continue
        nblk = (rows.size + block_size - 1) // block_size
        sorted_ids[pos:pos + rows.size] = rows
        expert_ids[pos // block_size: pos // block_size + nblk] = e
        pos += nblk * block_size
    return sorted_ids, expert_ids, np.array([pos], dtype=np.int32)


def silu_and_mul(x):
    """out[..., j] = silu(x[..., j]) * x[..., H + j], fp32 math, rounded once."""
    x = torch.as_tensor(x).cpu()
    h = x.shape[-1] // 2
    gate, up = x[..., :h].float(), x[..., h:].float()
    return (gate * torch.sigmoid(gate) * up).to(x.dtype)


def moe_sum(x, topk_ids=None, expert_map=None):
    """out[t, h] = sum over slots of x[t, slot, h] in fp32; slots whose id is negative,
    beyond the map, or mapped to a negative value contribute zero
    (src/native/cuda/ops/moe_sum/kernel.cuh:24-38)."""
    x = torch.as_tensor(x).cpu()
    xf = x.float()
    if topk_ids is not None:
        ids = torch.as_tensor(topk_ids).cpu().to(torch.int64)
        active = ids >= 0
        if expert_map is not None:
            emap = torch.as_tensor(expert_map).cpu().to(torch.int64)
            inside = active & (ids < emap.numel())
            mapped = torch.full_like(ids, -1)
            mapped[inside] = emap[ids[inside]]
            active = inside & (mapped >= 0)
        xf = xf * active.unsqueeze(-1)
    return xf.sum(dim=1).to(x.dtype)


def moe_w4a16_gemm(a, q, scales, zeros, sorted_token_ids, expert_ids, num_tokens_post_pad,
                   topk_weights, block_size: int, top_k: int, mul_topk_weights: bool,
                   num_bits: int = 4, bias=None) -> torch.Tensor:
    """fp32 [M*top_k, N]; row r (a flat routing id) = a[r // top_k] @ dequant(W[expert of r]).

    a: [M, K]; q: [E, K, N] integers; scales: [E, G, N]; zeros: [E, G, N] integers or None.
    Rows never routed keep zero.  Routing loop as tests/test_moe_wna16_gemm.py:413-440.
    """
    a = torch.as_tensor(a).cpu().float()
    m = a.shape[0]
    n = quant._as_np(q).shape[2]
    out = torch.zeros((m * top_k, n), dtype=torch.float32)
    sorted_ids = quant._as_np(sorted_token_ids)
    experts = quant._as_np(expert_ids)
    cutoff = int(quant._as_np(num_tokens_post_pad).reshape(-1)[0])
    tw = None if topk_weights is None else torch.as_tensor(topk_weights).cpu().float().reshape(-1)
    cache: dict[int, torch.Tensor] = {}
    for blk, e in enumerate(experts.tolist()):
        if blk * block_size >= cutoff:
            break
        if e < 0:
            continue
        if e not in cache:
            cache[e] = quant.dequantize(quant._as_np(q)[e], torch.as_tensor(scales)[e],
                                        None if zeros is None else quant._as_np(zeros)[e], num_bits)
        rows = sorted_ids[blk * block_size:(blk + 1) * block_size]
        rows = rows[rows < m * top_k].astype(np.int64)
        if rows.size == 0:
            continue
        r = torch.as_tensor(rows)
        val = a[r // top_k] @ cache[e]
        if bias is not None:
            val = val + torch.as_tensor(bias).cpu().float()[e]
        if mul_topk_weights:
            val = val * tw[r].unsqueeze(-1)
        out[r] = val
    return out


def topk_sigmoid(gating_output, e_score_correction_bias, is_padding, topk: int, renormalize: bool,
                 routed_scaling_factor: float):
    """Returns (weights f32 [T,k], ids i64 [T,k], token_expert_indices i32 [T,k]).

    tests/test_topk_sigmoid.py:352-381 of the reference, with the two details its kernel adds
    (src/native/cuda/nvidia/ops/topk_sigmoid/kernel.cuh:103-106,55-64): a non-finite score counts as
    0, and equal selection scores go to the smaller expert index (a stable descending sort)."""
    g = torch.as_tensor(gating_output).cpu()
    scores = torch.sigmoid(g.to(torch.float32))
    scores = torch.where(torch.isfinite(scores), scores, torch.zeros_like(scores))
    selection = scores if e_score_correction_bias is None else scores + torch.as_tensor(e_score_correction_bias).cpu()
    ids = torch.argsort(selection, dim=-1, descending=True, stable=True)[:, :topk]
    weights = scores.gather(1, ids)
    if renormalize:
        denominator = weights.sum(dim=-1, keepdim=True)
        weights = weights / torch.where(denominator > 0, denominator, torch.ones_like(denominator))
    weights = weights * routed_scaling_factor
    if is_padding is not None:
        ids = ids.masked_fill(torch.as_tensor(is_padding).cpu().bool().unsqueeze(-1), -1)
    t = g.shape[0]
    tei = (torch.arange(topk, dtype=torch.int32).unsqueeze(0).expand(t, -1) * t
           + torch.arange(t, dtype=torch.int32).unsqueeze(-1))
    return weights, ids, tei


def moe_wna16_gemm(x, quantized_weight, scales, zero_points, bit: int, topk_weights, sorted_token_ids, expert_ids,
                   num_tokens_post_pad, block_size_m: int, top_k: int) -> torch.Tensor:
    """fp32 [M, top_k, N] for the plain layout: quantized_weight [E, N, K] integers, scales [E, N, G],
    zero_points [E, N, G] integers or None (tests/test_moe_wna16_gemm.py:384-442 of the reference;
    its bfloat16 / 8-bit rounding model is NOT restated: the tolerance of that case covers it)."""
    q = quant._as_np(quantized_weight).transpose(0, 2, 1)
    s = torch.as_tensor(scales).permute(0, 2, 1)
    z = None if zero_points is None else quant._as_np(zero_points).transpose(0, 2, 1)
    m = torch.as_tensor(x).shape[0]
    out = moe_w4a16_gemm(x, q, s, z, sorted_token_ids, expert_ids, num_tokens_post_pad, topk_weights, block_size_m,
                         top_k, topk_weights is not None, num_bits=bit)
    return out.reshape(m, top_k, -1)


def get_cutlass_moe_mm_data(topk_ids, num_experts: int, n: int, k: int, is_gated: bool = True,
                            with_blockscale: bool = False):
    """Returns (expert_offsets, problem_sizes1, problem_sizes2, input_permutation, output_permutation,
    blockscale_offsets or None) as int32 numpy arrays, routes of one expert placed by ascending route
    index (the reference places them in any order, tests/test_get_cutlass_moe_mm_data.py:412-491)."""
    ids = quant._as_np(topk_ids).astype(np.int64)
    topk = ids.shape[1]
    flat = ids.reshape(-1)
    valid = (flat >= 0) & (flat < num_experts)
    counts = np.bincount(flat[valid], minlength=num_experts)
    offsets = np.concatenate(([0], np.cumsum(counts))).astype(np.int32)
    swap = not with_blockscale and flat.size <= 64
    n1 = 2 * n if is_gated else n
    if swap:
        ps1 = np.stack((np.full(num_experts, n1), counts, np.full(num_experts, k)), axis=1)
        ps2 = np.stack((np.full(num_experts, k), counts, np.full(num_experts, n)), axis=1)
    else:
        ps1 = np.stack((counts, np.full(num_experts, n1), np.full(num_experts, k)), axis=1)
        ps2 = np.stack((counts, np.full(num_experts, k), np.full(num_experts, n)), axis=1)
    in_perm = np.full(flat.size, -1, dtype=np.int32)
    out_perm = np.full(flat.size, -1, dtype=np.int32)
    cursor = offsets[:-1].astype(np.int64).copy()
    for route, e in enumerate(flat.tolist()):
        if 0 <= e < num_experts:
            in_perm[cursor[e]] = route // topk
            out_perm[route] = cursor[e]
            cursor[e] += 1
        elif e == -1:
            out_perm[route] = offsets[-1]
    scale_offsets = None
    if with_blockscale:
        scale_offsets = np.concatenate(([0], np.cumsum((counts + 127) // 128 * 128))).astype(np.int32)
    return offsets, ps1.astype(np.int32), ps2.astype(np.int32), in_perm, out_perm, scale_offsets
