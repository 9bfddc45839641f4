"""CPU oracle for the int4/int8 weight-only quantised linear path (TEST INFRASTRUCTURE ONLY).

This module is the checker, never the product: only tests, the smoke check and
the CPU-baseline leg of the benchmark may import it.  Everything here is a
restatement, in numpy / CPU torch, of what the reference's own tests define
for this path:

* GPTQ packing            -- tests/test_gptq_marlin_repack.py:137-147
* AWQ packing             -- tests/test_awq_marlin_repack.py:116-132
* Marlin tile packing     -- tests/test_gptq_marlin_repack.py:150-211 (same helper in
                             tests/test_awq_marlin_repack.py:135-196)
* act-order repack        -- tests/test_gptq_marlin_repack.py:45-49
* dequantise-then-matmul  -- tests/test_moe_wna16_gemm.py:397-404,437

The Marlin packing is written here as a closed-form index map (which (k, n)
lands in which bit-field of which output word) instead of the reference's
permutation-list construction; `tests/golden/make_golden.py` checks the two
agree on every variant and stores the resulting vectors.

Parity status: repack is pinned bit-exactly by the reference's helper (golden
vectors committed).  The GEMM value oracle follows the reference's
dequantise-then-matmul formula; the reference holds no golden GEMM values for
the Marlin path, so GEMM parity is "unpinned" beyond that formula.
"""

from __future__ import annotations

import numpy as np
import torch

# vLLM scalar-type ids accepted by the reference
# (src/base/moe_wna16_marlin_gemm.h:172-184).
UINT4B8 = 1125899907892224  # GPTQ symmetric, implicit zero point 8
UINT4 = 1125899906843648  # AWQ, explicit zero points
UINT8B128 = 1125899923621888

_AWQ_ORDER_4 = (0, 4, 1, 5, 2, 6, 3, 7)
_AWQ_ORDER_8 = (0, 2, 1, 3)


def _as_np(x) -> np.ndarray:
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy()
    return np.asarray(x)


def gptq_pack(unpacked, num_bits: int = 4) -> np.ndarray:
    """[K, N] integers -> int32 [K/pf, N]; field i of a word is row pf*(k/pf)+i.

    Follows tests/test_gptq_marlin_repack.py:137-147.
    """
    w = _as_np(unpacked).astype(np.uint32)
    pf = 32 // num_bits
    k, n = w.shape
    w = w.reshape(k // pf, pf, n)
    out = np.zeros((k // pf, n), dtype=np.uint32)
    for i in range(pf):
        out |= w[:, i, :] << np.uint32(num_bits * i)
    return out.view(np.int32)


def gptq_unpack(packed, num_bits: int = 4) -> np.ndarray:
    p = _as_np(packed).view(np.uint32)
    pf = 32 // num_bits
    mask = np.uint32((1 << num_bits) - 1)
    rows, n = p.shape
    out = np.empty((rows, pf, n), dtype=np.uint8)
    for i in range(pf):
        out[:, i, :] = (p >> np.uint32(num_bits * i)) & mask
    return out.reshape(rows * pf, n)


def awq_pack(unpacked, num_bits: int = 4) -> np.ndarray:
    """[K, N] integers -> int32 [K, N/pf]; logical column j sits in field order[j].

    Follows tests/test_awq_marlin_repack.py:116-132.
    """
    w = _as_np(unpacked).astype(np.uint32)
    pf = 32 // num_bits
    order = _AWQ_ORDER_4 if num_bits == 4 else _AWQ_ORDER_8
    k, n = w.shape
    w = w.reshape(k, n // pf, pf)
    out = np.zeros((k, n // pf), dtype=np.uint32)
    for logical, field in enumerate(order):
        out |= w[:, :, logical] << np.uint32(num_bits * field)
    return out.view(np.int32)


def awq_unpack(packed, num_bits: int = 4) -> np.ndarray:
    p = _as_np(packed).view(np.uint32)
    pf = 32 // num_bits
    order = _AWQ_ORDER_4 if num_bits == 4 else _AWQ_ORDER_8
    mask = np.uint32((1 << num_bits) - 1)
    k, words = p.shape
    out = np.empty((k, words, pf), dtype=np.uint8)
    for logical, field in enumerate(order):
        out[:, :, logical] = (p >> np.uint32(num_bits * field)) & mask
    return out.reshape(k, words * pf)


def marlin_source_index(size_k: int, size_n: int, num_bits: int, is_a_8bit: bool):
    """For every output (word, field) give the (k, n) it holds.

    Returns (k_idx, n_idx), both int64 arrays of shape [K*N/pf, pf], where the
    first axis is the flat word index of the [K/16, N*16/pf] output.

    Closed form of the layout produced by tests/test_gptq_marlin_repack.py:150-211:
    the output is a sequence of 1024-element chunks; with 16-bit activations a
    chunk is a 16(k) x 64(n) block, with 8-bit activations a 32(k) x 32(n) block;
    inside a chunk the words are ordered lane-major (32 "lanes", the threads of
    an m16n8k16 fragment) and each word mixes two n columns 8 apart with four
    (or eight) k rows.
    """
    pf = 32 // num_bits
    n_words = size_k * size_n // pf
    word = np.arange(n_words, dtype=np.int64)[:, None]
    field = np.arange(pf, dtype=np.int64)[None, :]
    words_per_chunk = 1024 // pf
    chunk = word // words_per_chunk
    inner = word % words_per_chunk
    if not is_a_8bit:
        chunks_per_row = size_n // 64
        k0 = (chunk // chunks_per_row) * 16
        n0 = (chunk % chunks_per_row) * 64
        if num_bits == 4:
            lane, sub = inner // 4, inner % 4
            k = 2 * (lane % 4) + (field >> 2) + 8 * (field & 1)
            n = lane // 4 + 8 * ((field >> 1) & 1) + 16 * sub
        else:
            lane, sub, half = inner // 8, (inner // 2) % 4, inner % 2
            k = 2 * (lane % 4) + (field >> 1) + 8 * (field & 1)
            n = lane // 4 + 8 * half + 16 * sub + 0 * field
    else:
        chunks_per_row = size_n // 32
        k0 = (chunk // chunks_per_row) * 32
        n0 = (chunk % chunks_per_row) * 32
        if num_bits == 4:
            lane, sub, half = inner // 4, (inner // 2) % 2, inner % 2
            k = 4 * (lane % 4) + (field >> 1) + 16 * (field & 1)
            n = lane // 4 + 8 * half + 16 * sub + 0 * field
        else:
            lane, sub, q = inner // 8, (inner // 4) % 2, inner % 4
            k = 4 * (lane % 4) + field + 16 * (q % 2)
            n = lane // 4 + 8 * (q // 2) + 16 * sub + 0 * field
    return (k0 + k), (n0 + n)


def marlin_pack(unpacked, num_bits: int = 4, is_a_8bit: bool = False) -> np.ndarray:
    """[K, N] integers -> int32 [K/16, N*16/pf] in the Marlin tile layout."""
    w = _as_np(unpacked).astype(np.uint32)
    size_k, size_n = w.shape
    pf = 32 // num_bits
    k_idx, n_idx = marlin_source_index(size_k, size_n, num_bits, is_a_8bit)
    vals = w[k_idx, n_idx]
    shifts = (np.arange(pf, dtype=np.uint32) * np.uint32(num_bits))[None, :]
    words = np.bitwise_or.reduce(vals << shifts, axis=1).astype(np.uint32)
    return words.reshape(size_k // 16, size_n * 16 // pf).view(np.int32)


def marlin_unpack(packed, size_k: int, size_n: int, num_bits: int = 4,
                  is_a_8bit: bool = False) -> np.ndarray:
    """Inverse of `marlin_pack`: int32 [K/16, N*16/pf] -> uint8 [K, N]."""
    p = _as_np(packed).view(np.uint32).reshape(-1)
    pf = 32 // num_bits
    k_idx, n_idx = marlin_source_index(size_k, size_n, num_bits, is_a_8bit)
    shifts = (np.arange(pf, dtype=np.uint32) * np.uint32(num_bits))[None, :]
    vals = (p[:, None] >> shifts) & np.uint32((1 << num_bits) - 1)
    out = np.empty((size_k, size_n), dtype=np.uint8)
    out[k_idx, n_idx] = vals
    return out


def marlin_unpack_w4(packed, size_k: int, size_n: int) -> np.ndarray:
    """`marlin_unpack` for 4-bit weights with 16-bit activations, written as reshapes and one
    transpose so that full-size matrices (4096 x 28672) unpack in well under a second.
    Same index map as `marlin_source_index`: word [kt][nb * 128 + (4 * l4 + c) * 4 + sub], field
    f = 4 * f2 + 2 * f1 + f0 holds k = 16 kt + 8 f0 + 2 c + f2, n = 64 nb + 16 sub + 8 f1 + l4.
    tests/test_oracle_golden.py checks it against `marlin_unpack`."""
    p = np.ascontiguousarray(_as_np(packed)).view(np.uint8).reshape(size_k // 16, size_n // 64, 8, 4, 4, 4)
    vals = np.stack((p & np.uint8(0xF), p >> np.uint8(4)), axis=-1)    # field = 2 * byte + nibble (little endian)
    vals = vals.reshape(size_k // 16, size_n // 64, 8, 4, 4, 2, 2, 2)  # kt nb l4 c sub f2 f1 f0
    out = vals.transpose(0, 7, 3, 5, 1, 4, 6, 2)                       # kt f0 c f2 | nb sub f1 l4
    return np.ascontiguousarray(out).reshape(size_k, size_n)


def gptq_marlin_repack(b_q_weight, perm, size_k: int, size_n: int, num_bits: int = 4,
                       is_a_8bit: bool = False) -> np.ndarray:
    """GPTQ-packed [K/pf, N] (+ optional act-order `perm` [K]) -> Marlin layout.

    Expected result per tests/test_gptq_marlin_repack.py:45-49: the Marlin
    packing of `unpacked[perm]`.
    """
    w = gptq_unpack(b_q_weight, num_bits)
    assert w.shape == (size_k, size_n)
    perm = _as_np(perm)
    if perm.size:
        w = w[perm.astype(np.int64)]
    return marlin_pack(w, num_bits, is_a_8bit)


def awq_marlin_repack(b_q_weight, size_k: int, size_n: int, num_bits: int = 4,
                      is_a_8bit: bool = False) -> np.ndarray:
    """AWQ-packed [K, N/pf] -> Marlin layout (tests/test_awq_marlin_repack.py:21-50)."""
    w = awq_unpack(b_q_weight, num_bits)
    assert w.shape == (size_k, size_n)
    return marlin_pack(w, num_bits, is_a_8bit)


def pack_zeros(zeros, num_bits: int = 4) -> np.ndarray:
    """[G, N] integer zero points -> int32 [G, N/pf], field j = column pf*(n/pf)+j.

    The reference fixes only the SHAPE of `b_zeros` ([.., G, N/pack_factor] int32,
    src/base/moe_wna16_marlin_gemm.h:231-240); this sequential field order is
    the layout this library defines for it.
    """
    z = _as_np(zeros).astype(np.uint32)
    pf = 32 // num_bits
    g, n = z.shape
    z = z.reshape(g, n // pf, pf)
    out = np.zeros((g, n // pf), dtype=np.uint32)
    for j in range(pf):
        out |= z[:, :, j] << np.uint32(num_bits * j)
    return out.view(np.int32)


def dequantize(q, scales, zeros=None, num_bits: int = 4) -> torch.Tensor:
    """fp32 weights [K, N] = (q - zp) * scale, scale/zero per group along K.

    q: [K, N] integers; scales: [G, N]; zeros: [G, N] integers or None
    (None -> zp = 2**(bits-1)).  tests/test_moe_wna16_gemm.py:397-404 with the
    weight stored [K, N] instead of [N, K].
    """
    qf = torch.as_tensor(_as_np(q).astype(np.float32))
    s = torch.as_tensor(scales).float().cpu()
    k = qf.shape[0]
    group = k // s.shape[0]
    s = s.repeat_interleave(group, dim=0)
    if zeros is None:
        zp = float(1 << (num_bits - 1))
    else:
        zp = torch.as_tensor(_as_np(zeros).astype(np.float32)).repeat_interleave(group, dim=0)
    return (qf - zp) * s


def dequantize_float8(q, scales) -> torch.Tensor:
    """fp32 weights [K, N] = float8_e4m3fn(byte) * scale, scale per group along K.

    q: [K, N] bytes, each the bit pattern of a float8_e4m3fn number (the weight type the operator
    accepts as `kFloat8E4M3Fn`, four weights per 32-bit word: src/base/moe_wna16_marlin_gemm.h:172-200);
    scales: [G, N].  The reference's tests hold no float8 case: this follows the type's definition
    (torch's own conversion) and the grouped-scale rule of `dequantize` above.
    """
    values = torch.from_numpy(np.ascontiguousarray(_as_np(q).astype(np.uint8))).view(torch.float8_e4m3fn).float()
    s = torch.as_tensor(scales).float().cpu()
    return values * s.repeat_interleave(values.shape[0] // s.shape[0], dim=0)


def w4a16_gemm(a, q, scales, zeros=None, num_bits: int = 4, bias=None) -> torch.Tensor:
    """fp32 [M, N] = a.float() @ dequantize(q) (+ bias); fp32 accumulate.

    tests/test_moe_wna16_gemm.py:437 (`input.float() @ weights.T`).
    """
    w = dequantize(q, scales, zeros, num_bits)
    out = torch.as_tensor(a).float().cpu() @ w
    if bias is not None:
        out = out + torch.as_tensor(bias).float().cpu()
    return out
