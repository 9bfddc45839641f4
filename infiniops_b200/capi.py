"""ctypes view of ``libinfiniops_b200.so`` (the C ABI declared in ``include/infiniops_b200.h``).

The functions here take torch tensors only to read ``data_ptr()`` / shapes / strides; the
arithmetic is entirely in the CUDA library.  There is no fallback: if the library is
missing or a call returns a non-zero status, an exception is raised.
"""

from __future__ import annotations

import ctypes
import pathlib

import torch

_LIB_PATH = pathlib.Path(__file__).resolve().parent / "lib" / "libinfiniops_b200.so"

F32, F16, BF16, I32, I64, U32 = range(6)
QTYPE_UINT4B8 = 1125899907892224
QTYPE_UINT4 = 1125899906843648
QTYPE_UINT8B128 = 1125899923621888
QTYPE_UINT8 = 1125899906844672
QTYPE_FLOAT8_E4M3FN = 2814749767172868

_DTYPE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: I32,
          torch.int64: I64, torch.uint32: U32}

_vp, _i64, _int, _sz, _dbl = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t, ctypes.c_double

# name -> (restype, argtypes); every name must also be declared in include/infiniops_b200.h
PROTOTYPES = {
    "infiniops_b200_last_error": (ctypes.c_char_p, []),
    "infiniops_b200_version": (ctypes.c_char_p, []),
    "infiniops_b200_swap_device": (_int, [_int, _vp]),
    "infiniops_b200_thread_scratch": (_vp, [_int, _sz, _vp]),
    "infiniops_b200_gemm_scratch_prepare": (_int, [_vp, _sz, _vp]),
    "infiniops_b200_selftest_bounded_wait": (_int, [_vp, _sz, _vp, _vp]),
    "infiniops_b200_static_scratch_status": (_int, [_vp]),
    "infiniops_b200_gptq_marlin_repack": (_int, [_vp, _vp, _i64, _i64, _int, _int, _vp, _vp]),
    "infiniops_b200_awq_marlin_repack": (_int, [_vp, _i64, _i64, _int, _int, _vp, _vp]),
    "infiniops_b200_topk_softmax": (_int, [_vp, _int, _vp, _vp, _int, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
    "infiniops_b200_grouped_topk": (_int, [_vp, _int, _vp, _int, _i64, _i64, _i64, _i64, _i64, _int, _dbl, _int,
                                           _vp, _vp, _vp]),
    "infiniops_b200_moe_align_block_size_scratch_bytes": (_sz, [_i64, _i64]),
    "infiniops_b200_moe_align_block_size": (_int, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp,
                                                   _sz, _vp]),
    "infiniops_b200_silu_and_mul": (_int, [_vp, _vp, _int, _int, _vp, _vp, _vp, _vp]),
    "infiniops_b200_moe_sum": (_int, [_vp, _int, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _int, _i64, _i64, _vp,
                                      _i64, _i64, _vp, _vp]),
    "infiniops_b200_scratch_status": (_int, [_vp, _vp]),
    "infiniops_b200_marlin_gemm_scratch_bytes": (_sz, [_i64, _i64, _i64]),
    "infiniops_b200_marlin_gemm_act_order_scratch_bytes": (_sz, [_i64, _i64, _i64]),
    "infiniops_b200_marlin_gemm": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp,
                                          _sz, _vp]),
    "infiniops_b200_marlin_gemm_static_scratch": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64,
                                                         _vp, _vp]),
    "infiniops_b200_moe_wna16_marlin_gemm_scratch_bytes": (_sz, [_i64, _i64, _i64, _i64, _i64, _i64]),
    "infiniops_b200_moe_wna16_marlin_gemm": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                                    _int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _sz,
                                                    _vp]),
}

MAX_PEERS = 7


class GemmProblem(ctypes.Structure):
    """`iob_gemm_problem` of include/infiniops_b200.h."""
    _fields_ = [("a", _vp), ("b_q_weight", _vp), ("b_bias", _vp), ("b_scales", _vp), ("b_zeros", _vp), ("out", _vp),
                ("size_m", _i64), ("size_n", _i64), ("size_k", _i64), ("num_groups", _i64),
                ("out_ld", _i64), ("out_col0", _i64), ("n_peers", _int), ("peer_out", _vp * MAX_PEERS),
                ("scale_layout", _int), ("g_idx", _vp), ("perm", _vp)]


class PeerSignal(ctypes.Structure):
    """`iob_peer_signal` of include/infiniops_b200.h."""
    _fields_ = [("done_counter", _vp), ("epoch", _vp), ("n_peers", _int), ("peer_flags", _vp * MAX_PEERS),
                ("flag_slot", _int)]


MAX_COPIES = 16


class PeerCopy(ctypes.Structure):
    """`iob_peer_copy`."""
    _fields_ = [("src", _vp), ("dst", _vp * MAX_PEERS), ("rows", _i64), ("row_bytes", _i64), ("pitch_bytes", _i64)]


class RoutedOptions(ctypes.Structure):
    """`iob_routed_options`."""
    _fields_ = [("scale_layout", _int), ("a_sorted", _int), ("out_sorted", _int), ("fuse_silu", _int),
                ("g_idx", _vp), ("perm", _vp), ("route_position", _vp), ("block_rows", _vp), ("row_dest", _vp),
                ("dest_base", _vp * (MAX_PEERS + 1)), ("n_dest", _int),
                ("signal", ctypes.POINTER(PeerSignal))]


class EpContext(ctypes.Structure):
    """`iob_ep_context`."""
    _fields_ = [("world", _int), ("rank", _int), ("top_k", _i64), ("hidden", _i64), ("inter", _i64),
                ("experts_per_rank", _i64), ("capacity", _i64), ("moe_block_size", _i64), ("a_dtype", _int),
                ("b_type_id", _i64), ("arena", _vp * (MAX_PEERS + 1)), ("flags", _vp * (MAX_PEERS + 1)), ("ctrl", _vp)]


class ExpertWeightsC(ctypes.Structure):
    """`iob_expert_weights`."""
    _fields_ = [("w13", _vp), ("s13", _vp), ("z13", _vp), ("groups13", _i64), ("w2", _vp), ("s2", _vp), ("z2", _vp),
                ("groups2", _i64), ("w13_interleaved", _int)]


PROTOTYPES.update({
    "infiniops_b200_moe_wna16_marlin_gemm_ex": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                                              _i64, _int, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp,
                                                              ctypes.POINTER(RoutedOptions), _vp, _sz, _vp]),
    "infiniops_b200_topk_softmax_align": (_int, [_vp, _int, _vp, _vp, _int, _int, _dbl, _vp, _vp, _vp, _i64, _i64, _i64,
                                                 _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _sz, _vp]),
    "infiniops_b200_grouped_topk_align": (_int, [_vp, _int, _vp, _int, _i64, _i64, _i64, _i64, _i64, _int, _dbl, _int,
                                                 _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _sz, _vp]),
    "infiniops_b200_moe_gather_sum": (_int, [_vp, _int, _vp, _i64, _i64, _i64, _vp, _vp]),
    "infiniops_b200_topk_sigmoid": (_int, [_vp, _int, _vp, _vp, _int, _dbl, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
    "infiniops_b200_get_cutlass_moe_mm_data": (_int, [_vp, _i64, _i64, _i64, _i64, _i64, _int, _vp, _vp, _vp, _vp, _vp,
                                                      _vp, _vp]),
    "infiniops_b200_moe_wna16_gemm": (_int, [_vp, _int, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64,
                                             _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    "infiniops_b200_ep_arena_bytes": (_sz, [_int, _i64, _i64]),
    "infiniops_b200_ep_workspace_bytes": (_sz, [ctypes.POINTER(EpContext)]),
    "infiniops_b200_ep_moe_layer": (_int, [ctypes.POINTER(EpContext), ctypes.POINTER(ExpertWeightsC), _vp, _vp, _vp,
                                           _i64, _vp, _vp, _sz, _vp]),
    "infiniops_b200_marlin_gemm_placed": (_int, [ctypes.POINTER(GemmProblem), _int, _i64, ctypes.POINTER(PeerSignal),
                                                 _vp, _sz, _vp]),
    "infiniops_b200_marlin_gemm_batch_scratch_bytes": (_sz, []),
    "infiniops_b200_marlin_gemm_batch": (_int, [ctypes.POINTER(GemmProblem), _int, _int, _i64,
                                                ctypes.POINTER(PeerSignal), _vp, _sz, _vp]),
    "infiniops_b200_peer_alloc": (_int, [_sz, ctypes.POINTER(_vp)]),
    "infiniops_b200_peer_free": (_int, [_vp]),
    "infiniops_b200_peer_export": (_int, [_vp, ctypes.c_char_p]),
    "infiniops_b200_peer_open": (_int, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "infiniops_b200_peer_close": (_int, [_vp]),
    "infiniops_b200_peer_wait": (_int, [_vp, _int, _int, _vp, _vp, _vp]),
    "infiniops_b200_peer_broadcast": (_int, [ctypes.POINTER(PeerCopy), _int, _int, ctypes.POINTER(PeerSignal), _vp]),
})

_lib = None


def lib() -> ctypes.CDLL:
    """Load the CUDA library, or fail loudly: there is no CPU or PyTorch fallback."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(f"{_LIB_PATH} is missing: run `python -m infiniops_b200.build` "
                               "(the operators have no fallback implementation)")
        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = handle
    return _lib


class Error(RuntimeError):
    pass


def _check(status: int) -> None:
    if status != 0:
        raise Error(f"status {status}: {lib().infiniops_b200_last_error().decode()}")


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(stream) -> ctypes.c_void_p:
    if stream is None:
        stream = torch.cuda.current_stream().cuda_stream
    return ctypes.c_void_p(stream)


_scratch: dict = {}


def scratch(device, nbytes: int, tag: str = "gemm") -> torch.Tensor:
    """A zero-initialised scratch buffer per (device, purpose) that only grows (test / bench
    convenience).  The GEMM keeps counters it expects to find zeroed, so it never shares a
    buffer with the token sort."""
    index = torch.device(device).index
    key = (torch.cuda.current_device() if index is None else index, tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def gptq_marlin_repack(b_q_weight, perm, size_k, size_n, num_bits, is_a_8bit, out, stream=None):
    p = perm if perm is not None and perm.numel() else None
    _check(lib().infiniops_b200_gptq_marlin_repack(_ptr(b_q_weight), _ptr(p), size_k, size_n, num_bits,
                                                   int(is_a_8bit), _ptr(out), _stream(stream)))


def awq_marlin_repack(b_q_weight, size_k, size_n, num_bits, is_a_8bit, out, stream=None):
    _check(lib().infiniops_b200_awq_marlin_repack(_ptr(b_q_weight), size_k, size_n, num_bits, int(is_a_8bit),
                                                  _ptr(out), _stream(stream)))


def topk_softmax(gating, bias, is_padding, renormalize, topk_weights, topk_indices, token_expert_indices,
                 stream=None):
    t, e = gating.shape
    _check(lib().infiniops_b200_topk_softmax(_ptr(gating), _DTYPE[gating.dtype], _ptr(bias), _ptr(is_padding),
                                             int(renormalize), _ptr(topk_weights), _ptr(topk_indices),
                                             _DTYPE[topk_indices.dtype], _ptr(token_expert_indices), t, e,
                                             topk_weights.shape[1], _stream(stream)))


def topk_sigmoid(gating, bias, is_padding, renormalize, routed_scaling_factor, topk_weights, topk_ids,
                 token_expert_indices, stream=None):
    t, e = gating.shape
    _check(lib().infiniops_b200_topk_sigmoid(_ptr(gating), _DTYPE[gating.dtype], _ptr(bias), _ptr(is_padding),
                                             int(renormalize), float(routed_scaling_factor), _ptr(topk_weights),
                                             _ptr(topk_ids), _DTYPE[topk_ids.dtype], _ptr(token_expert_indices), t, e,
                                             topk_weights.shape[1], _stream(stream)))


def grouped_topk(scores, bias, num_expert_group, topk_group, topk, renormalize, routed_scaling_factor,
                 scoring_func, topk_values, topk_indices, stream=None):
    t, e = scores.shape
    _check(lib().infiniops_b200_grouped_topk(_ptr(scores), _DTYPE[scores.dtype], _ptr(bias), _DTYPE[bias.dtype], t,
                                             e, num_expert_group, topk_group, topk, int(renormalize),
                                             float(routed_scaling_factor), scoring_func, _ptr(topk_values),
                                             _ptr(topk_indices), _stream(stream)))


def moe_align_block_size(topk_ids, expert_map, num_experts, block_size, sorted_token_ids, experts_ids,
                         num_tokens_post_pad, stream=None):
    numel = topk_ids.numel()
    need = lib().infiniops_b200_moe_align_block_size_scratch_bytes(numel, num_experts)
    buf = scratch(topk_ids.device, need, "align") if need else None
    _check(lib().infiniops_b200_moe_align_block_size(_ptr(topk_ids), _ptr(expert_map), numel, num_experts,
                                                     block_size, _ptr(sorted_token_ids), sorted_token_ids.numel(),
                                                     _ptr(experts_ids), experts_ids.numel(),
                                                     _ptr(num_tokens_post_pad), _ptr(buf),
                                                     0 if buf is None else buf.numel(), _stream(stream)))


def _sort_scratch(device, numel, num_experts):
    need = lib().infiniops_b200_moe_align_block_size_scratch_bytes(numel, num_experts)
    return scratch(device, need, "align") if need else None


def topk_softmax_align(gating, bias, is_padding, renormalize, topk_weights, topk_ids, token_expert_indices,
                       expert_map, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad, sigmoid=False,
                       routed_scaling_factor=1.0, stream=None):
    """Router and token sort in one call (one launch while tokens x top_k <= 1024)."""
    t, e = gating.shape
    buf = _sort_scratch(gating.device, topk_ids.numel(), e)
    _check(lib().infiniops_b200_topk_softmax_align(
        _ptr(gating), _DTYPE[gating.dtype], _ptr(bias), _ptr(is_padding), int(renormalize), int(sigmoid),
        float(routed_scaling_factor), _ptr(topk_weights), _ptr(topk_ids), _ptr(token_expert_indices), t, e,
        topk_weights.shape[1], _ptr(expert_map), block_size, _ptr(sorted_token_ids), sorted_token_ids.numel(),
        _ptr(experts_ids), experts_ids.numel(), _ptr(num_tokens_post_pad), _ptr(buf),
        0 if buf is None else buf.numel(), _stream(stream)))


def grouped_topk_align(scores, bias, num_expert_group, topk_group, topk, renormalize, routed_scaling_factor,
                       scoring_func, topk_values, topk_ids, expert_map, block_size, sorted_token_ids, experts_ids,
                       num_tokens_post_pad, stream=None):
    t, e = scores.shape
    buf = _sort_scratch(scores.device, topk_ids.numel(), e)
    _check(lib().infiniops_b200_grouped_topk_align(
        _ptr(scores), _DTYPE[scores.dtype], _ptr(bias), _DTYPE[bias.dtype], t, e, num_expert_group, topk_group, topk,
        int(renormalize), float(routed_scaling_factor), scoring_func, _ptr(topk_values), _ptr(topk_ids),
        _ptr(expert_map), block_size, _ptr(sorted_token_ids), sorted_token_ids.numel(), _ptr(experts_ids),
        experts_ids.numel(), _ptr(num_tokens_post_pad), _ptr(buf), 0 if buf is None else buf.numel(),
        _stream(stream)))


def moe_gather_sum(rows, position, out, stream=None):
    """out[t] = sum over slots of rows[position[t, slot]] (negative position: nothing)."""
    t, k = position.shape
    _check(lib().infiniops_b200_moe_gather_sum(_ptr(rows), _DTYPE[rows.dtype], _ptr(position), t, k, rows.shape[-1],
                                               _ptr(out), _stream(stream)))


def silu_and_mul(x, out, stream=None):
    nd = out.dim()
    arr = ctypes.c_int64 * nd
    _check(lib().infiniops_b200_silu_and_mul(_ptr(x), _ptr(out), _DTYPE[x.dtype], nd, arr(*out.shape),
                                             arr(*x.stride()), arr(*out.stride()), _stream(stream)))


def moe_sum(x, out, topk_ids=None, expert_map=None, stream=None):
    t, k, h = x.shape
    st, ss, sh = x.stride()
    ids_t, ids_s = (0, 0) if topk_ids is None else topk_ids.stride()
    _check(lib().infiniops_b200_moe_sum(_ptr(x), _DTYPE[x.dtype], t, k, h, st, ss, sh, _ptr(topk_ids),
                                        I32 if topk_ids is None else _DTYPE[topk_ids.dtype], ids_t, ids_s,
                                        _ptr(expert_map), 0 if expert_map is None else expert_map.numel(),
                                        0 if expert_map is None else expert_map.stride(0), _ptr(out),
                                        _stream(stream)))


def scratch_status(buf, stream=None) -> int:
    """0 unless a bounded on-device wait of a GEMM kernel using `buf` ever expired."""
    return lib().infiniops_b200_scratch_status(_ptr(buf), _stream(stream))


def marlin_gemm(a, b_q_weight, b_bias, b_scales, b_zeros, b_type_id, size_m, size_n, size_k, out, stream=None,
                scratch_buf=None, g_idx=None, perm=None):
    """`g_idx` / `perm` (int32 [size_k], both or neither): activation order."""
    if perm is None and g_idx is None:
        need = lib().infiniops_b200_marlin_gemm_scratch_bytes(size_m, size_n, size_k)
        buf = scratch_buf if scratch_buf is not None else scratch(a.device, need)
        _check(lib().infiniops_b200_marlin_gemm(_ptr(a), _DTYPE[a.dtype], _ptr(b_q_weight), _ptr(b_bias),
                                                _ptr(b_scales), _ptr(b_zeros), b_type_id, size_m, size_n, size_k,
                                                b_scales.shape[-2], _ptr(out), _ptr(buf), buf.numel(), _stream(stream)))
        return
    need = lib().infiniops_b200_marlin_gemm_act_order_scratch_bytes(size_m, size_n, size_k)
    buf = scratch_buf if scratch_buf is not None else scratch(a.device, need)
    problem = GemmProblem()
    problem.a, problem.b_q_weight, problem.b_bias = a.data_ptr(), b_q_weight.data_ptr(), _ptr(b_bias)
    problem.b_scales, problem.b_zeros, problem.out = b_scales.data_ptr(), _ptr(b_zeros), out.data_ptr()
    problem.size_m, problem.size_n, problem.size_k, problem.num_groups = size_m, size_n, size_k, b_scales.shape[-2]
    problem.g_idx, problem.perm = _ptr(g_idx), _ptr(perm)
    _check(lib().infiniops_b200_marlin_gemm_placed(ctypes.byref(problem), _DTYPE[a.dtype], b_type_id, None, _ptr(buf),
                                                   buf.numel(), _stream(stream)))


def marlin_gemm_static_scratch(a, b_q_weight, b_bias, b_scales, b_zeros, b_type_id, size_m, size_n, size_k, out,
                               stream=None):
    """The dense GEMM on the library's built-in scratch array: for callers that cannot allocate
    device memory.  Nothing is allocated here either (no torch tensor is created)."""
    _check(lib().infiniops_b200_marlin_gemm_static_scratch(_ptr(a), _DTYPE[a.dtype], _ptr(b_q_weight), _ptr(b_bias),
                                                           _ptr(b_scales), _ptr(b_zeros), b_type_id, size_m, size_n,
                                                           size_k, b_scales.shape[-2], _ptr(out), _stream(stream)))


def moe_wna16_marlin_gemm(a, b_q_weight, b_bias, b_scales, b_zeros, sorted_token_ids, expert_ids,
                          num_tokens_past_padded, topk_weights, moe_block_size, top_k, mul_topk_weights, b_type_id,
                          size_m, size_n, size_k, out, stream=None, scratch_buf=None, scale_layout=0, a_sorted=False,
                          out_sorted=False, fuse_silu=False, g_idx=None, perm=None, route_position=None, block_rows=None):
    e = b_q_weight.shape[0]
    need = lib().infiniops_b200_moe_wna16_marlin_gemm_scratch_bytes(size_m, top_k, size_n, size_k, e,
                                                                    moe_block_size)
    buf = scratch_buf if scratch_buf is not None else scratch(a.device, need)
    options = RoutedOptions()
    options.scale_layout, options.a_sorted, options.out_sorted = scale_layout, int(a_sorted), int(out_sorted)
    options.fuse_silu = int(fuse_silu)
    options.g_idx = None if g_idx is None else g_idx.data_ptr()
    options.perm = None if perm is None else perm.data_ptr()
    options.route_position = None if route_position is None else route_position.data_ptr()
    options.block_rows = None if block_rows is None else block_rows.data_ptr()
    _check(lib().infiniops_b200_moe_wna16_marlin_gemm_ex(
        _ptr(a), _DTYPE[a.dtype], _ptr(b_q_weight), _ptr(b_bias), _ptr(b_scales), _ptr(b_zeros),
        _ptr(sorted_token_ids), _ptr(expert_ids), _ptr(num_tokens_past_padded), _ptr(topk_weights), moe_block_size,
        top_k, int(mul_topk_weights), b_type_id, size_m, size_n, size_k, b_scales.shape[-2], e,
        sorted_token_ids.numel(), _ptr(out), ctypes.byref(options), _ptr(buf), buf.numel(), _stream(stream)))


def gemm_problem(a, b_q_weight, b_bias, b_scales, b_zeros, out, size_m, size_n, size_k, out_ld=0, out_col0=0,
                 peer_out=(), scale_layout=0) -> GemmProblem:
    """One entry of a problem list.  `out` may be a tensor or a raw device address; `peer_out` are the
    addresses of the other GPUs' result matrices (already mapped into this process)."""
    g = GemmProblem()
    g.a, g.b_q_weight, g.b_scales = a.data_ptr(), b_q_weight.data_ptr(), b_scales.data_ptr()
    g.b_bias = None if b_bias is None else b_bias.data_ptr()
    g.b_zeros = None if b_zeros is None else b_zeros.data_ptr()
    g.out = out if isinstance(out, int) else out.data_ptr()
    g.size_m, g.size_n, g.size_k, g.num_groups = size_m, size_n, size_k, b_scales.shape[-2]
    g.out_ld, g.out_col0, g.n_peers, g.scale_layout = out_ld, out_col0, len(peer_out), scale_layout
    for i, ptr in enumerate(peer_out):
        g.peer_out[i] = ptr
    return g


def peer_copy(src_ptr: int, dst_ptrs, rows: int, row_bytes: int, pitch_bytes: int) -> PeerCopy:
    c = PeerCopy()
    c.src, c.rows, c.row_bytes, c.pitch_bytes = src_ptr, rows, row_bytes, pitch_bytes
    for i, ptr in enumerate(dst_ptrs):
        c.dst[i] = ptr
    return c


def peer_broadcast(copies, n_peers: int, signal=None, stream=None):
    """`copies`: a ctypes array `(PeerCopy * n)(...)`, at most MAX_COPIES entries (build it once)."""
    _check(lib().infiniops_b200_peer_broadcast(copies, len(copies), n_peers,
                                               None if signal is None else ctypes.byref(signal), _stream(stream)))


def problem_array(problems):
    return (GemmProblem * len(problems))(*problems)


def marlin_gemm_batch(problems, a_dtype, b_type_id, scratch_buf, signal=None, stream=None):
    """`problems`: a ctypes array from `problem_array` (build it once, outside the hot loop)."""
    _check(lib().infiniops_b200_marlin_gemm_batch(problems, len(problems), _DTYPE[a_dtype], b_type_id,
                                                  None if signal is None else ctypes.byref(signal),
                                                  _ptr(scratch_buf), scratch_buf.numel(), _stream(stream)))


def marlin_gemm_placed(problem, a_dtype, b_type_id, scratch_buf, signal=None, stream=None):
    _check(lib().infiniops_b200_marlin_gemm_placed(ctypes.byref(problem), _DTYPE[a_dtype], b_type_id,
                                                   None if signal is None else ctypes.byref(signal),
                                                   _ptr(scratch_buf), scratch_buf.numel(), _stream(stream)))
