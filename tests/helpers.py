"""Problem builders shared by the GPU parity tests (inputs per the benchmark configurations)."""

from __future__ import annotations

import numpy as np
import torch

from oracle import quant as oq


def make_quantized(k, n, group_size, dtype, has_zeros, seed, device="cuda"):
    """Random int4 weights [K, N], scales |N(0,1)|*0.01+1e-3, optional int4 zeros [G, N]."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (k, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8)
    groups = 1 if group_size in (-1, k) else k // group_size
    scales = (torch.randn((groups, n), generator=gen).abs() * 0.01 + 1e-3).to(dtype)
    zeros = torch.randint(0, 16, (groups, n), generator=gen, dtype=torch.int32).numpy().astype(np.uint8) \
        if has_zeros else None
    return q, scales, zeros


def to_device_weights(q, scales, zeros, source="gptq", device="cuda"):
    """Packs on the CPU with the oracle's GPTQ/AWQ packers and returns device tensors
    (source-packed weight, scales, packed zeros)."""
    packed = oq.gptq_pack(q, 4) if source == "gptq" else oq.awq_pack(q, 4)
    packed_t = torch.from_numpy(packed).to(device)
    zeros_t = None if zeros is None else torch.from_numpy(oq.pack_zeros(zeros, 4)).to(device)
    return packed_t, scales.to(device), zeros_t


def rel_max_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    return float((got.float().cpu() - ref.float().cpu()).abs().max() / ref.float().abs().max().clamp_min(1e-30))
