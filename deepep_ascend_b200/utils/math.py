"""Numeric helpers: FP8 (e4m3, 1x128 block scales) casting in plain PyTorch, difference metrics,
alignment arithmetic and tensor hashing.

The casting functions are the fp32 PyTorch statement of what the fused dispatch kernels compute, and are
what the numerics tests compare the kernels with (parity: deep_ep/utils/math.py:5-103).
"""
from typing import Tuple

import torch

FP8_E4M3_MAX = 448.0
FP8_BLOCK = 128


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - cosine-like similarity of (x+1, y+1) in float64; 0 means identical."""
    x, y = x.double() + 1, y.double() + 1
    denominator = (x * x + y * y).sum()
    if denominator == 0:
        return 0.0
    return float(1 - 2 * (x * y).sum() / denominator)


def ceil_div(x: int, y: int) -> int:
    return (x + y - 1) // y


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def per_token_cast_to_fp8(x: torch.Tensor, round_scale: bool = False,
                          use_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantize ``x [m, n]`` to e4m3 with one scale per (token, 128 channels).

    amax is clamped to 1e-4, ``q = x * (448 / amax)`` in fp32 rounded to nearest-even, and the returned
    scale is ``amax / 448`` (the dequantization factor).  With ``round_scale`` the dequantization factor is
    rounded up to a power of two first (``q = x / 2^ceil(log2(amax/448))``); with ``use_ue8m0`` four such
    exponents are packed into one int32 per 512 channels.
    """
    assert x.dim() == 2
    m, n = x.shape
    aligned_n = align(n, FP8_BLOCK)
    xp = torch.nn.functional.pad(x.float(), (0, aligned_n - n)).view(m, aligned_n // FP8_BLOCK, FP8_BLOCK)
    amax = xp.abs().amax(dim=2).clamp(1e-4)
    if round_scale or use_ue8m0:
        sf = torch.exp2(torch.ceil(torch.log2(amax / FP8_E4M3_MAX)))
        q = (xp * (1.0 / sf).unsqueeze(2))
    else:
        sf = amax / FP8_E4M3_MAX
        q = xp * (FP8_E4M3_MAX / amax).unsqueeze(2)
    q = q.clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX).to(torch.float8_e4m3fn).view(m, aligned_n)[:, :n].contiguous()
    if use_ue8m0:
        exps = (sf.view(torch.int32) >> 23).to(torch.uint8)
        pad = align(exps.shape[1], 4) - exps.shape[1]
        exps = torch.nn.functional.pad(exps, (0, pad))
        return q, exps.contiguous().view(torch.int32)
    return q, sf


def per_token_cast_back(x_fp8: torch.Tensor, x_scales: torch.Tensor) -> torch.Tensor:
    """Dequantize the output of :func:`per_token_cast_to_fp8` (fp32 or packed UE8M0 scales) to bf16."""
    if x_fp8.numel() == 0:
        return x_fp8.to(torch.bfloat16)
    assert x_fp8.dim() == 2
    m, n = x_fp8.shape
    aligned_n = align(n, FP8_BLOCK)
    num_blocks = aligned_n // FP8_BLOCK
    xp = torch.nn.functional.pad(x_fp8.float(), (0, aligned_n - n)).view(m, -1, FP8_BLOCK)
    if x_scales.dtype == torch.int32:
        x_scales = (x_scales.contiguous().view(torch.uint8).to(torch.int32) << 23).view(torch.float32)
    x_scales = x_scales.reshape(m, -1)[:, :num_blocks].float()
    return (xp * x_scales.unsqueeze(2)).view(m, aligned_n)[:, :n].to(torch.bfloat16).contiguous()


def inplace_unique(x: torch.Tensor, num_slots: int) -> None:
    """Replace each row of ``x`` by its distinct non-negative values (descending), padded with -1."""
    assert x.dim() == 2
    counts = torch.zeros((x.size(0), num_slots + 1), dtype=x.dtype, device=x.device)
    counts.scatter_add_(1, x.masked_fill(x < 0, num_slots), torch.ones_like(x))
    present = counts[:, :num_slots] > 0
    ids = torch.arange(num_slots, device=x.device, dtype=x.dtype).expand_as(present)
    ids = torch.where(present, ids, torch.full_like(ids, -1))
    ids = torch.sort(ids, dim=-1, descending=True).values
    x.fill_(-1)
    width = min(num_slots, x.size(1))
    x[:, :width] = ids[:, :width]


def create_grouped_scores(scores: torch.Tensor, group_idx: torch.Tensor, num_groups: int) -> torch.Tensor:
    """Zero the scores of every expert group not listed in ``group_idx`` (group-limited gating)."""
    num_tokens, num_experts = scores.shape
    scores = scores.view(num_tokens, num_groups, -1)
    mask = torch.zeros((num_tokens, num_groups), dtype=torch.bool, device=scores.device)
    mask = mask.scatter_(1, group_idx, True).unsqueeze(-1).expand_as(scores)
    return (scores * mask).view(num_tokens, num_experts)


def hash_tensor(t: torch.Tensor) -> int:
    """Order-independent 32-bit-word checksum used by the determinism stress tests."""
    flat = t.contiguous().view(torch.uint8).flatten()
    pad = (-flat.numel()) % 4
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    return int(flat.view(torch.int32).sum(dtype=torch.int64).item())


def hash_tensors(*tensors) -> int:
    value = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            value ^= hash_tensors(*t)
        elif isinstance(t, torch.Tensor):
            value ^= hash_tensor(t)
    return value


def count_bytes(*tensors) -> int:
    total = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            total += count_bytes(*t)
        elif t is not None:
            total += t.numel() * t.element_size()
    return total


def logfmt10_roundtrip(x: torch.Tensor) -> torch.Tensor:
    """What a bf16 tensor ``[..., H]`` (H a multiple of 128) looks like after the LogFMT-10 coding of the low-latency
    combine (``use_logfmt=True``): per group of 128 channels the magnitudes are rounded to 510 equal steps of log2
    between the smallest non-zero and the largest magnitude of the group (at most 32 octaves), the sign is kept, zeros
    stay zero.  Returns fp32.  The device code evaluates log2 / exp2 with the hardware approximations, so single values can
    land on a neighbouring step; compare with a tolerance of one step."""
    xf = x.float()
    g = xf.reshape(*xf.shape[:-1], xf.shape[-1] // 128, 128)
    mag = g.abs()
    amax = mag.amax(dim=-1, keepdim=True)
    amin = torch.where(mag > 0, mag, torch.full_like(mag, float('inf'))).amin(dim=-1, keepdim=True)
    hi = torch.log2(amax.clamp_min(1e-38))
    lo = torch.maximum(torch.log2(amin.clamp(1e-38, 3e38)), hi - 32.0)
    step = (hi - lo) / 510.0
    inv = torch.where(step > 0, 1.0 / step, torch.zeros_like(step))
    code = torch.round(((torch.log2(mag.clamp_min(1e-38)) - lo) * inv).clamp(0, 510))
    dec = torch.exp2(lo + code * step)
    out = torch.where(mag > 0, torch.sign(g) * dec, torch.zeros_like(g))
    return out.reshape(xf.shape)
