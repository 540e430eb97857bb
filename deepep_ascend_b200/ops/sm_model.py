"""Analytical SM-count selection for the dispatch / combine kernels on B200.

Same structure as the reference model (deep_ep/buffers/elastic.py:1253-1369): the kernel is bounded by the
NVLink traffic of the rank; find the number of SMs whose aggregate per-SM issue rate covers that bandwidth,
add 25 % headroom, round up to an even count of at least 4, and use at least 64 SMs when the caller does not
intend to overlap communication with compute.

Differences: one flat NVLink domain (no RDMA terms), and the per-SM constants are B200 measurements of THIS
library's kernels rather than the reference's H800-era constants (200 / 50 GB/s).
"""
import math

from ..utils.math import align

# Per-SM throughput of THIS library's fused kernels on B200, GB/s, from the SM sweeps of `bench.py --sweep-sms` /
# `--min-sms` (8192 tokens, hidden 7168, top-8 of 256):
#   * write side = dispatch with the fused bf16 -> e4m3 cast: 24 SMs deliver 600 GB/s of received rows at EP4 (SM-bound: 64 SMs
#     reach 720) and 614 GB/s at EP8 (95 % of the 64-SM rate), i.e. 25 GB/s of rows per SM while the cast is the limit and about
#     40 GB/s of NVLink stores per SM once the link is; 40 is what reproduces "24 SMs are within 5 % of the link" at EP8;
#   * read side = the pull of combine: 24 SMs deliver 800 GB/s at EP4 (96 % of the 64-SM rate), at least 33 GB/s per SM with
#     the fp32 reduction included.  (The reference's 200 / 50 GB/s are constants of its own copy kernels on H800.)
SM_READ_GBS = 35.0
SM_WRITE_GBS = 40.0
NVLINK_GBS = 770.0     # measured peer-copy bandwidth per direction on this pool's B200s


def expected_topk_groups(num_experts: int, num_groups: int, num_topk: int) -> float:
    """Expected number of distinct groups (ranks) hit by a uniform top-k over ``num_experts`` experts."""
    if num_groups <= 1:
        return 1.0
    per_group = num_experts // num_groups
    return num_groups * (1 - math.comb(num_experts - per_group, num_topk) / math.comb(num_experts, num_topk))


def theoretical_num_sms(num_ranks: int, num_experts: int, num_topk: int, nvlink_gbs: float = 0, sm_read_gbs: float = 0,
                        sm_write_gbs: float = 0, prefer_overlap_with_compute: bool = True, num_device_sms: int = 148) -> int:
    nvlink_gbs = nvlink_gbs or NVLINK_GBS
    sm_read_gbs = sm_read_gbs or SM_READ_GBS
    sm_write_gbs = sm_write_gbs or SM_WRITE_GBS
    if num_ranks <= 1:
        num_sms = num_device_sms if not prefer_overlap_with_compute else 64
        return min(num_sms, num_device_sms)
    hit = expected_topk_groups(num_experts, num_ranks, num_topk)
    # per unit of bytes written to peers: each token is read once and written `hit` times
    sm_read = 1.0 / hit
    sm_write = 1.0
    nvlink_traffic = 1.0 - 1.0 / num_ranks
    need = max(nvlink_gbs / nvlink_traffic * sm_read / sm_read_gbs, nvlink_gbs / nvlink_traffic * sm_write / sm_write_gbs)
    num_sms = align(max(4, math.ceil(need * 1.25)), 2)
    if not prefer_overlap_with_compute:
        num_sms = max(num_sms, 64)
    return min(num_sms, num_device_sms)
