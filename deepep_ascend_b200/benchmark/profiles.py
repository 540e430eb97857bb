"""Named benchmark sizes.  ``canonical`` and ``smoke`` are the reference's (tests/benchmark/profiles.py:27-49);
``headline`` is the shape its README numbers are quoted on (8192 tokens, top-8 of 256 experts)."""
from dataclasses import dataclass
from types import MappingProxyType
from typing import Mapping, Optional

from .workload import Manifest, WorkloadSpec, build_manifest


@dataclass(frozen=True)
class Profile:
    name: str
    world_size: int
    num_tokens: int
    hidden: int
    num_topk: int
    num_experts: int
    seed: int
    warmups: int
    iterations: int
    unbalanced_ratio: float = 1.0
    masked_ratio: float = 0.0


PROFILES: Mapping[str, Profile] = MappingProxyType({
    'canonical': Profile('canonical', 8, 4096, 7168, 6, 256, 0, 30, 30),
    'headline': Profile('headline', 8, 8192, 7168, 8, 256, 0, 5, 20),
    'smoke': Profile('smoke', 8, 16, 128, 2, 8, 0, 1, 1),
})


def profile_spec(profile: Profile, world_size: Optional[int] = None) -> WorkloadSpec:
    return WorkloadSpec(world_size or profile.world_size, profile.num_tokens, profile.hidden, profile.num_topk, profile.num_experts,
                        profile.seed, profile.unbalanced_ratio, profile.masked_ratio)


def profile_manifest(profile: Profile, world_size: Optional[int] = None) -> Manifest:
    return build_manifest(profile_spec(profile, world_size))
