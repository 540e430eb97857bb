"""Seeded routing workload with a fingerprint.

Every rank's ``topk_idx`` / ``topk_weights`` are generated from ``random.Random(seed + rank)`` (pure Python, so the same
manifest comes out on every platform and library version), written to ``workload.json`` and protected by a SHA-256 over the
canonical JSON of its contents: two benchmark reports are comparable only if their fingerprints are equal.
Parity: tests/utils/ep_benchmark_manifest.py:77-238 of the reference.
"""
import hashlib
import json
import os
import random
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Dict, Tuple, Union

SCHEMA_VERSION = 1
GENERATOR_VERSION = 1


@dataclass(frozen=True)
class WorkloadSpec:
    world_size: int
    num_tokens: int
    hidden: int
    num_topk: int
    num_experts: int
    seed: int = 0
    unbalanced_ratio: float = 1.0      # scores of the experts of rank 0 are multiplied by this (>= 1)
    masked_ratio: float = 0.0          # probability that a selection is dropped (-1)

    def __post_init__(self) -> None:
        if self.world_size < 1:
            raise ValueError('world_size must be positive')
        if self.num_tokens <= 0 or self.hidden <= 0:
            raise ValueError('num_tokens and hidden must be positive')
        if self.num_experts <= 0 or self.num_experts % self.world_size != 0:
            raise ValueError('num_experts must be a positive multiple of world_size')
        if not 0 < self.num_topk <= self.num_experts:
            raise ValueError('num_topk must be in [1, num_experts]')
        if self.unbalanced_ratio < 1.0:
            raise ValueError('unbalanced_ratio must be at least one')
        if not 0.0 <= self.masked_ratio <= 1.0:
            raise ValueError('masked_ratio must be in [0, 1]')


@dataclass(frozen=True)
class RankWorkload:
    rank: int
    num_tokens: int
    topk_idx: Tuple[Tuple[int, ...], ...]
    topk_weights: Tuple[Tuple[float, ...], ...]


@dataclass(frozen=True)
class Manifest:
    spec: WorkloadSpec
    ranks: Tuple[RankWorkload, ...]
    fingerprint: str

    def to_dict(self) -> Dict[str, Any]:
        d = _payload(self.spec, self.ranks)
        d['fingerprint'] = self.fingerprint
        return d


def _rank_workload(spec: WorkloadSpec, rank: int) -> RankWorkload:
    rng = random.Random(spec.seed + rank)
    num_tokens = max(1, spec.num_tokens - rank)        # ranks differ in size on purpose
    per_rank = spec.num_experts // spec.world_size
    idx_rows, w_rows = [], []
    for _ in range(num_tokens):
        scores = [rng.random() * (spec.unbalanced_ratio if e < per_rank else 1.0) for e in range(spec.num_experts)]
        chosen = sorted(range(spec.num_experts), key=lambda e: (scores[e], e), reverse=True)[:spec.num_topk]
        rng.shuffle(chosen)
        weights = [scores[e] for e in chosen]
        for lane in range(spec.num_topk):
            if rng.random() < spec.masked_ratio:
                chosen[lane], weights[lane] = -1, 0.0
        idx_rows.append(tuple(chosen))
        w_rows.append(tuple(weights))
    return RankWorkload(rank, num_tokens, tuple(idx_rows), tuple(w_rows))


def _payload(spec: WorkloadSpec, ranks: Tuple[RankWorkload, ...]) -> Dict[str, Any]:
    return {'schema_version': SCHEMA_VERSION, 'generator_version': GENERATOR_VERSION, 'spec': asdict(spec),
            'ranks': [asdict(r) for r in ranks]}


def fingerprint_of(spec: WorkloadSpec, ranks: Tuple[RankWorkload, ...]) -> str:
    text = json.dumps(_payload(spec, ranks), sort_keys=True, separators=(',', ':'))
    return hashlib.sha256(text.encode('ascii')).hexdigest()


def build_manifest(spec: WorkloadSpec) -> Manifest:
    ranks = tuple(_rank_workload(spec, r) for r in range(spec.world_size))
    return Manifest(spec, ranks, fingerprint_of(spec, ranks))


def write_text_atomic(path: Union[str, Path], text: str) -> None:
    """Write next to the target, fsync, rename: readers never see a half-written artifact."""
    path = Path(path)
    tmp = path.with_name(path.name + '.tmp.%d' % os.getpid())
    with open(tmp, 'w', encoding='utf-8') as f:
        f.write(text)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def write_manifest(path: Union[str, Path], manifest: Manifest) -> None:
    write_text_atomic(path, json.dumps(manifest.to_dict(), indent=1, sort_keys=True) + '\n')


def load_manifest(path: Union[str, Path]) -> Manifest:
    d = json.loads(Path(path).read_text(encoding='utf-8'))
    if d.get('schema_version') != SCHEMA_VERSION or d.get('generator_version') != GENERATOR_VERSION:
        raise ValueError('unsupported workload manifest version')
    spec = WorkloadSpec(**d['spec'])
    ranks = tuple(RankWorkload(r['rank'], r['num_tokens'], tuple(tuple(row) for row in r['topk_idx']),
                               tuple(tuple(row) for row in r['topk_weights'])) for r in d['ranks'])
    fp = fingerprint_of(spec, ranks)
    if d.get('fingerprint') != fp:
        raise ValueError('workload manifest fingerprint does not match its contents')
    return Manifest(spec, ranks, fp)
