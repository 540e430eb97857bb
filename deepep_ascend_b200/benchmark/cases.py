"""The API-mode matrix: handle copy x expert alignment x dispatch precision x number of biases x stream plumbing.

Parity: tests/utils/ep_benchmark_manifest.py:9-75 of the reference (144 cases; a case that uses ``previous_event`` always
allocates on the communication stream, which is why the count is 2*2*2*3*(2*2 + 2) and not 192).
"""
from dataclasses import dataclass
from itertools import product
from typing import Tuple

CORRECTNESS_OPERATIONS = ('dispatch', 'expanded_dispatch', 'cached_dispatch', 'cached_expanded_padding', 'combine', 'reduced_combine')
PERFORMANCE_OPERATIONS = ('dispatch', 'expanded_dispatch', 'cached_dispatch', 'combine', 'reduced_combine')


@dataclass(frozen=True)
class ModeCase:
    do_handle_copy: bool
    expert_alignment: int
    use_fp8_dispatch: bool
    num_bias: int
    with_previous_event: bool
    async_with_compute_stream: bool
    allocate_on_comm_stream: bool

    @property
    def case_id(self) -> str:
        return ('ep-{}-align{}-bias{}-hcopy{}-prev{}-async{}-alloc{}'.format(
            'fp8' if self.use_fp8_dispatch else 'bf16', self.expert_alignment, self.num_bias, int(self.do_handle_copy),
            int(self.with_previous_event), int(self.async_with_compute_stream), int(self.allocate_on_comm_stream)))

    @property
    def suite(self) -> str:
        """``performance`` cases use no stream plumbing, so their timings compare across backends; the others are
        ``functional``."""
        plumbing = self.with_previous_event or self.async_with_compute_stream or self.allocate_on_comm_stream
        return 'functional' if plumbing else 'performance'


def enumerate_mode_cases() -> Tuple[ModeCase, ...]:
    cases = []
    for hcopy, align, fp8, bias, prev, async_ in product((True, False), (128, 1), (True, False), (0, 1, 2), (False, True), (False, True)):
        for alloc in ((True,) if prev else (False, True)):
            cases.append(ModeCase(hcopy, align, fp8, bias, prev, async_, alloc))
    return tuple(cases)


def select_cases(spec: str) -> Tuple[ModeCase, ...]:
    """``all`` | ``performance`` | ``functional`` | comma-separated case ids."""
    cases = enumerate_mode_cases()
    if spec == 'all':
        return cases
    if spec in ('performance', 'functional'):
        return tuple(c for c in cases if c.suite == spec)
    by_id = {c.case_id: c for c in cases}
    wanted = [s for s in spec.split(',') if s]
    unknown = [s for s in wanted if s not in by_id]
    if unknown:
        raise ValueError('unknown case id(s): ' + ', '.join(unknown))
    return tuple(by_id[s] for s in wanted)
