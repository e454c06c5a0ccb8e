"""PowerSGD gradient compression (ddp_comm_hooks/powerSGD_hook.py in the reference: ``PowerSGDState``,
``powerSGD_hook``): rank-``r`` approximation of each bucket viewed as a square matrix, one power iteration per step,
error feedback. The arithmetic is ``distributed.algorithms.powerSGD_hook``; the state object here gives it the
reference's constructor."""
from ... import algorithms as _a


class PowerSGDState(dict):
    """State of :func:`powerSGD_hook`. ``start_powerSGD_iter`` iterations are plain all-reduces first (the early
    gradients change too fast for a low-rank warm start to help)."""

    def __init__(self, process_group=None, matrix_approximation_rank: int = 1, start_powerSGD_iter: int = 0,
                 use_error_feedback: bool = True, warm_start: bool = True, random_seed: int = 0, **_ignored):
        super().__init__(process_group=process_group, rank=int(matrix_approximation_rank), seed=int(random_seed))
        self.process_group = process_group
        self.matrix_approximation_rank = int(matrix_approximation_rank)
        self.start_powerSGD_iter = int(start_powerSGD_iter)
        self.use_error_feedback, self.warm_start = use_error_feedback, warm_start
        self.iter = 0

    def maybe_increase_iter(self, bucket) -> None:
        if bucket.is_last():
            self.iter += 1


def powerSGD_hook(state, bucket):
    if isinstance(state, PowerSGDState):
        if state.iter < state.start_powerSGD_iter:
            state.maybe_increase_iter(bucket)
            return _a.allreduce_hook(state.process_group, bucket)
        state.maybe_increase_iter(bucket)
        if not state.use_error_feedback:
            state.pop("err", None)
        if not state.warm_start:
            state.pop("q", None)
    return _a.powerSGD_hook(state, bucket)
