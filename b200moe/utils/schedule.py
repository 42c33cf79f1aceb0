"""Learning-rate schedule (reference implementation/nnfunctions.py:19-35)."""
import math

__all__ = ["learning_rate_schedule", "learning_rate_schedule_wrapper"]


def learning_rate_schedule(t, a_max, a_min, t_w, t_c):
    """Linear warm-up to ``a_max`` over ``t_w`` steps, cosine decay to ``a_min``
    on ``[t_w, t_c]``, then constant ``a_min``."""
    if t < t_w:
        return t / t_w * a_max
    if t <= t_c:
        phase = (t - t_w) / (t_c - t_w)
        return a_min + 0.5 * (1.0 + math.cos(phase * math.pi)) * (a_max - a_min)
    return a_min


def learning_rate_schedule_wrapper(a_max, a_min, t_w, t_c):
    def scheduler(t):
        return learning_rate_schedule(t, a_max, a_min, t_w, t_c)
    return scheduler
