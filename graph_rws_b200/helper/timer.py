"""SpMM timing hook with the reference's names (helper/timer.py:7-19).

The reference's ``spmm_tc`` blocks the host on a CUDA event inside every call
(core/helper/timer.h:38-41) and returns the elapsed milliseconds; ``BCSRSPMMFunction`` feeds them
to ``record_spmm_time`` (layers/layer.py:51).  Here timing is opt-in (``core.set_spmm_timing``):
when it is off the recorded value is 0.0 and nothing synchronises.
"""
_SPMM_TIMINGS = []


def record_spmm_time(t):
    _SPMM_TIMINGS.append(t)


def reset_spmm_timings():
    del _SPMM_TIMINGS[:]


def spmm_timings():
    return list(_SPMM_TIMINGS)


def get_avg_spmm_time():
    if not _SPMM_TIMINGS:
        return 0.0
    return sum(_SPMM_TIMINGS) / len(_SPMM_TIMINGS)
