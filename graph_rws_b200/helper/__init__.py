from .timer import record_spmm_time, reset_spmm_timings, get_avg_spmm_time, spmm_timings  # noqa: F401
