from .timer import record_spmm_time, reset_spmm_timings, get_avg_spmm_time, spmm_timings  # noqa: F401
from .engine import train_step_full, train_step_full_sharded, train_step_sampled  # noqa: F401,E402
