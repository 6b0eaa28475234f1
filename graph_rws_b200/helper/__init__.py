from .timer import record_spmm_time, reset_spmm_timings, get_avg_spmm_time, spmm_timings  # noqa: F401
from .engine import (GraphedStep, graphed_full_step, graphed_sampled_step, layer0_inputs, train_epoch_node_sampling, train_step_full, train_step_full_sharded,  # noqa: F401,E402
                     train_step_sampled)  # noqa: F401,E402
