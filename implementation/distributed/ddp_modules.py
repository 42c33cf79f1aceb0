from b200moe.parallel.ddp import DDPWraper, ShardedOptimizer, sync_grad  # noqa: F401
from b200moe.parallel.fsdp import FSDPWrapperPipelined  # noqa: F401
from b200moe.parallel.hooks import (async_weight_wrapper_backward_next, async_weight_wrapper_next,  # noqa: F401
                                    free_weight, free_weight_backward, sync_weight_wrapper,
                                    sync_weight_wrapper_backward, wait_prefetched_weight,
                                    wait_prefetched_weight_backward)
