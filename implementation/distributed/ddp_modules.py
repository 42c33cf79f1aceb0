from b200moe.parallel.ddp import DDPWraper, ShardedOptimizer, sync_grad  # noqa: F401
from b200moe.parallel.fsdp import FSDPWrapperPipelined  # noqa: F401
