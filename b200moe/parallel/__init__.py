from .fsdp import FSDPWrapperPipelined, FlatShards  # noqa: F401
from .ddp import DDPWraper, ShardedOptimizer  # noqa: F401
from .pipeline import pipelined_train, pipelined_train_overlap  # noqa: F401
