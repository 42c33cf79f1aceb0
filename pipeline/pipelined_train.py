from b200moe.parallel.pipeline import pipelined_train  # noqa: F401
