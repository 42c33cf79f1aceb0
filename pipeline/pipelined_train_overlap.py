from b200moe.parallel.pipeline import (backward_with_router_loss, pipelined_train_overlap,  # noqa: F401
                                       router_loss_metrics)
