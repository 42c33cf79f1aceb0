from b200moe.ops.functional import (cross_entropy, dot_product_att, gradient_clippling, gradient_clipping,  # noqa: F401
                                    sample_output, silu, softmax)
from b200moe.utils.schedule import learning_rate_schedule, learning_rate_schedule_wrapper  # noqa: F401
