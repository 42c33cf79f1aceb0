from b200moe.ops.functional import clip_gradient, cross_entropy, log_softmax, softmax  # noqa: F401
