from b200moe.optim.adamw import AdamW  # noqa: F401
