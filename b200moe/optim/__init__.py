from .adamw import AdamW, adamw_update_  # noqa: F401
