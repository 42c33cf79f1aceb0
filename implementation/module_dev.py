from b200moe.models.module_dev import ModuleStack  # noqa: F401
