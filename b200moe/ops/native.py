"""Loader and Python bindings of the in-tree sm_100a extension (placeholder
until the first kernels land: reports that nothing is available)."""


def has(op: str) -> bool:
    return False
