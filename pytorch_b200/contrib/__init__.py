from . import module  # noqa: F401
