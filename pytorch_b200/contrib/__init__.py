from . import function  # noqa: F401
from . import module  # noqa: F401
