"""The slice of ``grilly.nn`` the quantized path rides on: ``Module``,
``Parameter``, ``Linear``, ``Sequential`` and ``functional.linear``."""
from . import functional  # noqa: F401
from .modules import Linear, Module, Parameter, Sequential  # noqa: F401
