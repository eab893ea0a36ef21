"""evox_b200: the population-batched generation step of EvoX as hand-written B200 (sm_100a) kernels.

Importing the package loads `libevox_b200.so` (built by `python -m evox_b200._build`); there is
no CPU implementation behind these classes.
"""

from . import _cabi  # noqa: F401  (fails loudly when the kernels are not built)
from . import algorithms, core, operators, ops, problems, workflows
from .core import ModuleBase, Mutable, Parameter

__all__ = ["algorithms", "core", "operators", "problems", "workflows", "ModuleBase", "Mutable", "Parameter"]
