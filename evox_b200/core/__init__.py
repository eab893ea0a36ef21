"""Minimal host-side programming model of the generation step.

The names and call protocol follow the reference's core layer so that code written against it
reads the same here: `ModuleBase` / `Parameter` / `Mutable` (evox/core/module.py:22-94) and the
`Algorithm` / `Problem` / `Workflow` / `Monitor` roles (evox/core/components.py:17-170).
`use_state` and `vmap` (evox/core/module.py:153-260) are provided for modules whose steps run in-place
kernels: see `functional.py`.
"""

from .components import Algorithm, Monitor, Problem, Workflow
from .functional import use_state, vmap
from .module import ModuleBase, Mutable, Parameter

__all__ = ["ModuleBase", "Mutable", "Parameter", "Algorithm", "Problem", "Workflow", "Monitor", "use_state", "vmap"]
