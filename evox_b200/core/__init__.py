"""Minimal host-side programming model of the generation step.

The names and call protocol follow the reference's core layer so that code written against it
reads the same here: `ModuleBase` / `Parameter` / `Mutable` (evox/core/module.py:22-94) and the
`Algorithm` / `Problem` / `Workflow` / `Monitor` roles (evox/core/components.py:17-170).
Only what the generation step needs is provided; tracing helpers (compile, vmap, use_state) are
not part of this package.
"""

from .components import Algorithm, Monitor, Problem, Workflow
from .module import ModuleBase, Mutable, Parameter

__all__ = ["ModuleBase", "Mutable", "Parameter", "Algorithm", "Problem", "Workflow", "Monitor"]
