from .pso import PSO

__all__ = ["PSO"]
