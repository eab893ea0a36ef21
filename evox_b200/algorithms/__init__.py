from .es import OpenES, VirtualLoRAES
from .pso import PSO

__all__ = ["PSO", "OpenES", "VirtualLoRAES"]
