from .es import OpenES, VirtualLoRAES
from .mo import NSGA2, RVEA
from .pso import PSO

__all__ = ["PSO", "OpenES", "VirtualLoRAES", "NSGA2", "RVEA"]
