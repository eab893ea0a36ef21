from .es import OpenES, VirtualLoRAES
from .mo import NSGA2, RVEA
from .cso import CSO
from .pso import PSO

__all__ = ["PSO", "CSO", "OpenES", "VirtualLoRAES", "NSGA2", "RVEA"]
