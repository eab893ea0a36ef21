from .es import ARS, OpenES, VirtualLoRAES
from .mo import NSGA2, RVEA
from .cso import CSO
from .pso import PSO

__all__ = ["PSO", "CSO", "OpenES", "ARS", "VirtualLoRAES", "NSGA2", "RVEA"]
