from .es import ARS, OpenES, PersistentES, VirtualLoRAES
from .mo import NSGA2, RVEA
from .clpso import CLPSO
from .cso import CSO
from .pso import PSO

__all__ = ["PSO", "CSO", "CLPSO", "OpenES", "ARS", "PersistentES", "VirtualLoRAES", "NSGA2", "RVEA"]
