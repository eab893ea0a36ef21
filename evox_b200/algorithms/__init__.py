from .es import ARS, DES, SNES, OpenES, PersistentES, VirtualLoRAES
from .hype import HypE
from .mo import NSGA2, NSGA3, RVEA, RVEAa
from .clpso import CLPSO
from .cso import CSO
from .de import DE
from .pso import PSO
from .slpso import SLPSOGS, SLPSOUS

__all__ = ["PSO", "CSO", "DE", "CLPSO", "SLPSOGS", "SLPSOUS", "OpenES", "ARS", "PersistentES", "SNES", "DES", "VirtualLoRAES", "NSGA2", "NSGA3", "RVEA", "RVEAa", "HypE"]
