from . import numerical
from .virtual_lora_problem import VirtualLoRAProblem

__all__ = ["numerical", "VirtualLoRAProblem"]
