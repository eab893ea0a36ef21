from .eval_monitor import EvalMonitor
from .std_workflow import StdWorkflow

__all__ = ["StdWorkflow", "EvalMonitor"]
