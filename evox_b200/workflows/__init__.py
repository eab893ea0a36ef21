from .std_workflow import StdWorkflow

__all__ = ["StdWorkflow"]
