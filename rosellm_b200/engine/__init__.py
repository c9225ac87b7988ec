from .context import HostBatch, StepContext, Workspace, build_host_batch
from .runner import ModelRunner, OutOfPages, StepEntry

__all__ = ["HostBatch", "ModelRunner", "OutOfPages", "StepContext", "StepEntry", "Workspace", "build_host_batch"]
