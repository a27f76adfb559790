"""Event system: monotonic u64 phase counters, task-graph metadata, validator."""

from .table import SCOPE_LOCAL, SCOPE_SYS, EventSpec, EventTable, NotifyEdge, TaskSpec, WaitEdge
from .validator import validate

__all__ = ["SCOPE_LOCAL", "SCOPE_SYS", "EventSpec", "EventTable", "WaitEdge", "NotifyEdge", "TaskSpec", "validate"]
