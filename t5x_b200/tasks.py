"""Importing this module registers the tasks that ship with the framework (role of
t5x/tasks.py, which imports seqio task definitions for their registration side effect)."""
from t5x_b200.data import tasks as _tasks

_tasks.register_synthetic_tasks()
TaskRegistry = _tasks.TaskRegistry
MixtureRegistry = _tasks.MixtureRegistry
