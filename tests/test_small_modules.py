"""Small modules: the import-time garbage-collector switch and the task registration module
(t5x/disable_gc_during_import_test.py)."""
import gc
import importlib

from t5x_b200 import disable_gc_during_import as gc_switch


def test_gc_is_suspended_between_start_and_stop_only_when_asked(monkeypatch):
  assert gc.isenabled()
  monkeypatch.delenv("T5X_B200_DISABLE_GC_DURING_IMPORT", raising=False)
  monkeypatch.delenv("EXPERIMENTAL_DISABLE_GC_DURING_IMPORT", raising=False)
  gc_switch.start()
  assert gc.isenabled() and not gc_switch.enabled()
  gc_switch.stop()
  for name in ("T5X_B200_DISABLE_GC_DURING_IMPORT", "EXPERIMENTAL_DISABLE_GC_DURING_IMPORT"):
    monkeypatch.setenv(name, "true")
    assert gc_switch.enabled()
    gc_switch.start()
    try:
      assert not gc.isenabled()
      gc_switch.start()            # a second start changes nothing
      assert not gc.isenabled()
    finally:
      gc_switch.stop()
    assert gc.isenabled()
    gc_switch.stop()               # and neither does a second stop
    assert gc.isenabled()
    monkeypatch.delenv(name)
  # the collector was off before: stop() leaves it off
  monkeypatch.setenv("T5X_B200_DISABLE_GC_DURING_IMPORT", "1")
  gc.disable()
  try:
    gc_switch.start()
    gc_switch.stop()
    assert not gc.isenabled()
  finally:
    gc.enable()


def test_importing_tasks_registers_the_shipped_tasks():
  tasks = importlib.import_module("t5x_b200.tasks")
  assert "synthetic_span_corruption" in tasks.TaskRegistry
  assert hasattr(tasks, "MixtureRegistry")
