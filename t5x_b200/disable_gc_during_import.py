"""Suspends the cyclic garbage collector while large modules are imported
(role of t5x/disable_gc_during_import.py:36-64).

Importing torch and the model code allocates many long-lived objects; every generation-2
collection in the middle of that walks all of them. With `T5X_B200_DISABLE_GC_DURING_IMPORT=1`
(or `EXPERIMENTAL_DISABLE_GC_DURING_IMPORT=true`, the reference's switch) the collector is
off between `start()` and `stop()`, which the entry points bracket their imports with.
"""
import gc
import os

_was_enabled = None


def enabled() -> bool:
  v = os.environ.get("T5X_B200_DISABLE_GC_DURING_IMPORT",
                     os.environ.get("EXPERIMENTAL_DISABLE_GC_DURING_IMPORT", ""))
  return v.lower() in ("1", "true", "yes")


def start() -> None:
  global _was_enabled
  if enabled() and _was_enabled is None:
    _was_enabled = gc.isenabled()
    gc.disable()


def stop() -> None:
  global _was_enabled
  if _was_enabled is not None:
    if _was_enabled:
      gc.enable()
    gc.collect()
    _was_enabled = None


start()
