"""Host-side helpers of bench.py that need no GPU."""
import importlib.util
import os
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def _bench():
  spec = importlib.util.spec_from_file_location("bench_module", os.path.join(HERE, "..", "bench.py"))
  mod = importlib.util.module_from_spec(spec)
  spec.loader.exec_module(mod)
  return mod


def test_watchdog_fires_only_without_a_finish():
  bench = _bench()
  fired = []
  late = bench.Watchdog(0.05, lambda: fired.append("late"))
  late.start()
  time.sleep(0.2)
  assert fired == ["late"]
  on_time = bench.Watchdog(0.2, lambda: fired.append("on_time"))
  on_time.start()
  on_time.finish()
  time.sleep(0.3)
  assert fired == ["late"]


def test_default_microbatches_cover_every_gpu_count():
  bench = _bench()
  for n in (1, 2, 4, 8):
    m = bench.default_microbatches("xxl", n) if "default_microbatches" in dir(bench) else 1
    assert m >= 1 and 128 % (n * m) == 0
