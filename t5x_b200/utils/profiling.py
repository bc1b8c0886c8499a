"""Step-range profiling hook: `--profile_steps a:b` on the launch scripts (or
`T5X_B200_PROFILE_STEPS=a:b`) records train steps a..b-1 with `torch.profiler` (CPU activity
plus CUDA kernels through CUPTI when a GPU is present) and writes, per rank,

  <model_dir>/profile/steps_<a>_<b>.rank<r>.trace.json   a Chrome / Perfetto trace
  <model_dir>/profile/steps_<a>_<b>.rank<r>.kernels.txt  kernels by total device time

The reference annotates steps for an external profiler (`jax.profiler.StepTraceAnnotation`,
t5x/trainer.py:562) and has no capture flag of its own; here the NVTX range per step plays that
role and this hook is the self-contained capture. Steps outside the range run unprofiled, so
the hook costs nothing when it is idle.
"""
from __future__ import annotations

import logging
import os
from typing import Optional, Tuple

import torch

_ENV = "T5X_B200_PROFILE_STEPS"


def parse_step_range(spec: Optional[str]) -> Optional[Tuple[int, int]]:
  """'a:b' -> (a, b) with b > a; 'a' -> (a, a + 1); None / '' -> None."""
  if not spec:
    return None
  first, sep, last = spec.partition(":")
  a = int(first)
  b = int(last) if sep and last else a + 1
  if a < 0 or b <= a:
    raise ValueError(f"--profile_steps wants 'first:last' with last > first >= 0, got {spec!r}")
  return a, b


class StepProfiler:
  """Drives one `torch.profiler` capture over a half-open range of train steps."""

  def __init__(self, steps: Optional[Tuple[int, int]], out_dir: Optional[str], rank: int = 0,
               top: int = 40):
    self.steps, self.out_dir, self.rank, self.top = steps, out_dir, rank, top
    self._prof = None
    self.written = []

  @classmethod
  def from_environment(cls, out_dir: Optional[str], rank: int = 0) -> "StepProfiler":
    return cls(parse_step_range(os.environ.get(_ENV)), out_dir, rank)

  @property
  def active(self) -> bool:
    return self._prof is not None

  def step_begin(self, step: int) -> None:
    if self.steps is None or self.out_dir is None or self._prof is not None:
      return
    if not self.steps[0] <= step < self.steps[1]:
      return
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
      acts.append(torch.profiler.ProfilerActivity.CUDA)
    self._prof = torch.profiler.profile(activities=acts, record_shapes=False)
    self._prof.__enter__()
    logging.info("profiling train steps %d..%d", self.steps[0], self.steps[1] - 1)

  def step_end(self, step: int) -> None:
    if self._prof is None:
      return
    if step + 1 >= self.steps[1]:
      self.finish()

  def finish(self) -> None:
    """Stops a running capture and writes its files (also called when training ends inside
    the range)."""
    prof, self._prof = self._prof, None
    if prof is None:
      return
    if torch.cuda.is_available():
      torch.cuda.synchronize()
    prof.__exit__(None, None, None)
    a, b = self.steps
    base = os.path.join(self.out_dir, "profile", f"steps_{a}_{b}.rank{self.rank}")
    os.makedirs(os.path.dirname(base), exist_ok=True)
    prof.export_chrome_trace(base + ".trace.json")
    key = "self_cuda_time_total" if torch.cuda.is_available() else "self_cpu_time_total"
    with open(base + ".kernels.txt", "w") as f:
      f.write(prof.key_averages().table(sort_by=key, row_limit=self.top))
    self.written = [base + ".trace.json", base + ".kernels.txt"]
    self.steps = None  # one capture per run
    logging.info("profile written: %s", ", ".join(self.written))
