"""Learning-rate schedules by factor string (t5x/utils.py:850-923)."""
from __future__ import annotations

import math
from typing import Callable


def create_learning_rate_scheduler(factors: str = "constant * linear_warmup * rsqrt_decay",
                                   base_learning_rate: float = 0.5, warmup_steps: int = 1000,
                                   decay_factor: float = 0.5, steps_per_decay: int = 20000,
                                   steps_per_cycle: int = 100000, step_offset: int = 0,
                                   min_learning_rate: float = 1e-8) -> Callable[[int], float]:
  """`factors` is a '*'-separated product of: constant, linear_warmup, linear_decay,
  rsqrt_decay, rsqrt_normalized_decay, decay_every, cosine_decay."""
  names = [n.strip() for n in factors.split("*")]
  for n in names:
    if n not in ("constant", "linear_warmup", "linear_decay", "rsqrt_decay",
                 "rsqrt_normalized_decay", "decay_every", "cosine_decay"):
      raise ValueError("Unknown factor %s." % n)

  def step_fn(step) -> float:
    step = max(0, int(step) - step_offset)
    ret = 1.0
    for name in names:
      if name == "constant":
        ret *= base_learning_rate
      elif name == "linear_warmup":
        ret *= min(1.0, step / warmup_steps)
      elif name == "linear_decay":
        ret *= base_learning_rate * min(step / warmup_steps,
                                        1.0 + decay_factor * (warmup_steps - step))
      elif name == "rsqrt_decay":
        ret /= math.sqrt(max(step, warmup_steps))
      elif name == "rsqrt_normalized_decay":
        ret *= math.sqrt(warmup_steps)
        ret /= math.sqrt(max(step, warmup_steps))
      elif name == "decay_every":
        ret *= decay_factor ** (step // steps_per_decay)
      elif name == "cosine_decay":
        progress = max(0.0, (step - warmup_steps) / float(steps_per_cycle))
        ret *= max(0.0, 0.5 * (1.0 + math.cos(math.pi * (progress % 1.0))))
    return float(max(ret, min_learning_rate))

  return step_fn
