"""Trainer for expert-parallel models (t5x/contrib/moe/trainer.py:39-149)."""
from __future__ import annotations

from typing import Optional

from t5x_b200 import trainer as trainer_lib
from t5x_b200.contrib.moe import training_utils
from t5x_b200.utils import tree as tree_utils


class MoeTrainer(trainer_lib.Trainer):
  """Standard trainer plus the expert-gradient convention.

  In the reference, pjit averages every gradient over the whole ('expert','data') batch axis,
  so the gradients of expert-sharded weights come out `num_expert_partitions` times too small
  and the trainer multiplies them back (`sharded_match_fn`, default `.*expert.*`). Here the
  sum over replicas is explicit: dense parameters are summed over all data x expert ranks,
  expert parameters only over the ranks that hold the same experts (the pure data axis), so
  expert gradients are already exact. `num_expert_partitions` and `sharded_match_fn` are
  accepted for API parity; `scale_expert_grads=True` applies the reference's factor for
  callers that feed mean-reduced gradients."""

  def __init__(self, model, train_state, partitioner, eval_names, summary_dir, train_state_axes,
               rng, learning_rate_fn, num_microbatches: Optional[int], num_expert_partitions: int,
               sharded_match_fn=training_utils.match_fn(r".*expert.*"),
               weight_metrics_computer=None, scale_expert_grads: bool = False):
    super().__init__(model=model, train_state=train_state, partitioner=partitioner,
                     eval_names=eval_names, summary_dir=summary_dir,
                     train_state_axes=train_state_axes, rng=rng,
                     learning_rate_fn=learning_rate_fn, num_microbatches=num_microbatches,
                     weight_metrics_computer=weight_metrics_computer)
    self._num_expert_partitions = num_expert_partitions
    self._sharded_match_fn = sharded_match_fn
    self._scale_expert_grads = scale_expert_grads

  def _train_step(self, train_state, batch, step_num):
    step = int(step_num)
    lr = float(self._learning_rate_fn(step))
    grads, metrics, _ = trainer_lib.accumulate_grads_microbatched(
        self._model, train_state, batch, self._get_step_rng(step), self._num_microbatches)
    if self._scale_expert_grads:
      flat = tree_utils.flatten_dict(grads)
      for name, g in flat.items():
        if self._sharded_match_fn(name):
          g.mul_(float(self._num_expert_partitions))
    return trainer_lib.apply_grads(train_state, grads, metrics, lr,
                                   self._weight_metrics_computer)
