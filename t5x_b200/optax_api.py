"""The `optax` names that reference gin files bind (`import optax` resolves here).

In the reference, `optax.adamw(...)` is a gradient transformation that `optimizers.chain` or
`optimizers.wrap_optax_optimizer` turns into an optimizer definition; `t5x.optimizers.adamw`
is the already wrapped form. This module provides the first kind on top of the
transformations implemented in `t5x_b200.optimizers`.
"""
from t5x_b200 import optimizers as _o

GradientTransformation = _o.GradientTransformation

# gradient transformations
clip = _o.clip
clip_by_global_norm = _o.clip_by_global_norm
scale = _o.scale
scale_by_learning_rate = _o.scale_by_learning_rate
trace = _o.trace
scale_by_adam = _o.scale_by_adam
scale_by_belief = _o.scale_by_belief
scale_by_yogi = _o.scale_by_yogi
scale_by_radam = _o.scale_by_radam
scale_by_rms = _o.scale_by_rms
scale_by_rss = _o.scale_by_rss
scale_by_lion = _o.scale_by_lion
scale_by_trust_ratio = _o.scale_by_trust_ratio
add_decayed_weights = _o.add_decayed_weights
add_noise = _o.add_noise


def chain(*transforms):
  return _o.chain_transforms(*transforms)


# optimizers as (unwrapped) gradient transformations
sgd = _o._sgd
adam = _o._adam
adamw = _o._adamw
lion = _o._lion
lamb = _o._lamb
lars = _o._lars
adagrad = _o._adagrad
adabelief = _o._adabelief
radam = _o._radam
rmsprop = _o._rmsprop
yogi = _o._yogi
noisy_sgd = _o._noisy_sgd
fromage = _o._fromage

# schedules
warmup_cosine_decay_schedule = _o.warmup_cosine_decay_schedule
