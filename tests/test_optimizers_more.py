"""Every wrapped optimizer: it minimises a quadratic, its logical-axes tree mirrors its state
tree, and its serialised state restores to the same trajectory; AdamW's moments inherit the
parameters' axes; further ones against `torch.optim` (the cases of t5x/optimizers_test.py)."""
import pytest
import torch

from t5x_b200 import optimizers
from t5x_b200.utils import tree

ALL = {
    "sgd": lambda: optimizers.sgd(None),
    "sgd_momentum": lambda: optimizers.sgd(None, momentum=0.9),
    "sgd_nesterov": lambda: optimizers.sgd(None, momentum=0.9, nesterov=True),
    "adam": lambda: optimizers.adam(None),
    "adamw": lambda: optimizers.adamw(None, weight_decay=1e-3),
    "lion": lambda: optimizers.lion(None),
    "lamb": lambda: optimizers.lamb(None),
    "lars": lambda: optimizers.lars(None, trust_coefficient=0.05),
    "adagrad": lambda: optimizers.adagrad(None),
    "adabelief": lambda: optimizers.adabelief(None),
    "radam": lambda: optimizers.radam(None),
    "rmsprop": lambda: optimizers.rmsprop(None),
    "rmsprop_momentum": lambda: optimizers.rmsprop(None, momentum=0.9),
    "yogi": lambda: optimizers.yogi(None),
    "noisy_sgd": lambda: optimizers.noisy_sgd(None, eta=1e-4),
    "fromage": lambda: optimizers.fromage(0.02),
}
LR = {"lion": 0.01, "lars": 0.5, "fromage": 0.02, "lamb": 0.02, "adagrad": 0.3, "yogi": 0.05}


def _params():
  torch.manual_seed(0)
  return {"dense": {"kernel": torch.randn(6, 4), "bias": torch.randn(4)},
          "embedding": torch.randn(5, 6)}


AXES = {"dense": {"kernel": ("embed", "mlp"), "bias": ("mlp",)}, "embedding": ("vocab", "embed")}


def _grads(params):
  """Gradient of 0.5 * sum((p - 1)^2)."""
  return tree.tree_map(lambda p: p - 1.0, params)


def _loss(params):
  return float(sum(((p - 1.0) ** 2).sum() for p in tree.flatten_dict(params).values()))


@pytest.mark.parametrize("name", sorted(ALL))
def test_optimizer_minimises_a_quadratic(name):
  opt = ALL[name]().create(_params())
  start = _loss(opt.target)
  for _ in range(60):
    opt = opt.apply_gradient(_grads(opt.target), learning_rate=LR.get(name, 0.05))
  assert int(opt.state.step) == 60
  assert _loss(opt.target) < 0.5 * start, (name, start, _loss(opt.target))


@pytest.mark.parametrize("name", sorted(ALL))
def test_logical_axes_mirror_the_state(name):
  opt_def = ALL[name]()
  opt_def.set_param_axes(AXES)
  opt = opt_def.create(_params())
  axes = opt_def.derive_logical_axes(opt, AXES)
  assert axes.target == AXES
  state_leaves = tree.flatten_dict(opt.state.param_states)
  axes_leaves = tree.flatten_dict(axes.state.param_states,
                                  is_leaf=lambda x: not isinstance(x, dict))
  assert set(state_leaves) == set(axes_leaves)
  for k, v in state_leaves.items():
    a = axes_leaves[k]
    if a is not None:  # a per-parameter slot: same rank as its tensor
      assert len(a) == v.dim(), (k, a, tuple(v.shape))


def test_adamw_moments_inherit_the_parameter_axes():
  opt_def = optimizers.adamw(None, weight_decay=1e-3)
  opt_def.set_param_axes(AXES)
  opt = opt_def.create(_params())
  axes = tree.flatten_dict(opt_def.derive_logical_axes(opt, AXES).state.param_states,
                           is_leaf=lambda x: not isinstance(x, dict))
  moments = {k: v for k, v in axes.items() if v is not None}
  assert len(moments) == 6   # mu and nu of three parameters
  assert sorted(tuple(v) for k, v in moments.items() if k.endswith("dense/kernel")) == \
      [("embed", "mlp"), ("embed", "mlp")]
  assert all(v is None for k, v in axes.items() if k.endswith("count"))


@pytest.mark.parametrize("name", ["adamw", "sgd_momentum", "lion", "rmsprop", "adagrad"])
def test_serialised_state_resumes_the_same_trajectory(name):
  lr = LR.get(name, 0.05)
  opt = ALL[name]().create(_params())
  for _ in range(3):
    opt = opt.apply_gradient(_grads(opt.target), learning_rate=lr)
  sd = opt.state_dict()
  assert set(sd) == {"target", "state"} and int(sd["state"]["step"]) == 3
  # plain nested dicts of tensors: what the checkpoint writer takes
  assert all(isinstance(v, torch.Tensor) or isinstance(v, (int, float))
             for v in tree.flatten_dict(sd).values())
  fresh = ALL[name]().create(tree.tree_map(torch.zeros_like, _params()))
  resumed = fresh.restore_state(sd)
  a = opt.apply_gradient(_grads(opt.target), learning_rate=lr)
  b = resumed.apply_gradient(_grads(resumed.target), learning_rate=lr)
  for k, v in tree.flatten_dict(a.target).items():
    torch.testing.assert_close(tree.flatten_dict(b.target)[k], v)
  assert int(b.state.step) == 4


@pytest.mark.parametrize("mine,theirs", [
    (lambda: optimizers.rmsprop(None, decay=0.9, eps=1e-8),
     lambda ps: torch.optim.RMSprop(ps, lr=0.05, alpha=0.9, eps=1e-8)),
    (lambda: optimizers.adagrad(None, initial_accumulator_value=0.1, eps=1e-10),
     lambda ps: torch.optim.Adagrad(ps, lr=0.05, initial_accumulator_value=0.1, eps=1e-10)),
    (lambda: optimizers.sgd(None, momentum=0.9, nesterov=True),
     lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9, nesterov=True)),
])
def test_further_optimizers_against_torch_optim(mine, theirs):
  params = _params()
  leaves = [torch.nn.Parameter(p.clone()) for p in tree.flatten_dict(params).values()]
  ref = theirs(leaves)
  opt = mine().create(params)
  for _ in range(4):
    for p in leaves:
      p.grad = p.detach() - 1.0
    ref.step()
    opt = opt.apply_gradient(_grads(opt.target), learning_rate=0.05)
  for got, want in zip(tree.flatten_dict(opt.target).values(), leaves):
    torch.testing.assert_close(got, want.detach(), rtol=2e-4, atol=2e-5)


def test_global_norm_clip_and_decay_mask_in_a_chain():
  mask = {"dense": {"kernel": True, "bias": False}, "embedding": True}
  opt_def = optimizers.chain([optimizers.clip_by_global_norm(1.0),
                              optimizers.add_decayed_weights(0.1, mask=mask),
                              optimizers.scale(-1.0)])
  params = tree.tree_map(torch.ones_like, _params())
  grads = tree.tree_map(lambda p: torch.full_like(p, 10.0), params)
  out = opt_def.create(params).apply_gradient(grads)
  n = sum(p.numel() for p in tree.flatten_dict(params).values())
  clipped = 10.0 / (10.0 * n ** 0.5)   # every entry after scaling the global norm to 1
  assert float(out.target["dense"]["bias"][0]) == pytest.approx(1.0 - clipped, rel=1e-5)
  assert float(out.target["dense"]["kernel"][0, 0]) == pytest.approx(1.0 - clipped - 0.1, rel=1e-5)
