"""Adafactor factor rules for MoE parameter axes (t5x/contrib/moe/adafactor_utils.py)."""
from t5x_b200 import adafactor

FactorDim = adafactor.FactorDim


def logical_factor_rules():
  """The standard rules plus the MoE axes: experts are a batch of independent matrices, the
  expert hidden dimension factors like `mlp`, router outputs are not factored."""
  rules = dict(adafactor.standard_logical_factor_rules())
  rules.update({
      "expert": FactorDim.BATCH,
      "expert_hidden": FactorDim.COLUMN,
      "expert_mlp": FactorDim.COLUMN,
      "unmodeled": FactorDim.NONE,
  })
  return rules
