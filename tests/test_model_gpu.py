"""The bf16 CUDA path of the T5 model against the fp32 CPU path (same weights, same batch)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(device, dtype):
  from t5x_b200 import adafactor, models
  from t5x_b200.data import vocabularies
  from t5x_b200.models.t5 import network
  cfg = network.T5Config(vocab_size=2048, dtype=dtype, emb_dim=256, num_heads=4,
                         num_encoder_layers=2, num_decoder_layers=2, head_dim=64, mlp_dim=512,
                         mlp_activations=("gelu", "linear"), dropout_rate=0.0)
  torch.manual_seed(0)
  module = network.Transformer(cfg, device=device)
  vocab = vocabularies.PassThroughVocabulary(2048)
  opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0,
                            logical_factor_rules=adafactor.standard_logical_factor_rules())
  return models.EncoderDecoderModel(module, vocab, vocab, opt, z_loss=1e-4)


def _batch(device):
  g = torch.Generator().manual_seed(1)
  enc = torch.randint(3, 2000, (4, 128), generator=g)
  enc[:, 100:] = 0
  tgt = torch.randint(3, 2000, (4, 32), generator=g)
  tgt[:, 28:] = 0
  dec_in = torch.cat([torch.zeros(4, 1, dtype=torch.long), tgt[:, :-1]], 1)
  b = {"encoder_input_tokens": enc, "decoder_target_tokens": tgt, "decoder_input_tokens": dec_in,
       "decoder_loss_weights": (tgt > 0).float()}
  return {k: v.to(device) for k, v in b.items()}


def test_loss_and_grads_match_cpu_fp32():
  from t5x_b200 import trainer as trainer_lib
  from t5x_b200.models import base
  from t5x_b200.ops import native
  cpu_model = _build("cpu", "float32")
  gpu_model = _build("cuda", "bfloat16")
  gpu_model.module.load_state_dict(cpu_model.module.state_dict())
  pc = base.module_param_tree(cpu_model.module)
  pg = base.module_param_tree(gpu_model.module)
  trainer_lib.attach_compute_buffers(pg, bf16_copy=True, main_grad=True)
  lc, _ = cpu_model.loss_fn(pc, _batch("cpu"), None)
  lc.backward()
  before = native.launch_count()
  lg, _ = gpu_model.loss_fn(pg, _batch("cuda"), None)
  lg.backward()
  native.check_status()
  assert native.launch_count() > before
  assert abs(float(lg) - float(lc)) / abs(float(lc)) < 2e-2
  from t5x_b200.utils import tree
  fc, fg = tree.flatten_dict(pc), tree.flatten_dict(pg)
  grads = trainer_lib._collect_grads(fg)
  worst = 0.0
  for k in fc:
    a, b = grads[k].float().cpu(), fc[k].grad.float()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    worst = max(worst, 1 - cos)
    assert cos > 0.98, (k, cos)
