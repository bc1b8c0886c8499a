"""In-kernel dropout (csrc/dropout.cu) and the fused mixture-of-experts router (csrc/router.cu)
against plain PyTorch fp32 statements of the same ops."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _host_mask(seed, site, n_keys, rate):
  from t5x_b200.ops import native
  return torch.tensor([native.dropout_keep_host(seed, site, i, rate) for i in range(n_keys)])


@pytest.mark.parametrize("cols", [64, 40, 7])
def test_dropout_mask_is_shared_along_the_sequence_and_matches_the_host_generator(cols):
  from t5x_b200.ops import native
  torch.manual_seed(0)
  batch, length, rate, seed, site = 3, 5, 0.25, 99, 4
  x = torch.randn(batch * length, cols, device="cuda").bfloat16()
  y = native.dropout_rows(x, rate, seed, site, group_rows=length, col_group=1)
  keep = _host_mask(seed, site, batch * cols, rate).view(batch, 1, cols).cuda()
  want = torch.where(keep, x.view(batch, length, cols).float() / (1 - rate),
                     torch.zeros((), device="cuda")).bfloat16()
  assert torch.equal(y.view(batch, length, cols), want)
  # a block of rows with its global offset draws the same mask as the whole tensor
  lo = 4
  part = native.dropout_rows(x[lo:lo + 7].contiguous(), rate, seed, site, group_rows=length,
                             col_group=1, row_offset=lo)
  assert torch.equal(part, y[lo:lo + 7])


def test_dropout_autograd_and_statistics():
  from t5x_b200.ops import functional as F, reference as ref
  ref.set_dropout_seed(17)
  x = torch.ones(8, 128, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  y = F.dropout(x, 0.1, True, broadcast_dims=(-2,))
  assert bool((y[:, 0:1] == y).all())                      # shared along the length axis
  kept = (y[:, 0] != 0).float().mean()
  assert abs(float(kept) - 0.9) < 0.02
  y.sum().backward()
  assert torch.equal(x.grad, y.detach())                   # gradient of sum = the mask / keep
  z = F.dropout(x, 0.1, True, broadcast_dims=(-2,))        # next site: another mask
  assert not torch.equal(z, y)
  ref.set_dropout_seed(17)
  again = F.dropout(x, 0.1, True, broadcast_dims=(-2,))    # same seed, same site: same mask
  assert torch.equal(again, y)
  ref.set_dropout_seed(None)


def test_attention_value_dropout_equals_dropping_attention_weights():
  """Scaling the rows of v by the per-(batch, key, head) keep mask equals applying that mask
  to the attention weights, broadcast over queries."""
  from t5x_b200.ops import functional as F, reference as ref
  torch.manual_seed(2)
  b, lq, lk, h, d = 2, 16, 24, 3, 64
  q = torch.randn(b, lq, h, d, device="cuda").bfloat16()
  k = torch.randn(b, lk, h, d, device="cuda").bfloat16()
  v = torch.randn(b, lk, h, d, device="cuda").bfloat16()
  ref.set_dropout_seed(5)
  vd = F.attention_value_dropout(v, 0.5, True)
  ref.set_dropout_seed(None)
  mask = (vd.float().abs().sum(-1) != 0)                    # [b, lk, h]
  w = torch.softmax(torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()), -1)
  w = w * mask.permute(0, 2, 1)[:, :, None, :].float() / 0.5
  want = torch.einsum("bhqk,bkhd->bqhd", w, v.float())
  got = ref.attention(q, k, vd)
  assert (got.float() - want).abs().max() / want.abs().max() < 2e-2
  assert 0.3 < float(mask.float().mean()) < 0.7


def _router_reference(x, w, k, capacity):
  """fp32 statement of the tokens-choose router with autograd."""
  logits = x.float() @ w
  probs = torch.softmax(logits, -1)
  gate, index = torch.topk(probs, k, dim=-1)
  t, e = probs.shape
  flat = index.t().reshape(-1)
  hits = (flat[None, :] == torch.arange(e, device=x.device)[:, None]).to(torch.int32)
  position = torch.cumsum(hits, 1).gather(0, flat[None, :]).squeeze(0).long() - 1
  position = position.view(k, t).t()
  kept = position < capacity
  flat_slot = torch.where(kept, index * capacity + position, torch.full_like(position, -1))
  z = torch.logsumexp(logits, -1).pow(2).mean()
  mask = torch.zeros_like(probs).scatter_(1, index, 1.0)
  aux = (mask.mean(0) * probs.mean(0)).mean() * float(e * e)
  dispatched = kept.any(1).float().sum()
  metrics = torch.stack([aux, z, 1.0 - dispatched / t, kept.float().sum() / (e * capacity),
                         (gate * kept.float()).sum() / dispatched.clamp(min=1.0)])
  return gate * kept.float(), aux, z, index, flat_slot, metrics


@pytest.mark.parametrize("tokens,d,experts,k,cf", [(1000, 256, 8, 1, 1.25), (777, 768, 8, 2, 1.0),
                                                   (4096, 512, 64, 2, 2.0), (300, 128, 40, 4, 0.5)])
def test_fused_router_matches_reference(tokens, d, experts, k, cf):
  from t5x_b200.contrib.moe import layers
  torch.manual_seed(tokens + experts)
  x = (torch.randn(tokens, d, device="cuda") * 0.7).bfloat16().requires_grad_(True)
  w = (torch.randn(d, experts, device="cuda") * 0.05).requires_grad_(True)
  cap = layers.expert_capacity(tokens, experts, cf, k)
  gate, aux, z, index, flat_slot, m = layers._FusedRouterFn.apply(x, w, k, cap)
  xr = x.detach().clone().requires_grad_(True)
  wr = w.detach().clone().requires_grad_(True)
  gate_r, aux_r, z_r, index_r, slot_r, m_r = _router_reference(xr, wr, k, cap)
  assert torch.equal(index.long(), index_r)
  assert torch.equal(flat_slot.long(), slot_r)
  torch.testing.assert_close(gate, gate_r, rtol=1e-4, atol=1e-6)
  torch.testing.assert_close(m[:5], m_r, rtol=1e-4, atol=1e-6)
  coef = torch.randn(tokens, k, device="cuda")
  (0.3 * aux + 0.7 * z + (gate * coef).sum()).backward()
  (0.3 * aux_r + 0.7 * z_r + (gate_r * coef).sum()).backward()
  torch.testing.assert_close(w.grad, wr.grad, rtol=2e-3, atol=2e-5)
  err = (x.grad.float() - xr.grad.float()).norm() / xr.grad.float().norm()
  assert float(err) < 8e-3
  from t5x_b200.ops import native
  native.check_status()
