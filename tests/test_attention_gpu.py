"""tcgen05 flash attention (forward and backward) against the fp32 PyTorch statement."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
  a, b = a.float(), b.float()
  return ((a - b).norm() / (b.norm() + 1e-12)).item()


CASES = [
    # B, H, Lq, Lk, bias, bidirectional, causal, key_mask, segments
    (2, 4, 512, 512, True, True, False, True, False),
    (2, 4, 114, 114, True, False, True, True, False),
    (2, 4, 114, 512, False, True, False, True, False),
    (3, 2, 128, 128, True, True, False, False, True),
    (1, 2, 200, 300, True, True, False, True, True),
    (2, 3, 64, 40, False, True, True, False, False),
]
# beyond the short-range forward kernel: the streaming forward with the same backward
LONG_CASES = [
    (1, 2, 640, 640, True, True, False, True, False),
    (1, 2, 1024, 1024, True, False, True, False, False),
    (1, 2, 300, 2048, False, True, False, True, False),
    (1, 2, 2048, 2048, True, True, False, True, True),
]
TOL = 8e-3


@pytest.mark.parametrize("kernel", ["stream", "classic"])
@pytest.mark.parametrize("case", CASES + LONG_CASES)
def test_flash_attention_matches_reference(case, kernel, monkeypatch):
  from t5x_b200.ops import attention as A
  from t5x_b200.ops import native
  from t5x_b200.ops import reference as ref
  B, H, Lq, Lk, use_bias, bidir, causal, use_mask, use_seg = case
  monkeypatch.setenv("T5X_B200_ATTN_FWD", kernel)
  if A.forward_kernel(Lq, Lk, 64) != kernel:
    pytest.skip("the short-range forward kernel does not cover this shape")
  torch.manual_seed(0)
  dev = "cuda"
  q = (torch.randn(B, Lq, H, 64, device=dev) * 0.5).bfloat16().requires_grad_(True)
  k = (torch.randn(B, Lk, H, 64, device=dev) * 0.5).bfloat16().requires_grad_(True)
  v = torch.randn(B, Lk, H, 64, device=dev).bfloat16().requires_grad_(True)
  table = (torch.randn(H, 32, device=dev) * 0.5).requires_grad_(True) if use_bias else None
  key_mask = None
  if use_mask:
    lens = torch.randint(Lk // 2, Lk + 1, (B,), device=dev)
    key_mask = torch.arange(Lk, device=dev)[None, :] < lens[:, None]
  qseg = kseg = None
  if use_seg:
    qseg = (torch.arange(Lq, device=dev)[None, :] * 3 // Lq + 1).expand(B, Lq).contiguous()
    kseg = (torch.arange(Lk, device=dev)[None, :] * 3 // Lk + 1).expand(B, Lk).contiguous()
  do = torch.randn(B, Lq, H, 64, device=dev).bfloat16()

  out = A.flash_attention(q, k, v, bias_table=table, bidirectional=bidir, key_mask=key_mask,
                          causal=causal, q_segment_ids=qseg, kv_segment_ids=kseg)
  out.backward(do)
  native.check_status()
  got = [out.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone(),
         table.grad.clone() if use_bias else None]
  q.grad = k.grad = v.grad = None
  if use_bias:
    table.grad = None
  bias = None
  if use_bias:
    bias = ref.relative_position_bias(table, Lq, Lk, bidir)
  exp = ref.attention(q.float(), k.float(), v.float(), bias=bias, key_mask=key_mask,
                      causal=causal, q_segment_ids=qseg, kv_segment_ids=kseg)
  exp.backward(do.float())
  want = [exp.detach(), q.grad, k.grad, v.grad, table.grad if use_bias else None]
  names = ["out", "dq", "dk", "dv", "dbias"]
  for n, g, w in zip(names, got, want):
    if w is None:
      continue
    assert rel(g, w) < TOL, (n, rel(g, w))


@pytest.mark.parametrize("kernel", ["stream", "classic"])
def test_rows_with_every_key_hidden_are_uniform(kernel, monkeypatch):
  """A query whose keys are all masked attends uniformly (the mask is an additive -1e10, not
  -inf), and gradients flow through such rows as they do through the additive form."""
  from t5x_b200.ops import attention as A
  from t5x_b200.ops import native
  from t5x_b200.ops import reference as ref
  monkeypatch.setenv("T5X_B200_ATTN_FWD", kernel)
  torch.manual_seed(1)
  B, H, Lq, Lk = 2, 2, 130, 260
  q = (torch.randn(B, Lq, H, 64, device="cuda") * 0.5).bfloat16().requires_grad_(True)
  k = (torch.randn(B, Lk, H, 64, device="cuda") * 0.5).bfloat16().requires_grad_(True)
  v = torch.randn(B, Lk, H, 64, device="cuda").bfloat16().requires_grad_(True)
  table = (torch.randn(H, 32, device="cuda") * 0.5).requires_grad_(True)
  # segments: queries of segment 3 find no key at all; batch row 1 has every key padded away
  qseg = torch.ones(B, Lq, dtype=torch.int32, device="cuda")
  qseg[:, 100:] = 3
  kseg = torch.ones(B, Lk, dtype=torch.int32, device="cuda")
  kseg[:, 200:] = 2
  key_mask = torch.ones(B, Lk, dtype=torch.bool, device="cuda")
  key_mask[1] = False
  do = torch.randn(B, Lq, H, 64, device="cuda").bfloat16()
  out = A.flash_attention(q, k, v, bias_table=table, key_mask=key_mask, q_segment_ids=qseg,
                          kv_segment_ids=kseg)
  out.backward(do)
  native.check_status()
  got = [out.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone()]
  q.grad = k.grad = v.grad = None
  exp = ref.attention(q.float(), k.float(), v.float(),
                      bias=ref.relative_position_bias(table, Lq, Lk, True), key_mask=key_mask,
                      q_segment_ids=qseg, kv_segment_ids=kseg)
  exp.backward(do.float())
  uniform = v.detach().float().mean(dim=1)  # [B, H, D]
  assert rel(out[1, 5].float(), uniform[1]) < TOL and rel(out[0, 120].float(), uniform[0]) < TOL
  for n, g, w in zip(["out", "dq", "dk", "dv"], got, [exp.detach(), q.grad, k.grad, v.grad]):
    assert rel(g, w) < TOL, (n, rel(g, w))


@pytest.mark.parametrize("shape", [(2, 3, 200, 200, True), (1, 2, 130, 1100, False),
                                   (2, 2, 384, 256, False)])
def test_head_dim_128_forward_and_backward(shape):
  """head_dim 128 (T5 1.0 3B / 11B): the streaming forward and the one-block-at-a-time
  backward against fp32, with bias, padding mask and (first case) causal masking."""
  from t5x_b200.ops import attention as A
  from t5x_b200.ops import native
  from t5x_b200.ops import reference as ref
  B, H, Lq, Lk, causal = shape
  torch.manual_seed(2)
  q = (torch.randn(B, Lq, H, 128, device="cuda") * 0.3).bfloat16().requires_grad_(True)
  k = (torch.randn(B, Lk, H, 128, device="cuda") * 0.3).bfloat16().requires_grad_(True)
  v = torch.randn(B, Lk, H, 128, device="cuda").bfloat16().requires_grad_(True)
  table = (torch.randn(H, 32, device="cuda") * 0.5).requires_grad_(True)
  lens = torch.randint(Lk // 2, Lk + 1, (B,), device="cuda")
  key_mask = torch.arange(Lk, device="cuda")[None, :] < lens[:, None]
  do = torch.randn(B, Lq, H, 128, device="cuda").bfloat16()
  assert A.flash_supported(q, k, v, None, None)
  out = A.flash_attention(q, k, v, bias_table=table, bidirectional=not causal,
                          key_mask=key_mask, causal=causal)
  out.backward(do)
  native.check_status()
  got = [out.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone(), table.grad.clone()]
  q.grad = k.grad = v.grad = table.grad = None
  exp = ref.attention(q.float(), k.float(), v.float(),
                      bias=ref.relative_position_bias(table, Lq, Lk, not causal),
                      key_mask=key_mask, causal=causal)
  exp.backward(do.float())
  for n, g, w in zip(["out", "dq", "dk", "dv", "dbias"], got,
                     [exp.detach(), q.grad, k.grad, v.grad, table.grad]):
    assert rel(g, w) < TOL, (n, rel(g, w))


@pytest.mark.parametrize("length", [96, 300, 1100])
def test_prefix_lm_visibility_from_per_token_codes(length):
  """Prefix-LM masks (causal, fully visible inside the prefix, packed segments, padding) built
  inside the kernels from per-token codes, against the dense mask of the fp32 statement."""
  from t5x_b200.ops import functional as F
  from t5x_b200.ops import attention as A
  from t5x_b200.ops import native
  from t5x_b200.ops import reference as ref
  torch.manual_seed(3)
  B, H, L = 2, 2, length
  q = (torch.randn(B, L, H, 64, device="cuda") * 0.5).bfloat16().requires_grad_(True)
  k = (torch.randn(B, L, H, 64, device="cuda") * 0.5).bfloat16().requires_grad_(True)
  v = torch.randn(B, L, H, 64, device="cuda").bfloat16().requires_grad_(True)
  table = (torch.randn(H, 32, device="cuda") * 0.5).requires_grad_(True)
  pos = torch.arange(L, device="cuda")
  # two packed segments; each starts with a prefix of a third of its length; the tail is padding
  seg = torch.where(pos < L // 2, 1, 2)[None].expand(B, L).contiguous()
  start = torch.where(pos < L // 2, 0, L // 2)
  in_prefix = ((pos - start) < L // 6)[None].expand(B, L).contiguous()
  valid = (pos < L - L // 10)[None].expand(B, L).contiguous()
  mask = ref.PrefixLMMask(in_prefix, valid, seg)
  assert A.flash_supported(q, k, v, None, mask)
  do = torch.randn(B, L, H, 64, device="cuda").bfloat16()
  out = F.attention(q, k, v, bias_table=table, bidirectional=False, extra_mask=mask)
  out.backward(do)
  native.check_status()
  got = [out.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone(), table.grad.clone()]
  q.grad = k.grad = v.grad = table.grad = None
  exp = ref.attention(q.float(), k.float(), v.float(),
                      bias=ref.relative_position_bias(table, L, L, False),
                      extra_mask=mask.bool())
  exp.backward(do.float())
  for n, g, w in zip(["out", "dq", "dk", "dv", "dbias"], got,
                     [exp.detach(), q.grad, k.grad, v.grad, table.grad]):
    assert rel(g, w) < TOL, (n, rel(g, w))
