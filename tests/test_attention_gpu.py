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


@pytest.mark.parametrize("case", CASES)
def test_flash_attention_matches_reference(case):
  from t5x_b200.ops import attention as A
  from t5x_b200.ops import native
  from t5x_b200.ops import reference as ref
  B, H, Lq, Lk, use_bias, bidir, causal, use_mask, use_seg = case
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
    assert rel(g, w) < 2e-2, (n, rel(g, w))
