"""Micro-benchmarks of the native kernels against the library ops they replace.

  python -m t5x_b200.ops.bench_kernels gemm [--pair 0|1|2]
  python -m t5x_b200.ops.bench_kernels attention

Timing: CUDA events on the launching stream after 3 warm-up calls; between timed calls a
256 MB buffer is overwritten so that operands do not stay in L2.
"""
from __future__ import annotations

import argparse
import json

import torch

from t5x_b200.ops import native

_FLUSH = None


def _flush_l2():
  global _FLUSH
  if _FLUSH is None:
    _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
  _FLUSH.fill_(1)


def time_ms(fn, iters: int = 10, warmup: int = 3) -> float:
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  total = 0.0
  for _ in range(iters):
    _flush_l2()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    total += e0.elapsed_time(e1)
  return total / iters


# (M, N, K, a transposed, b transposed): the XXL train step's dense shapes for one 16-sequence
# microbatch (8192 encoder / 1824 decoder tokens), forward, dgrad and wgrad forms.
GEMM_SHAPES = [
    (8192, 4096, 4096, 0, 0), (8192, 10240, 4096, 0, 0), (8192, 4096, 10240, 0, 0),
    (8192, 4096, 4096, 0, 1), (4096, 10240, 8192, 1, 0), (4096, 4096, 8192, 1, 0),
    (1824, 4096, 4096, 0, 0), (1824, 10240, 4096, 0, 0), (4096, 4096, 1824, 1, 0),
    (1824, 32128, 4096, 0, 0), (4096, 4096, 4096, 0, 0), (16384, 8192, 8192, 0, 0),
]


def bench_gemm(pair_modes=(0, 1)):
  rows = []
  for (M, N, K, ta, tb) in GEMM_SHAPES:
    A = (torch.randn(K, M, device="cuda").bfloat16().t() if ta
         else torch.randn(M, K, device="cuda").bfloat16())
    B = (torch.randn(N, K, device="cuda").bfloat16().t() if tb
         else torch.randn(K, N, device="cuda").bfloat16())
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * M * N * K
    row = {"M": M, "N": N, "K": K, "ta": ta, "tb": tb}
    for mode in pair_modes:
      native.gemm_set_pair_mode(mode)
      ms = time_ms(lambda: native.gemm(A, B, out=out))
      row[f"ours_pair{mode}_tflops"] = round(flops / ms / 1e9, 1)
    native.gemm_set_pair_mode(1)
    native.check_status()
    ms = time_ms(lambda: torch.matmul(A, B, out=out))
    row["cublas_tflops"] = round(flops / ms / 1e9, 1)
    rows.append(row)
    print(json.dumps(row), flush=True)
  return rows


def bench_attention():
  """Forward (both kernels where the short-range one applies) and forward + backward times of
  the flash-attention kernels with the T5 relative bias, against torch SDPA without a bias."""
  import os
  from t5x_b200.ops import attention as attn
  rows = []
  shapes = [(16, 64, 512, 512, 64), (16, 64, 114, 512, 64), (16, 64, 114, 114, 64),
            (4, 64, 2048, 2048, 64), (8, 32, 1024, 1024, 128)]
  for (b, h, lq, lk, d) in shapes:
    q = torch.randn(b, lq, h, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, lk, h, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, lk, h, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    table = torch.randn(h, 32, device="cuda")
    fwd = lambda: attn.flash_attention(q, k, v, bias_table=table, bidirectional=True)
    flops = 4.0 * b * h * lq * lk * d
    row = {"b": b, "h": h, "lq": lq, "lk": lk, "d": d}
    for kernel in ("stream", "classic"):
      os.environ["T5X_B200_ATTN_FWD"] = kernel
      if attn.forward_kernel(lq, lk, d) != kernel:
        continue
      with torch.no_grad():
        ms = time_ms(fwd)
      row[f"fwd_{kernel}_ms"] = round(ms, 3)
      row[f"fwd_{kernel}_tflops"] = round(flops / ms / 1e9, 1)
    os.environ.pop("T5X_B200_ATTN_FWD", None)
    if d == 64:
      o = fwd()
      do = torch.randn_like(o)
      row["fwd_bwd_ms"] = round(time_ms(lambda: torch.autograd.grad(fwd(), (q, k, v), do)), 3)
    qs, ks, vs = (t.detach().transpose(1, 2) for t in (q, k, v))
    row["sdpa_fwd_ms_no_bias"] = round(time_ms(
        lambda: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, scale=1.0)), 3)
    rows.append(row)
    print(json.dumps(row), flush=True)
  native.check_status()
  return rows


def gemm_one(m: int, n: int, k: int, iters: int, pair: int):
  """A few launches of one GEMM shape (the small case for profiler captures)."""
  a = torch.randn(m, k, device="cuda").bfloat16()
  b = torch.randn(k, n, device="cuda").bfloat16()
  out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
  native.gemm_set_pair_mode(pair)
  ms = time_ms(lambda: native.gemm(a, b, out=out), iters=iters, warmup=2)
  native.check_status()
  print(json.dumps({"M": m, "N": n, "K": k, "pair": pair, "ms": round(ms, 4),
                    "tflops": round(2.0 * m * n * k / ms / 1e9, 1)}))


def attention_one(b: int, h: int, lq: int, lk: int, iters: int):
  """A few forward + backward launches of one attention shape."""
  from t5x_b200.ops import attention as attn
  q = torch.randn(b, lq, h, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  k = torch.randn(b, lk, h, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  v = torch.randn(b, lk, h, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  table = torch.randn(h, 32, device="cuda")
  do = torch.randn(b, lq, h, 64, device="cuda", dtype=torch.bfloat16)
  fn = lambda: torch.autograd.grad(
      attn.flash_attention(q, k, v, bias_table=table, bidirectional=True), (q, k, v), do)
  ms = time_ms(fn, iters=iters, warmup=2)
  native.check_status()
  print(json.dumps({"b": b, "h": h, "lq": lq, "lk": lk, "fwd_bwd_ms": round(ms, 4)}))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("what", choices=["gemm", "attention", "gemm-one", "attention-one"])
  ap.add_argument("--pair", type=int, nargs="*", default=[0, 1])
  ap.add_argument("--shape", type=int, nargs="*", default=[])
  ap.add_argument("--iters", type=int, default=3)
  args = ap.parse_args()
  if args.what == "gemm":
    bench_gemm(tuple(args.pair))
  elif args.what == "gemm-one":
    m, n, k = args.shape or [8192, 8192, 4096]
    gemm_one(m, n, k, args.iters, args.pair[0] if args.pair else 1)
  elif args.what == "attention-one":
    b, h, lq, lk = args.shape or [16, 64, 512, 512]
    attention_one(b, h, lq, lk, args.iters)
  else:
    bench_attention()


if __name__ == "__main__":
  main()
