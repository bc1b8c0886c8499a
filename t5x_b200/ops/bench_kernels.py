"""Micro-benchmarks of the native kernels against the library ops they replace.

  python -m t5x_b200.ops.bench_kernels gemm [--pair 0|1|2]
  python -m t5x_b200.ops.bench_kernels attention

Timing: CUDA events on the launching stream after 3 warm-up calls; between timed calls a
256 MB buffer is overwritten so that operands do not stay in L2.
"""
from __future__ import annotations

import argparse
import json
import os

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


def _measured_hbm_gbs() -> float:
  path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                      "MEASURED_PEAKS.json")
  try:
    return float(json.load(open(path))["hbm_gbs"])
  except (OSError, KeyError, ValueError):
    return 6650.0  # the fallback figure of this pool


def bench_streaming():
  """The kernels whose bound is memory traffic, each against the bytes its algorithm has to
  move (inputs read once, outputs written once) and the measured copy bandwidth: one JSON line
  per kernel with time, achieved GB/s and the fraction of the copy figure. A kernel that fails
  prints its error and the run goes on."""
  from t5x_b200 import decoding_fast
  peak = _measured_hbm_gbs()
  dev = "cuda"
  bf = dict(device=dev, dtype=torch.bfloat16)

  def report(name, fn, nbytes, **extra):
    try:
      ms = time_ms(fn)
      native.check_status()
      gbs = nbytes / ms / 1e6
      print(json.dumps({"kernel": name, "ms": round(ms, 4), "mbytes": round(nbytes / 1e6, 1),
                        "gb_s": round(gbs, 1), "of_measured_copy": round(gbs / peak, 3),
                        **extra}), flush=True)
    except Exception as e:  # pylint: disable=broad-except
      print(json.dumps({"kernel": name, "error": f"{type(e).__name__}: {e}"}), flush=True)

  # RMSNorm over XXL activations of one microbatch (16384 x 4096)
  T, d = 16384, 4096
  x = torch.randn(T, d, **bf)
  scale = torch.ones(d, device=dev)
  report("rmsnorm_fwd", lambda: native.rmsnorm_fwd(x, scale, 1e-6), 2 * T * d * 2, rows=T, d=d)
  _, rstd = native.rmsnorm_fwd(x, scale, 1e-6)
  dy = torch.randn(T, d, **bf)
  dscale = torch.zeros(d, device=dev)
  report("rmsnorm_bwd", lambda: native.rmsnorm_bwd(dy, x, scale, rstd, None, dscale),
         3 * T * d * 2, rows=T, d=d)
  dres = torch.randn(T, d, **bf)
  report("rmsnorm_bwd_with_residual_grad",
         lambda: native.rmsnorm_bwd(dy, x, scale, rstd, dres, dscale), 4 * T * d * 2)
  # gated GELU backward on the saved [T, 2 * d_ff] pre-activations
  ff = 10240
  h = torch.randn(T, 2 * ff, **bf)
  dg = torch.randn(T, ff, **bf)
  report("gated_gelu_bwd", lambda: native.gated_gelu_bwd_(dg, h), (T * ff + 2 * 2 * T * ff) * 2)
  # dropout with a mask shared along the length axis
  from t5x_b200.ops import functional as F
  xb = torch.randn(32, 512, d, **bf)
  report("dropout_broadcast_over_length",
         lambda: F.dropout(xb, 0.1, True, broadcast_dims=(-2,)), 2 * xb.numel() * 2)
  # embedding gather
  table = torch.randn(32128, d, **bf)
  ids = torch.randint(0, 32128, (T,), device=dev)
  report("embedding_fwd", lambda: native.embedding_fwd(ids, table), 2 * T * d * 2)
  # optimizers on one XXL MLP kernel (4096 x 10240 fp32)
  from t5x_b200 import adafactor
  n = d * ff
  p = torch.randn(d, ff, device=dev)
  p.bf16 = p.to(torch.bfloat16)
  g = torch.randn(d, ff, device=dev) * 1e-2
  opt = adafactor.Adafactor(decay_rate=0.8, step_offset=0)
  state = opt.init_param_state(p, "mlp/wi_0/kernel") if hasattr(opt, "init_param_state") else None
  if state is not None:
    hp = opt.hyper_params.replace(learning_rate=0.01) if hasattr(opt.hyper_params, "replace") \
        else opt.hyper_params
    step = torch.tensor(3)
    # p read and written in fp32, g read twice (statistics, then the update), bf16 copy written
    report("adafactor_factored_update",
           lambda: opt.apply_param_gradient(3, hp, p, state, g, "mlp/wi_0/kernel"),
           n * (4 + 4 + 2 * 4 + 2))
  from t5x_b200.ops import comm
  mu, nu = torch.zeros_like(p), torch.zeros_like(p)
  outs = comm._ptr_array([p.bf16.data_ptr()])
  report("adamw_step", lambda: native.adamw_step_(p, g, mu, nu, outs, lr=1e-3, b1=0.9, b2=0.999,
                                                   eps=1e-8, eps_root=0.0, weight_decay=0.01,
                                                   step=3),
         n * (2 * 4 + 4 + 4 * 4 + 2))
  # decode-step attention at the XL decode shapes (batch 64, beam 4, 32 heads)
  b, k, H, D, L, Le = 64, 4, 32, 64, 129, 512
  rows = b * k
  qkv = torch.randn(rows, 3, H, D, **bf)
  ck = torch.randn(b, k, H, L, D, **bf)
  cv = torch.randn(b, k, H, L, D, **bf)
  anc = torch.arange(k, device=dev, dtype=torch.int32)[None, :, None].expand(b, k, L).contiguous()
  bias = torch.randn(H, L, device=dev)
  out = torch.empty(rows, H, D, **bf)
  cur = torch.tensor([L - 2], device=dev, dtype=torch.int32)
  report("decode_self_attention_full_cache",
         lambda: decoding_fast.decode_self_attention(qkv[:, 0], qkv[:, 1], qkv[:, 2], ck, cv, anc,
                                                     bias, cur, out, k),
         2 * rows * H * (L - 1) * D * 2, rows=rows, heads=H, cached_positions=L - 2)
  lc = -(-L // 32) * 32
  ck2 = torch.randn(b, k, H, lc, D, **bf)
  cvt = torch.randn(b, k, H, D, lc, **bf)
  report("decode_self_attention_mma_full_cache",
         lambda: decoding_fast.decode_self_attention_mma(qkv[:, 0], qkv[:, 1], qkv[:, 2], ck2, cvt,
                                                         anc, bias, cur, out, k, L),
         2 * rows * H * (L - 1) * D * 2, rows=rows, heads=H, cached_positions=L - 2)
  ek = torch.randn(b, H, Le, D, **bf)
  ev = torch.randn(b, H, Le, D, **bf)
  mask = torch.ones(b, Le, device=dev, dtype=torch.uint8)
  report("decode_cross_attention",
         lambda: decoding_fast.decode_cross_attention(qkv[:, 0], ek, ev, mask, out, k),
         2 * b * H * Le * D * 2, rows=rows, heads=H, keys=Le)
  kq = torch.randn(b, Le, H, D, **bf)
  kp, vt = decoding_fast.cross_kv_layout(kq, kq)
  report("decode_cross_attention_mma",
         lambda: decoding_fast.decode_cross_attention_mma(qkv[:, 0], kp, vt, mask, out, k, Le),
         2 * b * H * Le * D * 2, rows=rows, heads=H, keys=Le)
  # beam step over [rows, vocab] fp32 logits
  V = 32128
  logits = torch.randn(rows, V, device=dev)
  scratch = native.BeamStepScratch(b, k, V, dev)
  Ld = 130
  st = dict(live_lp=torch.zeros(b, k, device=dev),
            live_seqs=torch.zeros(b, k, Ld, dtype=torch.int64, device=dev),
            fin_seqs=torch.zeros(b, k, Ld, dtype=torch.int64, device=dev),
            fin_scores=torch.full((b, k), -1e7, device=dev),
            fin_flags=torch.zeros(b, k, dtype=torch.bool, device=dev),
            ancestry=anc[:, :, :Ld].contiguous() if L >= Ld else
            torch.zeros(b, k, Ld, dtype=torch.int32, device=dev),
            cur=torch.zeros(1, dtype=torch.int32, device=dev),
            terminated=torch.zeros(1, dtype=torch.bool, device=dev))

  def one_beam_step():
    st["cur"].zero_()
    native.beam_step(logits, batch=b, beams=k, eos_id=1, alpha=0.6, min_brevity=1.0,
                     scratch=scratch, **st)
  report("beam_step", one_beam_step, rows * V * 4, rows=rows, vocab=V)
  tok_logits = torch.randn(rows, V, device=dev)
  report("sample_tokens_topk40",
         lambda: native.sample_tokens(tok_logits, temperature=1.0, topk=40, topp=0.0,
                                      rescale_log_probs=True, seed=1, stream_id=0),
         rows * V * 4, rows=rows, vocab=V)


def _graph_us(fns, reps: int = 5) -> float:
  """Microseconds per call of `fns` replayed as one CUDA graph (median of `reps` replays): the
  way the decode step issues them, free of the host's launch cost."""
  for f in fns:
    f()
  torch.cuda.synchronize()
  g = torch.cuda.CUDAGraph()
  with torch.cuda.graph(g):
    for f in fns:
      f()
  g.replay()
  torch.cuda.synchronize()
  times = []
  for _ in range(reps):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    times.append(e0.elapsed_time(e1))
  return sorted(times)[len(times) // 2] * 1e3 / len(fns)


def bench_skinny():
  """The decode-step GEMMs of T5.1.1-XL (256 rows = batch 64 x beam 4): this library's GEMM
  plain and with K cut into slices (with the finishing kernel that adds the residual and applies
  the next norm), against cuBLAS (torch.matmul), and against the time the weights alone need at
  the measured copy bandwidth. Each figure is the time per GEMM inside a CUDA graph of 20
  GEMMs over 20 different weight matrices (more bytes than L2 holds, so the weights are cold)."""
  peak = _measured_hbm_gbs()
  rows, nw = 256, 20
  for name, K, N in [("qkv", 2048, 6144), ("attn_out", 2048, 2048), ("wo", 5120, 2048)]:
    a = torch.randn(rows, K, device="cuda").bfloat16()
    wts = [(torch.randn(K, N, device="cuda") * 0.02).bfloat16() for _ in range(nw)]
    res = torch.randn(rows, N, device="cuda").bfloat16()
    scale = torch.ones(N, device="cuda")
    out = torch.empty(rows, N, device="cuda", dtype=torch.bfloat16)
    ws = torch.zeros(rows * N, dtype=torch.float32, device="cuda")
    row = {"gemm": name, "M": rows, "K": K, "N": N,
           "weight_stream_us": round(K * N * 2 / peak / 1e3, 2)}
    row["plain_us"] = round(_graph_us([(lambda w=w: native.gemm(a, w, out=out)) for w in wts]), 2)
    for s_ in (2, 4, 8):
      if K % s_ or (K // s_) % 64:
        continue
      row[f"splitk{s_}_norm_us"] = round(_graph_us(
          [(lambda w=w: native.gemm_splitk_norm(a, w, s_, residual=res, scale=scale, eps=1e-6,
                                                workspace=ws)) for w in wts]), 2)
    if native.gemm_skinny_splits(rows, N, K) > 0:
      # K split over a cluster, partial products added through distributed shared memory
      row["cluster_splits"] = native.gemm_skinny_splits(rows, N, K)
      row["cluster_us"] = round(_graph_us(
          [(lambda w=w: native.gemm_skinny(a, w, residual=res, out=out)) for w in wts]), 2)
      hn = torch.empty_like(out)
      row["cluster_norm_us"] = round(_graph_us(
          [(lambda w=w: native.rmsnorm_fwd(native.gemm_skinny(a, w, residual=res, out=out), scale,
                                           1e-6, out=hn)) for w in wts]), 2)
    row["cublas_us"] = round(_graph_us([(lambda w=w: torch.matmul(a, w, out=out)) for w in wts]), 2)
    print(json.dumps(row), flush=True)
  K, N = 2048, 5120
  a = torch.randn(rows, K, device="cuda").bfloat16()
  w0 = [(torch.randn(K, N, device="cuda") * 0.02).bfloat16() for _ in range(nw)]
  w1 = [(torch.randn(K, N, device="cuda") * 0.02).bfloat16() for _ in range(nw)]
  print(json.dumps({
      "gemm": "wi_0 | wi_1 with gated GELU", "M": rows, "K": K, "N": N,
      "weight_stream_us": round(2 * K * N * 2 / peak / 1e3, 2),
      "fused_us": round(_graph_us([(lambda i=i: native.gemm(a, w0[i], b2=w1[i]))
                                   for i in range(nw)]), 2),
      "cublas_two_gemms_us": round(_graph_us(
          [(lambda i=i: (torch.matmul(a, w0[i]), torch.matmul(a, w1[i]))) for i in range(nw)]), 2)}))
  native.check_status()


def gemm_trace(m: int, n: int, k: int, splits: int):
  """Where the time of one small GEMM goes: per-CTA timestamps of the phases of its first tile
  (`t5x_gemm_set_trace`), in microseconds after the first CTA's entry; median and maximum over
  the CTAs. The weights are cold (fresh matrix after an L2 flush), the activations warm."""
  import ctypes
  a = torch.randn(m, k, device="cuda").bfloat16()
  ws = torch.zeros(m, n, dtype=torch.float32, device="cuda")
  sms = torch.cuda.get_device_properties(0).multi_processor_count
  trace = torch.zeros(sms * 8, dtype=torch.int64, device="cuda")
  l = native.lib()
  l.t5x_gemm_set_trace.argtypes = [ctypes.c_void_p]
  names = ["entry", "setup_done", "first_loads_issued", "first_operands_landed", "last_mma_issued",
           "accumulator_complete", "epilogue_done", "exit"]
  if splits == 0:  # the cluster split-K kernel records its own phases
    names = ["entry", "setup_done", "first_loads_issued", "first_operands_landed",
             "accumulator_complete", "tile_parked", "peer_rows_received", "rows_stored"]
  native.gemm_set_pair_mode(0)
  rows = []
  for it in range(4):
    w = (torch.randn(k, n, device="cuda") * 0.02).bfloat16()
    _flush_l2()
    native.gemm(a, a.t()[:, :64].contiguous())  # keeps the activations in L2 after the flush
    torch.cuda.synchronize()
    trace.zero_()
    l.t5x_gemm_set_trace(trace.data_ptr())
    try:
      if splits == 0:
        native.gemm_skinny(a, w)
      elif splits > 1:
        native.gemm_splitk(a, w, splits, workspace=ws, workspace_is_clear=True)
      else:
        native.gemm(a, w)
    finally:
      l.t5x_gemm_set_trace(None)
    torch.cuda.synchronize()
    t = trace.view(sms, 8).cpu()
    t = t[t[:, 0] > 0]
    if it == 0 or not len(t):
      continue  # first launch: descriptor encoding and attribute set-up
    rel = (t - t[:, 0].min()).double() / 1e3
    rows.append({"ctas": int(len(t)),
                 **{nm: [round(float(rel[:, i].median()), 2), round(float(rel[:, i].max()), 2)]
                    for i, nm in enumerate(names)}})
  native.check_status()
  for r in rows:
    print(json.dumps({"M": m, "N": n, "K": k, "splits": splits, "us_median_max": r}))


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
  ap.add_argument("what", choices=["gemm", "attention", "gemm-one", "attention-one", "streaming", "skinny",
                                   "gemm-trace"])
  ap.add_argument("--splits", type=int, default=4,
                  help="gemm-trace: K slices of the atomic split-K path; 1: plain; 0: the cluster kernel")
  ap.add_argument("--pair", type=int, nargs="*", default=[0, 1])
  ap.add_argument("--shape", type=int, nargs="*", default=[])
  ap.add_argument("--iters", type=int, default=3)
  args = ap.parse_args()
  if args.what == "gemm":
    bench_gemm(tuple(args.pair))
  elif args.what == "gemm-one":
    m, n, k = args.shape or [8192, 8192, 4096]
    gemm_one(m, n, k, args.iters, args.pair[0] if args.pair else 1)
  elif args.what == "streaming":
    bench_streaming()
  elif args.what == "skinny":
    bench_skinny()
  elif args.what == "gemm-trace":
    m, n, k = args.shape or [256, 2048, 2048]
    gemm_trace(m, n, k, args.splits)
  elif args.what == "attention-one":
    b, h, lq, lk = args.shape or [16, 64, 512, 512]
    attention_one(b, h, lq, lk, args.iters)
  else:
    bench_attention()


if __name__ == "__main__":
  main()
