"""Times the fused tensor-parallel GEMMs against their NCCL + GEMM equivalents.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      --master-port 29620 -m t5x_b200.parallel.bench_tp [--rows 8192] [--iters 20]

For the T5.1.1-XXL projections (d_model 4096, 64 heads x 64, d_ff 10240) with `--rows` rows of
activations in total, every rank times with CUDA events (max over ranks reported):

  all-gather -> GEMM   `t5x_gemm_allgather_bf16`  vs  NCCL all_gather_into_tensor + GEMM
  GEMM -> reduce-scatter `t5x_gemm_reducescatter_bf16` + inbox sum  vs  GEMM + NCCL reduce_scatter

and prints, per shape, the times, the time of the GEMM alone, and the roofline: the slower of
FLOPs / (measured GEMM throughput) and bytes over NVLink / (770 GB/s per direction).
Operands are re-randomised buffers larger than L2 in rotation (4 sets).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _time(fn, iters: int, warmup: int = 3) -> float:
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  dist.barrier()
  e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  e0.record()
  for _ in range(iters):
    fn()
  e1.record()
  torch.cuda.synchronize()
  t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
  dist.all_reduce(t, op=dist.ReduceOp.MAX)
  return float(t[0])


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--rows", type=int, default=8192)
  ap.add_argument("--iters", type=int, default=20)
  args = ap.parse_args()
  from t5x_b200.ops import native
  from t5x_b200.parallel import state as pstate, tp_fused
  torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
  pstate.init_distributed("nccl")
  st = pstate.setup_mesh(model_size=int(os.environ["WORLD_SIZE"]))
  T, r = st.model_size, st.model_rank
  M, d, inner, dff = args.rows, 4096, 4096, 10240
  m = M // T
  ar = tp_fused.arena()
  dev = st.device
  rnd = lambda *s: (torch.randn(*s, device=dev) * 0.05).to(torch.bfloat16)
  rows = []

  # ---- all-gather -> GEMM: q projection [d, inner/T] and gated wi [d, dff/T] x 2 ----
  for name, n, gated in (("q_proj", inner // T, False), ("mlp_wi", dff // T, True)):
    w0, w1 = rnd(d, n), rnd(d, n)
    h_sp = [rnd(m, d) for _ in range(4)]
    full = torch.empty(M, d, dtype=torch.bfloat16, device=dev)
    i = [0]

    def fused():
      blk = tp_fused._gather_block(h_sp[i[0] % 4])
      tp_fused.gemm_allgather(blk, M, d, w0, b2=w1 if gated else None)
      blk.release()
      i[0] += 1

    def nccl():
      dist.all_gather_into_tensor(full, h_sp[i[0] % 4], group=st.model_group)
      native.gemm(full, w0, b2=w1 if gated else None)
      i[0] += 1

    def alone():
      native.gemm(full, w0, b2=w1 if gated else None)

    t_f, t_n, t_g = _time(fused, args.iters), _time(nccl, args.iters), _time(alone, args.iters)
    flops = 2.0 * M * d * n * (2 if gated else 1)
    link = (T - 1) * m * d * 2 / (NVLINK_GBS * 1e9) * 1e3   # ms to pull the other blocks
    rows.append({"op": f"allgather->gemm {name}", "M": M, "N": n, "K": d, "fused_ms": t_f,
                 "nccl_ms": t_n, "gemm_ms": t_g, "link_ms": link,
                 "roofline_ms": max(t_g, link), "of_roofline": max(t_g, link) / t_f,
                 "gemm_tflops": flops / t_g / 1e9})

  # ---- GEMM -> reduce-scatter: attention out [inner/T, d] and wo [dff/T, d] ----
  for name, k in (("attn_out", inner // T), ("mlp_wo", dff // T)):
    w = rnd(k, d)
    a = [rnd(M, k) for _ in range(4)]
    part = torch.empty(M, d, dtype=torch.bfloat16, device=dev)
    outb = torch.empty(m, d, dtype=torch.bfloat16, device=dev)
    i = [0]

    def fused():
      tp_fused._reduce_scatter(a[i[0] % 4], w)
      i[0] += 1

    def nccl():
      native.gemm(a[i[0] % 4], w, out=part)
      dist.reduce_scatter_tensor(outb, part, group=st.model_group)
      i[0] += 1

    def alone():
      native.gemm(a[i[0] % 4], w, out=part)

    t_f, t_n, t_g = _time(fused, args.iters), _time(nccl, args.iters), _time(alone, args.iters)
    flops = 2.0 * M * d * k
    link = (T - 1) * m * d * 2 / (NVLINK_GBS * 1e9) * 1e3
    rows.append({"op": f"gemm->reducescatter {name}", "M": M, "N": d, "K": k, "fused_ms": t_f,
                 "nccl_ms": t_n, "gemm_ms": t_g, "link_ms": link,
                 "roofline_ms": max(t_g, link), "of_roofline": max(t_g, link) / t_f,
                 "gemm_tflops": flops / t_g / 1e9})
  native.check_status()
  if st.rank == 0:
    for row in rows:
      print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()}))
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
