"""Builds the native sm_100a library in-tree.

Every ``csrc/*.cu`` file is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``
and linked into ``t5x_b200/lib/libt5x_b200.so``; the result is loaded with ctypes by
:mod:`t5x_b200.ops.native`. nvcc cross-compiles without a GPU present.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CSRC = os.path.join(ROOT, "csrc")
LIB_DIR = os.path.join(ROOT, "t5x_b200", "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libt5x_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
  cand = os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
  return cand if os.path.exists(cand) else "nvcc"


def sources() -> list[str]:
  return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime() -> float:
  return max([os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC)
              if f.endswith((".cuh", ".h"))] + [0.0])


def _compile(src: str, verbose: bool, ptxas_v: bool) -> str:
  obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
  newest = max(os.path.getmtime(src), _headers_mtime())
  if os.path.exists(obj) and os.path.getmtime(obj) >= newest:
    return obj
  cmd = [_nvcc(), *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
  if ptxas_v:
    cmd[1:1] = ["-Xptxas", "-v"]
  if verbose:
    print(" ".join(cmd), flush=True)
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
  if ptxas_v or verbose:
    sys.stderr.write(r.stderr)
  return obj


def build(verbose: bool = False, force: bool = False, ptxas_v: bool = False) -> str:
  """Compiles what is out of date and links the shared library. Returns its path."""
  os.makedirs(OBJ_DIR, exist_ok=True)
  srcs = sources()
  if force:
    for f in os.listdir(OBJ_DIR):
      os.remove(os.path.join(OBJ_DIR, f))
  with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
    objs = list(ex.map(lambda s: _compile(s, verbose, ptxas_v), srcs))
  if (not os.path.exists(LIB_PATH)) or any(os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs):
    cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH, *objs]
    if verbose:
      print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
      raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
  return LIB_PATH


if __name__ == "__main__":
  print(build(verbose=True, force="--force" in sys.argv, ptxas_v="--ptxas-v" in sys.argv))
