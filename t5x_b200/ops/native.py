"""ctypes binding of the in-tree sm_100a library (``t5x_b200/lib/libt5x_b200.so``).

The library exports a plain C ABI: device pointers, sizes and a CUDA stream. The
wrappers here take ``torch`` tensors, check dtypes/contiguity, pass
``tensor.data_ptr()`` and the current stream, and raise ``NativeError`` with the
library's message when a call is rejected. On a machine with a GPU a missing
library is an error (there is no silent fallback); without a GPU the pure
PyTorch reference ops in :mod:`t5x_b200.ops.reference` are what runs.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib",
                         "libt5x_b200.so")
_lib = None
_lock = threading.Lock()


class NativeError(RuntimeError):
  pass


class KernelStatusError(RuntimeError):
  """A kernel gave up on a bounded wait (or flagged non-finite values)."""


STATUS_NAMES = {
    0: "ok", 1: "timeout: TMA producer", 2: "timeout: MMA issuer", 3: "timeout: epilogue",
    4: "timeout: peer flag", 5: "bad argument", 6: "non-finite value",
}

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _declare(lib):
  lib.t5x_last_error.restype = ctypes.c_char_p
  lib.t5x_launch_count.restype = c_ll
  lib.t5x_read_status.argtypes = [ctypes.POINTER(c_int), c_void_p]
  lib.t5x_gemm_bf16.argtypes = [
      c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll,
      c_ll, c_ll, c_int, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_ll, c_void_p, c_void_p,
      c_ll, c_float, c_int, c_void_p]
  lib.t5x_rmsnorm_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                                  c_void_p]
  lib.t5x_rmsnorm_bwd.argtypes = [c_void_p] * 7 + [c_int, c_int, c_void_p]
  lib.t5x_gated_gelu_bwd.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_int, c_void_p]
  lib.t5x_gated_gelu_fwd.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_void_p]
  lib.t5x_embedding_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int,
                                    c_void_p]
  lib.t5x_embedding_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int,
                                    c_void_p]
  lib.t5x_cast_f32_bf16.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_void_p]
  lib.t5x_ce_stats.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                               c_int, c_ll, c_int, c_void_p]
  lib.t5x_ce_grad.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                              c_int, c_ll, c_ll, c_int, c_float, c_float, c_float, c_void_p]
  lib.t5x_adafactor_scratch_floats.restype = c_ll
  lib.t5x_adafactor_scratch_floats.argtypes = [c_int, c_int, c_int]
  lib.t5x_adafactor_factored.argtypes = [
      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_void_p, c_int,
      c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_float, c_float, c_float, c_float,
      c_int, c_void_p]
  lib.t5x_adafactor_unfactored.argtypes = [
      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_void_p, c_int, c_int, c_int,
      c_float, c_float, c_float, c_float, c_float, c_float, c_float, c_float, c_int, c_void_p]
  lib.t5x_adafactor_stats.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float,
                                      c_void_p]
  lib.t5x_adafactor_ema.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                    c_int, c_int, c_float, c_int, c_void_p]
  lib.t5x_adafactor_usq.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                    c_int, c_int, c_int, c_int, c_void_p]
  lib.t5x_adafactor_apply.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll,
                                      c_void_p, c_int, c_int, c_int, c_ll, c_float, c_float,
                                      c_float, c_float, c_float, c_float, c_int, c_void_p]
  lib.t5x_adafactor_unfactored_stats.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                 c_ll, c_float, c_float, c_int, c_void_p]
  lib.t5x_adafactor_unfactored_apply.argtypes = [
      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_ll, c_void_p, c_int, c_int, c_int,
      c_ll, c_float, c_float, c_float, c_float, c_float, c_float, c_int, c_void_p]
  return lib


def available() -> bool:
  """True when the shared library exists (it may still need a GPU to run)."""
  return os.path.exists(_LIB_PATH)


def lib():
  """Loads the library (building it first if it is missing and nvcc is present)."""
  global _lib
  if _lib is not None:
    return _lib
  with _lock:
    if _lib is None:
      if not os.path.exists(_LIB_PATH):
        from t5x_b200.ops import build as _build
        _build.build()
      _lib = _declare(ctypes.CDLL(_LIB_PATH))
      _declare_optional(_lib)
  return _lib


def _declare_optional(l):
  """Entry points added by later source files; declared only when present."""
  for name, argtypes in _OPTIONAL_SIGNATURES.items():
    if hasattr(l, name):
      getattr(l, name).argtypes = argtypes


_OPTIONAL_SIGNATURES: dict = {}


def register_signature(name: str, argtypes) -> None:
  _OPTIONAL_SIGNATURES[name] = argtypes
  if _lib is not None and hasattr(_lib, name):
    getattr(_lib, name).argtypes = argtypes


def launch_count() -> int:
  """Kernels launched by the native library so far in this process."""
  return int(lib().t5x_launch_count())


class chained_launches:
  """Context: kernels of this library that support it are launched as programmatic dependents
  of the kernel before them on the stream, so that their set-up (barriers, TMEM, descriptor
  fetches) overlaps that kernel's tail. Level 2 also promises that the B operand of every GEMM
  issued inside is a constant weight, which those GEMMs then request before they wait for
  their predecessor. For sequences of short kernels (a decode step); captured into CUDA graphs
  as programmatic dependencies. Applies to the calling thread."""

  def __init__(self, level: int = 2):
    self.level = int(level)

  def __enter__(self):
    l = lib()
    l.t5x_set_chained_launches.argtypes = [c_int]
    l.t5x_set_chained_launches(self.level)
    return self

  def __exit__(self, *exc):
    lib().t5x_set_chained_launches(0)
    return False


def use_native(t: torch.Tensor) -> bool:
  """Native kernels run for CUDA tensors; on a GPU the library is mandatory."""
  return t.is_cuda


def _check(rc: int, what: str) -> None:
  if rc != 0:
    raise NativeError(f"{what}: {lib().t5x_last_error().decode()}")


def stream_ptr() -> int:
  return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> int:
  return 0 if t is None else t.data_ptr()


def check_status() -> None:
  """Synchronises the current stream and raises if a kernel reported a failure."""
  words = (c_int * 8)()
  code = lib().t5x_read_status(words, stream_ptr())
  if code < 0:
    raise NativeError(lib().t5x_last_error().decode())
  if code != 0:
    raise KernelStatusError(
        f"kernel {words[1]} block {words[2]} reported '{STATUS_NAMES.get(code, code)}' "
        f"(payload {words[3]}, {words[4]})")


def _raise_status(words) -> None:
  code = int(words[0])
  raise KernelStatusError(
      f"kernel {int(words[1])} block {int(words[2])} reported '{STATUS_NAMES.get(code, code)}' "
      f"(payload {int(words[3])}, {int(words[4])})")


class StatusPoller:
  """Watches the device status words from inside a training loop without stalling it.

  `poll()` looks at the copy enqueued by an earlier `poll()` if that copy has completed
  (raising `KernelStatusError` when a kernel gave up on a bounded wait: a peer that never
  raised its flag, a barrier that ran out) and enqueues the next copy behind the work launched
  so far. A failure is therefore reported one or two steps after it happened, and the host
  never waits for the GPU. `check()` is the blocking form for points where the state leaves
  the loop (checkpoints, the end of training)."""

  def __init__(self):
    self._host = torch.zeros(8, dtype=torch.int32).pin_memory()
    self._event = None

  def poll(self) -> None:
    if self._event is not None:
      if not self._event.query():
        return
      if int(self._host[0]) != 0:
        words = self._host.clone()
        self._event = None
        check_status()  # synchronises and clears the device words
        _raise_status(words)
    l = lib()
    l.t5x_status_copy_async.argtypes = [c_void_p, c_void_p]
    _check(l.t5x_status_copy_async(self._host.data_ptr(), stream_ptr()), "status_copy_async")
    self._event = torch.cuda.Event()
    self._event.record()

  def check(self) -> None:
    self._event = None
    check_status()


# ----------------------------------------------------------------------------
# GEMM
# ----------------------------------------------------------------------------
EPI_PLAIN, EPI_GATED_GELU, EPI_RESIDUAL = 0, 1, 2


def _mat_layout(t: torch.Tensor, rows: int, cols: int):
  """Returns (mn_major, ld, batch_stride) for a [..., rows, cols] operand whose contraction
  dim is `cols` when K-major. Accepts row-major or its transpose view."""
  if t.stride(-1) == 1:
    return 0, t.stride(-2), (t.stride(0) if t.dim() == 3 else 0)
  if t.stride(-2) == 1:
    return 1, t.stride(-1), (t.stride(0) if t.dim() == 3 else 0)
  raise NativeError(f"operand with strides {t.stride()} is neither row- nor column-major")


def gemm(a: torch.Tensor, b: torch.Tensor, *, out: Optional[torch.Tensor] = None,
         out_dtype: torch.dtype = torch.bfloat16, accumulate: bool = False,
         residual: Optional[torch.Tensor] = None, b2: Optional[torch.Tensor] = None,
         save_h: Optional[torch.Tensor] = None, alpha: float = 1.0,
         max_ctas: int = 0) -> torch.Tensor:
  """out[..., M, N] (+)= a[..., M, K] @ b[..., K, N]   (bf16 inputs, fp32 accumulation).

  `a` and `b` may be arbitrary 2-D/3-D views whose last two dims are row-major or
  transposed-row-major (no copy is made: the tensor-core descriptors read either).
  With `b2` the gated-GELU epilogue runs: out = gelu(a @ b) * (a @ b2); `save_h`
  ([M, 2N], bf16) then receives the two pre-activations side by side.
  `residual` adds a bf16 tensor of the output's shape in the epilogue.
  """
  assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
  batch = a.shape[0] if a.dim() == 3 else 1
  M, K = a.shape[-2], a.shape[-1]
  K2, N = b.shape[-2], b.shape[-1]
  assert K == K2, (a.shape, b.shape)
  a_mn, lda, abs_ = _mat_layout(a, M, K)
  # b as a [K, N] matrix: "K-major" for the kernel means memory [N, K] with K contiguous.
  if b.stride(-2) == 1:
    b_mn, ldb = 0, b.stride(-1)
  elif b.stride(-1) == 1:
    b_mn, ldb = 1, b.stride(-2)
  else:
    raise NativeError(f"b with strides {b.stride()} is neither row- nor column-major")
  bbs = b.stride(0) if b.dim() == 3 else 0
  if out is None:
    shape = (batch, M, N) if a.dim() == 3 else (M, N)
    out = torch.empty(shape, dtype=out_dtype, device=a.device)
  assert out.stride(-1) == 1 and out.shape[-2:] == (M, N), (out.shape, out.stride(), M, N)
  epi = EPI_PLAIN
  r_ptr, ldr, rbs = 0, 0, 0
  if residual is not None:
    assert residual.dtype == torch.bfloat16 and residual.stride(-1) == 1
    epi = EPI_RESIDUAL
    r_ptr, ldr = residual.data_ptr(), residual.stride(-2)
    rbs = residual.stride(0) if residual.dim() == 3 else 0
  h0 = h1 = 0
  ldh = 0
  b2_ptr = 0
  if b2 is not None:
    assert b2.stride() == b.stride() and b2.shape == b.shape
    epi = EPI_GATED_GELU
    b2_ptr = b2.data_ptr()
    if save_h is not None:
      assert save_h.dtype == torch.bfloat16 and save_h.shape[-1] == 2 * N and save_h.stride(-1) == 1
      h0 = save_h.data_ptr()
      h1 = h0 + N * 2
      ldh = save_h.stride(-2)
  rc = lib().t5x_gemm_bf16(
      a.data_ptr(), b.data_ptr(), b2_ptr, out.data_ptr(), M, N, K, batch, lda, ldb,
      out.stride(-2), abs_, bbs, out.stride(0) if out.dim() == 3 else 0, a_mn, b_mn,
      1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0, epi, r_ptr, ldr, rbs, h0,
      h1, ldh, alpha, max_ctas, stream_ptr())
  _check(rc, "gemm")
  return out


# ----------------------------------------------------------------------------
# Normalisation / activations / embedding
# ----------------------------------------------------------------------------
def gemm_splitk(a: torch.Tensor, b: torch.Tensor, splits: int, *,
                residual: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                workspace: Optional[torch.Tensor] = None,
                workspace_is_clear: bool = False) -> torch.Tensor:
  """out[M, N] (bf16) = a[M, K] @ b[K, N] (+ residual) with K cut into `splits` slices whose
  partial products are added atomically into an fp32 workspace. For skinny problems (decode
  steps: M of a few hundred rows) this puts `splits` times more CTAs on the weight stream
  than one CTA per output tile would. `workspace_is_clear`: the caller's workspace is zero on
  entry and is left zero on return (the finishing kernel clears what it reads), so a sequence
  of such GEMMs over one workspace needs no fill kernel at all."""
  M, K = a.shape
  N = b.shape[1]
  assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.stride(1) == 1
  assert b.stride(1) == 1, "b must be row-major [K, N]"
  if splits <= 1 or K % splits or (K // splits) % 64 or N % 4:
    return gemm(a, b, out=out, residual=residual)
  ks = K // splits
  ws = workspace if workspace is not None else torch.empty(M, N, dtype=torch.float32,
                                                           device=a.device)
  ws = ws.view(-1)[:M * N].view(M, N)
  keep_clear = workspace_is_clear and workspace is not None
  if not keep_clear:
    ws.zero_()
  rc = lib().t5x_gemm_bf16(
      a.data_ptr(), b.data_ptr(), 0, ws.data_ptr(), M, N, ks, splits, a.stride(0), b.stride(0), N,
      ks, ks * b.stride(0), 0, 0, 1, 1, 2, EPI_PLAIN, 0, 0, 0, 0, 0, 0, 1.0, 0, stream_ptr())
  _check(rc, "gemm_splitk")
  if out is None:
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
  assert out.is_contiguous() and (residual is None or residual.is_contiguous())
  l = lib()
  if keep_clear:
    l.t5x_f32_to_bf16_residual_clear.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_void_p]
    _check(l.t5x_f32_to_bf16_residual_clear(ws.data_ptr(), ptr(residual), out.data_ptr(), M * N,
                                            stream_ptr()), "f32_to_bf16_residual_clear")
  else:
    l.t5x_f32_to_bf16_residual.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_void_p]
    _check(l.t5x_f32_to_bf16_residual(ws.data_ptr(), ptr(residual), out.data_ptr(), M * N,
                                      stream_ptr()), "f32_to_bf16_residual")
  return out


def gemm_skinny_splits(M: int, N: int, K: int) -> int:
  """Cluster size `gemm_skinny` would use for this shape; 0 when it does not cover it."""
  l = lib()
  l.t5x_gemm_skinny_splits.argtypes = [c_int, c_int, c_int]
  return int(l.t5x_gemm_skinny_splits(M, N, K))


def gemm_skinny(a: torch.Tensor, b: torch.Tensor, *, residual: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, splits: Optional[int] = None,
                alpha: float = 1.0) -> Optional[torch.Tensor]:
  """out[M, N] (bf16) = alpha * a[M, K] @ b[K, N] (+ residual) for few rows: K is cut over the
  CTAs of a thread-block cluster, which add their partial products through distributed shared
  memory and store finished bf16 rows (no workspace, no second kernel). `b` may be row-major
  [K, N] or a transposed view of a row-major [N, K] matrix. Returns None when the shape is not
  covered (N % 128, K % 64, more tiles than SMs); callers then use `gemm` / `gemm_splitk`."""
  M, K = a.shape
  N = b.shape[1]
  if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or a.stride(1) != 1 or M == 0:
    return None
  if b.stride(1) == 1:
    b_mn, ldb = 1, b.stride(0)
  elif b.stride(0) == 1:
    b_mn, ldb = 0, b.stride(1)
  else:
    return None
  s = gemm_skinny_splits(M, N, K) if splits is None else int(splits)
  if s <= 0 or a.stride(0) % 8 or ldb % 8 or (a.data_ptr() | b.data_ptr()) & 15:
    return None
  if residual is not None and (residual.stride(1) != 1 or residual.stride(0) % 4 or
                               residual.dtype != torch.bfloat16):
    return None
  if out is None:
    out = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
  assert out.stride(1) == 1 and out.stride(0) % 4 == 0 and out.dtype == torch.bfloat16
  l = lib()
  l.t5x_gemm_skinny_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                     c_ll, c_ll, c_ll, c_ll, c_int, c_int, c_float, c_void_p]
  _check(l.t5x_gemm_skinny_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), ptr(residual), M, N, K,
                                a.stride(0), ldb, out.stride(0),
                                residual.stride(0) if residual is not None else 0, b_mn, s,
                                float(alpha), stream_ptr()), "gemm_skinny")
  return out


def gemm_splitk_norm(a: torch.Tensor, b: torch.Tensor, splits: int, *, residual: torch.Tensor,
                     scale: torch.Tensor, eps: float, workspace: torch.Tensor):
  """(x, h): x = a @ b + residual (bf16), h = rmsnorm(x) * scale, with K cut into `splits`
  slices added atomically into `workspace` (fp32, zero on entry, zero again on return) and one
  finishing kernel per row doing the residual add, the rounding and the norm. Falls back to
  the separate kernels when the shape does not split."""
  M, K = a.shape
  N = b.shape[1]
  if splits <= 1 or K % splits or (K // splits) % 64 or N % 8 or N > 8192 or b.stride(1) != 1:
    x = gemm_splitk(a, b, splits, residual=residual, workspace=workspace,
                    workspace_is_clear=True)
    return x, rmsnorm_fwd(x, scale, eps)[0]
  ks = K // splits
  ws = workspace.view(-1)[:M * N].view(M, N)
  rc = lib().t5x_gemm_bf16(
      a.data_ptr(), b.data_ptr(), 0, ws.data_ptr(), M, N, ks, splits, a.stride(0), b.stride(0), N,
      ks, ks * b.stride(0), 0, 0, 1, 1, 2, EPI_PLAIN, 0, 0, 0, 0, 0, 0, 1.0, 0, stream_ptr())
  _check(rc, "gemm_splitk")
  x = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
  h = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
  assert residual is None or residual.is_contiguous()
  l = lib()
  l.t5x_finish_residual_rmsnorm.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_int, c_int, c_float, c_void_p]
  _check(l.t5x_finish_residual_rmsnorm(ws.data_ptr(), ptr(residual), scale.data_ptr(),
                                       x.data_ptr(), h.data_ptr(), M, N, float(eps),
                                       stream_ptr()), "finish_residual_rmsnorm")
  return x, h


def wgrad_splits(M: int, N: int, K: int) -> int:
  """How many K slices a weight-gradient GEMM [M, K] @ [K, N] should be cut into: 1 unless
  the output has too few tiles to occupy the SMs and K is long (small models: a 768 x 768
  gradient over 131072 tokens is 18 output tiles)."""
  tiles = -(-M // 128) * -(-N // 256)
  sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
  if tiles * 2 > sms or K < 8192:
    return 1
  splits = min(sms // tiles, K // 2048)
  while splits > 1 and (K % splits or (K // splits) % 64):
    splits -= 1
  return max(1, splits)


def gemm_splitk_accumulate(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, splits: int,
                           accumulate: bool) -> torch.Tensor:
  """out[M, N] (fp32) (+)= a[M, K] @ b[K, N] with K cut into `splits` slices whose products
  are added atomically into `out` (cleared first unless `accumulate`). Operand layouts as in
  `gemm`."""
  assert out.dtype == torch.float32 and out.is_contiguous()
  M, K = a.shape
  N = b.shape[1]
  ks = K // splits
  a_mn, lda, _ = _mat_layout(a, M, K)
  if b.stride(-2) == 1:
    b_mn, ldb = 0, b.stride(-1)
  else:
    b_mn, ldb = 1, b.stride(-2)
  a_step = ks * lda if a_mn else ks       # elements between consecutive K slices
  b_step = ks * ldb if b_mn else ks
  if not accumulate:
    out.zero_()
  rc = lib().t5x_gemm_bf16(
      a.data_ptr(), b.data_ptr(), 0, out.data_ptr(), M, N, ks, splits, lda, ldb, N, a_step,
      b_step, 0, a_mn, b_mn, 1, 2, EPI_PLAIN, 0, 0, 0, 0, 0, 0, 1.0, 0, stream_ptr())
  _check(rc, "gemm_splitk_accumulate")
  return out


def gemm_set_pair_mode(mode: int) -> None:
  """0: one CTA per tile always; 1: CTA pairs (256 x 256 tiles) where the shape suits them
  (default); 2: CTA pairs always."""
  l = lib()
  l.t5x_gemm_set_pair_mode.argtypes = [c_int]
  _check(l.t5x_gemm_set_pair_mode(mode), "gemm_set_pair_mode")


def rmsnorm_fwd(x: torch.Tensor, scale: torch.Tensor, eps: float,
                out: Optional[torch.Tensor] = None):
  d = x.shape[-1]
  x2 = x.reshape(-1, d)
  assert x2.is_contiguous() and x.dtype == torch.bfloat16 and scale.dtype == torch.float32
  if out is not None:
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() == x2.numel()
  y = torch.empty_like(x2) if out is None else out.view(x2.shape)
  rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
  _check(lib().t5x_rmsnorm_fwd(x2.data_ptr(), scale.data_ptr(), y.data_ptr(), rstd.data_ptr(),
                               x2.shape[0], d, eps, stream_ptr()), "rmsnorm_fwd")
  return y.view(x.shape), rstd


def rmsnorm_bwd(dy, x, scale, rstd, dres: Optional[torch.Tensor], dscale: torch.Tensor):
  """Returns dx (+ dres). Accumulates into `dscale` (fp32 [d])."""
  d = x.shape[-1]
  dy2, x2 = dy.reshape(-1, d), x.reshape(-1, d)
  assert dy2.is_contiguous() and x2.is_contiguous()
  dx = torch.empty_like(x2)
  dres2 = None
  if dres is not None:
    dres2 = dres.reshape(-1, d)
    assert dres2.is_contiguous()
  _check(lib().t5x_rmsnorm_bwd(dy2.data_ptr(), x2.data_ptr(), scale.data_ptr(), rstd.data_ptr(),
                               ptr(dres2), dx.data_ptr(), dscale.data_ptr(), x2.shape[0], d,
                               stream_ptr()), "rmsnorm_bwd")
  return dx.view(x.shape)


def gated_gelu_bwd_(dg: torch.Tensor, h: torch.Tensor, write_g: bool = False) -> None:
  """In place: h=[h0|h1] -> [dh0|dh1]; with `write_g`, dg -> g (the recomputed activation)."""
  dff = dg.shape[-1]
  dg2, h2 = dg.view(-1, dff), h.view(-1, 2 * dff)
  _check(lib().t5x_gated_gelu_bwd(dg2.data_ptr(), h2.data_ptr(), dg2.shape[0], dff, h2.stride(0),
                                  dg2.stride(0), int(write_g), stream_ptr()), "gated_gelu_bwd")


def gated_gelu_fwd(h: torch.Tensor) -> torch.Tensor:
  dff = h.shape[-1] // 2
  h2 = h.view(-1, 2 * dff)
  g = torch.empty((h2.shape[0], dff), dtype=h.dtype, device=h.device)
  _check(lib().t5x_gated_gelu_fwd(h2.data_ptr(), g.data_ptr(), h2.shape[0], dff, h2.stride(0),
                                  g.stride(0), stream_ptr()), "gated_gelu_fwd")
  return g.view(*h.shape[:-1], dff)


def embedding_fwd(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
  assert ids.dtype == torch.int64 and table.dtype == torch.bfloat16 and table.is_contiguous()
  ids_c = ids.contiguous()
  out = torch.empty((*ids.shape, table.shape[1]), dtype=torch.bfloat16, device=table.device)
  _check(lib().t5x_embedding_fwd(ids_c.data_ptr(), table.data_ptr(), out.data_ptr(),
                                 ids_c.numel(), table.shape[1], vocab_start, table.shape[0],
                                 stream_ptr()), "embedding_fwd")
  return out


def embedding_bwd_(ids: torch.Tensor, dout: torch.Tensor, dtable: torch.Tensor,
                   vocab_start: int = 0) -> None:
  assert dtable.dtype == torch.float32 and dtable.is_contiguous() and dout.is_contiguous()
  ids_c = ids.contiguous()
  _check(lib().t5x_embedding_bwd(ids_c.data_ptr(), dout.data_ptr(), dtable.data_ptr(),
                                 ids_c.numel(), dtable.shape[1], vocab_start, dtable.shape[0],
                                 stream_ptr()), "embedding_bwd")


def cast_f32_bf16_(src: torch.Tensor, dst: torch.Tensor) -> None:
  """dst (bf16, possibly a column slice of a wider matrix) <- src (fp32, 2-D)."""
  assert src.dtype == torch.float32 and dst.dtype == torch.bfloat16 and src.dim() == 2
  assert src.stride(1) == 1 and dst.stride(1) == 1 and src.shape == dst.shape
  _check(lib().t5x_cast_f32_bf16(src.data_ptr(), dst.data_ptr(), src.shape[0], src.shape[1],
                                 src.stride(0), dst.stride(0), stream_ptr()), "cast")


# ----------------------------------------------------------------------------
# Cross entropy
# ----------------------------------------------------------------------------
def ce_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int = 0):
  rows, v = logits.shape
  assert logits.stride(1) == 1 and targets.dtype == torch.int64
  stats = torch.empty((rows, 4), dtype=torch.float32, device=logits.device)
  arg_val = torch.empty(rows, dtype=torch.float32, device=logits.device)
  arg_idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
  _check(lib().t5x_ce_stats(logits.data_ptr(), int(logits.dtype == torch.float32),
                            targets.data_ptr(), stats.data_ptr(), arg_val.data_ptr(),
                            arg_idx.data_ptr(), rows, v, logits.stride(0), vocab_start,
                            stream_ptr()), "ce_stats")
  return stats, arg_val, arg_idx


def ce_grad(logits, targets, lse, row_scale, z_loss, confidence, low_confidence,
            vocab_start: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
  rows, v = logits.shape
  if out is None:
    out = torch.empty((rows, v), dtype=torch.bfloat16, device=logits.device)
  _check(lib().t5x_ce_grad(logits.data_ptr(), int(logits.dtype == torch.float32),
                           targets.data_ptr(), lse.data_ptr(), row_scale.data_ptr(),
                           out.data_ptr(), rows, v, logits.stride(0), out.stride(0), vocab_start,
                           z_loss, confidence, low_confidence, stream_ptr()), "ce_grad")
  return out


register_signature("t5x_gemm_ce_tiles", [c_int])
register_signature("t5x_gemm_ce_stats", [c_void_p, c_void_p, c_int, c_int, c_int, c_ll, c_ll, c_int,
                                         c_int, c_float, c_void_p, c_int, c_void_p, c_void_p,
                                         c_void_p, c_void_p])
register_signature("t5x_gemm_ce_grad", [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_int,
                                        c_ll, c_ll, c_int, c_int, c_float, c_void_p, c_int,
                                        c_void_p, c_void_p, c_float, c_float, c_float, c_void_p])
register_signature("t5x_ce_merge", [c_void_p] * 7 + [c_int, c_int, c_int, c_int, c_void_p])


def _b_layout(b: torch.Tensor):
  """(mn_major, ld) of b as the [K, N] operand of the GEMM kernels."""
  if b.stride(-2) == 1:
    return 0, b.stride(-1)
  if b.stride(-1) == 1:
    return 1, b.stride(-2)
  raise NativeError(f"b with strides {b.stride()} is neither row- nor column-major")


def gemm_ce_stats(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, alpha: float = 1.0,
                  vocab_start: int = 0):
  """Cross-entropy statistics of logits = alpha * h[M, K] @ w[K, N] without storing the
  logits: the GEMM epilogue folds every 256-column tile into softmax partials, which a second
  small kernel merges. Returns what `ce_stats` returns: stats [M, 4] = (max, sum exp(x - max),
  target logit, sum x), arg_val [M], arg_idx [M] (vocabulary id of the largest logit)."""
  assert h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and targets.dtype == torch.int64
  M, K = h.shape
  N = w.shape[1]
  a_mn, lda, _ = _mat_layout(h, M, K)
  b_mn, ldb = _b_layout(w)
  tiles = int(lib().t5x_gemm_ce_tiles(N))
  dev = h.device
  part = torch.empty((M, tiles, 4), dtype=torch.float32, device=dev)
  arg = torch.empty((M, tiles), dtype=torch.int32, device=dev)
  tlogit = torch.zeros(M, dtype=torch.float32, device=dev)
  t = targets.contiguous()
  _check(lib().t5x_gemm_ce_stats(h.data_ptr(), w.data_ptr(), M, N, K, lda, ldb, a_mn, b_mn,
                                 float(alpha), t.data_ptr(), vocab_start, part.data_ptr(),
                                 arg.data_ptr(), tlogit.data_ptr(), stream_ptr()), "gemm_ce_stats")
  stats = torch.empty((M, 4), dtype=torch.float32, device=dev)
  arg_val = torch.empty(M, dtype=torch.float32, device=dev)
  arg_idx = torch.empty(M, dtype=torch.int32, device=dev)
  _check(lib().t5x_ce_merge(part.data_ptr(), arg.data_ptr(), tlogit.data_ptr(), t.data_ptr(),
                            stats.data_ptr(), arg_val.data_ptr(), arg_idx.data_ptr(), M, tiles,
                            vocab_start, N, stream_ptr()), "ce_merge")
  return stats, arg_val, arg_idx


def gemm_ce_grad(h: torch.Tensor, w: torch.Tensor, targets: torch.Tensor, lse: torch.Tensor,
                 row_scale: torch.Tensor, z_loss: float, confidence: float,
                 low_confidence: float, alpha: float = 1.0, vocab_start: int = 0) -> torch.Tensor:
  """dlogits [M, N] (bf16) of the cross-entropy over logits = alpha * h @ w, with the logits
  recomputed tile by tile inside the GEMM instead of read from memory."""
  M, K = h.shape
  N = w.shape[1]
  a_mn, lda, _ = _mat_layout(h, M, K)
  b_mn, ldb = _b_layout(w)
  out = torch.empty((M, N), dtype=torch.bfloat16, device=h.device)
  _check(lib().t5x_gemm_ce_grad(h.data_ptr(), w.data_ptr(), out.data_ptr(), out.stride(0), M, N,
                                K, lda, ldb, a_mn, b_mn, float(alpha),
                                targets.contiguous().data_ptr(), vocab_start,
                                lse.contiguous().data_ptr(), row_scale.contiguous().data_ptr(),
                                float(z_loss), float(confidence), float(low_confidence),
                                stream_ptr()), "gemm_ce_grad")
  return out


# ----------------------------------------------------------------------------
# Adafactor
# ----------------------------------------------------------------------------
AF_PARAM_SCALE, AF_CLIP, AF_WD, AF_MOMENTUM, AF_MAX_SCALE, AF_SKIP_NAN = 1, 2, 4, 8, 16, 32


def adafactor_scratch_floats(batch: int, rows: int, cols: int) -> int:
  return int(lib().t5x_adafactor_scratch_floats(batch, rows, cols))


def adafactor_factored_(p, g, v_rvec, v_cvec, m, p_bf16, scratch, *, batch, rows, cols,
                        row_is_normalized, lr, decay, eps1, eps2, clip_threshold, weight_decay,
                        beta1, max_param_scale, flags, ld_bf16=0, bf16_batch_stride=0) -> None:
  _check(lib().t5x_adafactor_factored(
      p.data_ptr(), g.data_ptr(), v_rvec.data_ptr(), v_cvec.data_ptr(), ptr(m), ptr(p_bf16),
      ld_bf16, bf16_batch_stride, scratch.data_ptr(), batch, rows, cols, int(row_is_normalized),
      lr, decay, eps1, eps2, clip_threshold, weight_decay, beta1, max_param_scale, flags,
      stream_ptr()), "adafactor_factored")


def adafactor_unfactored_(p, g, v, m, p_bf16, scratch, *, batch, rows, cols, lr, decay, eps1, eps2,
                          clip_threshold, weight_decay, beta1, max_param_scale, flags, ld_bf16=0,
                          bf16_batch_stride=0) -> None:
  _check(lib().t5x_adafactor_unfactored(
      p.data_ptr(), g.data_ptr(), v.data_ptr(), ptr(m), ptr(p_bf16), ld_bf16, bf16_batch_stride,
      scratch.data_ptr(), batch, rows, cols, lr, decay, eps1, eps2, clip_threshold, weight_decay,
      beta1, max_param_scale, flags, stream_ptr()), "adafactor_unfactored")


def adafactor_stats_(p, g, scratch, batch, rows, cols, eps1) -> None:
  _check(lib().t5x_adafactor_stats(p.data_ptr(), g.data_ptr(), scratch.data_ptr(), batch, rows,
                                   cols, eps1, stream_ptr()), "adafactor_stats")


def adafactor_ema_(v_rvec, v_cvec, scratch, batch, rows, cols, global_rows, global_cols,
                   row_is_normalized, decay, skip_nan) -> None:
  _check(lib().t5x_adafactor_ema(v_rvec.data_ptr(), v_cvec.data_ptr(), scratch.data_ptr(), batch,
                                 rows, cols, global_rows, global_cols, int(row_is_normalized),
                                 decay, int(skip_nan), stream_ptr()), "adafactor_ema")


def adafactor_usq_(g, v_rvec, v_cvec, scratch, batch, rows, cols, global_rows, global_cols,
                   row_is_normalized, use_clip) -> None:
  _check(lib().t5x_adafactor_usq(g.data_ptr(), v_rvec.data_ptr(), v_cvec.data_ptr(),
                                 scratch.data_ptr(), batch, rows, cols, global_rows, global_cols,
                                 int(row_is_normalized), int(use_clip), stream_ptr()),
         "adafactor_usq")


def adafactor_apply_(p, g, m, p_bf16, scratch, batch, rows, cols, n_global, *, lr, eps2,
                     clip_threshold, weight_decay, beta1, max_param_scale, flags, ld_bf16=0,
                     bf16_batch_stride=0) -> None:
  _check(lib().t5x_adafactor_apply(p.data_ptr(), g.data_ptr(), ptr(m), ptr(p_bf16), ld_bf16,
                                   bf16_batch_stride, scratch.data_ptr(), batch, rows, cols,
                                   n_global, lr, eps2, clip_threshold, weight_decay, beta1,
                                   max_param_scale, flags, stream_ptr()), "adafactor_apply")


def adafactor_unfactored_stats_(p, g, v, scratch, batch, n, decay, eps1, skip_nan) -> None:
  _check(lib().t5x_adafactor_unfactored_stats(p.data_ptr(), g.data_ptr(), v.data_ptr(),
                                              scratch.data_ptr(), batch, n, decay, eps1,
                                              int(skip_nan), stream_ptr()),
         "adafactor_unfactored_stats")


def adafactor_unfactored_apply_(p, g, v, m, p_bf16, scratch, batch, rows, cols, n_global, *, lr,
                                eps2, clip_threshold, weight_decay, beta1, max_param_scale, flags,
                                ld_bf16=0, bf16_batch_stride=0) -> None:
  _check(lib().t5x_adafactor_unfactored_apply(
      p.data_ptr(), g.data_ptr(), v.data_ptr(), ptr(m), ptr(p_bf16), ld_bf16, bf16_batch_stride,
      scratch.data_ptr(), batch, rows, cols, n_global, lr, eps2, clip_threshold, weight_decay,
      beta1, max_param_scale, flags, stream_ptr()), "adafactor_unfactored_apply")


# ----------------------------------------------------------------------------
# Dropout (in-kernel counter-based mask)
# ----------------------------------------------------------------------------
c_ull, c_uint = ctypes.c_ulonglong, ctypes.c_uint
register_signature("t5x_dropout_bf16", [c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_ll, c_int,
                                        c_int, c_ull, c_uint, c_float, c_void_p])
register_signature("t5x_dropout_keep_host", [c_ull, c_uint, c_ull, c_float])


def dropout_rows(x: torch.Tensor, rate: float, seed: int, stream_id: int, *, group_rows: int,
                 col_group: int, row_offset: int = 0, out: Optional[torch.Tensor] = None
                 ) -> torch.Tensor:
  """out[r, c] = x[r, c] * keep(key) / (1 - rate) for a 2-D bf16 view x [R, C] with
  key = ((r + row_offset) // group_rows) * ceil(C / col_group) + c // col_group. The mask is a
  pure function of (seed, stream_id, key), so calling this again on a gradient with the same
  three numbers applies the mask of the forward pass."""
  assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.stride(1) == 1
  if out is None:
    out = torch.empty_like(x)
  assert out.shape == x.shape and out.stride(1) == 1
  _check(lib().t5x_dropout_bf16(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1],
                                x.stride(0), out.stride(0), row_offset, group_rows, col_group,
                                seed & ((1 << 64) - 1), stream_id & 0xFFFFFFFF, float(rate),
                                stream_ptr()), "dropout")
  return out


def dropout_keep_host(seed: int, stream_id: int, key: int, rate: float) -> bool:
  """The device generator's keep decision for one key, evaluated on the host."""
  return bool(lib().t5x_dropout_keep_host(seed & ((1 << 64) - 1), stream_id & 0xFFFFFFFF,
                                          int(key), float(rate)))


# ----------------------------------------------------------------------------
# Beam search step, sampling, top-k / top-p masks
# ----------------------------------------------------------------------------
register_signature("t5x_beam_chunks", [c_int])
register_signature("t5x_beam_step", [c_void_p, c_ll, c_int, c_int, c_int, c_int, c_int, c_float,
                                     c_float] + [c_void_p] * 13)
register_signature("t5x_sample_tokens", [c_void_p, c_ll, c_int, c_int, c_void_p, c_float, c_int,
                                         c_void_p, c_float, c_int, c_ull, c_uint, c_void_p,
                                         c_void_p, c_void_p])
register_signature("t5x_topk_topp_mask", [c_void_p, c_ll, c_void_p, c_ll, c_int, c_int, c_int,
                                          c_void_p, c_float, c_float, c_void_p])


class BeamStepScratch:
  """Device scratch of `beam_step` for a fixed (batch, beams, vocab)."""

  def __init__(self, batch: int, beams: int, vocab: int, device):
    s = int(lib().t5x_beam_chunks(vocab))
    rows = batch * beams
    self.f = torch.empty(rows * s * (2 + 2 * beams), dtype=torch.float32, device=device)
    self.i = torch.empty(rows * s * 2 * beams, dtype=torch.int32, device=device)
    self.flags = torch.zeros(batch, dtype=torch.uint8, device=device)
    self.ticket = torch.zeros(1, dtype=torch.int32, device=device)


def beam_step(logits: torch.Tensor, *, batch: int, beams: int, eos_id: int, alpha: float,
              min_brevity: float, live_lp, live_seqs, fin_seqs, fin_scores, fin_flags, ancestry,
              cur, terminated, scratch: BeamStepScratch) -> None:
  """One beam-search step in place (see csrc/beam.cu): `logits` [batch * beams, V] fp32 are
  the logits of the tokens at position `cur` (device int32 scalar, advanced by the call)."""
  assert logits.dtype == torch.float32 and logits.stride(1) == 1
  assert live_seqs.dtype == torch.int64 and fin_seqs.dtype == torch.int64
  assert ancestry.dtype == torch.int32 and cur.dtype == torch.int32
  assert fin_flags.dtype == torch.bool and terminated.dtype == torch.bool
  for t in (live_lp, live_seqs, fin_seqs, fin_scores, fin_flags, ancestry):
    assert t.is_contiguous()
  _check(lib().t5x_beam_step(
      logits.data_ptr(), logits.stride(0), batch, beams, live_seqs.shape[2], logits.shape[1],
      eos_id, float(alpha), float(min_brevity), live_lp.data_ptr(), live_seqs.data_ptr(),
      fin_seqs.data_ptr(), fin_scores.data_ptr(), fin_flags.data_ptr(), ancestry.data_ptr(),
      cur.data_ptr(), terminated.data_ptr(), scratch.f.data_ptr(), scratch.i.data_ptr(),
      scratch.flags.data_ptr(), scratch.ticket.data_ptr(), stream_ptr()), "beam_step")


def _row_array(v, rows: int, device):
  """(device pointer or 0, scalar) for a value that is either a Python number or per row."""
  if isinstance(v, torch.Tensor) and v.dim() > 0:
    t = v.to(device=device, dtype=torch.float32).reshape(-1).contiguous()
    assert t.numel() == rows
    return t, 0.0
  return None, float(v)


def sample_tokens(logits: torch.Tensor, *, temperature, topk: int, topp, rescale_log_probs: bool,
                  seed: int, stream_id: int):
  """(tokens int64 [rows], log_probs fp32 [rows]) drawn from logits [rows, V] fp32 with
  temperature scaling and a top-k or top-p mask (one kernel; csrc/beam.cu)."""
  assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
  rows, v = logits.shape
  t_arr, t_s = _row_array(temperature, rows, logits.device)
  p_arr, p_s = _row_array(topp if topp else 0.0, rows, logits.device)
  tokens = torch.empty(rows, dtype=torch.int64, device=logits.device)
  lps = torch.empty(rows, dtype=torch.float32, device=logits.device)
  _check(lib().t5x_sample_tokens(
      logits.data_ptr(), logits.stride(0), rows, v, ptr(t_arr), t_s, int(topk or 0), ptr(p_arr),
      p_s, int(bool(rescale_log_probs)), seed & ((1 << 64) - 1), stream_id & 0xFFFFFFFF,
      tokens.data_ptr(), lps.data_ptr(), stream_ptr()), "sample_tokens")
  return tokens, lps


def topk_topp_mask(logits: torch.Tensor, topk: int, topp, replace_val: float) -> torch.Tensor:
  """logits with everything outside the top-k / top-p set replaced by `replace_val`."""
  x = logits.reshape(-1, logits.shape[-1])
  x = x if (x.dtype == torch.float32 and x.stride(1) == 1) else x.float().contiguous()
  out = torch.empty_like(x)
  p_arr, p_s = _row_array(topp if topp is not None else 0.0, x.shape[0], x.device)
  _check(lib().t5x_topk_topp_mask(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0),
                                  x.shape[0], x.shape[1], int(topk or 0), ptr(p_arr), p_s,
                                  float(replace_val), stream_ptr()), "topk_topp_mask")
  return out.view(logits.shape)


# ----------------------------------------------------------------------------
# Mixture-of-experts router
# ----------------------------------------------------------------------------
register_signature("t5x_moe_router_parts", [c_int])
register_signature("t5x_moe_router_fwd", [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int] + [c_void_p] * 9)
register_signature("t5x_moe_router_bwd", [c_void_p, c_ll, c_void_p, c_int, c_int, c_int, c_int,
                                          c_int] + [c_void_p] * 9 + [c_ll, c_void_p, c_void_p,
                                                                     c_void_p])
register_signature("t5x_moe_router_dw_tiles", [c_int])

ROUTER_MAX_EXPERTS, ROUTER_MAX_CHOICES = 64, 4


def moe_router_fwd(x: torch.Tensor, w: torch.Tensor, k: int, capacity: int):
  """x [T, d] bf16, w [d, E] fp32 -> dict of probs [T, E], lse [T], index [T, k] (int32),
  gate [T, k] (zero for choices that lost their slot), flat_slot [T, k] (int32, -1 = dropped),
  stats [E, 4], metrics [8] (auxiliary_loss, router_z_loss, fraction_tokens_left_behind,
  expert_usage, router_confidence, tokens dispatched)."""
  assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
  assert w.dtype == torch.float32 and w.is_contiguous()
  t, d = x.shape
  e = w.shape[1]
  dev = x.device
  parts = int(lib().t5x_moe_router_parts(t))
  f32, i32 = dict(dtype=torch.float32, device=dev), dict(dtype=torch.int32, device=dev)
  out = dict(probs=torch.empty(t, e, **f32), lse=torch.empty(t, **f32),
             index=torch.empty(t, k, **i32), gate=torch.empty(t, k, **f32),
             flat_slot=torch.empty(t, k, **i32), stats=torch.empty(e, 4, **f32),
             metrics=torch.zeros(8, **f32))
  part = torch.empty(parts, 1 + e, **f32)
  _check(lib().t5x_moe_router_fwd(
      x.data_ptr(), x.stride(0), w.data_ptr(), t, d, e, k, capacity, out["probs"].data_ptr(),
      out["lse"].data_ptr(), out["index"].data_ptr(), out["gate"].data_ptr(),
      out["flat_slot"].data_ptr(), out["stats"].data_ptr(), out["metrics"].data_ptr(),
      part.data_ptr(), stream_ptr()), "moe_router_fwd")
  return out


def moe_router_bwd(x, w, k: int, capacity: int, fwd: dict, dgate: torch.Tensor,
                   coef: torch.Tensor, need_dx: bool = True):
  """(dx [T, d] bf16 or None, dw [d, E] fp32) from the gate gradients [T, k] and
  coef = [d loss / d auxiliary_loss, d loss / d router_z_loss] (device fp32)."""
  t, d = x.shape
  e = w.shape[1]
  dlogits = torch.empty(t, e, dtype=torch.float32, device=x.device)
  dx = torch.empty(t, d, dtype=torch.bfloat16, device=x.device) if need_dx else None
  dw = torch.empty(d, e, dtype=torch.float32, device=x.device)
  dgate = dgate.float().contiguous()
  dw_part = torch.empty(int(lib().t5x_moe_router_dw_tiles(t)) * d * e, dtype=torch.float32,
                        device=x.device)
  _check(lib().t5x_moe_router_bwd(
      x.data_ptr(), x.stride(0), w.data_ptr(), t, d, e, k, capacity, fwd["probs"].data_ptr(),
      fwd["lse"].data_ptr(), fwd["index"].data_ptr(), fwd["flat_slot"].data_ptr(),
      dgate.data_ptr(), fwd["stats"].data_ptr(), coef.data_ptr(), dlogits.data_ptr(), ptr(dx),
      d, dw.data_ptr(), dw_part.data_ptr(), stream_ptr()), "moe_router_bwd")
  return dx, dw


# ----------------------------------------------------------------------------
# AdamW
# ----------------------------------------------------------------------------
register_signature("t5x_adamw_step", [c_void_p, c_void_p, c_void_p, c_void_p,
                                      ctypes.POINTER(c_void_p), c_int, c_void_p, c_ll, c_float,
                                      c_float, c_float, c_float, c_float, c_float, c_int, c_void_p,
                                      c_void_p])


def adamw_step_(p, g, mu, nu, bf16_out_ptrs, bf16_mc: int = 0, *, lr, b1, b2, eps, eps_root,
                weight_decay, step: int, clip_scale: Optional[torch.Tensor] = None) -> None:
  """One fused AdamW step on a contiguous fp32 parameter (csrc/adamw.cu). `bf16_out_ptrs`: a
  ctypes array of device pointers to the bf16 working copies that receive the new weights;
  `clip_scale`: a one-element device tensor multiplying the gradient, or None."""
  _check(lib().t5x_adamw_step(p.data_ptr(), g.data_ptr(), mu.data_ptr(), nu.data_ptr(),
                              bf16_out_ptrs, len(bf16_out_ptrs), bf16_mc, p.numel(), float(lr),
                              float(b1), float(b2), float(eps), float(eps_root),
                              float(weight_decay), int(step), ptr(clip_scale), stream_ptr()),
         "adamw_step")
