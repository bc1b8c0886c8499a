"""The allocation-free Adafactor entry point, called through its exported C symbol.

`t5x_adafactor_factored_static` serves embedders that cannot allocate device memory when they
step the optimizer (a host that owns the whole device heap through its own pool, a callback in
which cudaMalloc is off limits because it synchronises the device, a C program with no tensor
library): its scratch is a fixed array inside the library instead of a caller buffer. This test
drives it the way such a caller would - raw device pointers through ctypes - twice in a row
(the second call meets the first call's leftovers in the shared scratch) and checks the
parameter, both second-moment vectors and the bf16 copy against the caller-scratch entry
point, and that an oversized request is refused with a message. It sits in a file that pytest
collects last so that a failure here cannot hide the other tests of a stop-at-first-failure run.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "t5x_b200", "lib",
                   "libt5x_b200.so")
vp, ci, cl, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _lib():
  lib = ctypes.CDLL(LIB)
  lib.t5x_last_error.restype = ctypes.c_char_p
  lib.t5x_adafactor_scratch_floats.restype = cl
  lib.t5x_adafactor_scratch_floats.argtypes = [ci, ci, ci]
  lib.t5x_adafactor_factored_static_max_floats.restype = cl
  lib.t5x_adafactor_factored.argtypes = [vp, vp, vp, vp, vp, vp, cl, cl, vp, ci, ci, ci, ci] + \
      [cf] * 8 + [ci, vp]
  lib.t5x_adafactor_factored_static.argtypes = [vp, vp, vp, vp, vp, vp, cl, cl, ci, ci, ci, ci] + \
      [cf] * 8 + [ci, vp]
  return lib


def rel(a, b):
  a, b = a.float(), b.float()
  return ((a - b).norm() / (b.norm() + 1e-12)).item()


def test_static_scratch_entry_point_matches_caller_scratch_twice():
  lib = _lib()
  torch.manual_seed(11)
  R, C = 768, 2048
  flags = 1 | 2  # parameter scale + RMS clipping
  hyper = (0.01, 0.8, 1e-30, 1e-3, 1.0, 0.0, 0.0, 0.0)
  stream = torch.cuda.current_stream().cuda_stream

  def fresh():
    p = torch.randn(R, C, device="cuda") * 0.05
    vr = torch.rand(R, device="cuda") * 1e-4
    vc = torch.rand(C, device="cuda") * 1e-4
    pb = torch.zeros(R, C, device="cuda", dtype=torch.bfloat16)
    return p, vr, vc, pb

  p_a, vr_a, vc_a, pb_a = fresh()
  p_b, vr_b, vc_b, pb_b = (t.clone() for t in (p_a, vr_a, vc_a, pb_a))
  scratch = torch.empty(lib.t5x_adafactor_scratch_floats(1, R, C), device="cuda")
  assert scratch.numel() <= lib.t5x_adafactor_factored_static_max_floats()
  for call in range(2):
    g = torch.randn(R, C, device="cuda") * 0.01
    rc = lib.t5x_adafactor_factored(p_a.data_ptr(), g.data_ptr(), vr_a.data_ptr(),
                                    vc_a.data_ptr(), None, pb_a.data_ptr(), C, 0,
                                    scratch.data_ptr(), 1, R, C, 1, *hyper, flags, stream)
    assert rc == 0, lib.t5x_last_error().decode()
    rc = lib.t5x_adafactor_factored_static(p_b.data_ptr(), g.data_ptr(), vr_b.data_ptr(),
                                           vc_b.data_ptr(), None, pb_b.data_ptr(), C, 0, 1, R, C,
                                           1, *hyper, flags, stream)
    assert rc == 0, lib.t5x_last_error().decode()
    torch.cuda.synchronize()
    assert rel(p_b, p_a) < 1e-5, f"call {call}: parameter differs"
    assert rel(vr_b, vr_a) < 1e-5 and rel(vc_b, vc_a) < 1e-5, f"call {call}: moments differ"
    assert rel(pb_b, pb_a) < 4e-3, f"call {call}: bf16 copy differs"
    assert bool(torch.isfinite(p_b).all())


def test_static_scratch_entry_point_rejects_oversized_request():
  lib = _lib()
  limit = lib.t5x_adafactor_factored_static_max_floats()
  R = C = 300_000  # 2 * (R + C) + 4 floats > 1 Mi
  assert lib.t5x_adafactor_scratch_floats(1, R, C) > limit
  dummy = torch.zeros(8, device="cuda")
  rc = lib.t5x_adafactor_factored_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                         dummy.data_ptr(), None, None, 0, 0, 1, R, C, 1, 0.01, 0.8,
                                         1e-30, 1e-3, 1.0, 0.0, 0.0, 0.0, 3,
                                         torch.cuda.current_stream().cuda_stream)
  assert rc != 0
  assert b"scratch" in lib.t5x_last_error()
