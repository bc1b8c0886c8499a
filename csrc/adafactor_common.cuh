// Types shared by the Adafactor kernels and their NVLink-fused variants.
#pragma once
#include "common.cuh"

namespace t5x {

struct AdafactorScalars {  // per batch element, in scratch
  float psq;   // sum p^2
  float usq;   // sum u^2
  float vsum;  // sum of the normalised second-moment vector (T5X "v_row")
  float pad;
};

struct AfHyper {
  float lr, eps2, clip_threshold, weight_decay, beta1, max_param_scale;
  int multiply_by_parameter_scale, use_clip, use_wd, use_momentum, use_max_scale, skip_nan;
};

__device__ __forceinline__ float af_update_scale(const AdafactorScalars& s, float n,
                                                 const AfHyper& h) {
  float scale = h.lr;
  if (h.multiply_by_parameter_scale) {
    float ps = fmaxf(sqrtf(s.psq / n), h.eps2);
    if (h.use_max_scale) ps = fminf(ps, h.max_param_scale);
    scale *= ps;
  }
  if (h.use_clip) {
    // a NaN anywhere in the update makes its RMS NaN, and max(1, NaN) is NaN in the reference
    // (jnp.maximum): the whole parameter's update is then NaN and, with skip_nan_updates, the
    // whole parameter keeps its value. fmaxf alone would drop the NaN.
    const float rms = sqrtf(s.usq / n) / h.clip_threshold;
    scale /= isnan(rms) ? rms : fmaxf(1.f, rms);
  }
  return scale;
}

inline AfHyper af_hyper(float lr, float eps2, float clip_threshold, float weight_decay, float beta1,
                 float max_param_scale, int flags) {
  AfHyper h;
  h.lr = lr;
  h.eps2 = eps2;
  h.clip_threshold = clip_threshold;
  h.weight_decay = weight_decay;
  h.beta1 = beta1;
  h.max_param_scale = max_param_scale;
  h.multiply_by_parameter_scale = (flags >> 0) & 1;
  h.use_clip = (flags >> 1) & 1;
  h.use_wd = (flags >> 2) & 1;
  h.use_momentum = (flags >> 3) & 1;
  h.use_max_scale = (flags >> 4) & 1;
  h.skip_nan = (flags >> 5) & 1;
  return h;
}

}  // namespace t5x
