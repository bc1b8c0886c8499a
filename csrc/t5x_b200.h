/* Public C declarations of libt5x_b200.so that are meant to be called without the Python
 * package. All pointers are device pointers; `stream` is a cudaStream_t passed as void*.
 * Every function returns 0 on success and a negative value after recording a message that
 * t5x_last_error() returns. */
#ifndef T5X_B200_H_
#define T5X_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

const char* t5x_last_error(void);

/* Number of fp32 scratch values t5x_adafactor_factored needs for a [batch, rows, cols]
 * parameter. */
long long t5x_adafactor_scratch_floats(int batch, int rows, int cols);

/* Factored Adafactor update of an fp32 parameter p[batch, rows, cols] with gradient g; the
 * caller provides `scratch` (t5x_adafactor_scratch_floats values). v_rvec[batch, rows] and
 * v_cvec[batch, cols] are the second-moment vectors, m an optional momentum buffer, p_bf16 an
 * optional bf16 copy of the updated parameter. `flags` is a bit set: 1 multiply by parameter
 * scale, 2 RMS clipping, 4 weight decay, 8 momentum, 16 cap the parameter scale, 32 skip NaN
 * updates. */
int t5x_adafactor_factored(void* p, const void* g, void* v_rvec, void* v_cvec, void* m,
                           void* p_bf16, long long ld_bf16, long long bf16_batch_stride,
                           void* scratch, int batch, int rows, int cols, int row_is_normalized,
                           float lr, float decay, float eps1, float eps2, float clip_threshold,
                           float weight_decay, float beta1, float max_param_scale, int flags,
                           void* stream);

/* The same update for callers that cannot allocate device memory. (This entry point has no
 * counterpart in the reference framework; it exists for embedders of this library.)
 *
 * Who needs it: a host program that gave the whole device heap to its own pool or arena and
 * must not see a cudaMalloc behind its back; code that steps the optimizer from a callback or
 * a latency-critical section where cudaMalloc/cudaFree are off limits because they
 * synchronise the device; a plain C or C++ program that links this library without a tensor
 * library to allocate with. Instead of a caller buffer, the scratch is one fixed array inside
 * the library's device image.
 *
 * Rules of use:
 *  - Limit: t5x_adafactor_scratch_floats(batch, rows, cols) must not exceed
 *    t5x_adafactor_factored_static_max_floats() (1 Mi floats = 4 MiB; e.g. one 4096 x 10240
 *    matrix needs 28,676). Larger requests are rejected with an error and nothing runs. Every
 *    GPU that loads the library holds those 4 MiB until the process exits.
 *  - It calls no cudaMalloc, cudaFree or other allocating routine; inputs and outputs are
 *    still the caller's.
 *  - The first call on each device looks up the array's device address and the SM count and
 *    caches them. Make that first call with the device current and before any stream
 *    capture begins.
 *  - All calls on a device share the one array, and the array keeps the previous call's
 *    contents (the entry point clears what has to start at zero). Two calls whose kernels can
 *    overlap on the GPU - different streams without an ordering between them - race on it;
 *    issue them on one stream or order them with events. */
long long t5x_adafactor_factored_static_max_floats(void);
int t5x_adafactor_factored_static(void* p, const void* g, void* v_rvec, void* v_cvec, void* m,
                                  void* p_bf16, long long ld_bf16, long long bf16_batch_stride,
                                  int batch, int rows, int cols, int row_is_normalized, float lr,
                                  float decay, float eps1, float eps2, float clip_threshold,
                                  float weight_decay, float beta1, float max_param_scale,
                                  int flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* T5X_B200_H_ */
