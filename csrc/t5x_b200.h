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
 * updates. p, g, v_rvec and v_cvec must not be null and m must not be null when flag 8 is
 * set (the call is rejected otherwise); p and g need only 4-byte alignment (16-byte aligned
 * pointers with cols % 4 == 0 take the faster 16-byte loads). */
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

/* ---- GEMM (tcgen05): C[batch, M, N] (+)= alpha * A[batch, M, K] @ B[batch, K, N] ----
 * bf16 operands, fp32 accumulation; leading dimensions and batch strides in elements.
 * a_mn_major / b_mn_major: 0 = the contraction dim is contiguous, 1 = the M (N) dim is.
 * out_fp32: C is fp32 (else bf16); accumulate: 0 store, 1 add to C, 2 add atomically (several
 * K slices as batches into one C). epilogue: 0 plain, 1 gated GELU (C = gelu(A B) * (A B2),
 * optional copies of both products in H0 / H1), 2 add the bf16 matrix R. */
int t5x_gemm_bf16(const void* A, const void* B, const void* B2, void* C, int M, int N, int K,
                  int batch, long long lda, long long ldb, long long ldc,
                  long long a_batch_stride, long long b_batch_stride, long long c_batch_stride,
                  int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int epilogue,
                  const void* R, long long ldr, long long r_batch_stride, void* H0, void* H1,
                  long long ldh, float alpha, int max_ctas, void* stream);

/* ---- tensor parallelism with the collective inside the GEMM kernel ----
 * The M rows are split evenly over `world` ranks (rows_per_rank each). Peer pointers are the
 * other ranks' buffers as mapped into this process (symmetric memory).
 *
 * Ordering between ranks is carried by signal words instead of barrier kernels: every rank
 * owns 32 uint32 (zero at start) that all ranks map (sig_local = this rank's own,
 * sig_peers[r] = rank r's as mapped here), and every call of either GEMM takes an `epoch` one
 * larger than the previous call on the group; all ranks make the same calls in the same order.
 * exit_count: one zeroed uint32 of this GPU's memory shared by both GEMMs.
 *
 * all-gather -> GEMM: A is this rank's [M, K] buffer with only block `rank` filled; the kernel
 * announces that, waits for each peer's announcement and pulls block r from a_peers[r] (same
 * layout) while it multiplies. `flags`: t5x_gemm_allgather_flag_words(world, rows_per_rank)
 * uint32 of this GPU's memory, zero on entry and on exit. K % 32 == 0. epilogue 0 or 1.
 *
 * GEMM -> reduce-scatter: the bf16 partial product (+ R) is stored row block by row block to
 * c_peers[r], this rank's slot [rows_per_rank, ldc] of rank r's inbox; the kernel then raises
 * this rank's "scattered" signal. The owner adds its `world` slots with
 * t5x_slot_sum_wait_bf16 (sig = sig_local + 16), which first waits for every peer's signal of
 * that epoch. Successive calls must alternate between two inboxes. */
int t5x_gemm_allgather_flag_words(int world, int rows_per_rank);
int t5x_gemm_allgather_bf16(void* A, const void* const* a_peers, int world, int rank,
                            int rows_per_rank, void* flags, const void* B, const void* B2,
                            void* C, int M, int N, int K, long long ldb, long long ldc,
                            int b_mn_major, int epilogue, void* H0, void* H1, long long ldh,
                            void* sig_local, void* const* sig_peers, unsigned int epoch,
                            void* exit_count, void* stream);
int t5x_gemm_reducescatter_bf16(const void* A, const void* B, void* const* c_peers, int world,
                                int rank, int rows_per_rank, int M, int N, int K, long long lda,
                                long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                                const void* R, long long ldr, void* sig_local,
                                void* const* sig_peers, unsigned int epoch, void* exit_count,
                                void* stream);
int t5x_slot_sum_bf16(const void* slots, int num_slots, long long n, const void* residual,
                      void* dst, void* stream);
int t5x_slot_sum_wait_bf16(const void* slots, int num_slots, long long n, const void* residual,
                           void* dst, const void* sig, int world, int rank, unsigned int epoch,
                           void* stream);

/* Stream-ordered barrier over `world` ranks through signal pads (one per rank, as mapped
 * here; (channel + 1) * 16 uint32 each, zero at start). `epoch` >= 1 and increasing per
 * channel. A rank that never arrives makes the wait give up after `spin_limit` polls and
 * records a status (t5x_read_status) instead of hanging. */
int t5x_comm_barrier(const void* const* pads, int rank, int world, int channel,
                     unsigned int epoch, unsigned long long spin_limit, void* stream);

/* Synchronises `stream` and copies the device status words (kernel id, reason, indices) to
 * `words[8]`; returns the reason code (0 = none) and clears it. */
int t5x_read_status(int* words, void* stream);

/* The same words copied to `host_dst` (8 ints of pinned host memory) by an asynchronous copy
 * enqueued on `stream`; nothing is synchronised or cleared. Read `host_dst` once an event
 * recorded after this call has completed. */
int t5x_status_copy_async(int* host_dst, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* T5X_B200_H_ */
