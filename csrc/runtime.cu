// Host runtime shared by all kernels: error strings, the per-device status
// buffer that bounded waits report into, device properties and the tensor-map
// (TMA descriptor) cache.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace t5x {

static thread_local char g_err[512] = {0};

int set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return -1;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  uint64_t w[14];
  bool operator==(const MapKey& o) const { return memcmp(w, o.w, sizeof(w)) == 0; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t v : k.w) {
      h ^= v;
      h *= 1099511628211ull;
    }
    return static_cast<size_t>(h);
  }
};

static std::mutex g_map_mu;
static std::unordered_map<MapKey, CUtensorMap*, MapKeyHash> g_maps;

const CUtensorMap* get_tensor_map(const void* base, int elem_bytes, int rank, const uint64_t* dims,
                                  const uint64_t* strides_bytes, const uint32_t* box,
                                  int swizzle_128b) {
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.w[0] = reinterpret_cast<uint64_t>(base);
  key.w[1] = (static_cast<uint64_t>(elem_bytes) << 32) | (static_cast<uint64_t>(rank) << 8) |
             static_cast<uint64_t>(swizzle_128b);
  for (int i = 0; i < rank; ++i) {
    key.w[2 + i] = dims[i];
    key.w[6 + i] = (i > 0) ? strides_bytes[i - 1] : 0;
    key.w[10 + i] = box[i];
  }
  std::lock_guard<std::mutex> lk(g_map_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) return it->second;

  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return nullptr;
  }
  if ((reinterpret_cast<uint64_t>(base) & 15) != 0) {
    set_error("tensor map base %p is not 16-byte aligned", base);
    return nullptr;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstr[5];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      gstr[i - 1] = strides_bytes[i - 1];
      if (gstr[i - 1] % 16 != 0) {
        set_error("tensor map stride %llu is not a multiple of 16 bytes",
                  (unsigned long long)gstr[i - 1]);
        return nullptr;
      }
    }
  }
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUtensorMap* m = new CUtensorMap;
  CUresult r = enc(m, dt, rank, const_cast<void*>(base), gdims, gstr, gbox, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    delete m;
    set_error("cuTensorMapEncodeTiled failed with %d (rank %d, dims %llu x %llu, box %u x %u)",
              (int)r, rank, (unsigned long long)dims[0],
              (unsigned long long)(rank > 1 ? dims[1] : 1), box[0], rank > 1 ? box[1] : 1);
    return nullptr;
  }
  if (g_maps.size() > 65536) {  // unbounded growth guard: descriptors are cheap to rebuild
    for (auto& kv : g_maps) delete kv.second;
    g_maps.clear();
  }
  g_maps.emplace(key, m);
  return m;
}

struct DeviceState {
  int* status = nullptr;
  int sms = 0;
};
static std::mutex g_dev_mu;
static DeviceState g_dev[64];

static DeviceState& dev_state() {
  int d = 0;
  cudaGetDevice(&d);
  std::lock_guard<std::mutex> lk(g_dev_mu);
  DeviceState& s = g_dev[d];
  if (s.status == nullptr) {
    cudaMalloc(&s.status, kStatusWords * sizeof(int));
    cudaMemset(s.status, 0, kStatusWords * sizeof(int));
    cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, d);
  }
  return s;
}

static std::atomic<long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launches() { return g_launches.load(std::memory_order_relaxed); }

int* device_status_buffer() { return dev_state().status; }
int num_sms() { return dev_state().sms; }

}  // namespace t5x

T5X_API const char* t5x_last_error() { return t5x::g_err; }

// Copies the status words of the current device to `out` (kStatusWords ints)
// after synchronising `stream`, then clears them. Returns the status code.
T5X_API int t5x_read_status(int* out, void* stream) {
  int* s = t5x::device_status_buffer();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int host[t5x::kStatusWords];
  if (cudaMemcpyAsync(host, s, sizeof(host), cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return t5x::set_error("status copy failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (cudaStreamSynchronize(st) != cudaSuccess)
    return t5x::set_error("stream sync failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (host[0] != 0) cudaMemsetAsync(s, 0, sizeof(host), st);
  if (out) memcpy(out, host, sizeof(host));
  return host[0];
}

// Enqueues, on `stream`, a copy of the status words to `host_dst` (kStatusWords ints of pinned
// host memory) and returns at once. The caller reads `host_dst` after an event recorded behind
// this call has completed; the words are not cleared. A training loop uses this to notice a
// kernel that gave up on a wait without stalling its launch queue.
T5X_API int t5x_status_copy_async(int* host_dst, void* stream) {
  if (host_dst == nullptr) return t5x::set_error("status copy: null destination");
  int* s = t5x::device_status_buffer();
  if (cudaMemcpyAsync(host_dst, s, t5x::kStatusWords * sizeof(int), cudaMemcpyDeviceToHost,
                      static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return t5x::set_error("status copy failed: %s", cudaGetErrorString(cudaGetLastError()));
  return 0;
}

// Number of kernels this library has launched in this process (all devices).
T5X_API long long t5x_launch_count() { return t5x::launches(); }

namespace t5x {
static thread_local int g_chained = 0;  // per host thread: only the caller's launches change
bool chained_launches() { return g_chained != 0; }
bool chained_launches_constant_b() { return g_chained == 2; }
}  // namespace t5x
// Applies to the calling host thread. 0 (default): ordinary launches. 1: kernels that support it are launched as programmatic
// dependents of their predecessor on the stream (their prologue overlaps its tail). 2: as 1,
// and the caller promises that the B operand of every GEMM it issues is constant (weights that
// no kernel in flight writes), so that the GEMMs request B before they wait for the predecessor.
T5X_API int t5x_set_chained_launches(int level) {
  t5x::g_chained = level < 0 ? 0 : (level > 2 ? 2 : level);
  return 0;
}

T5X_API int t5x_num_sms() { return t5x::num_sms(); }
T5X_API int t5x_abi_version() { return 1; }
