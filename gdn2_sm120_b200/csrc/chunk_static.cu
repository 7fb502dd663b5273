// gdn2_chunk_forward_static: the chunk forward for callers that are not allowed to allocate.
//
// Some hosts of this library cannot hand it a freshly allocated workspace: an inference server that
// carves up all device memory once at start-up and forbids any allocator call afterwards, a plugin
// whose enqueue hook runs inside someone else's memory plan, a control loop with a hard latency
// budget where an allocator call (which may synchronise the device) is not acceptable.  For them the
// workspace and scratch of the chunk forward live in a fixed array inside the library image instead.
//
// Consequences the caller must know:
//   * the array has a fixed size: batch * (full_tokens / 64) * heads <= GDN2_STATIC_MAX_CHUNK_HEADS
//     (64), about 9 MiB; larger problems are rejected with GDN2_ERR_TOO_LARGE.  Every GPU that loads
//     the library holds those 9 MiB until the process exits.
//   * the first call on each device looks up the array's device address (a one-off driver query that
//     may load the module); make that first call before starting any stream capture.
//   * all calls on a device share the one array and it keeps whatever the previous call left in it.
//     The status word is cleared at the start of each call; every tile is rewritten before it is
//     read.  Two calls whose kernels overlap on the GPU (different streams, no dependency) race on
//     the array: serialise them.
//   * no cudaMalloc / cudaFree / allocating library routine is called here.

#include <mutex>

#include "chunk_common.cuh"

namespace gdn2 {

int launch_chunk_forward(const void*, const void*, const void*, const void*, const void*, const void*,
                         const float*, void*, float*, float*, uint8_t*, uint8_t*, int64_t, int64_t, int64_t,
                         int64_t, int, int, int, float, int, cudaStream_t);
int64_t chunk_status_offset(int64_t, int64_t, int64_t);

namespace {

constexpr int64_t kStaticMaxChunkHeads = GDN2_STATIC_MAX_CHUNK_HEADS;
// inference workspace (chunk-end decays + status block) followed by the forward scratch tiles
constexpr int64_t kStaticWorkspaceBytes = kStaticMaxChunkHeads * kBlobD + kStatusBytes;
constexpr int64_t kStaticBytes = kStaticWorkspaceBytes + kStaticMaxChunkHeads * (kTileU + kFwdTilesBytes);
static_assert(kStaticWorkspaceBytes % 256 == 0, "the scratch part must keep the array's alignment");

// Device-resident scratch.  In host code this name is only a handle for cudaGetSymbolAddress, never
// a pointer that a kernel may be given.
static __device__ __align__(256) unsigned char g_static_workspace[kStaticBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_device_address[kMaxDevices] = {nullptr};
int64_t g_last_status_offset[kMaxDevices];  // status word of the most recent call's layout; valid once the address is

// Once per device, with that device current: resolve the array's device address.
int static_workspace_for_current_device(unsigned char** out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  if (dev < 0 || dev >= kMaxDevices) return GDN2_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_device_address[dev] == nullptr) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_workspace);
    if (err != cudaSuccess || address == nullptr) {
      record_cuda_error(err);
      return GDN2_ERR_LAUNCH;
    }
    g_device_address[dev] = static_cast<unsigned char*>(address);
  }
  *out = g_device_address[dev];
  return GDN2_OK;
}

}  // namespace
}  // namespace gdn2

extern "C" int gdn2_chunk_forward_static(const void* q, const void* k, const void* v, const void* g,
                                         const void* beta, const void* w, const float* initial_state,
                                         void* out, float* final_state, int64_t batch, int64_t time,
                                         int64_t heads, int64_t full_tokens, int dtype, int g_dtype,
                                         float scale, void* stream) {
  using namespace gdn2;
  if (!q || !k || !v || !g || !beta || !w || !out) return GDN2_ERR_NULL_POINTER;
  if (batch <= 0 || heads <= 0 || time <= 0) return GDN2_ERR_BAD_SHAPE;
  // whole chunks only, or rounded up over a partial last chunk (its missing tokens are identity steps)
  if (full_tokens <= 0 || full_tokens % GDN2_CHUNK != 0 || full_tokens >= time + GDN2_CHUNK) return GDN2_ERR_BAD_RANGE;
  if (!valid_seq_dtype(dtype) || !valid_gate_dtype(g_dtype, dtype)) return GDN2_ERR_BAD_DTYPE;
  // reject anything that does not fit the fixed array (checked without overflow)
  const int64_t n_chunks = full_tokens / GDN2_CHUNK;
  if (batch > kStaticMaxChunkHeads || heads > kStaticMaxChunkHeads || n_chunks > kStaticMaxChunkHeads ||
      batch * heads > kStaticMaxChunkHeads || batch * heads * n_chunks > kStaticMaxChunkHeads)
    return GDN2_ERR_TOO_LARGE;
  const void* need16[] = {q, k, v, g, beta, w, initial_state, out, final_state};
  for (const void* ptr : need16) {
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return GDN2_ERR_ALIGNMENT;
  }
  unsigned char* workspace = nullptr;
  const int st = static_workspace_for_current_device(&workspace);
  if (st != GDN2_OK) return st;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < kMaxDevices) {
      std::lock_guard<std::mutex> lock(g_setup_mutex);
      g_last_status_offset[dev] = chunk_status_offset(batch, full_tokens, heads);
    }
  }
  // same kernels as gdn2_chunk_forward (inference layout); the launcher clears the status word
  return launch_chunk_forward(q, k, v, g, beta, w, initial_state, out, final_state, nullptr, workspace,
                              workspace + kStaticWorkspaceBytes, batch, time, heads, full_tokens, 0, dtype,
                              g_dtype, scale, 0, static_cast<cudaStream_t>(stream));
}

extern "C" int gdn2_chunk_static_read_status(void* stream) {
  using namespace gdn2;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  if (dev < 0 || dev >= kMaxDevices) return GDN2_ERR_DEVICE;
  const unsigned char* base = nullptr;
  int64_t offset = 0;
  {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    base = g_device_address[dev];
    offset = g_last_status_offset[dev];
  }
  if (base == nullptr) return GDN2_ERR_UNSUPPORTED;  // no static call has run on this device yet
  int host = 0;
  err = cudaMemcpyAsync(&host, base + offset, sizeof(int), cudaMemcpyDeviceToHost,
                        static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  return host;
}
