// extern "C" entry points of libgdn2_b200.so: argument validation + kernel launches.
// No allocation, no synchronisation, no exceptions cross this boundary.

#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <mutex>

#include "common.cuh"

namespace gdn2 {

// launchers defined next to their kernels
int launch_token_forward(const void*, const void*, const void*, const void*, const void*,
                         const void*, const float*, void*, float*, float*, int64_t, int64_t,
                         int64_t, int64_t, int64_t, int, int, float, int, cudaStream_t);
int launch_token_t1_zero(const void*, const void*, const void*, const void*, void*, float*,
                         int64_t, int64_t, int, float, int, cudaStream_t);
int launch_token_dstate_scan(const void*, const void*, const void*, const void*, const void*,
                             const float*, float*, float*, int64_t, int64_t, int64_t, int64_t,
                             int64_t, int, int, float, cudaStream_t);
int launch_token_chunk_vjp(const void*, const void*, const void*, const void*, const void*,
                           const void*, const void*, const float*, const float*, void*, void*,
                           void*, void*, void*, void*, int64_t, int64_t, int64_t, int64_t,
                           int64_t, int, int, float, cudaStream_t);

int64_t chunk_workspace_bytes(int64_t, int64_t, int64_t, int);
int64_t chunk_scratch_bytes(int64_t, int64_t, int64_t, int);
int64_t chunk_status_offset(int64_t, int64_t, int64_t);
int launch_chunk_forward(const void*, const void*, const void*, const void*, const void*, const void*,
                         const float*, void*, float*, float*, uint8_t*, uint8_t*, int64_t, int64_t, int64_t,
                         int64_t, int, int, int, float, int, cudaStream_t);

int launch_chunk_backward(const void*, const void*, const void*, const void*, const void*, const void*,
                          const void*, const float*, const float*, float*, const uint8_t*, uint8_t*, void*,
                          void*, void*, void*, void*, void*, float*, int64_t, int64_t, int64_t, int64_t, int,
                          int, float, int, cudaStream_t);
int launch_debug_wait_expires(int* status, uint32_t max_polls, cudaStream_t stream);
int launch_gate_prologue(const void*, const void*, const void*, const void*, const void*, void*, void*, void*,
                         void*, void*, float*, float*, int64_t, int, int, cudaStream_t);
int launch_gate_prologue_vjp(const void*, const void*, const void*, const void*, const void*, const float*,
                             const float*, const void*, const void*, const void*, const void*, const void*,
                             void*, void*, void*, void*, void*, int64_t, int, int, cudaStream_t);

namespace {
thread_local char g_cuda_error[256] = {0};
}

void record_cuda_error(cudaError_t err) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", cudaGetErrorName(err),
                cudaGetErrorString(err));
}

// ---- optional per-kernel timing of the chunk entry points -----------------------------------------
// Events 0..2 bracket the two kernels of gdn2_chunk_forward, 3..5 those of gdn2_chunk_backward.
// One event set per device (events belong to the device that was current when they were created),
// all state behind one mutex; meant for one measuring thread per device.
namespace {
constexpr int kProfileDevices = 64;
struct ProfileSet {
  cudaEvent_t events[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  bool recorded[2] = {false, false};
};
bool g_profile_on = false;
ProfileSet g_profile[kProfileDevices];
std::mutex g_profile_mutex;
}  // namespace

void profile_mark(int index, cudaStream_t stream) {
  if (!g_profile_on) return;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kProfileDevices) return;
  std::lock_guard<std::mutex> lock(g_profile_mutex);
  ProfileSet& set = g_profile[device];
  if (set.events[index] == nullptr && cudaEventCreate(&set.events[index]) != cudaSuccess) return;
  if (cudaEventRecord(set.events[index], stream) != cudaSuccess) {
    (void)cudaGetLastError();
    set.recorded[index / 3] = false;
    return;
  }
  if (index == 0) set.recorded[0] = false;
  if (index == 3) set.recorded[1] = false;
  if (index == 2) set.recorded[0] = true;
  if (index == 5) set.recorded[1] = true;
}

// Opt a kernel in to more than 48 KiB of dynamic shared memory, once per (kernel, device): launches
// after the first make no attribute call (cheaper, and nothing but the launch itself happens on the
// stream's behalf, which keeps the entry points usable under stream capture).
namespace {
struct SmemOptIn { const void* kernel; uint64_t devices; int bytes; };
SmemOptIn g_smem_opt_in[64];
int g_smem_opt_in_count = 0;
std::mutex g_smem_opt_in_mutex;
}  // namespace

cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  const uint64_t bit = 1ull << (device & 63);
  std::lock_guard<std::mutex> lock(g_smem_opt_in_mutex);
  SmemOptIn* entry = nullptr;
  for (int i = 0; i < g_smem_opt_in_count; ++i) {
    if (g_smem_opt_in[i].kernel == kernel) { entry = &g_smem_opt_in[i]; break; }
  }
  if (entry != nullptr && (entry->devices & bit) != 0 && entry->bytes >= bytes) return cudaSuccess;
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (err != cudaSuccess) return err;
  if (entry == nullptr && g_smem_opt_in_count < 64) {
    entry = &g_smem_opt_in[g_smem_opt_in_count++];
    *entry = SmemOptIn{kernel, 0, bytes};
  }
  if (entry != nullptr) {
    if (entry->bytes != bytes) { entry->bytes = bytes; entry->devices = 0; }
    entry->devices |= bit;
  }
  return cudaSuccess;
}

int check_launch() {
  const cudaError_t err = cudaGetLastError();
  if (err == cudaSuccess) return GDN2_OK;
  record_cuda_error(err);
  return GDN2_ERR_LAUNCH;
}

namespace {

inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

int check_shape(int64_t B, int64_t T, int64_t H) {
  if (B <= 0 || H <= 0 || T < 0) return GDN2_ERR_BAD_SHAPE;
  // element offsets are 64-bit, but keep every product representable
  const int64_t limit = int64_t(1) << 46;
  if (B > limit || H > limit || T > limit) return GDN2_ERR_TOO_LARGE;
  if (B * H > limit || (T > 0 && B * H > limit / T)) return GDN2_ERR_TOO_LARGE;
  return GDN2_OK;
}

int check_range(int64_t T, int64_t t_begin, int64_t t_end) {
  if (t_begin < 0 || t_end < t_begin || t_end > T) return GDN2_ERR_BAD_RANGE;
  return GDN2_OK;
}

int check_types(int dtype, int g_dtype) {
  if (!valid_seq_dtype(dtype) || !valid_gate_dtype(g_dtype, dtype)) return GDN2_ERR_BAD_DTYPE;
  return GDN2_OK;
}

}  // namespace
}  // namespace gdn2

using namespace gdn2;

extern "C" {

int gdn2_version(void) { return 200; /* 0.2.0: row-major WY tiles, scratch kinds */ }

const char* gdn2_status_string(int status) {
  switch (status) {
    case GDN2_OK: return "ok";
    case GDN2_ERR_NULL_POINTER: return "a required pointer is NULL";
    case GDN2_ERR_BAD_SHAPE: return "batch and heads must be positive and time non-negative";
    case GDN2_ERR_BAD_DTYPE: return "unsupported dtype code (q/k/v/beta/w: bf16 or fp16; g: same or fp32)";
    case GDN2_ERR_BAD_RANGE: return "token range must satisfy 0 <= t_begin <= t_end <= T";
    case GDN2_ERR_ALIGNMENT: return "a pointer does not satisfy the required alignment";
    case GDN2_ERR_UNSUPPORTED: return "shape or option not supported by this entry point";
    case GDN2_ERR_LAUNCH: return "CUDA reported an error at launch (see gdn2_last_cuda_error)";
    case GDN2_ERR_DEVICE: return "the current device is not a compute-capability 10.x GPU";
    case GDN2_ERR_TOO_LARGE: return "problem size exceeds the launch grid or 64-bit index budget";
    default: return "unknown status";
  }
}

const char* gdn2_last_cuda_error(void) { return g_cuda_error; }

int gdn2_device_supported(void) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  int major = 0;
  err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  return major == 10 ? 1 : 0;
}

namespace {
inline bool valid_prologue(int prologue) {
  return (prologue & ~(GDN2_PROLOGUE_NORMALIZE_QK | GDN2_PROLOGUE_ACTIVATE_GATES)) == 0;
}

int token_forward_checked(const void* q, const void* k, const void* v, const void* g, const void* beta,
                          const void* w, const float* initial_state, void* out, float* final_state,
                          float* boundaries, int64_t batch, int64_t time, int64_t heads, int64_t t_begin,
                          int64_t t_end, int dtype, int g_dtype, float scale, int prologue, void* stream) {
  if (!q || !k || !v || !g || !beta || !w || !out) return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, time, heads);
  if (st != GDN2_OK) return st;
  if ((st = check_range(time, t_begin, t_end)) != GDN2_OK) return st;
  if ((st = check_types(dtype, g_dtype)) != GDN2_OK) return st;
  if (!valid_prologue(prologue)) return GDN2_ERR_UNSUPPORTED;
  if (!aligned(initial_state, 4) || !aligned(final_state, 4) || !aligned(boundaries, 4))
    return GDN2_ERR_ALIGNMENT;
  return launch_token_forward(q, k, v, g, beta, w, initial_state, out, final_state, boundaries,
                              batch, time, heads, t_begin, t_end, dtype, g_dtype, scale, prologue,
                              static_cast<cudaStream_t>(stream));
}

int token_t1_zero_checked(const void* q, const void* k, const void* v, const void* w, void* out,
                          float* final_state, int64_t batch, int64_t heads, int dtype, float scale,
                          int prologue, void* stream) {
  if (!q || !k || !v || !w || !out || !final_state) return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, 1, heads);
  if (st != GDN2_OK) return st;
  if (!valid_seq_dtype(dtype)) return GDN2_ERR_BAD_DTYPE;
  if (!valid_prologue(prologue)) return GDN2_ERR_UNSUPPORTED;
  if (!aligned(final_state, 4)) return GDN2_ERR_ALIGNMENT;
  return launch_token_t1_zero(q, k, v, w, out, final_state, batch, heads, dtype, scale, prologue,
                              static_cast<cudaStream_t>(stream));
}
}  // namespace

int gdn2_token_forward(const void* q, const void* k, const void* v, const void* g,
                       const void* beta, const void* w, const float* initial_state, void* out,
                       float* final_state, float* boundaries, int64_t batch, int64_t time,
                       int64_t heads, int64_t t_begin, int64_t t_end, int dtype, int g_dtype,
                       float scale, void* stream) {
  return token_forward_checked(q, k, v, g, beta, w, initial_state, out, final_state, boundaries, batch, time,
                               heads, t_begin, t_end, dtype, g_dtype, scale, 0, stream);
}

int gdn2_token_forward_fused(const void* q, const void* k, const void* v, const void* g,
                             const void* beta, const void* w, const float* initial_state, void* out,
                             float* final_state, int64_t batch, int64_t time, int64_t heads,
                             int64_t t_begin, int64_t t_end, int dtype, int g_dtype, float scale,
                             int prologue, void* stream) {
  return token_forward_checked(q, k, v, g, beta, w, initial_state, out, final_state, nullptr, batch, time,
                               heads, t_begin, t_end, dtype, g_dtype, scale, prologue, stream);
}

int gdn2_token_forward_t1_zero(const void* q, const void* k, const void* v, const void* w,
                               void* out, float* final_state, int64_t batch, int64_t heads,
                               int dtype, float scale, void* stream) {
  return token_t1_zero_checked(q, k, v, w, out, final_state, batch, heads, dtype, scale, 0, stream);
}

int gdn2_token_forward_t1_zero_fused(const void* q, const void* k, const void* v, const void* w,
                                     void* out, float* final_state, int64_t batch, int64_t heads,
                                     int dtype, float scale, int prologue, void* stream) {
  return token_t1_zero_checked(q, k, v, w, out, final_state, batch, heads, dtype, scale, prologue, stream);
}

int gdn2_token_dstate_scan(const void* q, const void* k, const void* g, const void* beta,
                           const void* d_out, const float* d_final_state, float* d_boundaries,
                           float* d_initial_state, int64_t batch, int64_t time, int64_t heads,
                           int64_t t_begin, int64_t t_end, int dtype, int g_dtype, float scale,
                           void* stream) {
  if (!q || !k || !g || !beta || !d_out || !d_boundaries) return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, time, heads);
  if (st != GDN2_OK) return st;
  if ((st = check_range(time, t_begin, t_end)) != GDN2_OK) return st;
  if ((st = check_types(dtype, g_dtype)) != GDN2_OK) return st;
  if (!aligned(d_final_state, 4) || !aligned(d_boundaries, 4) || !aligned(d_initial_state, 4))
    return GDN2_ERR_ALIGNMENT;
  return launch_token_dstate_scan(q, k, g, beta, d_out, d_final_state, d_boundaries,
                                  d_initial_state, batch, time, heads, t_begin, t_end, dtype,
                                  g_dtype, scale, static_cast<cudaStream_t>(stream));
}

int gdn2_token_chunk_vjp(const void* q, const void* k, const void* v, const void* g,
                         const void* beta, const void* w, const void* d_out,
                         const float* boundaries, const float* d_boundaries, void* dq, void* dk,
                         void* dv, void* dg, void* dbeta, void* dw, int64_t batch, int64_t time,
                         int64_t heads, int64_t t_begin, int64_t t_end, int dtype, int g_dtype,
                         float scale, void* stream) {
  if (!q || !k || !v || !g || !beta || !w || !d_out || !boundaries || !d_boundaries || !dq ||
      !dk || !dv || !dg || !dbeta || !dw)
    return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, time, heads);
  if (st != GDN2_OK) return st;
  if ((st = check_range(time, t_begin, t_end)) != GDN2_OK) return st;
  if ((st = check_types(dtype, g_dtype)) != GDN2_OK) return st;
  if (!aligned(boundaries, 16) || !aligned(d_boundaries, 16)) return GDN2_ERR_ALIGNMENT;
  if (t_begin == t_end) return GDN2_OK;
  return launch_token_chunk_vjp(q, k, v, g, beta, w, d_out, boundaries, d_boundaries, dq, dk, dv,
                                dg, dbeta, dw, batch, time, heads, t_begin, t_end, dtype,
                                g_dtype, scale, static_cast<cudaStream_t>(stream));
}

int64_t gdn2_chunk_workspace_bytes(int64_t batch, int64_t full_tokens, int64_t heads, int training) {
  if (batch <= 0 || heads <= 0 || full_tokens <= 0 || full_tokens % GDN2_CHUNK != 0) return GDN2_ERR_BAD_SHAPE;
  if (check_shape(batch, full_tokens, heads) != GDN2_OK) return GDN2_ERR_TOO_LARGE;
  return chunk_workspace_bytes(batch, full_tokens, heads, training);
}

int64_t gdn2_chunk_scratch_bytes(int64_t batch, int64_t full_tokens, int64_t heads, int kind) {
  if (batch <= 0 || heads <= 0 || full_tokens <= 0 || full_tokens % GDN2_CHUNK != 0) return GDN2_ERR_BAD_SHAPE;
  if (kind < 0 || kind > 2) return GDN2_ERR_BAD_SHAPE;
  if (check_shape(batch, full_tokens, heads) != GDN2_OK) return GDN2_ERR_TOO_LARGE;
  return chunk_scratch_bytes(batch, full_tokens, heads, kind);
}

namespace {
int chunk_forward_checked(const void* q, const void* k, const void* v, const void* g, const void* beta,
                          const void* w, const float* initial_state, void* out, float* final_state,
                          float* chunk_boundaries, void* workspace, void* scratch, int64_t batch, int64_t time,
                          int64_t heads, int64_t full_tokens, int training, int dtype, int g_dtype, float scale,
                          int prologue, void* stream) {
  if (!q || !k || !v || !g || !beta || !w || !out || !workspace || !scratch) return GDN2_ERR_NULL_POINTER;
  if (training && !chunk_boundaries) return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, time, heads);
  if (st != GDN2_OK) return st;
  // whole chunks only, or rounded up over a partial last chunk (its missing tokens are identity steps)
  if (full_tokens <= 0 || full_tokens % GDN2_CHUNK != 0 || full_tokens >= time + GDN2_CHUNK) return GDN2_ERR_BAD_RANGE;
  if ((st = check_types(dtype, g_dtype)) != GDN2_OK) return st;
  // the fused prologue is a forward-only feature: backward differentiates the activated tensors
  if (!valid_prologue(prologue) || (prologue != 0 && training)) return GDN2_ERR_UNSUPPORTED;
  const void* need16[] = {q, k, v, g, beta, w, initial_state, out, final_state, chunk_boundaries, workspace,
                          scratch};
  for (const void* ptr : need16) {
    if (!aligned(ptr, 16)) return GDN2_ERR_ALIGNMENT;
  }
  return launch_chunk_forward(q, k, v, g, beta, w, initial_state, out, final_state, chunk_boundaries,
                              static_cast<uint8_t*>(workspace), static_cast<uint8_t*>(scratch), batch, time,
                              heads, full_tokens, training, dtype, g_dtype, scale, prologue,
                              static_cast<cudaStream_t>(stream));
}
}  // namespace

int gdn2_chunk_forward(const void* q, const void* k, const void* v, const void* g,
                       const void* beta, const void* w, const float* initial_state, void* out,
                       float* final_state, float* chunk_boundaries, void* workspace, void* scratch,
                       int64_t batch, int64_t time, int64_t heads, int64_t full_tokens, int training,
                       int dtype, int g_dtype, float scale, void* stream) {
  return chunk_forward_checked(q, k, v, g, beta, w, initial_state, out, final_state, chunk_boundaries, workspace,
                               scratch, batch, time, heads, full_tokens, training, dtype, g_dtype, scale, 0,
                               stream);
}

int gdn2_chunk_forward_fused(const void* q, const void* k, const void* v, const void* g,
                             const void* beta, const void* w, const float* initial_state, void* out,
                             float* final_state, void* workspace, void* scratch, int64_t batch, int64_t time,
                             int64_t heads, int64_t full_tokens, int dtype, int g_dtype, float scale,
                             int prologue, void* stream) {
  return chunk_forward_checked(q, k, v, g, beta, w, initial_state, out, final_state, nullptr, workspace, scratch,
                               batch, time, heads, full_tokens, 0, dtype, g_dtype, scale, prologue, stream);
}

namespace {
int chunk_backward_checked(const void* q, const void* k, const void* v, const void* g, const void* beta,
                           const void* w, const void* d_out, const float* d_final_state,
                           const float* chunk_boundaries, float* d_boundaries, const void* workspace,
                           void* scratch, void* dq, void* dk, void* dv, void* dg, void* dbeta, void* dw,
                           float* d_initial_state, int64_t batch, int64_t time, int64_t heads,
                           int64_t full_tokens, int dtype, int g_dtype, float scale, int grads_f32,
                           void* stream) {
  if (!q || !k || !v || !g || !beta || !w || !d_out || !chunk_boundaries || !d_boundaries || !workspace ||
      !scratch || !dq || !dk || !dv || !dg || !dbeta || !dw)
    return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, time, heads);
  if (st != GDN2_OK) return st;
  // whole chunks only, or rounded up over a partial last chunk (its missing tokens are identity steps)
  if (full_tokens <= 0 || full_tokens % GDN2_CHUNK != 0 || full_tokens >= time + GDN2_CHUNK) return GDN2_ERR_BAD_RANGE;
  if ((st = check_types(dtype, g_dtype)) != GDN2_OK) return st;
  const void* need16[] = {q, k, v, g, beta, w, d_out, d_final_state, chunk_boundaries, d_boundaries, workspace,
                          scratch, dq, dk, dv, dg, dbeta, dw, d_initial_state};
  for (const void* ptr : need16) {
    if (!aligned(ptr, 16)) return GDN2_ERR_ALIGNMENT;
  }
  return launch_chunk_backward(q, k, v, g, beta, w, d_out, d_final_state, chunk_boundaries, d_boundaries,
                               static_cast<const uint8_t*>(workspace), static_cast<uint8_t*>(scratch), dq, dk,
                               dv, dg, dbeta, dw, d_initial_state, batch, time, heads, full_tokens, dtype,
                               g_dtype, scale, grads_f32, static_cast<cudaStream_t>(stream));
}
}  // namespace

int gdn2_chunk_backward(const void* q, const void* k, const void* v, const void* g, const void* beta,
                        const void* w, const void* d_out, const float* d_final_state,
                        const float* chunk_boundaries, float* d_boundaries, const void* workspace,
                        void* scratch, void* dq, void* dk, void* dv, void* dg, void* dbeta, void* dw,
                        float* d_initial_state, int64_t batch, int64_t time, int64_t heads,
                        int64_t full_tokens, int dtype, int g_dtype, float scale, void* stream) {
  return chunk_backward_checked(q, k, v, g, beta, w, d_out, d_final_state, chunk_boundaries, d_boundaries,
                                workspace, scratch, dq, dk, dv, dg, dbeta, dw, d_initial_state, batch, time,
                                heads, full_tokens, dtype, g_dtype, scale, 0, stream);
}

int gdn2_chunk_backward_f32grads(const void* q, const void* k, const void* v, const void* g, const void* beta,
                                 const void* w, const void* d_out, const float* d_final_state,
                                 const float* chunk_boundaries, float* d_boundaries, const void* workspace,
                                 void* scratch, float* dq, float* dk, float* dv, float* dg, float* dbeta,
                                 float* dw, float* d_initial_state, int64_t batch, int64_t time,
                                 int64_t heads, int64_t full_tokens, float scale, void* stream) {
  return chunk_backward_checked(q, k, v, g, beta, w, d_out, d_final_state, chunk_boundaries, d_boundaries,
                                workspace, scratch, dq, dk, dv, dg, dbeta, dw, d_initial_state, batch, time,
                                heads, full_tokens, GDN2_BF16, GDN2_FP32, scale, 1, stream);
}

int gdn2_chunk_read_status(const void* workspace, int64_t batch, int64_t full_tokens, int64_t heads,
                           void* stream) {
  if (!workspace) return GDN2_ERR_NULL_POINTER;
  if (batch <= 0 || heads <= 0 || full_tokens <= 0 || full_tokens % GDN2_CHUNK != 0) return GDN2_ERR_BAD_SHAPE;
  int host = 0;
  const uint8_t* src = static_cast<const uint8_t*>(workspace) + chunk_status_offset(batch, full_tokens, heads);
  cudaError_t err = cudaMemcpyAsync(&host, src, sizeof(int), cudaMemcpyDeviceToHost,
                                    static_cast<cudaStream_t>(stream));
  if (err == cudaSuccess) err = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  return host;
}

namespace {
// a group of pointers must be given completely or not at all; returns 1 / 0, or -1 when mixed
int group_state(std::initializer_list<const void*> ptrs) {
  int set = 0, total = 0;
  for (const void* ptr : ptrs) { ++total; set += ptr != nullptr; }
  return set == 0 ? 0 : (set == total ? 1 : -1);
}
}  // namespace

int gdn2_gate_prologue(const void* q_raw, const void* k_raw, const void* g_raw, const void* beta_raw,
                       const void* w_raw, void* q, void* k, void* g, void* beta, void* w,
                       float* inv_norm_q, float* inv_norm_k, int64_t batch, int64_t time, int64_t heads,
                       int dtype, int g_dtype, void* stream) {
  const int norm = group_state({q_raw, k_raw, q, k, inv_norm_q, inv_norm_k});
  const int gate = group_state({g_raw, beta_raw, w_raw, g, beta, w});
  if (norm < 0 || gate < 0 || norm + gate == 0) return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, time, heads);
  if (st != GDN2_OK) return st;
  if ((st = check_types(dtype, g_dtype)) != GDN2_OK) return st;
  for (const void* ptr : {q_raw, k_raw, g_raw, beta_raw, w_raw, (const void*)q, (const void*)k, (const void*)g,
                          (const void*)beta, (const void*)w}) {
    if (!aligned(ptr, 16)) return GDN2_ERR_ALIGNMENT;
  }
  if (time == 0) return GDN2_OK;
  return launch_gate_prologue(q_raw, k_raw, g_raw, beta_raw, w_raw, q, k, g, beta, w, inv_norm_q, inv_norm_k,
                              batch * time * heads, dtype, g_dtype, static_cast<cudaStream_t>(stream));
}

int gdn2_gate_prologue_vjp(const void* q_raw, const void* k_raw, const void* g_raw, const void* beta_raw,
                           const void* w_raw, const float* inv_norm_q, const float* inv_norm_k,
                           const void* dq, const void* dk, const void* dg, const void* dbeta, const void* dw,
                           void* dq_raw, void* dk_raw, void* dg_raw, void* dbeta_raw, void* dw_raw,
                           int64_t batch, int64_t time, int64_t heads, int dtype, int g_dtype, void* stream) {
  const int norm = group_state({q_raw, k_raw, inv_norm_q, inv_norm_k, dq, dk, dq_raw, dk_raw});
  const int gate = group_state({g_raw, beta_raw, w_raw, dg, dbeta, dw, dg_raw, dbeta_raw, dw_raw});
  if (norm < 0 || gate < 0 || norm + gate == 0) return GDN2_ERR_NULL_POINTER;
  int st = check_shape(batch, time, heads);
  if (st != GDN2_OK) return st;
  if ((st = check_types(dtype, g_dtype)) != GDN2_OK) return st;
  for (const void* ptr : {q_raw, k_raw, g_raw, beta_raw, w_raw, dq, dk, dg, dbeta, dw, (const void*)dq_raw,
                          (const void*)dk_raw, (const void*)dg_raw, (const void*)dbeta_raw, (const void*)dw_raw}) {
    if (!aligned(ptr, 16)) return GDN2_ERR_ALIGNMENT;
  }
  if (time == 0) return GDN2_OK;
  return launch_gate_prologue_vjp(q_raw, k_raw, g_raw, beta_raw, w_raw, inv_norm_q, inv_norm_k, dq, dk, dg,
                                  dbeta, dw, dq_raw, dk_raw, dg_raw, dbeta_raw, dw_raw, batch * time * heads,
                                  dtype, g_dtype, static_cast<cudaStream_t>(stream));
}

int gdn2_debug_wait_expires(void* workspace, int64_t batch, int64_t full_tokens, int64_t heads,
                            int64_t max_polls, void* stream) {
  if (!workspace) return GDN2_ERR_NULL_POINTER;
  if (batch <= 0 || heads <= 0 || full_tokens <= 0 || full_tokens % GDN2_CHUNK != 0) return GDN2_ERR_BAD_SHAPE;
  if (check_shape(batch, full_tokens, heads) != GDN2_OK) return GDN2_ERR_TOO_LARGE;
  if (!aligned(workspace, 16)) return GDN2_ERR_ALIGNMENT;
  const int64_t polls = max_polls < 1 ? 1 : (max_polls > (int64_t(1) << 20) ? (int64_t(1) << 20) : max_polls);
  int* status = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) +
                                       chunk_status_offset(batch, full_tokens, heads));
  return launch_debug_wait_expires(status, uint32_t(polls), static_cast<cudaStream_t>(stream));
}

}  // extern "C"

extern "C" int gdn2_profile_enable(int on) {
  std::lock_guard<std::mutex> lock(gdn2::g_profile_mutex);
  gdn2::g_profile_on = on != 0;
  for (auto& set : gdn2::g_profile) set.recorded[0] = set.recorded[1] = false;
  return GDN2_OK;
}

// Durations of the most recent forward / backward pair recorded on the current device.
extern "C" int gdn2_profile_chunk_kernels(float* prep_ms, float* scan_ms, float* bwd_scan_ms, float* vjp_ms) {
  if (prep_ms == nullptr || scan_ms == nullptr || bwd_scan_ms == nullptr || vjp_ms == nullptr) {
    return GDN2_ERR_NULL_POINTER;
  }
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) { gdn2::record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  if (device < 0 || device >= gdn2::kProfileDevices) return GDN2_ERR_DEVICE;
  float* out[4] = {prep_ms, scan_ms, bwd_scan_ms, vjp_ms};
  cudaEvent_t events[6];
  bool recorded[2];
  {
    std::lock_guard<std::mutex> lock(gdn2::g_profile_mutex);
    for (int i = 0; i < 6; ++i) events[i] = gdn2::g_profile[device].events[i];
    recorded[0] = gdn2::g_profile[device].recorded[0];
    recorded[1] = gdn2::g_profile[device].recorded[1];
  }
  for (int call = 0; call < 2; ++call) {
    out[2 * call][0] = out[2 * call + 1][0] = -1.f;
    if (!recorded[call]) continue;
    cudaEvent_t* ev = events + 3 * call;
    err = cudaEventSynchronize(ev[2]);
    if (err == cudaSuccess) err = cudaEventElapsedTime(out[2 * call], ev[0], ev[1]);
    if (err == cudaSuccess) err = cudaEventElapsedTime(out[2 * call + 1], ev[1], ev[2]);
    if (err != cudaSuccess) { gdn2::record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  }
  return GDN2_OK;
}
