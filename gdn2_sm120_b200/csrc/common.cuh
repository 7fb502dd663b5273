// Shared device/host helpers for the gdn2_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/gdn2_b200.h"

namespace gdn2 {

constexpr int kDim = GDN2_DIM;
constexpr int kTokenInterval = GDN2_TOKEN_INTERVAL;

// ---- typed scalar loads / stores through float --------------------------------
// bf16 -> fp32 is a 16-bit shift (exact); spelled out so that it runs on the integer pipe
__device__ __forceinline__ float to_float(__nv_bfloat16 x) {
  return __uint_as_float(uint32_t(__bfloat16_as_ushort(x)) << 16);
}
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(float x) { return x; }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}
template <>
__device__ __forceinline__ __half from_float<__half>(float x) {
  return __float2half_rn(x);
}
template <>
__device__ __forceinline__ float from_float<float>(float x) {
  return x;
}

template <typename T>
__device__ __forceinline__ float ldf(const void* base, int64_t index) {
  return to_float(static_cast<const T*>(base)[index]);
}
template <typename T>
__device__ __forceinline__ void stf(void* base, int64_t index, float value) {
  static_cast<T*>(base)[index] = from_float<T>(value);
}

// ---- state tile I/O: 128-bit when the base is 16-byte aligned ------------------
__device__ __forceinline__ void load4(const float* p, bool vec, float (&x)[4]) {
  if (vec) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
  } else {
    x[0] = p[0]; x[1] = p[1]; x[2] = p[2]; x[3] = p[3];
  }
}
__device__ __forceinline__ void store4(float* p, bool vec, const float (&x)[4]) {
  if (vec) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
  } else {
    p[0] = x[0]; p[1] = x[1]; p[2] = x[2]; p[3] = x[3];
  }
}

// ---- layer prologue (optional, fused into the forward kernels) ------------------------------
// bit flags of the `prologue` argument of the *_fused entry points
constexpr int kPrologueNorm = GDN2_PROLOGUE_NORMALIZE_QK;   // q, k are raw projections: L2-normalise them
constexpr int kPrologueGate = GDN2_PROLOGUE_ACTIVATE_GATES; // beta, w, g are pre-activations
constexpr float kPrologueEps = 1e-6f;

// The activations inside the forward kernels run on the special-function unit (ex2 / lg2 / rcp
// approximations, about 1e-6 relative, far below the 16-bit inputs' own rounding): the library routines
// (expf, log1pf, a full division) made the prologue half of the prep kernel's code and two thirds again
// of its time.  (The stand-alone activation kernel of a training step is memory-bound and keeps them.)
__device__ __forceinline__ float prologue_sigmoid(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + __expf(-x)));
  return r;
}
// log-decay g = -softplus(x) = -log(1 + e^x).  Small e^x: the series e - e^2/2 + e^3/3 (its first
// dropped term is below 2^-26 of the sum there; lg2 of a number next to 1 would lose the digits);
// softplus(x) equals x to fp32 precision beyond 20.
__device__ __forceinline__ float prologue_log_decay(float x) {
  const float e = __expf(fminf(x, 20.f));
  const float series = e * (1.f - e * (0.5f - e * 0.33333334f));
  const float direct = __logf(1.f + e);
  return x > 20.f ? -x : -(e < 0.00390625f ? series : direct);
}

// ---- host-side status helpers ---------------------------------------------------
void record_cuda_error(cudaError_t err);  // defined in api.cu
int check_launch();                       // cudaGetLastError -> status
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes);  // once per (kernel, device) opt-in (api.cu)
void profile_mark(int index, cudaStream_t stream);  // records timing event `index` when profiling is on (api.cu)

inline bool valid_seq_dtype(int d) { return d == GDN2_BF16 || d == GDN2_FP16; }
inline bool valid_gate_dtype(int d, int seq) { return d == seq || d == GDN2_FP32; }

// Dispatch a callable templated on <T, G> over the runtime dtype codes.
#define GDN2_DISPATCH_TYPES(dtype, g_dtype, ...)                         \
  do {                                                                   \
    if ((dtype) == GDN2_BF16) {                                          \
      using T = __nv_bfloat16;                                           \
      if ((g_dtype) == GDN2_FP32) { using G = float; __VA_ARGS__; }      \
      else { using G = __nv_bfloat16; __VA_ARGS__; }                     \
    } else {                                                             \
      using T = __half;                                                  \
      if ((g_dtype) == GDN2_FP32) { using G = float; __VA_ARGS__; }      \
      else { using G = __half; __VA_ARGS__; }                            \
    }                                                                    \
  } while (0)

}  // namespace gdn2
