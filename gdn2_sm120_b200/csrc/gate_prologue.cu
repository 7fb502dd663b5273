// Fused input prologue of a Gated DeltaNet-2 layer and its VJP: q/k L2 normalisation and gate
// activations in one pass over the sequence tensors instead of a dozen elementwise launches.
//
//   q^ = q / sqrt(sum_c q_c^2 + eps)      k^ likewise          (eps = 1e-6, fp32 arithmetic)
//   beta = sigmoid(beta_raw)              w = sigmoid(w_raw)
//   g = -softplus(g_raw) = -log(1 + exp(g_raw))                (a log-decay: finite and <= 0)
//
// The reference keeps these steps outside its primitive (README.md:127-131, docs/design.md:32-34 of
// the reference) and names the official implementation's flags for them, use_qk_l2norm_in_kernel and
// use_gate_in_kernel (src/gdn2_sm120/benchmark.py:230-231).  Here they are one memory-bound kernel
// in front of the chunk / token kernels and one behind their backward: a warp owns one (token, head)
// row of 128 channels, a lane 4 consecutive channels (8- or 16-byte accesses, fully coalesced), the
// row sums are warp shuffles.  Either group (normalisation, gates) can be switched off by passing
// NULL for its tensors.

#include "common.cuh"

namespace gdn2 {

namespace {

constexpr int kRowsPerBlock = 8;  // 8 warps, one row each
constexpr float kNormEps = 1e-6f;

template <typename T> struct Vec4 { using type = uint2; };
template <> struct Vec4<float> { using type = float4; };

template <typename T>
__device__ __forceinline__ void load4f(const void* base, int64_t idx, float (&x)[4]);
template <>
__device__ __forceinline__ void load4f<__nv_bfloat16>(const void* base, int64_t idx, float (&x)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + idx);
  x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xffff0000u);
  x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xffff0000u);
}
template <>
__device__ __forceinline__ void load4f<__half>(const void* base, int64_t idx, float (&x)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __half*>(base) + idx);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
  x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
template <>
__device__ __forceinline__ void load4f<float>(const void* base, int64_t idx, float (&x)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
}

template <typename T>
__device__ __forceinline__ void store4f(void* base, int64_t idx, const float (&x)[4]);
template <>
__device__ __forceinline__ void store4f<__nv_bfloat16>(void* base, int64_t idx, const float (&x)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + idx) =
      make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}
template <>
__device__ __forceinline__ void store4f<__half>(void* base, int64_t idx, const float (&x)[4]) {
  const __half2 lo = __floats2half2_rn(x[0], x[1]), hi = __floats2half2_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(static_cast<__half*>(base) + idx) =
      make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}
template <>
__device__ __forceinline__ void store4f<float>(void* base, int64_t idx, const float (&x)[4]) {
  *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = make_float4(x[0], x[1], x[2], x[3]);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
  return x;
}

__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + expf(-x)); }
// softplus with the usual guard: log1p(exp(x)) overflows for large x, where it equals x to fp32 precision
__device__ __forceinline__ float softplusf(float x) { return x > 20.f ? x : log1pf(expf(x)); }

struct PrologueParams {
  const void *q_raw, *k_raw, *g_raw, *beta_raw, *w_raw;
  void *q, *k, *g, *beta, *w;
  float *inv_q, *inv_k;
  int64_t rows;
};

template <typename T, typename G>
__global__ void __launch_bounds__(32 * kRowsPerBlock) gate_prologue_kernel(const PrologueParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * kRowsPerBlock + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const int64_t idx = row * kDim + 4 * lane;
  float x[4], y[4];
  if (p.q_raw != nullptr) {
    load4f<T>(p.q_raw, idx, x);
    const float inv = rsqrtf(warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]) + kNormEps);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = x[c] * inv;
    store4f<T>(p.q, idx, y);
    if (lane == 0) p.inv_q[row] = inv;
    load4f<T>(p.k_raw, idx, x);
    const float invk = rsqrtf(warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]) + kNormEps);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = x[c] * invk;
    store4f<T>(p.k, idx, y);
    if (lane == 0) p.inv_k[row] = invk;
  }
  if (p.g_raw != nullptr) {
    load4f<G>(p.g_raw, idx, x);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = -softplusf(x[c]);
    store4f<G>(p.g, idx, y);
    load4f<T>(p.beta_raw, idx, x);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = sigmoidf(x[c]);
    store4f<T>(p.beta, idx, y);
    load4f<T>(p.w_raw, idx, x);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = sigmoidf(x[c]);
    store4f<T>(p.w, idx, y);
  }
}

struct PrologueVjpParams {
  const void *q_raw, *k_raw, *g_raw, *beta_raw, *w_raw;
  const float *inv_q, *inv_k;
  const void *dq, *dk, *dg, *dbeta, *dw;          // cotangents of the activated tensors
  void *dq_raw, *dk_raw, *dg_raw, *dbeta_raw, *dw_raw;  // may alias the incoming cotangents
  int64_t rows;
};

template <typename T, typename G>
__global__ void __launch_bounds__(32 * kRowsPerBlock) gate_prologue_vjp_kernel(const PrologueVjpParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * kRowsPerBlock + (threadIdx.x >> 5);
  if (row >= p.rows) return;
  const int64_t idx = row * kDim + 4 * lane;
  float x[4], d[4], y[4];
  if (p.q_raw != nullptr) {
    // d(x / |x|) : dx = inv (dy - y^ (y^ . dy)),  y^ = x inv
    load4f<T>(p.q_raw, idx, x);
    load4f<T>(p.dq, idx, d);
    float inv = p.inv_q[row];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) { x[c] *= inv; dot = fmaf(x[c], d[c], dot); }
    dot = warp_sum(dot);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = inv * fmaf(-x[c], dot, d[c]);
    store4f<T>(p.dq_raw, idx, y);
    load4f<T>(p.k_raw, idx, x);
    load4f<T>(p.dk, idx, d);
    inv = p.inv_k[row];
    dot = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) { x[c] *= inv; dot = fmaf(x[c], d[c], dot); }
    dot = warp_sum(dot);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = inv * fmaf(-x[c], dot, d[c]);
    store4f<T>(p.dk_raw, idx, y);
  }
  if (p.g_raw != nullptr) {
    load4f<G>(p.g_raw, idx, x);
    load4f<G>(p.dg, idx, d);
#pragma unroll
    for (int c = 0; c < 4; ++c) y[c] = -sigmoidf(x[c]) * d[c];   // d(-softplus(x))/dx = -sigmoid(x)
    store4f<G>(p.dg_raw, idx, y);
    load4f<T>(p.beta_raw, idx, x);
    load4f<T>(p.dbeta, idx, d);
#pragma unroll
    for (int c = 0; c < 4; ++c) { const float s = sigmoidf(x[c]); y[c] = s * (1.f - s) * d[c]; }
    store4f<T>(p.dbeta_raw, idx, y);
    load4f<T>(p.w_raw, idx, x);
    load4f<T>(p.dw, idx, d);
#pragma unroll
    for (int c = 0; c < 4; ++c) { const float s = sigmoidf(x[c]); y[c] = s * (1.f - s) * d[c]; }
    store4f<T>(p.dw_raw, idx, y);
  }
}

}  // namespace

int launch_gate_prologue(const void* q_raw, const void* k_raw, const void* g_raw, const void* beta_raw,
                         const void* w_raw, void* q, void* k, void* g, void* beta, void* w, float* inv_q,
                         float* inv_k, int64_t rows, int dtype, int g_dtype, cudaStream_t stream) {
  const int64_t blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (blocks <= 0 || blocks > int64_t(0x7fffffff)) return GDN2_ERR_TOO_LARGE;
  PrologueParams p{q_raw, k_raw, g_raw, beta_raw, w_raw, q, k, g, beta, w, inv_q, inv_k, rows};
  GDN2_DISPATCH_TYPES(dtype, g_dtype,
                      (gate_prologue_kernel<T, G><<<unsigned(blocks), 32 * kRowsPerBlock, 0, stream>>>(p)));
  return check_launch();
}

int launch_gate_prologue_vjp(const void* q_raw, const void* k_raw, const void* g_raw, const void* beta_raw,
                             const void* w_raw, const float* inv_q, const float* inv_k, const void* dq,
                             const void* dk, const void* dg, const void* dbeta, const void* dw, void* dq_raw,
                             void* dk_raw, void* dg_raw, void* dbeta_raw, void* dw_raw, int64_t rows, int dtype,
                             int g_dtype, cudaStream_t stream) {
  const int64_t blocks = (rows + kRowsPerBlock - 1) / kRowsPerBlock;
  if (blocks <= 0 || blocks > int64_t(0x7fffffff)) return GDN2_ERR_TOO_LARGE;
  PrologueVjpParams p{q_raw, k_raw, g_raw, beta_raw, w_raw, inv_q, inv_k, dq, dk, dg, dbeta, dw,
                      dq_raw, dk_raw, dg_raw, dbeta_raw, dw_raw, rows};
  GDN2_DISPATCH_TYPES(dtype, g_dtype,
                      (gate_prologue_vjp_kernel<T, G><<<unsigned(blocks), 32 * kRowsPerBlock, 0, stream>>>(p)));
  return check_launch();
}

}  // namespace gdn2
