// Shared definitions of the 64-token tensor-core chunk path.
//
// Workspace ("WY blobs"): for every chunk-head ch = (b * n_chunks + c) * H + h the prep kernel
// writes operand-ready tiles that the scan kernels pull into shared memory with 1-D bulk
// copies and that backward reuses.  All tiles are "blocked" (see tc05.cuh), CS = 128, tf32
// values in fp32 containers:
//
//   Y    X[r = token i (64)][c = key k (128)]   RS = 4096   32 KiB   Y = (I+L)^-1 E
//   Ut   X[r = value v (128)][c = token i (64)] RS = 2048   32 KiB   U^T, U = (I+L)^-1 (w*v)
//   Q    X[r = token i (64)][c = key k (128)]   RS = 4096   32 KiB   scale * gamma * q
//   Kt   X[r = key k (128)][c = token j (64)]   RS = 2048   32 KiB   (k * gamma_end / gamma)^T
//   A    X[r = token i (64)][c = token j (64)]  RS = 2048   16 KiB   tril(Q_gamma Kbar^T)
//   D    float[128]                                         512 B    gamma_end
// and, for training calls only (consumed by backward, which contracts over the other index):
//   Yt   X[r = key k (128)][c = token i (64)]   RS = 2048   32 KiB   Y^T
//   Qt   X[r = key k (128)][c = token i (64)]   RS = 2048   32 KiB   Q_gamma^T
//   Kn   X[r = token j (64)][c = key k (128)]   RS = 4096   32 KiB   K_tail
//   At   X[r = token j (64)][c = token i (64)]  RS = 2048   16 KiB   A_qk^T
//   Tt   X[r = token j (64)][c = token i (64)]  RS = 2048   16 KiB   ((I+L)^-1)^T
//   Rn   X[r = token j (64)][c = value v (128)] RS = 4096   32 KiB   R = U - Y S_0 (forward scan)
//   dZ   X[r = token j (64)][c = value v (128)] RS = 4608, CS = 144   36 KiB   dZ = T^T dR (backward
//        scan; the padded strides are those of the shared-memory tile it is copied into)
//
// Arrays are stored one after another (struct of arrays), each n_ch entries long.
#pragma once

#include "common.cuh"
#include "tc05.cuh"

namespace gdn2 {

constexpr int kChunk = GDN2_CHUNK;  // 64

constexpr int64_t kBlobY = 32768, kBlobUt = 32768, kBlobQ = 32768, kBlobKt = 32768;
constexpr int64_t kBlobA = 16384, kBlobD = 512;
constexpr int64_t kBlobFwd = kBlobY + kBlobUt + kBlobQ + kBlobKt + kBlobA + kBlobD;
constexpr int64_t kBlobYt = 32768, kBlobQt = 32768, kBlobKn = 32768, kBlobAt = 16384, kBlobTt = 16384;
constexpr int64_t kBlobRn = 32768, kBlobDZ = 8 * 4608;

struct WsLayout {
  int64_t n_ch;
  bool training = false;
  __host__ __device__ int64_t off_y() const { return 0; }
  __host__ __device__ int64_t off_ut() const { return n_ch * kBlobY; }
  __host__ __device__ int64_t off_q() const { return n_ch * (kBlobY + kBlobUt); }
  __host__ __device__ int64_t off_kt() const { return n_ch * (kBlobY + kBlobUt + kBlobQ); }
  __host__ __device__ int64_t off_a() const { return n_ch * (kBlobY + kBlobUt + kBlobQ + kBlobKt); }
  __host__ __device__ int64_t off_d() const { return off_a() + n_ch * kBlobA; }
  __host__ __device__ int64_t off_status() const { return off_d() + n_ch * kBlobD; }
  // training-only arrays follow the status block
  __host__ __device__ int64_t off_yt() const { return off_status() + 256; }
  __host__ __device__ int64_t off_qt() const { return off_yt() + n_ch * kBlobYt; }
  __host__ __device__ int64_t off_kn() const { return off_qt() + n_ch * kBlobQt; }
  __host__ __device__ int64_t off_at() const { return off_kn() + n_ch * kBlobKn; }
  __host__ __device__ int64_t off_tt() const { return off_at() + n_ch * kBlobAt; }
  __host__ __device__ int64_t off_rn() const { return off_tt() + n_ch * kBlobTt; }
  __host__ __device__ int64_t off_dz() const { return off_rn() + n_ch * kBlobRn; }
  __host__ __device__ int64_t total() const {
    return training ? off_dz() + n_ch * kBlobDZ : off_status() + 256;
  }
};

// device status codes written to the workspace status word (0 = ok)
enum : int { kStatusOk = 0, kStatusBarrierTimeout = 1 };

// A wait that gives up: after the first timeout every later wait of the thread returns
// immediately, the kernel runs to completion on garbage and the host sees the status word.
struct BoundedWaiter {
  bool dead = false;
  int* status;
  __device__ explicit BoundedWaiter(int* s) : status(s) {}
  __device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity) {
    if (dead) return;
    if (!tc::mbar_wait(bar, parity, 1u << 20)) {
      dead = true;
      if (status != nullptr) atomicExch(status, kStatusBarrierTimeout);
    }
  }
};

// load 8 consecutive sequence elements (16-bit type: one 16-byte load; fp32: two)
template <typename T>
__device__ __forceinline__ void load8(const void* base, int64_t idx, float (&out)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const void* base, int64_t idx, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + idx);
  const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(wv[i] << 16);
    out[2 * i + 1] = __uint_as_float(wv[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const void* base, int64_t idx, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __half*>(base) + idx);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const void* base, int64_t idx, float (&out)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
  const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}

// 4 consecutive sequence elements, kept packed until they are needed (a prefetch then costs 2 or 4
// registers per group instead of 4 floats)
template <typename T> struct Raw4 { using type = uint2; };
template <> struct Raw4<float> { using type = float4; };
template <typename T>
__device__ __forceinline__ typename Raw4<T>::type load4_raw(const void* base, int64_t idx) {
  return *reinterpret_cast<const typename Raw4<T>::type*>(static_cast<const T*>(base) + idx);
}
template <typename T>
__device__ __forceinline__ void unpack4(typename Raw4<T>::type raw, float (&out)[4]);
template <>
__device__ __forceinline__ void unpack4<__nv_bfloat16>(uint2 raw, float (&out)[4]) {
  out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
  out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
}
template <>
__device__ __forceinline__ void unpack4<__half>(uint2 raw, float (&out)[4]) {
  const __half2* hh = reinterpret_cast<const __half2*>(&raw);
  const float2 a = __half22float2(hh[0]), c = __half22float2(hh[1]);
  out[0] = a.x; out[1] = a.y; out[2] = c.x; out[3] = c.y;
}
template <>
__device__ __forceinline__ void unpack4<float>(float4 raw, float (&out)[4]) {
  out[0] = raw.x; out[1] = raw.y; out[2] = raw.z; out[3] = raw.w;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

}  // namespace gdn2
