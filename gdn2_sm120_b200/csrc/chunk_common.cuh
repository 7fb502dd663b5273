// Shared definitions of the 64-token tensor-core chunk path.
//
// For every unit ch = (b * n_chunks + c) * H + h (one 64-token chunk of one head) the prep kernel
// writes the WY factors as plain row-major fp32 matrices holding tf32 values ("tiles"), ONE copy of
// each.  The forward scan and the reverse scan both consume them: the forward contracts over one index
// of a tile and the backward over the other, so one kernel reads a tile as a K-major operand and the
// other as an MN-major operand.  Tiled TMA loads put the same global bytes into shared memory in the
// layout each role needs (K-major: 128-byte swizzle; MN-major tf32: 128-byte swizzle with 32-byte
// atoms, the only MN-major form the tensor cores accept for 32-bit operands).  The orientation of a
// tile in global memory is the one its producer can store with full 128-byte lines: token-major for
// tiles made from registers, transposed for tiles read out of tensor memory (lane = row).
//
//   Q    [token i (64)][key k (128)]     32 KiB   scale * gamma * q            fwd K-major,  bwd MN-major
//   Kn   [token j (64)][key k (128)]     32 KiB   k * gamma_end / gamma        fwd MN-major, bwd K-major
//   Yt   [key k (128)][token i (64)]     32 KiB   Y^T, Y = (I+L)^-1 E          fwd MN-major, bwd K-major
//   At   [token j (64)][token i (64)]    16 KiB   tril(Q_gamma Kbar^T)^T       fwd MN-major, bwd K-major
//   Tt   [token j (64)][token i (64)]    16 KiB   ((I+L)^-1)^T                 bwd K-major (training only)
//        (both are zero where j > i: the quadrant j >= 32, i < 32 is neither written nor read, the
//        consumers keep those lines of their shared-memory tile at zero; 12 KiB move)
//   U    [token j (64)][value v (128)]   32 KiB   U = (I+L)^-1 (w*v)           forward only: copied into
//                                                                               tensor memory by threads
//   D    float[128]                      512 B    gamma_end
//
//   Rn   [token j (64)][value v (128)]   32 KiB   R = U - Y S_0   forward scan -> VJP kernel (K-major)
//
// One more per-unit array is a "blocked" tile (see tc05.cuh) that a bulk copy moves as it is:
//   dZ   X[r = token j (64)][c = value v (128)] RS = 4608, CS = 144   36 KiB   dZ = T^T dR
//        (reverse scan -> VJP kernel; the padded strides are those of the tile it is copied into)
//
// Buffers (caller-provided, struct of arrays, each array n_ch entries long):
//   workspace  D, a 256-byte status block, and for a training call what backward consumes:
//              Rn, Q, Kn, Yt, At, Tt
//   scratch    dead when the call returns: forward U (and Q, Kn, Yt, At for an inference call);
//              backward dZ
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "tc05.cuh"

namespace gdn2 {

constexpr int kChunk = GDN2_CHUNK;  // 64

constexpr int64_t kTileQ = 32768, kTileKn = 32768, kTileYt = 32768, kTileU = 32768;
constexpr int64_t kTileAt = 16384, kTileTt = 16384, kBlobD = 512;
constexpr int64_t kBlobRn = 32768, kBlobDZ = 8 * 4608;
constexpr int64_t kStatusBytes = 256;
constexpr int64_t kFwdTilesBytes = kTileQ + kTileKn + kTileYt + kTileAt;  // the tiles both scans read

// workspace: what a training forward leaves for backward (inference: D and the status block only)
struct WsLayout {
  int64_t n_ch;
  bool training = false;
  __host__ __device__ int64_t off_d() const { return 0; }
  __host__ __device__ int64_t off_status() const { return n_ch * kBlobD; }
  // training-only arrays follow the status block
  __host__ __device__ int64_t off_rn() const { return off_status() + kStatusBytes; }
  __host__ __device__ int64_t off_q() const { return off_rn() + n_ch * kBlobRn; }
  __host__ __device__ int64_t off_kn() const { return off_q() + n_ch * kTileQ; }
  __host__ __device__ int64_t off_yt() const { return off_kn() + n_ch * kTileKn; }
  __host__ __device__ int64_t off_at() const { return off_yt() + n_ch * kTileYt; }
  __host__ __device__ int64_t off_tt() const { return off_at() + n_ch * kTileAt; }
  __host__ __device__ int64_t total() const { return training ? off_tt() + n_ch * kTileTt : off_rn(); }
};

// scratch of one call
struct ScratchLayout {
  int64_t n_ch;
  __host__ __device__ int64_t off_u() const { return 0; }
  // inference calls only (a training call keeps these in its workspace)
  __host__ __device__ int64_t off_q() const { return n_ch * kTileU; }
  __host__ __device__ int64_t off_kn() const { return off_q() + n_ch * kTileQ; }
  __host__ __device__ int64_t off_yt() const { return off_kn() + n_ch * kTileKn; }
  __host__ __device__ int64_t off_at() const { return off_yt() + n_ch * kTileYt; }
  __host__ __device__ int64_t total_forward(bool training) const {
    return training ? n_ch * kTileU : n_ch * (kTileU + kFwdTilesBytes);
  }
  __host__ __device__ int64_t off_dz() const { return 0; }
  __host__ __device__ int64_t total_backward() const { return n_ch * kBlobDZ; }
};

// where the forward tile arrays of a call live
struct ForwardTiles {
  uint8_t *q, *kn, *yt, *at, *tt, *u;
};
inline ForwardTiles forward_tiles(uint8_t* workspace, uint8_t* scratch, int64_t n_ch, bool training) {
  const WsLayout ws{n_ch, training};
  const ScratchLayout sc{n_ch};
  ForwardTiles t;
  t.u = scratch + sc.off_u();
  if (training) {
    t.q = workspace + ws.off_q(); t.kn = workspace + ws.off_kn(); t.yt = workspace + ws.off_yt();
    t.at = workspace + ws.off_at(); t.tt = workspace + ws.off_tt();
  } else {
    t.q = scratch + sc.off_q(); t.kn = scratch + sc.off_kn(); t.yt = scratch + sc.off_yt();
    t.at = scratch + sc.off_at(); t.tt = nullptr;
  }
  return t;
}

// device status codes written to the workspace status word (0 = ok)
enum : int { kStatusOk = 0, kStatusBarrierTimeout = 1 };

__device__ __forceinline__ float poison_nan() { return __int_as_float(0x7fc00000); }

// A wait that gives up: after `limit` failed polls the thread records kStatusBarrierTimeout in the
// status word and every later wait of the thread returns immediately.  The kernel then runs to its
// end (shared resources such as TMEM are always released) and writes NaN instead of results, so the
// failure shows in the outputs themselves and not only in the status word.
struct BoundedWaiter {
  bool dead = false;
  int* status;
  uint32_t limit;
  __device__ explicit BoundedWaiter(int* s, uint32_t max_polls = (1u << 20)) : status(s), limit(max_polls) {}
  __device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity) {
    if (dead) return;
    if (!tc::mbar_wait(bar, parity, limit)) {
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

// ---- tensor maps (host) -------------------------------------------------------------------------
// cuTensorMapEncodeTiled through the runtime's driver entry point query: the library does not link
// against the driver API for this one call.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query) != cudaSuccess ||
        query != cudaDriverEntryPointSuccess) {
      return EncodeTiledFn(nullptr);
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Encoding a tensor map costs the host some 20 microseconds and a call needs a dozen of them; the
// maps depend only on addresses and shapes, which repeat from call to call (allocators hand the same
// blocks out again), so the last few hundred are kept.  Direct-mapped, one mutex.
struct TensorMapKey {
  uintptr_t base;
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4];
  int rank, type, swizzle;
  bool operator==(const TensorMapKey& o) const {
    bool same = base == o.base && rank == o.rank && type == o.type && swizzle == o.swizzle;
    for (int i = 0; i < 4; ++i) same = same && dims[i] == o.dims[i] && box[i] == o.box[i];
    for (int i = 0; i < 3; ++i) same = same && strides[i] == o.strides[i];
    return same;
  }
};

// rank 3 or 4; unused trailing entries of dims / strides / box are 1 / 0 / 1
inline bool encode_cached(CUtensorMap* tm, int rank, CUtensorMapDataType type, const void* base,
                          const cuuint64_t (&dims)[4], const cuuint64_t (&strides)[3], const cuuint32_t (&box)[4],
                          CUtensorMapSwizzle swizzle) {
  constexpr int kSlots = 512;
  struct Slot { bool used = false; TensorMapKey key; CUtensorMap map; };
  static Slot slots[kSlots];
  static std::mutex mutex;
  TensorMapKey key{reinterpret_cast<uintptr_t>(base), {dims[0], dims[1], dims[2], dims[3]},
                   {strides[0], strides[1], strides[2]}, {box[0], box[1], box[2], box[3]}, rank, int(type),
                   int(swizzle)};
  uint64_t h = key.base * 0x9E3779B97F4A7C15ull;
  h ^= (key.dims[2] + 0x632BE59BD9B4E019ull * key.strides[1]) + (uint64_t(key.box[1]) << 7) + (uint64_t(key.box[2]) << 17) +
       uint64_t(key.swizzle) * 31 + uint64_t(key.type) + uint64_t(rank) * 131 + key.dims[3] * 0x2545F4914F6CDD1Dull;
  h ^= h >> 29;
  Slot& slot = slots[h % kSlots];
  {
    std::lock_guard<std::mutex> lock(mutex);
    if (slot.used && slot.key == key) { *tm = slot.map; return true; }
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
  // OOB_FILL_NONE: the part of a load box outside the tensor reads as zero
  if (encode(tm, type, cuuint32_t(rank), const_cast<void*>(base), dims, strides, box, elem_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    return false;
  }
  std::lock_guard<std::mutex> lock(mutex);
  slot.used = true; slot.key = key; slot.map = *tm;
  return true;
}

// A contiguous [B, T, H, 128] sequence tensor seen as (channel, head, token, batch): a box
// (128, 1, 64, 1) is one head's 64-token chunk, landing in shared memory as dense [64][128] rows
// (`box_rows` tokens instead of 64 when given).  Tokens are a dimension of their own so that the last,
// partial chunk of a ragged sequence reads zeros beyond token T - 1 (and a store is clipped there).
inline bool encode_sequence_map(CUtensorMap* tm, const void* base, int64_t batch, int64_t time, int64_t heads,
                                int dtype, int box_rows = kChunk) {
  const cuuint64_t es = (dtype == GDN2_FP32) ? 4 : 2;
  const CUtensorMapDataType type = (dtype == GDN2_FP32)   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : (dtype == GDN2_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint64_t dims[4] = {cuuint64_t(kDim), cuuint64_t(heads), cuuint64_t(time), cuuint64_t(batch)};
  const cuuint64_t strides[3] = {cuuint64_t(kDim) * es, cuuint64_t(heads) * kDim * es,
                                 cuuint64_t(time) * heads * kDim * es};  // bytes, dimensions 1..3
  const cuuint32_t box[4] = {cuuint32_t(kDim), 1, cuuint32_t(box_rows), 1};
  return encode_cached(tm, 4, type, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

// An array of n_ch row-major fp32 tiles [rows][cols] seen as (col, row, unit): a box (32, rows, 1) is a
// slab of 32 columns of one tile, `rows` lines of 128 bytes in shared memory.  mn_major chooses the
// swizzle: 128-byte with 32-byte atoms (the tile is read as an MN-major operand, contraction over its
// rows) or plain 128-byte (K-major operand, contraction over its columns).
// (`box_rows` < rows: boxes of that many rows, for tiles whose zero quadrant is never moved.)
inline bool encode_tile_map(CUtensorMap* tm, const uint8_t* base, int64_t n_ch, int rows, int cols, bool mn_major,
                            int box_rows = 0) {
  const cuuint64_t dims[4] = {cuuint64_t(cols), cuuint64_t(rows), cuuint64_t(n_ch), 1};
  const cuuint64_t strides[3] = {cuuint64_t(cols) * 4, cuuint64_t(rows) * cols * 4, 0};
  const cuuint32_t box[4] = {32, cuuint32_t(box_rows > 0 ? box_rows : rows), 1, 1};
  return encode_cached(tm, 3, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, dims, strides, box,
                       mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
}
// The same array, whole tiles without swizzle (box (cols, rows, 1); cols <= 256): for tiles that threads read.
inline bool encode_plain_tile_map(CUtensorMap* tm, const uint8_t* base, int64_t n_ch, int rows, int cols) {
  const cuuint64_t dims[4] = {cuuint64_t(cols), cuuint64_t(rows), cuuint64_t(n_ch), 1};
  const cuuint64_t strides[3] = {cuuint64_t(cols) * 4, cuuint64_t(rows) * cols * 4, 0};
  const cuuint32_t box[4] = {cuuint32_t(cols), cuuint32_t(rows), 1, 1};
  return encode_cached(tm, 3, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

}  // namespace gdn2
