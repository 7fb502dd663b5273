// Tensor-core chunk backward (64-token chunks), two kernels that consume the WY tiles and
// residuals saved by the forward and the fp32 chunk-start states.  The reverse scan reads the very
// tiles the forward scan read, through tiled TMA loads in the other swizzle: what the forward
// contracted over columns it contracts over rows (K-major <-> MN-major operands, tc05.cuh).
//
//   chunk_bwd_scan_kernel  one CTA per (batch, head), chunks in reverse order.  The state
//                          cotangent lives transposed (dS^T: value rows x key columns) in TMEM:
//                              dR^T  = dO^T Aqk + dS^T Kt^T        dZ^T = dR^T T
//                              dS^T <- dS^T diag(d) + dO^T Qg - dR^T Y
//                          It writes dZ = T^T dR per chunk and the cotangent at every chunk start.
//   chunk_bwd_vjp_kernel   persistent, one CTA per SM walking over the (batch, chunk, head) units,
//                          all chunks independent.  With R = T (Z - E S_0) as the parametrisation
//                          (no Y / U needed):
//                              dv = dZ w, dw = dZ v             (dZ = T^T dR comes from the scan)
//                              [-dE ; dQg] = [dZ ; dO] S_0^T    dKt = R dS_1^T
//                              [-dL ; dA]  = [dZ ; dO] R^T      (strictly lower / lower part)
//                          then the Gram products' VJP with the same 16-token block anchors as the
//                          forward, and a per-channel chain (one thread = one key channel) that
//                          forms dq, dk, dbeta and the reverse cumulative sum for dg.
// A ragged length ends in a partial chunk: tokens past T - 1 carry no cotangent and get no gradient.
//
// Reference counterparts: boundary scan  src/gdn2_sm120/backward_parallel.py:721-1049,
// compact-WY VJP  src/gdn2_sm120/backward_wy.py:226-1168 (a 10-12 launch graph there).

#include <cuda.h>

#include <type_traits>

#include "chunk_common.cuh"

namespace gdn2 {

using namespace tc;

namespace {

constexpr int64_t kStateElems = int64_t(kDim) * kDim;

// =============================================================================================
// reverse scan
// =============================================================================================
constexpr int kBScanThreads = 512;
constexpr int kRsDot = 2064;   // dO^T tile: padded row-group stride (16-byte chunk stores, 4 tokens each)
constexpr int kCsZ = 144, kRsZ = 32 * kCsZ;  // dZ tile: the padded strides of the VJP kernel's [dZ ; dO] stack

struct BScanSmem {
  // swizzled operand tiles, slabs of 32 columns (tc05.cuh): Q is read MN-major, the others K-major
  alignas(1024) uint8_t kn[32768];   // Kn[j][k]: 4 slabs of 64 lines
  alignas(1024) uint8_t q[32768];    // Q[i][k]:  4 slabs of 64 lines
  alignas(1024) uint8_t yt[32768];   // Yt[k][j]: 2 slabs of 128 lines
  alignas(1024) uint8_t at[16384];   // At[j][i]: 2 slabs of 64 lines
  alignas(1024) uint8_t tt[16384];   // Tt[j][i]: 2 slabs of 64 lines
  alignas(128) uint8_t dot[16 * kRsDot];  // dO^T tile X[r = v][c = i], tf32, blocked (built from dO)
  alignas(128) uint8_t dz[kBlobDZ];  // dZ staging, natural tile X[r = j][c = v] with the padded strides
  alignas(16) float d[kDim];
  alignas(8) uint64_t bar_ak, bar_qy, bar_mma1, bar_mma2;
  uint32_t tmem_base;
};

struct BScanParams {
  const uint8_t* ws;        // workspace of the training forward (D; the tiles come through tensor maps)
  uint8_t* sc;              // scratch: receives dZ
  const void* d_out;        // [B,T,H,128]
  const float* ds_final;    // [B,H,128,128] or null
  float* d_bnd;             // [B, n_chunks+1, H,128,128]
  float* ds_init;           // [B,H,128,128] or null
  int* status;
  int64_t T, H, n_chunks, n_ch;
};

template <typename T>
__global__ void __launch_bounds__(kBScanThreads, 1)
chunk_bwd_scan_kernel(const BScanParams p, const __grid_constant__ CUtensorMap tm_at,
                      const __grid_constant__ CUtensorMap tm_tt, const __grid_constant__ CUtensorMap tm_kn,
                      const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_yt) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  BScanSmem& sm = *reinterpret_cast<BScanSmem*>(smem_raw);
  const WsLayout ws{p.n_ch, true};
  const ScratchLayout sc{p.n_ch};
  BoundedWaiter waiter(p.status);
  // a wait that ran out earlier (forward or backward) left garbage behind: results become NaN
  const bool upstream_failed = *static_cast<volatile const int*>(p.status) != kStatusOk;

  // 16 warps.  TMEM phases: warp & 3 = lane quadrant, warp >> 2 = quarter of the columns.
  // dO^T tile builder: warp = 4-token group tg, lane = 4-channel group.
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, part = warp >> 2;
  const int tg = warp;
  const int64_t bh = blockIdx.x;
  const int64_t b = bh / p.H, h = bh % p.H;
  constexpr uint32_t kColS = 0, kColR = 128, kColZ = 192;

  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&sm.bar_ak, 1);
    mbar_init(&sm.bar_qy, 1);
    mbar_init(&sm.bar_mma1, 1);
    mbar_init(&sm.bar_mma2, 1);
    fence_mbar_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = sm.tmem_base;
  const uint32_t lane_base = 32u * q4;
  const int vrow = 32 * q4 + lane;
  const int k0 = 32 * part, j0 = 16 * part;

  auto ch_of = [&](int64_t c) { return (b * p.n_chunks + c) * p.H + h; };
  auto load_ak = [&](int64_t c) {
    const int ch = int(ch_of(c));
    mbar_arrive_expect_tx(&sm.bar_ak, uint32_t(kTileAt + kTileKn + kTileTt - 2 * 4096));
    // At and Tt are zero for j >= 32, i < 32: three 32-row boxes each, the fourth quadrant stays zero
    tma_load_3d(sm.at, &tm_at, 0, 0, ch, &sm.bar_ak);
    tma_load_3d(sm.at + 8192, &tm_at, 32, 0, ch, &sm.bar_ak);
    tma_load_3d(sm.at + 8192 + 4096, &tm_at, 32, 32, ch, &sm.bar_ak);
#pragma unroll
    for (int s = 0; s < 4; ++s) tma_load_3d(sm.kn + s * 8192, &tm_kn, 32 * s, 0, ch, &sm.bar_ak);
    tma_load_3d(sm.tt, &tm_tt, 0, 0, ch, &sm.bar_ak);
    tma_load_3d(sm.tt + 8192, &tm_tt, 32, 0, ch, &sm.bar_ak);
    tma_load_3d(sm.tt + 8192 + 4096, &tm_tt, 32, 32, ch, &sm.bar_ak);
  };
  auto load_qy = [&](int64_t c) {
    const int64_t ch = ch_of(c);
    mbar_arrive_expect_tx(&sm.bar_qy, uint32_t(kTileQ + kTileYt + kBlobD));
#pragma unroll
    for (int s = 0; s < 4; ++s) tma_load_3d(sm.q + s * 8192, &tm_q, 32 * s, 0, int(ch), &sm.bar_qy);
#pragma unroll
    for (int s = 0; s < 2; ++s) tma_load_3d(sm.yt + s * 16384, &tm_yt, 32 * s, 0, int(ch), &sm.bar_qy);
    bulk_g2s(sm.d, p.ws + ws.off_d() + ch * kBlobD, uint32_t(kBlobD), &sm.bar_qy);
  };
  // dO of one chunk: 4 tokens x 4 channels per thread, still packed
  auto load_do = [&](int64_t c, typename Raw4<T>::type (&raw)[4]) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // past the end of a ragged sequence there is no cotangent: read the chunk's first token instead
      // (always there) and drop the value, so that no branch separates the loads
      const int64_t t = c * kChunk + 4 * tg + e;
      const typename Raw4<T>::type x =
          load4_raw<T>(p.d_out, ((b * p.T + (t < p.T ? t : c * kChunk)) * p.H + h) * kDim + 4 * lane);
      raw[e] = (t < p.T) ? x : typename Raw4<T>::type{};
    }
  };

  // lines 32..63 of the first slab of At and Tt (j >= 32, i < 32) are never loaded: zero, once
  for (int e = tid; e < 4096 / 16; e += kBScanThreads) {
    reinterpret_cast<float4*>(sm.at + 4096)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    reinterpret_cast<float4*>(sm.tt + 4096)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  fence_async_smem();
  typename Raw4<T>::type do_raw[4] = {};
  if (p.n_chunks > 0) {
    if (tid == 0) {
      load_ak(p.n_chunks - 1);
      load_qy(p.n_chunks - 1);
    }
    load_do(p.n_chunks - 1, do_raw);
  }

  // ---- dS^T <- dS_T^T (32 key rows of column v per thread); also becomes the last boundary slot ----
  {
    const float* src = (p.ds_final != nullptr) ? p.ds_final + bh * kStateElems + vrow : nullptr;
    float* slot = p.d_bnd + ((b * (p.n_chunks + 1) + p.n_chunks) * p.H + h) * kStateElems + vrow;
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = (src != nullptr) ? __float_as_uint(src[(k0 + j) * kDim]) : 0u;
#pragma unroll
    for (int j = 0; j < 32; ++j) slot[(k0 + j) * kDim] = __uint_as_float(r[j]);
    tmem_st32(tmem_addr(tb, lane_base, kColS + k0), r);
    tmem_wait_st();
  }

  uint32_t it = 0;
  for (int64_t c = p.n_chunks - 1; c >= 0; --c, ++it) {
    const uint32_t par = it & 1u;
    if (it > 0) {
      // previous iteration's second MMA group read dO^T, Qt, Yt and dR^T
      waiter.wait(&sm.bar_mma2, par ^ 1u);
      tc_fence_after();
      if (tid == 0) load_qy(c);
    }
    // ---- dO^T tile: one 16-byte chunk (4 tokens) per channel ------------------------------------------
    {
      float dv[4][4];
#pragma unroll
      for (int e = 0; e < 4; ++e) unpack4<T>(do_raw[e], dv[e]);
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        *reinterpret_cast<float4*>(sm.dot + blk_off<4>(4 * lane + f, 4 * tg, kRsDot, 128)) =
            make_float4(dv[0][f], dv[1][f], dv[2][f], dv[3][f]);
      }
    }
    if (it > 0) {
      // cotangent at the start of chunk c + 1 (= end of chunk c); off the MMA's critical path
      float* slot = p.d_bnd + ((b * (p.n_chunks + 1) + c + 1) * p.H + h) * kStateElems + vrow;
      uint32_t r[32];
      tmem_ld32(tmem_addr(tb, lane_base, kColS + k0), r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) slot[(k0 + j) * kDim] = __uint_as_float(r[j]);
    }
    fence_async_smem();
    waiter.wait(&sm.bar_ak, par);
    if (tid == 0) bulk_wait_read_all();  // the previous dZ tile has left its staging buffer
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const uint32_t d0 = smem_u32(sm.dot), a0 = smem_u32(sm.at), kn0 = smem_u32(sm.kn);
      const uint32_t id64 = idesc(128, 64, kFmtTF32, kMajorK, kMajorK);
      // dR^T = dO^T Aqk   (A: dO^T [v x i], B: At[j][i] read K-major)
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        mma_tf32_ss(tb + kColR, smem_desc(d0 + ks * 256, 128, kRsDot), smem_desc_sw128_k(a0, 8192, ks), id64,
                    ks > 0 ? 1u : 0u);
      }
      // dR^T += dS^T Kt^T (A: cotangent columns, K = 128 keys; B: Kn[j][k] read K-major)
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {
        mma_tf32_ts(tb + kColR, tb + kColS + ks * 8, smem_desc_sw128_k(kn0, 8192, ks), id64, 1u);
      }
      // dZ^T = dR^T T     (A: the accumulator just produced, K = 64 tokens; B: Tt[j][i] read K-major)
      const uint32_t tt0 = smem_u32(sm.tt);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        mma_tf32_ts(tb + kColZ, tb + kColR + ks * 8, smem_desc_sw128_k(tt0, 8192, ks), id64, ks > 0 ? 1u : 0u);
      }
      mma_commit(&sm.bar_mma1);
    }
    // the next chunk's dO is on its way while the tensor cores work
    if (c > 0) load_do(c - 1, do_raw);
    waiter.wait(&sm.bar_mma1, par);
    tc_fence_after();
    if (tid == 0 && c > 0) load_ak(c - 1);  // At / Kn are free again

    // ---- dZ out: 16 token columns of value row v into the staging tile X[r = j][c = v] ----------------
    {
      uint8_t* col = sm.dz + (vrow >> 2) * kCsZ + (vrow & 3) * 4;
      uint32_t r[16];
      tmem_ld16(tmem_addr(tb, lane_base, kColZ + j0), r);
      tmem_wait_ld();
#pragma unroll
      for (int jj = 0; jj < 16; ++jj) {
        const int j = j0 + jj;
        *reinterpret_cast<float*>(col + (j >> 3) * kRsZ + (j & 7) * 16) =
            (upstream_failed || waiter.dead) ? poison_nan() : to_tf32(__uint_as_float(r[jj]));
      }
    }
    // ---- decay: dS^T <- dS^T diag(d) -------------------------------------------------------------------
    waiter.wait(&sm.bar_qy, par);
    {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tb, lane_base, kColS + k0), r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sm.d[k0 + j]);
      tmem_st32(tmem_addr(tb, lane_base, kColS + k0), r);
      tmem_wait_st();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      bulk_s2g(p.sc + sc.off_dz() + ch_of(c) * kBlobDZ, sm.dz, uint32_t(kBlobDZ));
      bulk_commit();
      const uint32_t d0 = smem_u32(sm.dot), q0 = smem_u32(sm.q), y0 = smem_u32(sm.yt);
      const uint32_t id_pos = idesc(128, 128, kFmtTF32, kMajorK, kMajorMN);
      const uint32_t id_neg = idesc(128, 128, kFmtTF32, kMajorK, kMajorK, 1, 0);
      // dS^T += dO^T Qg   (K = 64 tokens; B: Q[i][k] read MN-major)
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        mma_tf32_ss(tb + kColS, smem_desc(d0 + ks * 256, 128, kRsDot), smem_desc_sw128_mn(q0, 8192, ks), id_pos, 1u);
      }
      // dS^T -= dR^T Y    (A: dR^T columns, K = 64 tokens; B: Yt[k][j] read K-major)
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        mma_tf32_ts(tb + kColS, tb + kColR + ks * 8, smem_desc_sw128_k(y0, 16384, ks), id_neg, 1u);
      }
      mma_commit(&sm.bar_mma2);
    }
  }

  // ---- cotangent of the initial state: slot 0 and d_initial_state ------------------------------------
  if (p.n_chunks > 0) {
    waiter.wait(&sm.bar_mma2, (it - 1) & 1u);
    tc_fence_after();
  }
  {
    float* slot = p.d_bnd + ((b * (p.n_chunks + 1)) * p.H + h) * kStateElems + vrow;
    float* init = (p.ds_init != nullptr) ? p.ds_init + bh * kStateElems + vrow : nullptr;
    uint32_t r[32];
    tmem_ld32(tmem_addr(tb, lane_base, kColS + k0), r);
    tmem_wait_ld();
    const bool failed = upstream_failed || waiter.dead;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float x = failed ? poison_nan() : __uint_as_float(r[j]);
      slot[(k0 + j) * kDim] = x;
      if (init != nullptr) init[(k0 + j) * kDim] = x;
    }
  }
  if (tid == 0) bulk_wait_all();  // the last dZ tile is in global memory before the CTA retires
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 256);
}


// =============================================================================================
// chunk VJP
// =============================================================================================
// 512 threads.  Elementwise phases: warp = 4-token group tg, lane = 4-channel group c4 (as in the
// forward prep kernel).  TMEM phases: warp & 3 = lane quadrant, warp >> 2 = share of the columns.
// Final chain: thread = (key channel, 16-token block).
constexpr int kVjpThreads = 512;
constexpr int kCsN = 144;              // natural 128-column tiles: padded chunk stride
constexpr int kRsN = 32 * kCsN;        // 4608
constexpr int kRsT = 2064;             // transposed 64-column tiles: padded row-group stride
constexpr int kCsS = 144;              // 64-column tiles written by scattered 4-byte stores
constexpr int kRsS = 16 * kCsS;        // 2304

// dynamic shared memory map (bytes).  Phase B = products with the states, phase C = Gram VJP.
constexpr int kOffStack = 0;                      // B: [dZ ; dO] X[r = 128][c = v], RS kRsN     73728 (dZ rows: bulk copy)
constexpr int kOffRn = kOffStack + 16 * kRsN;     // B: R[j][v], 4 swizzled slabs of 64 lines    32768
constexpr int kOffS0 = kOffRn + 32768;            // B: S_0[k][v], 4 swizzled slabs of 128 lines  65536
constexpr int kOffDs1 = kOffS0 + 65536;           // B: dS_1[k][64 v] half, 2 swizzled slabs      32768
static_assert(kOffS0 % 1024 == 0 && kOffDs1 % 1024 == 0, "swizzled tiles are 1024-byte aligned");
constexpr int kEndB = kOffDs1 + 32768;            // 204800
constexpr int kOffStack2 = 0;                     // C: [dL_I ; dA_I] for I = 0..3, X[r = 128][c = j], RS 2048   32768
constexpr int kOffDLt = 32768;                    // C: dL^T X[r = j][c = i], RS kRsS            18432
constexpr int kOffDAt = kOffDLt + 8 * kRsS;       // C: dA^T                                     18432
constexpr int kOffKIt = kOffDAt + 8 * kRsS;       // C: (K^I)^T X[r = k][c = j < 16 (I+1)], RS 512 (I+1) + 16
constexpr int kKItBytes = 16 * (528 + 1040 + 1552 + 2064);  // 82944
constexpr int kOffEat = kOffKIt + kKItBytes;      // C: E_a^T X[r = k][c = i], RS kRsT           33024
constexpr int kOffQat = kOffEat + 16 * kRsT;      // C: Q_a^T                                    33024
constexpr int kEndC = kOffQat + 16 * kRsT;        // 218624
// final chain: k and q of the unit as 16-bit [64][128] tiles over the dO rows of the stack (dk and dq
// replace them in place and leave by tiled TMA stores), the log-decay prefix G as an fp32 tile over
// the dS_1 buffer.  The next unit's prefetch keeps clear of both until the chain is over.
constexpr int kOffTileK = kOffStack + 8 * kRsN;   // 36864
constexpr int kOffTileQ = kOffTileK + 16384;
constexpr int kOffTileG = kOffDs1;
// beta (dbeta in place) has no 16 KiB hole left: its 16-token blocks 0..2 sit behind the dS_1 buffer,
// block 3 in the last 4 KiB of the dO rows; a chain thread works on one block, so it sees one base
constexpr int kOffTileB012 = kEndB;               // 204800, 12 KiB
constexpr int kOffTileB3 = kOffTileQ + 16384;     // 69632, 4 KiB
static_assert(kOffTileB3 + 4096 <= kOffRn, "chain tiles exceed the dO rows of the stack");
static_assert(kOffTileB012 + 12288 <= kEndC, "beta tile exceeds the free space behind the dS_1 buffer");
__device__ __forceinline__ int beta_tile_offset(int blk) { return blk < 3 ? kOffTileB012 + blk * 4096 : kOffTileB3; }
constexpr int kOffMisc = (kEndB > kEndC ? kEndB : kEndC);
struct VjpMisc {
  float part[16][kDim];   // exclusive prefixes of the log-decay per 4-token group
  float gend[kDim];
  float xe[4][kDim];      // per-block sum_j Kt_j dKt_j
  float xt[4][kDim];      // partial sums of dd = sum_v dS_1 * S_0, then the per-block sums of dG
  alignas(8) uint64_t bar_a, bar_s, bar_r, bar_m, bar_d;
  uint32_t tmem_base;
};
constexpr int kVjpSmemBytes = kOffMisc + int(sizeof(VjpMisc));
static_assert(kVjpSmemBytes <= 232448, "VJP kernel exceeds the 227 KiB shared-memory limit");

__device__ __forceinline__ int kit_rs(int I) { return 512 * (I + 1) + 16; }
__device__ __forceinline__ int kit_offset(int I) {
  return kOffKIt + 16 * ((I == 0) ? 0 : (I == 1) ? 528 : (I == 2) ? (528 + 1040) : (528 + 1040 + 1552));
}
__device__ __forceinline__ uint32_t d6_col(int I) { return (I == 3) ? 0u : (I == 2) ? 64u : (I == 1) ? 448u : 480u; }

struct VjpParams {
  const void *q, *k, *v, *g, *beta, *w, *d_out;
  const uint8_t* ws;    // workspace of the training forward (Rn)
  const uint8_t* sc;    // scratch: dZ written by the reverse scan
  const float* bnd;     // [B, n_chunks+1, H,128,128] forward states
  const float* d_bnd;   // same shape, cotangents
  void *dq, *dk, *dv, *dg, *dbeta, *dw;
  int* status;
  int64_t T, H, n_chunks, n_ch;
  float scale;
};
// tensor maps of the seven sequence tensors the VJP kernel reads (for L2 prefetches only)
struct VjpInputMaps {
  CUtensorMap q, k, v, g, beta, w, d_out;
};

template <typename T>
__device__ __forceinline__ void load4v(const void* base, int64_t idx, float (&out)[4]);
template <>
__device__ __forceinline__ void load4v<__nv_bfloat16>(const void* base, int64_t idx, float (&out)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + idx);
  out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
  out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
}
template <>
__device__ __forceinline__ void load4v<__half>(const void* base, int64_t idx, float (&out)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __half*>(base) + idx);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}
template <>
__device__ __forceinline__ void load4v<float>(const void* base, int64_t idx, float (&out)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
}

template <typename T>
__device__ __forceinline__ void store4v(void* base, int64_t idx, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4v<__nv_bfloat16>(void* base, int64_t idx, float a, float b, float c, float d) {
  *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + idx) = make_uint2(pack_bf16(a, b), pack_bf16(c, d));
}
template <>
__device__ __forceinline__ void store4v<float>(void* base, int64_t idx, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4v<__half>(void* base, int64_t idx, float a, float b, float c, float d) {
  const __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
  *reinterpret_cast<uint2*>(static_cast<__half*>(base) + idx) =
      make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// tf32 value of k times its anchored decay, as stored in the (K^I)^T tiles: `decay` alone, or
// `decay * far` for row blocks beyond the next one.  Tile build and chain both call this, so that the
// chain multiplies the Gram cotangents by exactly the operand values the tensor cores saw.
__device__ __forceinline__ float anchored_k(float k, float decay, float far, bool use_far) {
  return to_tf32(k * (use_far ? decay * far : decay));
}
// the same product for the tile itself, which only the tensor cores read (they drop the low bits themselves)
__device__ __forceinline__ float anchored_k_operand(float k, float decay, float far, bool use_far) {
  return to_tf32_operand(k * (use_far ? decay * far : decay));
}

__device__ __forceinline__ void tmem_ld8f(uint32_t taddr, float (&x)[8]) {
  uint32_t r[8];
  tmem_ld8(taddr, r);
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = __uint_as_float(r[i]);
}

// kF32Grads: dq, dk, dv, dbeta, dw leave as fp32 instead of the sequence dtype (the values before
// their final rounding; used by tests to judge the arithmetic apart from the 16-bit cast).
// kRagged: the sequence length is not a multiple of 64 and the last chunk of every (batch, head) is
// partial; only this instantiation carries the guards (they cost the others 6 %).
template <typename T, typename G, bool kF32Grads = false, bool kRagged = false>
__global__ void __launch_bounds__(kVjpThreads, 1)
chunk_bwd_vjp_kernel(const VjpParams p, const __grid_constant__ CUtensorMap tm_s0,
                     const __grid_constant__ CUtensorMap tm_ds, const __grid_constant__ CUtensorMap tm_rn,
                     const __grid_constant__ CUtensorMap tm_dq, const __grid_constant__ CUtensorMap tm_dk,
                     const __grid_constant__ CUtensorMap tm_dbeta, const __grid_constant__ VjpInputMaps tm_in) {
  using O = typename std::conditional<kF32Grads, float, T>::type;  // element type of dq, dk, dv, dbeta, dw
  extern __shared__ __align__(1024) uint8_t smem[];
  VjpMisc& ms = *reinterpret_cast<VjpMisc*>(smem + kOffMisc);
  const WsLayout ws{p.n_ch, true};
  const ScratchLayout sc{p.n_ch};
  BoundedWaiter waiter(p.status);
  // a wait that ran out earlier (forward or reverse scan) left garbage behind: gradients become NaN
  const bool upstream_failed = *static_cast<volatile const int*>(p.status) != kStatusOk;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, part = warp >> 2;
  const int tg = warp, c4 = lane, kc0 = 4 * lane;

  if (warp == 0) {
    tmem_alloc(&ms.tmem_base, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&ms.bar_a, 1);
    mbar_init(&ms.bar_r, 1);
    mbar_init(&ms.bar_m, 1);
    mbar_init(&ms.bar_d, 1);
    mbar_init(&ms.bar_s, 1);
    fence_mbar_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = ms.tmem_base;
  uint32_t mma_phase = 0;
  constexpr uint32_t kColD2 = 64, kColD3 = 128, kColD4 = 256, kColD5 = 320;

  // Everything the first MMA batch of a chunk-head reads arrives asynchronously: the dZ rows of the
  // stack and the residual R as 1-D bulk copies, S_0 and the first 64 value columns of dS_1 as tiled TMA
  // loads (128-byte swizzle) that put the row-major fp32 checkpoints into shared memory as K-major
  // operands, 32 value columns per slab (the tensor cores read the fp32 containers as tf32).  No
  // register staging.  The kernel is persistent: one SM takes in bytes at a limited rate, so the copies
  // for the CTA's next chunk-head are issued as soon as the last MMA of the current one has read shared
  // memory, and land during its final chain.
  // The chain keeps the dO rows of the stack and the dS_1 buffer for its own tiles, so the copies come in
  // two parts: S_0, R and dZ before the chain, the dS_1 half after it (bar_s expects both from the start).
  auto s0_slot_of = [&](int64_t ch_) {
    const int64_t h_ = ch_ % p.H, c_ = (ch_ / p.H) % p.n_chunks, b_ = ch_ / (p.H * p.n_chunks);
    return int((b_ * (p.n_chunks + 1) + c_) * p.H + h_);
  };
  auto issue_loads = [&](int64_t ch_) {
    mbar_arrive_expect_tx(&ms.bar_s, uint32_t(65536 + 32768));
#pragma unroll
    for (int sl = 0; sl < 4; ++sl) tma_load_3d(smem + kOffS0 + sl * 16384, &tm_s0, 32 * sl, 0, s0_slot_of(ch_), &ms.bar_s);
    mbar_arrive_expect_tx(&ms.bar_a, uint32_t(kBlobDZ + kBlobRn));
#pragma unroll
    for (int sl = 0; sl < 4; ++sl) tma_load_3d(smem + kOffRn + sl * 8192, &tm_rn, 32 * sl, 0, int(ch_), &ms.bar_a);
    bulk_g2s(smem + kOffStack, p.sc + sc.off_dz() + ch_ * kBlobDZ, uint32_t(kBlobDZ), &ms.bar_a);
  };
  auto issue_ds1 = [&](int64_t ch_) {
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
      tma_load_3d(smem + kOffDs1 + sl * 16384, &tm_ds, 32 * sl, 0, s0_slot_of(ch_) + int(p.H), &ms.bar_s);
    }
  };
  if (tid == 0 && int64_t(blockIdx.x) < p.n_ch) {
    issue_loads(blockIdx.x);
    issue_ds1(blockIdx.x);
  }

  uint32_t iter = 0;
  for (int64_t ch = blockIdx.x; ch < p.n_ch; ch += gridDim.x, ++iter) {
  const uint32_t par = iter & 1u;
  // (unit numbers fit 31 bits, the launcher checks: 32-bit divisions, a fraction of the 64-bit routine)
  const uint32_t bc32 = uint32_t(ch) / uint32_t(p.H);
  const int64_t h = uint32_t(ch) - bc32 * uint32_t(p.H);
  const int64_t b = bc32 / uint32_t(p.n_chunks);
  const int64_t c = bc32 - uint32_t(b) * uint32_t(p.n_chunks);
  const int64_t t0 = c * kChunk;
  auto seq_idx = [&](int tok) { return ((b * p.T + t0 + tok) * p.H + h) * int64_t(kDim); };
  // tokens of this chunk that exist: 64 except in the last chunk of a ragged sequence, whose missing
  // tokens read as zeros (the identity step) and whose gradients are not stored
  const int n_valid = kRagged ? int(min(int64_t(kChunk), p.T - t0)) : kChunk;
  auto there = [&](int tok) { return !kRagged || tok < n_valid; };            // does token `tok` of the chunk exist
  auto clamped = [&](int tok) { return kRagged ? min(tok, n_valid - 1) : tok; };  // a token that does
  const int ds1_slot = int((b * (p.n_chunks + 1) + c + 1) * p.H + h);
  // dd[k] += sum over the 64 value columns of half `hf` of dS_1[k][v] S_0[k][v], both read from their
  // shared-memory tiles.  The two tiles are swizzled alike (a line = 32 values of one key row, its
  // 16-byte pieces permuted by the row), so equal positions hold equal (k, v) and the order inside a
  // line does not matter for the sum.  Piece qd = tid + 512 x: line (qd >> 3) = slab * 128 + k, piece qd & 7.
  auto dd_half = [&](int hf) {
#pragma unroll
    for (int x = 0; x < 4; ++x) {
      const int qd = tid + 512 * x;
      const int line = qd >> 3, slab = line >> 7, kr = line & 127;
      const float4 ds = *reinterpret_cast<const float4*>(smem + kOffDs1 + slab * 16384 + kr * 128 + (qd & 7) * 16);
      const float4 s0 = *reinterpret_cast<const float4*>(smem + kOffS0 + (2 * hf + slab) * 16384 + kr * 128 + (qd & 7) * 16);
      float acc = ds.x * s0.x + ds.y * s0.y + ds.z * s0.z + ds.w * s0.w;
      // the 8 lanes of a line
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      // one owner per (half, slab, key row): partial sums in fixed slots, no atomics, so that the result
      // does not depend on the timing of the warps (xt is free until the end of the chain)
      if ((lane & 7) == 0) ms.xt[2 * hf + slab][kr] = acc;
    }
  };

  // ---- phase A: dO rows of the stack (rows 64 + i), natural tile with padded chunk stride, and the
  // log-decay sums of this thread's tokens
  float Gc[4][4];
  {
    float dv4[4][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // a token past the end of a ragged sequence: the last real token is read instead (no branch around
      // the loads, they are all issued back to back) and its value dropped below
      const int64_t idx = seq_idx(clamped(4 * tg + e)) + kc0;
      load4v<T>(p.d_out, idx, dv4[e]);
      load4v<G>(p.g, idx, Gc[e]);
    }
    if (kRagged && n_valid < kChunk) {  // CTA-uniform; false for every chunk but the last one of a sequence
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (!there(4 * tg + e)) {
#pragma unroll
          for (int f = 0; f < 4; ++f) dv4[e][f] = Gc[e][f] = 0.f;
        }
      }
    }
    if (!kF32Grads) {
      // the dk / dq tiles of the previous unit lie where the dO rows go: their stores must have read them
      if (tid == 0) bulk_wait_read_all();
      __syncthreads();
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 4 * tg + e;
      *reinterpret_cast<float4*>(smem + kOffStack + ((64 + i) >> 3) * kRsN + c4 * kCsN + (i & 7) * 16) =
          make_float4(dv4[e][0], dv4[e][1], dv4[e][2], dv4[e][3]);
      if (e > 0) {
#pragma unroll
        for (int f = 0; f < 4; ++f) Gc[e][f] += Gc[e - 1][f];
      }
    }
  }
#pragma unroll
  for (int f = 0; f < 4; ++f) ms.part[tg][kc0 + f] = Gc[3][f];
  waiter.wait(&ms.bar_a, par);
  waiter.wait(&ms.bar_s, par);
  dd_half(0);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  // ---- first MMA batch: M4 (first half) dKt^T = dS_1[:, v < 64] R[:, v < 64]^T ;
  //      M2 [-dL ; dA] = [dZ ; dO] R^T ;  M3 [-dE ; dQg]^T = S_0 [dZ ; dO]^T ------------------------------
  if (tid == 0) {
    tc_fence_after();
    const uint32_t st = smem_u32(smem + kOffStack), rn = smem_u32(smem + kOffRn);
    const uint32_t s0 = smem_u32(smem + kOffS0), d1 = smem_u32(smem + kOffDs1);
    const uint32_t id64 = idesc(128, 64, kFmtTF32, kMajorK, kMajorK);
    const uint32_t id128 = idesc(128, 128, kFmtTF32, kMajorK, kMajorK);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      mma_tf32_ss(tb + kColD4, smem_desc_sw128_k(d1, 16384, ks), smem_desc_sw128_k(rn, 8192, ks), id64,
                  ks > 0 ? 1u : 0u);
    }
    mma_commit(&ms.bar_r);  // the dS_1 buffer may be refilled once these have run
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      mma_tf32_ss(tb + kColD2, smem_desc(st + ks * 2 * kCsN, kCsN, kRsN), smem_desc_sw128_k(rn, 8192, ks), id64,
                  ks > 0 ? 1u : 0u);
    }
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      mma_tf32_ss(tb + kColD3, smem_desc_sw128_k(s0, 16384, ks), smem_desc(st + ks * 2 * kCsN, kCsN, kRsN), id128,
                  ks > 0 ? 1u : 0u);
    }
    mma_commit(&ms.bar_m);
    // the second 64 value columns of dS_1 replace the first as soon as their product has run
    waiter.wait(&ms.bar_r, 0);
    mbar_arrive_expect_tx(&ms.bar_d, 32768u);
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) tma_load_3d(smem + kOffDs1 + sl * 16384, &tm_ds, 64 + 32 * sl, 0, ds1_slot, &ms.bar_d);
  }
  // ---- under the tensor cores: log-decay prefixes, dv = dZ w, dw = dZ v, and the raw inputs of the
  // Gram operands.  Every load is issued before the first store: the outputs may alias the inputs as
  // far as the compiler knows, so a load placed after a store would wait for its round trip.
  if (tid < kDim) {
    float run = 0.f;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const float x = ms.part[t][tid];
      ms.part[t][tid] = run;
      run += x;
    }
    ms.gend[tid] = run;
  }
  const int mb = tg >> 2;
  float kk[4][4], qq[4][4], bb[4][4];
  {
    typename Raw4<T>::type wr[4], vr[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int64_t idx = seq_idx(clamped(4 * tg + e)) + kc0;  // see phase A
      wr[e] = load4_raw<T>(p.w, idx);
      vr[e] = load4_raw<T>(p.v, idx);
      load4v<T>(p.k, idx, kk[e]);
      load4v<T>(p.q, idx, qq[e]);
      load4v<T>(p.beta, idx, bb[e]);
    }
    if (kRagged && n_valid < kChunk) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (!there(4 * tg + e)) {
#pragma unroll
          for (int f = 0; f < 4; ++f) kk[e][f] = qq[e][f] = bb[e][f] = 0.f;
        }
      }
    }
    // (the ragged instantiation has the one, predicated copy of these stores: a second, unpredicated copy
    // for the warps whose tokens all exist made it slower, that kernel is close to the size of the
    // instruction cache)
    auto store_dv_dw = [&](auto guarded) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = 4 * tg + e;
        float4 dz = *reinterpret_cast<const float4*>(smem + kOffStack + (j >> 3) * kRsN + c4 * kCsN + (j & 7) * 16);
        if (upstream_failed || waiter.dead) dz = make_float4(poison_nan(), poison_nan(), poison_nan(), poison_nan());
        const int64_t idx = seq_idx(j) + kc0;
        float wv[4], vv[4];
        unpack4<T>(wr[e], wv);
        unpack4<T>(vr[e], vv);
        if (!decltype(guarded)::value || j < n_valid) {
          store4v<O>(p.dv, idx, dz.x * wv[0], dz.y * wv[1], dz.z * wv[2], dz.w * wv[3]);
          store4v<O>(p.dw, idx, dz.x * vv[0], dz.y * vv[1], dz.z * vv[2], dz.w * vv[3]);
        }
      }
    };
    if (!kRagged) store_dv_dw(std::false_type{});
    else store_dv_dw(std::true_type{});
  }
  // ---- M4 (second half) once the second half of dS_1 has landed -----------------------------------------
  waiter.wait(&ms.bar_d, par);
  dd_half(1);
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc_fence_after();
    const uint32_t rn = smem_u32(smem + kOffRn), d1 = smem_u32(smem + kOffDs1);
    const uint32_t id64 = idesc(128, 64, kFmtTF32, kMajorK, kMajorK);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      mma_tf32_ss(tb + kColD4, smem_desc_sw128_k(d1, 16384, ks), smem_desc_sw128_k(rn, 8192, 8 + ks), id64, 1u);
    }
    mma_commit(&ms.bar_r);
  }
  waiter.wait(&ms.bar_m, mma_phase & 1u);
  ++mma_phase;
  tc_fence_after();

  // ================================ phase C: Gram VJP =============================================
  // [-dL_raw ; dA_raw] out of TMEM: masked tiles [dL ; dA] (rows) and their transposes; the four
  // warps of a quadrant take 16 columns each.  These tiles lie over the [dZ ; dO] stack, whose last
  // readers (the first MMA batch and the dv / dw pass) are done; R and the dS_1 buffer may still be
  // read by the second half of M4 and are not touched before the wait further down.
  {
    const int r = 32 * q4 + lane, i = r & 63;
    // row of the stacked tile: the dL and dA rows of a 16-token block sit next to each other, so that
    // one N = 32 instruction multiplies both by (K^I)^T
    const int row2 = 32 * (i >> 4) + ((r < 64) ? 0 : 16) + (i & 15);
    uint8_t* tr_base = smem + ((r < 64) ? kOffDLt : kOffDAt);
    const int c0 = 16 * part;
    uint32_t raw[16];
    tmem_ld16(tmem_addr(tb, 32 * q4, kColD2 + c0), raw);
    tmem_wait_ld();
    float vals[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int col = c0 + j;
      const float x = __uint_as_float(raw[j]);
      vals[j] = to_tf32_operand((r < 64) ? ((col < i) ? -x : 0.f) : ((col <= i) ? x : 0.f));
      *reinterpret_cast<float*>(tr_base + (col >> 3) * kRsS + (i >> 2) * kCsS + (col & 7) * 16 + (i & 3) * 4) = vals[j];
    }
#pragma unroll
    for (int j4 = 0; j4 < 4; ++j4) {
      *reinterpret_cast<float4*>(smem + kOffStack2 + blk_off<4>(row2, c0 + 4 * j4, 2048, 128)) =
          make_float4(vals[4 * j4], vals[4 * j4 + 1], vals[4 * j4 + 2], vals[4 * j4 + 3]);
    }
  }
  // anchored Gram operands, transposed tiles X[r = channel][c = token] with padded row-group stride.
  // They overwrite R and the dS_1 buffer: the second half of M4 must have run.
  waiter.wait(&ms.bar_r, 1);
  tc_fence_after();
  {
    float eat[4][4], qat[4][4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int kc = kc0 + f;
        const float Gi = Gc[e][f] + ms.part[tg][kc];
        Gc[e][f] = Gi;
        const float anchored = __expf(Gi - ms.part[4 * mb][kc]);
        eat[e][f] = to_tf32_operand(bb[e][f] * kk[e][f] * anchored);
        qat[e][f] = to_tf32_operand(p.scale * qq[e][f] * anchored);
      }
    }
#pragma unroll
    for (int f = 0; f < 4; ++f) {
      const uint32_t off = blk_off<4>(kc0 + f, 4 * tg, kRsT, 128);
      *reinterpret_cast<float4*>(smem + kOffEat + off) = make_float4(eat[0][f], eat[1][f], eat[2][f], eat[3][f]);
      *reinterpret_cast<float4*>(smem + kOffQat + off) = make_float4(qat[0][f], qat[1][f], qat[2][f], qat[3][f]);
    }
    // (K^I)^T for every row block I >= the token's own block mb, three exponentials per element:
    //   I = mb      k exp(a_mb - G)                      (own block: >= 1, bounded by the 16-token contract)
    //   I = mb + 1  k exp(a_next - G)                    (a_next = start of the next block)
    //   I > mb + 1  k (exp(a_next - G) exp(a_I - a_next))
    // The final chain forms the same products with the same expressions (anchored_k below).
#pragma unroll
    for (int f = 0; f < 4; ++f) {
      const int kc = kc0 + f;
      const float a_mb = ms.part[4 * mb][kc];
      const float a_nx = (mb < 3) ? ms.part[4 * (mb + 1)][kc] : ms.gend[kc];
      const float c_nx = __expf(a_nx - a_mb);  // decay over the whole 16-token block
      float own[4], nb[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        own[e] = __expf(a_mb - Gc[e][f]);
        nb[e] = own[e] * c_nx;                 // exp(a_nx - G): the chain forms it the same way
      }
#pragma unroll
      for (int I = 0; I < 4; ++I) {
        if (I >= mb) {
          const float far = (I > mb + 1) ? __expf(ms.part[4 * I][kc] - a_nx) : 1.f;
          float val[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) val[e] = anchored_k_operand(kk[e][f], (I == mb) ? own[e] : nb[e], far, I > mb + 1);
          *reinterpret_cast<float4*>(smem + kit_offset(I) + blk_off<4>(kc, 4 * tg, kit_rs(I), 128)) =
              make_float4(val[0], val[1], val[2], val[3]);
        }
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (tid == 0) {
    tc_fence_after();
    const uint32_t s2 = smem_u32(smem + kOffStack2);
    const uint32_t dlt = smem_u32(smem + kOffDLt), dat = smem_u32(smem + kOffDAt);
    const uint32_t eat0 = smem_u32(smem + kOffEat), qat0 = smem_u32(smem + kOffQat);
    const uint32_t id32 = idesc(128, 32, kFmtTF32, kMajorK, kMajorK);
    // [dEa_I^T | dQa_I^T] (columns 32 I .. 32 I + 31) = (K^I)^T x the 32 stacked rows [dL_I ; dA_I]
#pragma unroll
    for (int I = 0; I < 4; ++I) {
      const uint32_t kit = smem_u32(smem + kit_offset(I));
      const uint32_t rs = uint32_t(kit_rs(I));
      for (int ks = 0; ks < 2 * (I + 1); ++ks) {
        mma_tf32_ss(tb + kColD5 + 32 * I, smem_desc(kit + ks * 256, 128, rs),
                    smem_desc(s2 + 4 * I * 2048 + ks * 256, 128, 2048), id32, ks > 0 ? 1u : 0u);
      }
    }
    // (dK^I)^T = Ea^T[:, block I] dL[block I, :] + Qa^T[:, block I] dA[block I, :]
#pragma unroll
    for (int I = 0; I < 4; ++I) {
      const uint32_t idn = idesc(128, 16 * (I + 1), kFmtTF32, kMajorK, kMajorK);
#pragma unroll
      for (int pt = 0; pt < 2; ++pt) {
        const uint32_t a_base = (pt ? qat0 : eat0) + 4 * I * 128;
        const uint32_t b_base = (pt ? dat : dlt) + 4 * I * kCsS;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          mma_tf32_ss(tb + d6_col(I), smem_desc(a_base + ks * 256, 128, kRsT),
                      smem_desc(b_base + ks * 2 * kCsS, kCsS, kRsS), idn, (pt | ks) ? 1u : 0u);
        }
      }
    }
    mma_commit(&ms.bar_m);
  }
  waiter.wait(&ms.bar_m, mma_phase & 1u);
  ++mma_phase;
  tc_fence_after();
  // shared memory (all but the small arrays of VjpMisc) is dead from here on: fetch the next chunk-head
  if (tid == 0 && ch + gridDim.x < p.n_ch) issue_loads(ch + gridDim.x);
  // The sequence tensors of the next chunk-head are read with per-thread loads, whose rate is set by the
  // bytes in flight over the latency: have its seven [64][128] tiles brought into L2 while the chain runs.
  if (tid == 64 && ch + gridDim.x < p.n_ch) {
    const int64_t ch_ = ch + gridDim.x;
    const int h_ = int(ch_ % p.H), t_ = int((ch_ / p.H) % p.n_chunks) * kChunk, b_ = int(ch_ / (p.H * p.n_chunks));
    tma_prefetch_l2_4d(&tm_in.d_out, 0, h_, t_, b_);
    tma_prefetch_l2_4d(&tm_in.g, 0, h_, t_, b_);
    tma_prefetch_l2_4d(&tm_in.w, 0, h_, t_, b_);
    tma_prefetch_l2_4d(&tm_in.v, 0, h_, t_, b_);
    tma_prefetch_l2_4d(&tm_in.k, 0, h_, t_, b_);
    tma_prefetch_l2_4d(&tm_in.q, 0, h_, t_, b_);
    tma_prefetch_l2_4d(&tm_in.beta, 0, h_, t_, b_);
  }
  // hand k, q and the log-decay prefix to the chain, which walks the tokens of one channel: these threads
  // hold them as 4 x 4 patches (the same values, and for G the same summation order, as the tiles above)
  {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int off = (4 * tg + e) * kDim + kc0;
      store4v<T>(smem + kOffTileK, off, kk[e][0], kk[e][1], kk[e][2], kk[e][3]);
      store4v<T>(smem + kOffTileQ, off, qq[e][0], qq[e][1], qq[e][2], qq[e][3]);
      store4v<T>(smem + beta_tile_offset(mb), (4 * (tg & 3) + e) * kDim + kc0, bb[e][0], bb[e][1], bb[e][2], bb[e][3]);
      store4v<float>(smem + kOffTileG, off, Gc[e][0], Gc[e][1], Gc[e][2], Gc[e][3]);
    }
    __syncthreads();
  }

  // ================================ per-channel chain ==============================================
  // One thread = one key channel over one 16-token block.  The log-decay G and the anchored operands
  // are re-evaluated with exactly the expressions (and summation order) used when the MMA tiles were
  // built, so that dG multiplies each Gram cotangent by the very tf32 value the tensor cores saw:
  // the row and column contributions of the Gram products to dG then cancel as they do exactly.
  {
    const int kc = tid & 127, blk = part;
    const bool failed = upstream_failed || waiter.dead;
    const float gend = ms.gend[kc];
    // dd[k] = sum_v dS_1[k][v] S_0[k][v]: read here, before xt is reused for the block sums of dG
    const float dd_k = (ms.xt[0][kc] + ms.xt[1][kc]) + (ms.xt[2][kc] + ms.xt[3][kc]);
    const float a_me = ms.part[4 * blk][kc];
    const float a_nx = (blk < 3) ? ms.part[4 * (blk + 1)][kc] : gend;
    // per-thread constants: everything but three exponentials per token comes from these
    const float e_ame = __expf(a_me);            // exp(G) = exp(G - a_me) e_ame
    const float c_nx = __expf(a_nx - a_me);      // exp(a_next - G) = exp(a_me - G) c_nx, as in the tile build
    const float t_end = __expf(gend - a_nx);     // exp(G_end - G) = exp(a_next - G) t_end
    const float far2 = (blk + 2 < 4) ? __expf(ms.part[4 * (blk + 2)][kc] - a_nx) : 1.f;  // row block blk + 2
    const float far3 = (blk + 3 < 4) ? __expf(ms.part[4 * (blk + 3)][kc] - a_nx) : 1.f;  // row block blk + 3
    // dG of a token goes back into the slot of the G tile this thread read its log-decay from (nobody else
    // touches it), and the two halves of the block run as a loop: the kernel is a long stretch of
    // straight-line code that every warp walks once per unit, and what it does not need to hold twice
    // saves instruction fetches
    float e_part = 0.f, tot = 0.f;
#pragma unroll 1
    for (int sb = 0; sb < 2; ++sb) {
      const int i0 = 16 * blk + 8 * sb;
      float Gb[8], kv[8], bv[8], sq[8], P3[8], P2[8], dG[8], x[8], y[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int off = (i0 + t) * kDim + kc;
        Gb[t] = ldf<float>(smem + kOffTileG, off);
        kv[t] = ldf<T>(smem + kOffTileK, off);
        sq[t] = p.scale * ldf<T>(smem + kOffTileQ, off);
        bv[t] = ldf<T>(smem + beta_tile_offset(blk), (8 * sb + t) * kDim + kc);
      }
      // row blocks I = blk + d that contain these tokens as columns, nearest first: the own block uses
      // exp(a_me - G), the others exp(a_next - G) (times the block-to-block factor from d = 2 on)
      tmem_ld8f(tmem_addr(tb, 32 * q4, d6_col(blk) + i0), x);  // dK^blk
      float nb[8];
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float own = __expf(a_me - Gb[t]);
        nb[t] = own * c_nx;
        Gb[t] = __expf(Gb[t] - a_me);  // from here on Gb holds the anchored decay exp(G - a_me)
        P3[t] = x[t] * own;
        dG[t] = -anchored_k(kv[t], own, 1.f, false) * x[t];
      }
      tmem_ld8f(tmem_addr(tb, 32 * q4, kColD4 + i0), x);  // dKt
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float et = nb[t] * t_end;
        const float kt = kv[t] * et;
        P3[t] = fmaf(x[t], et, P3[t]);
        e_part = fmaf(kt, x[t], e_part);
        dG[t] = fmaf(-kt, x[t], dG[t]);
      }
#pragma unroll
      for (int d = 1; d < 4; ++d) {
        if (blk + d < 4) {
          const float far = (d == 2) ? far2 : far3;
          tmem_ld8f(tmem_addr(tb, 32 * q4, d6_col(blk + d) + i0), x);  // dK^(blk + d)
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const float ex = (d > 1) ? nb[t] * far : nb[t];
            P3[t] = fmaf(x[t], ex, P3[t]);
            dG[t] = fmaf(-anchored_k(kv[t], nb[t], far, d > 1), x[t], dG[t]);
          }
        }
      }
      tmem_ld8f(tmem_addr(tb, 32 * q4, kColD3 + i0), x);  // -dE (state part)
      tmem_ld8f(tmem_addr(tb, 32 * q4, kColD5 + 32 * blk + 8 * sb), y);  // dEa
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const float ea = Gb[t], eg = ea * e_ame;
        const float de = -x[t], dea = y[t];
        P2[t] = fmaf(de, eg, dea * ea);
        const float bk = bv[t] * kv[t];
        dG[t] = fmaf(bk * eg, de, dG[t]);
        dG[t] = fmaf(to_tf32(bk * ea), dea, dG[t]);
      }
      tmem_ld8f(tmem_addr(tb, 32 * q4, kColD3 + 64 + i0), x);  // dQg (state part)
      tmem_ld8f(tmem_addr(tb, 32 * q4, kColD5 + 32 * blk + 16 + 8 * sb), y);  // dQa
#pragma unroll
      for (int t = 0; t < 8; ++t) {
        const int64_t idx = seq_idx(i0 + t) + kc;
        const float ea = Gb[t], eg = ea * e_ame;
        const float P1 = failed ? poison_nan() : fmaf(x[t], eg, y[t] * ea);
        const float dGt = fmaf(to_tf32(sq[t] * ea), y[t], fmaf(sq[t] * eg, x[t], dG[t]));
        const float dk_t = failed ? poison_nan() : fmaf(bv[t], P2[t], P3[t]);
        if (kF32Grads) {
          if (there(i0 + t)) {
            stf<O>(p.dq, idx, p.scale * P1);
            stf<O>(p.dk, idx, dk_t);
          }
        } else {
          // in place over q and k (this thread's own slots, already read): the tiles leave by TMA stores
          const int off = (i0 + t) * kDim + kc;
          stf<T>(smem + kOffTileQ, off, p.scale * P1);
          stf<T>(smem + kOffTileK, off, dk_t);
          stf<T>(smem + beta_tile_offset(blk), (8 * sb + t) * kDim + kc, failed ? poison_nan() : kv[t] * P2[t]);
        }
        if (kF32Grads && there(i0 + t)) stf<O>(p.dbeta, idx, failed ? poison_nan() : kv[t] * P2[t]);
        stf<float>(smem + kOffTileG, (i0 + t) * kDim + kc, dGt);
        tot += dGt;
      }
    }
    ms.xe[blk][kc] = e_part;
    __syncthreads();
    if (blk == 3) {
      const float end_term = ms.xe[0][kc] + ms.xe[1][kc] + ms.xe[2][kc] + ms.xe[3][kc] + __expf(gend) * dd_k;
      *reinterpret_cast<float*>(smem + kOffTileG + (63 * kDim + kc) * 4) += end_term;
      tot += end_term;
    }
    ms.xt[blk][kc] = tot;
    __syncthreads();
    float run = 0.f;
#pragma unroll
    for (int bq = 3; bq > 0; --bq) {
      if (bq > blk) run += ms.xt[bq][kc];
    }
    if (!kRagged) {
#pragma unroll
      for (int t = 15; t >= 0; --t) {
        run += ldf<float>(smem + kOffTileG, (16 * blk + t) * kDim + kc);
        stf<G>(p.dg, seq_idx(16 * blk + t) + kc, failed ? poison_nan() : run);
      }
    } else {
#pragma unroll
      for (int t = 15; t >= 0; --t) {
        run += ldf<float>(smem + kOffTileG, (16 * blk + t) * kDim + kc);
        if (16 * blk + t < n_valid) stf<G>(p.dg, seq_idx(16 * blk + t) + kc, failed ? poison_nan() : run);
      }
    }
  }
  // the next chunk-head reuses the arrays of VjpMisc and the TMEM columns
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) {
    if (!kF32Grads) {
      // (the boxes are clipped at token T - 1: rows of a partial last chunk that do not exist are dropped)
      tma_store_4d(&tm_dq, 0, int(h), int(t0), int(b), smem + kOffTileQ);
      tma_store_4d(&tm_dk, 0, int(h), int(t0), int(b), smem + kOffTileK);
#pragma unroll
      for (int bq = 0; bq < 4; ++bq) {  // (a box that starts past token T - 1 is dropped whole)
        tma_store_4d(&tm_dbeta, 0, int(h), int(t0) + 16 * bq, int(b), smem + beta_tile_offset(bq));
      }
      bulk_commit();
    }
    // the G tile is dead: the dS_1 half of the next chunk-head may land on it
    if (ch + gridDim.x < p.n_ch) issue_ds1(ch + gridDim.x);
  }
  }  // chunk-head loop
  if (tid == 0) bulk_wait_all();  // the last dq / dk tiles are in global memory before the CTA retires
  if (warp == 0) tmem_dealloc(tb, 512);
}

}  // namespace

// ---- launcher ---------------------------------------------------------------------------------------
int launch_chunk_backward(const void* q, const void* k, const void* v, const void* g, const void* beta,
                          const void* w, const void* d_out, const float* ds_final, const float* bnd,
                          float* d_bnd, const uint8_t* workspace, uint8_t* scratch, void* dq, void* dk, void* dv, void* dg,
                          void* dbeta, void* dw, float* ds_init, int64_t B, int64_t T, int64_t H,
                          int64_t full_tokens, int dtype, int g_dtype, float scale, int grads_f32,
                          cudaStream_t stream) {
  if (grads_f32 && !(dtype == GDN2_BF16 && g_dtype == GDN2_FP32)) return GDN2_ERR_UNSUPPORTED;
  const int64_t n_chunks = full_tokens / kChunk;
  const int64_t n_ch = B * n_chunks * H;
  if (n_ch <= 0 || n_ch > int64_t(0x7fffffff)) return GDN2_ERR_TOO_LARGE;
  const WsLayout ws{n_ch, true};
  // the status word is the one the forward cleared: a forward failure stays visible to backward
  int* status = reinterpret_cast<int*>(const_cast<uint8_t*>(workspace) + ws.off_status());
  cudaError_t err;

  profile_mark(3, stream);
  // the reverse scan's operands: the forward's tiles, each in the swizzle of the role backward reads it in
  CUtensorMap tm_at, tm_tt, tm_kn, tm_q, tm_yt;
  if (!encode_tile_map(&tm_at, workspace + ws.off_at(), n_ch, kChunk, kChunk, false, 32) ||
      !encode_tile_map(&tm_tt, workspace + ws.off_tt(), n_ch, kChunk, kChunk, false, 32) ||
      !encode_tile_map(&tm_kn, workspace + ws.off_kn(), n_ch, kChunk, kDim, false) ||
      !encode_tile_map(&tm_q, workspace + ws.off_q(), n_ch, kChunk, kDim, true) ||
      !encode_tile_map(&tm_yt, workspace + ws.off_yt(), n_ch, kDim, kChunk, false)) {
    return GDN2_ERR_LAUNCH;
  }
  BScanParams sp{workspace, scratch, d_out, ds_final, d_bnd, ds_init, status, T, H, n_chunks, n_ch};
  const int scan_smem = int(sizeof(BScanSmem));
  if (dtype == GDN2_BF16) {
    auto kernel = chunk_bwd_scan_kernel<__nv_bfloat16>;
    err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), scan_smem);
    if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
    kernel<<<unsigned(B * H), kBScanThreads, scan_smem, stream>>>(sp, tm_at, tm_tt, tm_kn, tm_q, tm_yt);
  } else {
    auto kernel = chunk_bwd_scan_kernel<__half>;
    err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), scan_smem);
    if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
    kernel<<<unsigned(B * H), kBScanThreads, scan_smem, stream>>>(sp, tm_at, tm_tt, tm_kn, tm_q, tm_yt);
  }
  int st = check_launch();
  if (st != GDN2_OK) return st;
  profile_mark(4, stream);

  int device = 0, sm_count = 0;
  err = cudaGetDevice(&device);
  if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  if (err != cudaSuccess || sm_count <= 0) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  CUtensorMap tm_s0, tm_ds;
  const int64_t n_slots = B * (n_chunks + 1) * H;
  if ((reinterpret_cast<uintptr_t>(bnd) & 15u) != 0 || (reinterpret_cast<uintptr_t>(d_bnd) & 15u) != 0 ||
      !encode_tile_map(&tm_s0, reinterpret_cast<const uint8_t*>(bnd), n_slots, kDim, kDim, false) ||
      !encode_tile_map(&tm_ds, reinterpret_cast<const uint8_t*>(d_bnd), n_slots, kDim, kDim, false)) {
    return GDN2_ERR_LAUNCH;
  }
  // dq and dk leave the VJP kernel as [64][128] tiles through tiled TMA stores (rows b * T + t in 31 bits)
  CUtensorMap tm_dq, tm_dk;
  if (B * T > int64_t(0x7fffffff)) return GDN2_ERR_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(dq) & 15u) != 0 || (reinterpret_cast<uintptr_t>(dk) & 15u) != 0 ||
      !encode_sequence_map(&tm_dq, dq, B, T, H, grads_f32 ? GDN2_FP32 : dtype) ||
      !encode_sequence_map(&tm_dk, dk, B, T, H, grads_f32 ? GDN2_FP32 : dtype)) {
    return GDN2_ERR_LAUNCH;
  }
  CUtensorMap tm_dbeta;
  if ((reinterpret_cast<uintptr_t>(dbeta) & 15u) != 0 ||
      !encode_sequence_map(&tm_dbeta, dbeta, B, T, H, grads_f32 ? GDN2_FP32 : dtype, 16)) {
    return GDN2_ERR_LAUNCH;
  }
  CUtensorMap tm_rn;
  if (!encode_tile_map(&tm_rn, workspace + ws.off_rn(), n_ch, kChunk, kDim, false)) return GDN2_ERR_LAUNCH;
  VjpInputMaps tm_in;
  {
    const void* bases[7] = {q, k, v, g, beta, w, d_out};
    CUtensorMap* maps[7] = {&tm_in.q, &tm_in.k, &tm_in.v, &tm_in.g, &tm_in.beta, &tm_in.w, &tm_in.d_out};
    for (int i = 0; i < 7; ++i) {
      if ((reinterpret_cast<uintptr_t>(bases[i]) & 15u) != 0 ||
          !encode_sequence_map(maps[i], bases[i], B, T, H, i == 3 ? g_dtype : dtype)) {
        return GDN2_ERR_LAUNCH;
      }
    }
  }
  VjpParams vp{q, k, v, g, beta, w, d_out, workspace, scratch, bnd, d_bnd, dq, dk, dv, dg, dbeta, dw,
               status, T, H, n_chunks, n_ch, scale};
  const unsigned vjp_grid = unsigned(n_ch < int64_t(sm_count) ? n_ch : int64_t(sm_count));
  const bool ragged = full_tokens > T;  // the last chunk of every (batch, head) is partial
  if (grads_f32) {
    auto kernel = ragged ? chunk_bwd_vjp_kernel<__nv_bfloat16, float, true, true>
                         : chunk_bwd_vjp_kernel<__nv_bfloat16, float, true, false>;
    err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kVjpSmemBytes);
    if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
    kernel<<<vjp_grid, kVjpThreads, kVjpSmemBytes, stream>>>(vp, tm_s0, tm_ds, tm_rn, tm_dq, tm_dk, tm_dbeta, tm_in);
  } else {
    GDN2_DISPATCH_TYPES(dtype, g_dtype, {
      auto kernel = ragged ? chunk_bwd_vjp_kernel<T, G, false, true> : chunk_bwd_vjp_kernel<T, G, false, false>;
      err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kVjpSmemBytes);
      if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
      kernel<<<vjp_grid, kVjpThreads, kVjpSmemBytes, stream>>>(vp, tm_s0, tm_ds, tm_rn, tm_dq, tm_dk, tm_dbeta, tm_in);
    });
  }
  st = check_launch();
  profile_mark(5, stream);
  return st;
}

}  // namespace gdn2
