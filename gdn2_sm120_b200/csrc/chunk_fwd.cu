// Tensor-core chunk forward (64-token chunks, compact-WY form), two kernels:
//
//   chunk_prep_kernel   persistent, one CTA per SM walking over the (batch, chunk, head) units, all
//                       chunks independent.  The raw inputs of the next unit arrive by tiled TMA
//                       loads under the tail of the current one (a CTA that starts a unit with
//                       per-thread loads spends a quarter of its time issuing them: the load/store
//                       unit's queue, not HBM, is the limit).  Builds the WY factors of the chunk
//                       and writes them as row-major tiles:
//                       cumulative log-decay, block-anchored Gram products on tf32 tcgen05 MMAs,
//                       blocked inverse of the unit lower-triangular system on CUDA cores (fp32),
//                       Y = T E and U^T = Z^T T^T on tf32 tcgen05 MMAs.
//   chunk_scan_kernel   one CTA per (batch, head), chunks in order.  The state lives transposed
//                       (S^T: value rows x key columns) in TMEM as the fp32 accumulator and is fed
//                       back as the tf32 A operand of the next MMAs without leaving TMEM:
//                           R^T  = U^T - S^T Y^T
//                           O^T  = S^T Qg^T + R^T Aqk^T
//                           S^T <- S^T diag(d) + R^T Kt
//                       The B operands are the prep kernel's row-major tiles, brought in by tiled
//                       TMA loads in the swizzled layout of their role (chunk_common.cuh).
//
// Math per chunk (reference: src/gdn2_sm120/reference.py:149-172, chunk.py:188-331, with the
// chunk length re-chosen as 64 and the decay normalisation anchored per 16-token block so that
// every exponent stays inside the contract "16-token prefix sums of g > -87"):
//   G_i = sum_{t<=i} g_t,  a_I = G at the start of block I = i / 16
//   L[i][j]   = sum_k beta k_i exp(G_i - a_I) * k_j exp(a_I - G_j)      (j < i)
//   Aqk[i][j] = sum_k scale q_i exp(G_i - a_I) * k_j exp(a_I - G_j)     (j <= i)
//   T = (I + L)^-1,  Y = T (beta k exp(G)),  U = T (w v)
//   Qg = scale q exp(G),  Kt = k exp(G_end - G),  d = exp(G_end)

#include "chunk_common.cuh"

namespace gdn2 {

using namespace tc;

namespace {

// ---------------------------------------------------------------------------------------------
// prep kernel
// ---------------------------------------------------------------------------------------------
// 512 threads: warp = 4-token group tg (0..15), lane = 4-channel group c4 (0..31).  A thread owns
// 4 tokens x 4 channels: one 16-byte chunk of every natural tile row (tokens x channels) and one
// 16-byte chunk (4 tokens) per channel of every transposed tile (channels x tokens).
// Shared-memory tiles written this way use padded strides so that the 8 lanes of a store phase hit
// 8 different 16-byte bank groups: natural tiles CS = 144 (chunk stride), transposed tiles RS = 2064.
constexpr int kPrepThreads = 512;
constexpr int kLd = 68;           // leading dimension of the fp32 64x64 scratch matrices (16-byte rows, banks shift by 4)
constexpr int kLdW = 20;          // leading dimension of the transposed 16x16 block products
constexpr int kCsN = 144;         // natural tiles: byte stride between 16-byte column chunks
constexpr int kRsN = 32 * kCsN;   // natural tiles of 128 fp32 columns: byte stride between 8-row groups (4608)
constexpr int kRsT = 2064;        // transposed tiles (64 fp32 columns): byte stride between 8-row groups
constexpr int kTileT = 16 * kRsT; // 33024 bytes

struct PrepSmem {
  // region 1: tf32 Gram A operand [E_anchored ; Q_anchored] X[r = 128][c = k];
  //           after the Gram products: fp32 scratch for L, T, A_qk and the block products
  alignas(128) uint8_t gram_a[16 * kRsN];               // 73728
  // region 2: tf32 Gram B operands K^I X[r = j < 16 (I + 1)][c = k]: 2 (I + 1) row groups each;
  //           after the Gram products: E^T at +0 and Z^T at +kTileT, tiles X[r = channel][c = j]
  alignas(128) uint8_t gram_b[20 * kRsN];               // 92160
  alignas(128) uint8_t tmat[32768];    // T tile X[r = i][c = j], tf32, RS 2048 (rows 64..127: filler of the M = 128
                                       // product, whose output rows nobody reads; v of the next unit is staged there)
  alignas(128) uint8_t stage_w[16384]; // w of the next unit
  float part[16][kDim];                // per 4-token group partial sums -> exclusive prefixes
  float gend[kDim];
  float nrm[16][2][4][2];              // fused prologue: per (warp, token group, token) sums of q^2, k^2 over 64 channels
  alignas(8) uint64_t bar[2];          // MMA commits
  alignas(8) uint64_t bar_ld[2];       // raw inputs of the next unit: {g, k, q} and {beta, v, w}
  uint32_t tmem_base;
};
// landing zones of the raw [64][128] input tiles of the next unit, in places that are dead by then:
// g, k, q over the fp32 scratch in region 1 (free once T is written, just before the last MMAs);
// beta behind E^T / Z^T in region 2, v in the filler rows of the T tile, w in its own buffer (free as
// soon as the Gram products are done, half a unit earlier)
constexpr int kStageK = 32768, kStageQ = 49152;                     // region 1: g at 0 (16 or 32 KiB)
constexpr int kStageBeta = 2 * kTileT;                              // region 2, behind the two transposed tiles
constexpr int kStageV = 16384;                                      // T tile, rows 64..127
constexpr uint32_t kStageTile16 = kChunk * kDim * 2;                // a 16-bit input tile
static_assert(kStageQ + kStageTile16 <= 16 * kRsN && kStageBeta + kStageTile16 <= 20 * kRsN, "staging exceeds its region");
static_assert(kStageBeta % 128 == 0, "TMA destinations are 128-byte aligned");

struct PrepParams {
  const void *q, *k, *v, *g, *beta, *w;
  uint8_t* ws;   // workspace (D, status)
  ForwardTiles tiles;  // the tile arrays (in the workspace for a training call, else in the scratch)
  int64_t T, H, n_chunks, n_ch;
  float scale;
  int training;  // also write T^T, which only backward consumes
  int prologue;  // kPrologueNorm | kPrologueGate: the inputs are raw projections / gate pre-activations
};

__device__ __forceinline__ int gram_b_offset(int I) { return kRsN * ((I == 0) ? 0 : (I == 1) ? 2 : (I == 2) ? 6 : 12); }
__device__ __forceinline__ int gram_col(int I) { return (I == 0) ? 0 : (I == 1) ? 16 : (I == 2) ? 48 : 96; }

// kPro: the instantiation that can apply the layer prologue to raw inputs (p.prologue says which parts);
// the plain instantiation carries none of that code.
template <typename T, typename G, bool kPro = false>
__global__ void __launch_bounds__(kPrepThreads, 1)
chunk_prep_kernel(const PrepParams p, const __grid_constant__ CUtensorMap tm_g,
                  const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_q,
                  const __grid_constant__ CUtensorMap tm_beta, const __grid_constant__ CUtensorMap tm_v,
                  const __grid_constant__ CUtensorMap tm_w) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  PrepSmem& sm = *reinterpret_cast<PrepSmem*>(smem_raw);
  const WsLayout ws{p.n_ch, p.training != 0};
  int* status = reinterpret_cast<int*>(p.ws + ws.off_status());
  BoundedWaiter waiter(status);
  const bool training = p.training != 0;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    mbar_init(&sm.bar_ld[0], 1);
    mbar_init(&sm.bar_ld[1], 1);
    fence_mbar_init();
  }

  // a warp holds two neighbouring token groups x 16 channel groups: a store of one token row per lane
  // then touches 16 lines of a blocked tile (two 16-byte pieces each) instead of 32
  const int tg = 2 * (warp >> 1) + (lane >> 4), c4 = 16 * (warp & 1) + (lane & 15);
  const int kc0 = 4 * c4;
  const int q4 = warp & 3, part = warp >> 2;  // TMEM lane quadrant of this warp, and its share of the columns

  // unit -> TMA coordinates (channel 0, head, first token of the chunk, batch row).  The last chunk of a
  // ragged sequence reaches past token T - 1: the loads fill those rows with zeros, which is the identity
  // step of the recurrence (no decay, no key, no query, no value).
  const int heads = int(p.H), chunks = int(p.n_chunks), n_ch = int(p.n_ch);
  constexpr uint32_t kStageTileG = kChunk * kDim * sizeof(G);
  auto issue_gkq = [&](int ch_) {
    const int h_ = ch_ % heads, bc = ch_ / heads, b_ = bc / chunks, t_ = (bc % chunks) * kChunk;
    mbar_arrive_expect_tx(&sm.bar_ld[0], kStageTileG + 2 * kStageTile16);
    tma_load_4d(sm.gram_a, &tm_g, 0, h_, t_, b_, &sm.bar_ld[0]);
    tma_load_4d(sm.gram_a + kStageK, &tm_k, 0, h_, t_, b_, &sm.bar_ld[0]);
    tma_load_4d(sm.gram_a + kStageQ, &tm_q, 0, h_, t_, b_, &sm.bar_ld[0]);
  };
  auto issue_bvw = [&](int ch_) {
    const int h_ = ch_ % heads, bc = ch_ / heads, b_ = bc / chunks, t_ = (bc % chunks) * kChunk;
    mbar_arrive_expect_tx(&sm.bar_ld[1], 3 * kStageTile16);
    tma_load_4d(sm.gram_b + kStageBeta, &tm_beta, 0, h_, t_, b_, &sm.bar_ld[1]);
    tma_load_4d(sm.tmat + kStageV, &tm_v, 0, h_, t_, b_, &sm.bar_ld[1]);
    tma_load_4d(sm.stage_w, &tm_w, 0, h_, t_, b_, &sm.bar_ld[1]);
  };
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0 && int(blockIdx.x) < n_ch) {
    issue_gkq(int(blockIdx.x));
    issue_bvw(int(blockIdx.x));
  }
  const uint32_t tb = sm.tmem_base;
  // this thread's 8- or 16-byte piece of row 4 tg + e of a staged [64][128] tile
  auto staged = [&](const uint8_t* tile, int e, int elem_bytes) {
    return tile + ((4 * tg + e) * kDim + kc0) * elem_bytes;
  };

  uint32_t par = 0;
  for (int ch = int(blockIdx.x); ch < n_ch; ch += int(gridDim.x), par ^= 1u) {
  const int ch_next = ch + int(gridDim.x);
  // tokens of this chunk that exist (64 except in the last chunk of a ragged sequence); only the fused
  // prologue needs to know: its activations do not map the zero fill to the identity step
  const int n_valid = kPro ? min(kChunk, int(p.T) - ((ch / heads) % chunks) * kChunk) : kChunk;
  // ---- the raw inputs were brought in while the previous unit was finishing; the log-decay is
  // consumed first: the prefix sums below need it alone ------------------------------------------------
  float Gc[4][4], kk[4][4], qq[4][4], bb[4][4];
  {
    using RawG = typename Raw4<G>::type;
    using RawT = typename Raw4<T>::type;
    RawG rg[4];
    RawT rk[4], rq[4];
    waiter.wait(&sm.bar_ld[0], par);
#pragma unroll
    for (int e = 0; e < 4; ++e) rg[e] = *reinterpret_cast<const RawG*>(staged(sm.gram_a, e, sizeof(G)));
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      rk[e] = *reinterpret_cast<const RawT*>(staged(sm.gram_a + kStageK, e, 2));
      rq[e] = *reinterpret_cast<const RawT*>(staged(sm.gram_a + kStageQ, e, 2));
    }
    const bool pro_norm = kPro && (p.prologue & kPrologueNorm) != 0;
    const bool pro_gate = kPro && (p.prologue & kPrologueGate) != 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float gv[4];
      unpack4<G>(rg[e], gv);
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        if (pro_gate) gv[f] = (4 * tg + e < n_valid) ? prologue_log_decay(gv[f]) : 0.f;
        Gc[e][f] = (e ? Gc[e - 1][f] : 0.f) + gv[f];
      }
    }
#pragma unroll
    for (int f = 0; f < 4; ++f) sm.part[tg][kc0 + f] = Gc[3][f];
    if (pro_norm) {
      // sums of q^2 and k^2 of this thread's four tokens over its four channels, then over the 16 lanes
      // that hold the other channels of the same tokens in this warp (the other 64 channels are in the
      // neighbouring warp: combined after the barrier)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float kf[4], qf[4];
        unpack4<T>(rk[e], kf);
        unpack4<T>(rq[e], qf);
        float sq = qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3];
        float sk = kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3];
#pragma unroll
        for (int off = 1; off < 16; off <<= 1) {
          sq += __shfl_xor_sync(0xffffffffu, sq, off);
          sk += __shfl_xor_sync(0xffffffffu, sk, off);
        }
        if ((lane & 15) == 0) {
          sm.nrm[warp][lane >> 4][e][0] = sq;
          sm.nrm[warp][lane >> 4][e][1] = sk;
        }
      }
    }
    waiter.wait(&sm.bar_ld[1], par);
    // v and w stay where they landed until Z is built, after the Gram products: nothing overwrites their
    // landing zones before the next unit's copies, which are issued after that
    RawT rb[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) rb[e] = *reinterpret_cast<const RawT*>(staged(sm.gram_b + kStageBeta, e, 2));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      unpack4<T>(rk[e], kk[e]);
      unpack4<T>(rq[e], qq[e]);
      unpack4<T>(rb[e], bb[e]);
      if (pro_norm) {
        const float inv_q = rsqrtf(sm.nrm[warp][lane >> 4][e][0] + sm.nrm[warp ^ 1][lane >> 4][e][0] + kPrologueEps);
        const float inv_k = rsqrtf(sm.nrm[warp][lane >> 4][e][1] + sm.nrm[warp ^ 1][lane >> 4][e][1] + kPrologueEps);
#pragma unroll
        for (int f = 0; f < 4; ++f) { qq[e][f] *= inv_q; kk[e][f] *= inv_k; }
      }
      if (pro_gate) {
#pragma unroll
        for (int f = 0; f < 4; ++f) bb[e][f] = (4 * tg + e < n_valid) ? prologue_sigmoid(bb[e][f]) : 0.f;
      }
    }
  }
  if (tid < kDim) {
    float run = 0.f;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const float x = sm.part[t][tid];
      sm.part[t][tid] = run;
      run += x;
    }
    sm.gend[tid] = run;
  }
  __syncthreads();

  // ---- per-thread decay table: everything except three exponentials per element comes from here ----
  const int mb = tg >> 2;  // 16-token block of this thread's tokens
  float a_mb[4], a_nx[4], e_amb[4], c_nx[4], t_end[4], t_far[2][4];
#pragma unroll
  for (int f = 0; f < 4; ++f) {
    const int kc = kc0 + f;
    a_mb[f] = sm.part[4 * mb][kc];
    a_nx[f] = (mb < 3) ? sm.part[4 * (mb + 1)][kc] : sm.gend[kc];
    e_amb[f] = __expf(a_mb[f]);
    c_nx[f] = __expf(a_nx[f] - a_mb[f]);  // decay over the whole 16-token block (<= 1)
    t_end[f] = __expf(sm.gend[kc] - a_nx[f]);
    // blocks further than the next one: exp(a_I - a_next), I = mb + 2, mb + 3
    t_far[0][f] = (mb + 2 < 4) ? __expf(sm.part[4 * (mb + 2)][kc] - a_nx[f]) : 0.f;
    t_far[1][f] = (mb + 3 < 4) ? __expf(sm.part[4 * (mb + 3)][kc] - a_nx[f]) : 0.f;
  }

  float* tile_q = reinterpret_cast<float*>(p.tiles.q + int64_t(ch) * kTileQ);
  float* tile_kn = reinterpret_cast<float*>(p.tiles.kn + int64_t(ch) * kTileKn);
  float ebar[4][4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const int i = 4 * tg + e;
    float ea[4], qa[4], kown[4], knb[4], qgam[4], ktail[4];
#pragma unroll
    for (int f = 0; f < 4; ++f) {
      const float Gi = Gc[e][f] + sm.part[tg][kc0 + f];
      const float anchored = __expf(Gi - a_mb[f]);   // <= 1
      const float own = __expf(a_mb[f] - Gi);        // >= 1, bounded by the 16-token contract
      const float nb = own * c_nx[f];                // exp(a_nx - G_i) <= 1: decay from token i to the next block start
      const float bk = bb[e][f] * kk[e][f];
      const float sq = p.scale * qq[e][f];
      ea[f] = to_tf32_operand(bk * anchored);
      qa[f] = to_tf32_operand(sq * anchored);
      ebar[e][f] = to_tf32_operand(bk * anchored * e_amb[f]);
      qgam[f] = to_tf32_operand(sq * anchored * e_amb[f]);
      kown[f] = to_tf32_operand(kk[e][f] * own);
      knb[f] = kk[e][f] * nb;
      ktail[f] = to_tf32_operand(knb[f] * t_end[f]);
    }
    // Gram A operand rows i (erase) and 64 + i (query), tf32, K-major, padded chunk stride
    *reinterpret_cast<float4*>(sm.gram_a + (i >> 3) * kRsN + c4 * kCsN + (i & 7) * 16) =
        make_float4(ea[0], ea[1], ea[2], ea[3]);
    *reinterpret_cast<float4*>(sm.gram_a + ((64 + i) >> 3) * kRsN + c4 * kCsN + (i & 7) * 16) =
        make_float4(qa[0], qa[1], qa[2], qa[3]);
    // Gram B operands: token i is a column of every row block I >= its own
    const uint32_t row_off = (i >> 3) * kRsN + c4 * kCsN + (i & 7) * 16;
    *reinterpret_cast<float4*>(sm.gram_b + gram_b_offset(mb) + row_off) =
        make_float4(kown[0], kown[1], kown[2], kown[3]);
    if (mb + 1 < 4) {
      *reinterpret_cast<float4*>(sm.gram_b + gram_b_offset(mb + 1) + row_off) =
          make_float4(to_tf32_operand(knb[0]), to_tf32_operand(knb[1]), to_tf32_operand(knb[2]), to_tf32_operand(knb[3]));
    }
#pragma unroll
    for (int far = 0; far < 2; ++far) {
      if (mb + 2 + far < 4) {
        *reinterpret_cast<float4*>(sm.gram_b + gram_b_offset(mb + 2 + far) + row_off) =
            make_float4(to_tf32_operand(knb[0] * t_far[far][0]), to_tf32_operand(knb[1] * t_far[far][1]),
                        to_tf32_operand(knb[2] * t_far[far][2]), to_tf32_operand(knb[3] * t_far[far][3]));
      }
    }
    // token-major tiles Q[i][k] and Kn[i][k]: the 16 lanes of a token write 256 consecutive bytes
    *reinterpret_cast<float4*>(tile_q + i * kDim + kc0) = make_float4(qgam[0], qgam[1], qgam[2], qgam[3]);
    *reinterpret_cast<float4*>(tile_kn + i * kDim + kc0) = make_float4(ktail[0], ktail[1], ktail[2], ktail[3]);
  }
  if (tid < kDim) {
    reinterpret_cast<float*>(p.ws + ws.off_d() + int64_t(ch) * kBlobD)[tid] = __expf(sm.gend[tid]);
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- Gram products on the tensor cores: P_I = [E_a ; Q_a] (K^I)^T -----------------------------
  if (tid == 0) {
    tc_fence_after();
    // the four anchored copies K^0 .. K^3 are stacked (16 + 32 + 48 + 64 = 160 rows) and their products
    // sit side by side in TMEM, so one N = 160 instruction per k-step reads the A tile once for all four
    const uint32_t id = idesc(128, 160, kFmtTF32, kMajorK, kMajorK);
    const uint32_t a0 = smem_u32(sm.gram_a), b0 = smem_u32(sm.gram_b);
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      mma_tf32_ss(tb, smem_desc(a0 + ks * 2 * kCsN, kCsN, kRsN), smem_desc(b0 + ks * 2 * kCsN, kCsN, kRsN), id,
                  ks > 0 ? 1u : 0u);
    }
    mma_commit(&sm.bar[0]);
  }
  waiter.wait(&sm.bar[0], par);
  tc_fence_after();
  // the Gram operands are dead: region 1 becomes fp32 scratch, region 2 receives E^T and Z^T
  float* Ln = reinterpret_cast<float*>(sm.gram_a);           // [64][kLd]   L
  float* Tn = Ln + 64 * kLd;                                  // [64][kLd]   T
  float* Tc = Tn + 64 * kLd;                                  // [64][kLd]   T transposed: Tc[j][i] = T[i][j]
  float* Wt = Tc + 64 * kLd;                                  // [3][16][kLdW] block products, transposed
  static_assert((3 * 64 * kLd + 3 * 16 * kLdW) * 4 <= 16 * kRsN, "fp32 scratch exceeds the Gram A region");
  uint8_t* et_tile = sm.gram_b;                               // E^T  X[r = k][c = j], tf32, RS kRsT
  uint8_t* zt_tile = sm.gram_b + kTileT;                      // Z^T  X[r = v][c = j], tf32, RS kRsT
  {
    // Z = w * v from the staged inputs (kept out of registers until now)
    float zz[4][4];
    const bool pro_gate = kPro && (p.prologue & kPrologueGate) != 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float vv[4], ww[4];
      unpack4<T>(*reinterpret_cast<const typename Raw4<T>::type*>(staged(sm.tmat + kStageV, e, 2)), vv);
      unpack4<T>(*reinterpret_cast<const typename Raw4<T>::type*>(staged(sm.stage_w, e, 2)), ww);
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        if (pro_gate) ww[f] = (4 * tg + e < n_valid) ? prologue_sigmoid(ww[f]) : 0.f;
        zz[e][f] = to_tf32_operand(vv[f] * ww[f]);
      }
    }
#pragma unroll
    for (int f = 0; f < 4; ++f) {
      const uint32_t off = blk_off<4>(kc0 + f, 4 * tg, kRsT, 128);
      *reinterpret_cast<float4*>(et_tile + off) = make_float4(ebar[0][f], ebar[1][f], ebar[2][f], ebar[3][f]);
      *reinterpret_cast<float4*>(zt_tile + off) = make_float4(zz[0][f], zz[1][f], zz[2][f], zz[3][f]);
    }
  }
  {
    // pull L (rows 0..63) into fp32 scratch and A_qk (rows 64..127) into the workspace;
    // the four warps of a quadrant take 16 columns each
    const int r = 32 * q4 + lane;  // TMEM lane = row of [E_a ; Q_a]
    const int i = r & 63;
    const int I_lo = (q4 & 1) * 2;
    const int my_I = I_lo + (lane >> 4);
    const int c0 = 16 * part;
    float* tile_at = reinterpret_cast<float*>(p.tiles.at + int64_t(ch) * kTileAt);
    uint32_t lo[16], hi[16];
    const bool need_lo = c0 < 16 * (I_lo + 1), need_hi = c0 < 16 * (I_lo + 2);
    if (need_lo) tmem_ld16(tmem_addr(tb, 32 * q4, gram_col(I_lo) + c0), lo);
    if (need_hi) tmem_ld16(tmem_addr(tb, 32 * q4, gram_col(I_lo + 1) + c0), hi);
    tmem_wait_ld();
    float vals[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const bool mine_lo = (my_I == I_lo);
      const float x = mine_lo ? (need_lo ? __uint_as_float(lo[j]) : 0.f) : (need_hi ? __uint_as_float(hi[j]) : 0.f);
      const int col = c0 + j;
      vals[j] = (r < 64) ? ((col < i) ? x : 0.f) : ((col <= i) ? to_tf32_operand(x) : 0.f);
    }
    if (r < 64) {
#pragma unroll
      for (int j4 = 0; j4 < 4; ++j4) {
        *reinterpret_cast<float4*>(Ln + i * kLd + c0 + 4 * j4) =
            make_float4(vals[4 * j4], vals[4 * j4 + 1], vals[4 * j4 + 2], vals[4 * j4 + 3]);
      }
    } else {
      // A_qk leaves transposed, At[j][i]: the 32 lanes of a warp (rows i) fill one 128-byte line per column j;
      // the quadrant j >= 32, i < 32 is zero and stays unwritten (nobody reads it)
      if (!(c0 >= 32 && i < 32)) {
#pragma unroll
        for (int j = 0; j < 16; ++j) tile_at[(c0 + j) * kChunk + i] = vals[j];
      }
    }
  }
  for (int e = tid; e < 64 * kLd / 4; e += kPrepThreads) {
    reinterpret_cast<float4*>(Tn)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    reinterpret_cast<float4*>(Tc)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  tc_fence_before();
  __syncthreads();
  // every thread has read v and w of this unit, the Gram operands are dead: beta, v, w of the next unit
  // start to arrive
  if (tid == 0 && ch_next < n_ch) issue_bvw(ch_next);

  // ---- T = (I + L)^-1, blocked: 16x16 diagonal blocks by substitution, the rest by block products.
  // T is kept in both orientations (Tn row-major, Tc column-major) and the block products W transposed,
  // so that both factors of every inner product are read as 16-byte vectors along the summed index.
  auto ld4 = [](const float* ptr) { return *reinterpret_cast<const float4*>(ptr); };
  if (tid < 64) {
    const int I = tid >> 4, cc = tid & 15;
    float x[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      float s = (r == cc) ? 1.f : 0.f;
#pragma unroll
      for (int m4 = 0; m4 < (r + 3) / 4; ++m4) {
        const float4 l = ld4(Ln + (16 * I + r) * kLd + 16 * I + 4 * m4);
        if (4 * m4 + 0 < r) s = fmaf(-l.x, x[4 * m4 + 0], s);
        if (4 * m4 + 1 < r) s = fmaf(-l.y, x[4 * m4 + 1], s);
        if (4 * m4 + 2 < r) s = fmaf(-l.z, x[4 * m4 + 2], s);
        if (4 * m4 + 3 < r) s = fmaf(-l.w, x[4 * m4 + 3], s);
      }
      x[r] = s;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) Tn[(16 * I + r) * kLd + 16 * I + cc] = x[r];
#pragma unroll
    for (int r4 = 0; r4 < 4; ++r4) {
      *reinterpret_cast<float4*>(Tc + (16 * I + cc) * kLd + 16 * I + 4 * r4) =
          make_float4(x[4 * r4], x[4 * r4 + 1], x[4 * r4 + 2], x[4 * r4 + 3]);
    }
  }
  __syncthreads();
  // Two levels of 2 x 2 blocking instead of one block row at a time (four barriers fewer):
  // level 1: the 16 x 16 blocks (1,0) and (3,2) complete the two 32 x 32 diagonal inverses P and Q,
  // level 2: T[32.., ..32) = -Q (L[32.., ..32) P).
  // level 1, W = L_IJ T_JJ for (I, J) = (1, 0), (3, 2)
  {
    const int pair = tid >> 8, r = (tid >> 4) & 15, cc = tid & 15;
    const int J = 2 * pair, I = J + 1;
    const float* lrow = Ln + (16 * I + r) * kLd + 16 * J;
    const float* tcol = Tc + (16 * J + cc) * kLd + 16 * J;
    // four independent chains (one per vector component): the sum is latency-bound otherwise
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int m4 = 0; m4 < 4; ++m4) {
      const float4 a = ld4(lrow + 4 * m4), b = ld4(tcol + 4 * m4);
      acc.x = fmaf(a.x, b.x, acc.x); acc.y = fmaf(a.y, b.y, acc.y);
      acc.z = fmaf(a.z, b.z, acc.z); acc.w = fmaf(a.w, b.w, acc.w);
    }
    Wt[(pair * 16 + cc) * kLdW + r] = (acc.x + acc.y) + (acc.z + acc.w);
  }
  __syncthreads();
  // level 1, T_IJ = -T_II W
  {
    const int pair = tid >> 8, r = (tid >> 4) & 15, cc = tid & 15;
    const int J = 2 * pair, I = J + 1;
    const float* trow = Tn + (16 * I + r) * kLd + 16 * I;
    const float* wcol = Wt + (pair * 16 + cc) * kLdW;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int m4 = 0; m4 < 4; ++m4) {
      const float4 a = ld4(trow + 4 * m4), b = ld4(wcol + 4 * m4);
      acc.x = fmaf(a.x, b.x, acc.x); acc.y = fmaf(a.y, b.y, acc.y);
      acc.z = fmaf(a.z, b.z, acc.z); acc.w = fmaf(a.w, b.w, acc.w);
    }
    const float s = (acc.x + acc.y) + (acc.z + acc.w);
    Tn[(16 * I + r) * kLd + 16 * J + cc] = -s;
    Tc[(16 * J + cc) * kLd + 16 * I + r] = -s;
  }
  __syncthreads();
  // level 2, W2 = L[32.., ..32) P, stored transposed over the (now dead) first 32 rows of L
  // A thread forms two entries of a column (rows r and r + 16): the column of the right factor is the
  // expensive read (a different 16-byte piece per lane, four shared-memory wavefronts), the row of the
  // left factor is a broadcast; the column is read once for both.
  float* W2t = Ln;  // W2t[c][r] = W2[r][c], leading dimension kLd
  {
    const int r = tid >> 5, cc = tid & 31;
    const float* lrow = Ln + (32 + r) * kLd;
    const float* pcol = Tc + cc * kLd;
    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
#pragma unroll
    for (int m4 = 0; m4 < 8; ++m4) {
      const float4 b = ld4(pcol + 4 * m4);
      const float4 a0 = ld4(lrow + 4 * m4), a1 = ld4(lrow + 16 * kLd + 4 * m4);
      acc0.x = fmaf(a0.x, b.x, acc0.x); acc0.y = fmaf(a0.y, b.y, acc0.y);
      acc0.z = fmaf(a0.z, b.z, acc0.z); acc0.w = fmaf(a0.w, b.w, acc0.w);
      acc1.x = fmaf(a1.x, b.x, acc1.x); acc1.y = fmaf(a1.y, b.y, acc1.y);
      acc1.z = fmaf(a1.z, b.z, acc1.z); acc1.w = fmaf(a1.w, b.w, acc1.w);
    }
    // rows 32.. of L are read above by other threads; W2t lives in rows 0..31, which nobody reads any more
    W2t[cc * kLd + r] = (acc0.x + acc0.y) + (acc0.z + acc0.w);
    W2t[cc * kLd + r + 16] = (acc1.x + acc1.y) + (acc1.z + acc1.w);
  }
  __syncthreads();
  // level 2, T[32 + r][c] = -sum_m Q[r][m] W2[m][c]
  {
    const int r = tid >> 5, cc = tid & 31;
    const float* qrow = Tn + (32 + r) * kLd + 32;
    const float* wcol = W2t + cc * kLd;
    float4 acc0 = make_float4(0.f, 0.f, 0.f, 0.f), acc1 = acc0;
#pragma unroll
    for (int m4 = 0; m4 < 8; ++m4) {
      const float4 b = ld4(wcol + 4 * m4);
      const float4 a0 = ld4(qrow + 4 * m4), a1 = ld4(qrow + 16 * kLd + 4 * m4);
      acc0.x = fmaf(a0.x, b.x, acc0.x); acc0.y = fmaf(a0.y, b.y, acc0.y);
      acc0.z = fmaf(a0.z, b.z, acc0.z); acc0.w = fmaf(a0.w, b.w, acc0.w);
      acc1.x = fmaf(a1.x, b.x, acc1.x); acc1.y = fmaf(a1.y, b.y, acc1.y);
      acc1.z = fmaf(a1.z, b.z, acc1.z); acc1.w = fmaf(a1.w, b.w, acc1.w);
    }
    const float s0 = (acc0.x + acc0.y) + (acc0.z + acc0.w), s1 = (acc1.x + acc1.y) + (acc1.z + acc1.w);
    Tn[(32 + r) * kLd + cc] = -s0;
    Tc[cc * kLd + 32 + r] = -s0;
    Tn[(48 + r) * kLd + cc] = -s1;
    Tc[cc * kLd + 48 + r] = -s1;
  }
  __syncthreads();
  // T as tf32 tile X[r = i][c = j] in shared memory (MMA operand); T^T[j][i] goes to the workspace when training
  {
    for (int e = tid; e < 64 * 16; e += kPrepThreads) {
      const int i = e & 63, c4t = e >> 6;  // consecutive threads -> consecutive rows -> contiguous 16-byte chunks
      const float4 tn = ld4(Tn + i * kLd + 4 * c4t);
      *reinterpret_cast<float4*>(sm.tmat + blk_off<4>(i, 4 * c4t, 2048, 128)) =
          make_float4(to_tf32_operand(tn.x), to_tf32_operand(tn.y), to_tf32_operand(tn.z), to_tf32_operand(tn.w));
    }
    if (training) {
      float* tile_tt = reinterpret_cast<float*>(p.tiles.tt + int64_t(ch) * kTileTt);
      for (int e = tid; e < 64 * 16; e += kPrepThreads) {
        const int j = e >> 4, c4t = e & 15;  // consecutive threads -> consecutive 16-byte pieces of a row
        if (j >= 32 && c4t < 8) continue;    // the zero quadrant j >= 32, i < 32 stays unwritten
        const float4 tc = ld4(Tc + j * kLd + 4 * c4t);
        *reinterpret_cast<float4*>(tile_tt + j * kChunk + 4 * c4t) =
            make_float4(to_tf32_operand(tc.x), to_tf32_operand(tc.y), to_tf32_operand(tc.z), to_tf32_operand(tc.w));
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();

  // ---- Y = T E (rows 0..63 of an M = 128 product) and U^T = Z^T T^T ----------------------------------
  if (tid == 0) {
    tc_fence_after();
    // region 1 (fp32 scratch) is dead: g, k, q of the next unit land there under the MMAs and the epilogue
    if (ch_next < n_ch) issue_gkq(ch_next);
    const uint32_t t0a = smem_u32(sm.tmat), e0 = smem_u32(et_tile), z0 = smem_u32(zt_tile);
    const uint32_t id_y = idesc(128, 128, kFmtTF32, kMajorK, kMajorK);
    const uint32_t id_u = idesc(128, 64, kFmtTF32, kMajorK, kMajorK);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      mma_tf32_ss(tb + 0, smem_desc(t0a + ks * 256, 128, 2048), smem_desc(e0 + ks * 256, 128, kRsT), id_y,
                  ks > 0 ? 1u : 0u);
    }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      mma_tf32_ss(tb + 128, smem_desc(z0 + ks * 256, 128, kRsT), smem_desc(t0a + ks * 256, 128, 2048), id_u,
                  ks > 0 ? 1u : 0u);
    }
    mma_commit(&sm.bar[1]);
  }
  waiter.wait(&sm.bar[1], par);
  tc_fence_after();
  {
    // Both accumulators leave transposed: a register holds one column, the 32 lanes of a warp hold 32
    // consecutive rows of it, which are 128 consecutive bytes of the row-major tile.
    // Y (lanes 0..63 = tokens i): Yt[k][i]; the four warps of quadrants 0 and 1 take 32 key columns each
    if (q4 < 2) {
      const int i = 32 * q4 + lane;
      float* tile_yt = reinterpret_cast<float*>(p.tiles.yt + int64_t(ch) * kTileYt) + i;
#pragma unroll
      for (int c0 = 32 * part; c0 < 32 * part + 32; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(tmem_addr(tb, 32 * q4, c0), r);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) tile_yt[(c0 + j) * kChunk] = to_tf32_operand(__uint_as_float(r[j]));
      }
    }
    // U^T (lanes = values v; kept in full fp32): U[j][v]; each warp of a quadrant takes 16 tokens
    {
      const int row = 32 * q4 + lane;
      const int c0 = 16 * part;
      float* tile_u = reinterpret_cast<float*>(p.tiles.u + int64_t(ch) * kTileU) + row;
      uint32_t r[16];
      tmem_ld16(tmem_addr(tb, 32 * q4, 128 + c0), r);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 16; ++j) tile_u[(c0 + j) * kDim] = __uint_as_float(r[j]);
    }
  }
  }  // units of this CTA
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 256);
}

// ---------------------------------------------------------------------------------------------
// scan kernel
// ---------------------------------------------------------------------------------------------
constexpr int kScanThreads = 512;

struct ScanSmem {
  // swizzled operand tiles, slabs of 32 columns (tc05.cuh): Yt and At and Kn are read MN-major, Q K-major
  alignas(1024) uint8_t yt[32768];   // Yt[k][i]: 2 slabs of 128 lines
  alignas(1024) uint8_t q[32768];    // Q[i][k]:  4 slabs of 64 lines
  alignas(1024) uint8_t kn[32768];   // Kn[j][k]: 4 slabs of 64 lines
  alignas(1024) uint8_t at[16384];   // At[j][i]: 2 slabs of 64 lines
  alignas(1024) float u[kChunk * kDim];  // U[j][v], plain rows: threads copy it into tensor memory
  alignas(128) float ck[kDim * kDim];    // training: the chunk-start state [k][v] on its way out (one bulk
                                         // store per chunk: 64 KiB of per-thread stores would hold up the chain)
  alignas(16) float d[kDim];
  alignas(8) uint64_t bar_yqa, bar_ut, bar_kt, bar_mma1, bar_mma2;
  uint32_t tmem_base;
};

struct ScanParams {
  const uint8_t* ws;   // workspace (D)
  const float* s_in;   // [B,H,128,128] or null
  void* out;           // [B,T,H,128]
  float* s_out;        // [B,H,128,128] or null
  float* bnd;          // [B, n_chunks+1, H,128,128] or null
  int* status;
  int64_t T, H, n_chunks, n_ch;
  uint8_t* ws_out;     // same workspace, writable (training: residual tiles)
  int training;
};

template <typename T>
__global__ void __launch_bounds__(kScanThreads, 1)
chunk_scan_kernel(const ScanParams p, const __grid_constant__ CUtensorMap tm_yt,
                  const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kn,
                  const __grid_constant__ CUtensorMap tm_at, const __grid_constant__ CUtensorMap tm_u) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  ScanSmem& sm = *reinterpret_cast<ScanSmem*>(smem_raw);
  const WsLayout ws{p.n_ch, p.training != 0};
  BoundedWaiter waiter(p.status);
  // a wait that ran out in the prep kernel left garbage tiles: results become NaN from the start
  const bool upstream_failed = *static_cast<volatile const int*>(p.status) != kStatusOk;

  // 16 warps: warp & 3 = TMEM lane quadrant (a warp reaches only the 32 lanes of its quadrant),
  // warp >> 2 = its quarter of the columns of whatever accumulator is being moved
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q4 = warp & 3, part = warp >> 2;
  const int64_t bh = blockIdx.x;
  const int64_t b = bh / p.H, h = bh % p.H;
  constexpr uint32_t kColS = 0, kColR = 128, kColO = 192;

  if (warp == 0) {
    tmem_alloc(&sm.tmem_base, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&sm.bar_yqa, 1);
    mbar_init(&sm.bar_ut, 1);
    mbar_init(&sm.bar_kt, 1);
    mbar_init(&sm.bar_mma1, 1);
    mbar_init(&sm.bar_mma2, 1);
    fence_mbar_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = sm.tmem_base;
  const uint32_t lane_base = 32u * q4;
  const int vrow = 32 * q4 + lane;   // value row of the transposed state = TMEM lane
  const int k0 = 32 * part;          // this thread's quarter of the 128 key columns
  const int i0 = 16 * part;          // ... and of the 64 token columns

  auto ch_of = [&](int64_t c) { return (b * p.n_chunks + c) * p.H + h; };
  auto load_yqa = [&](int64_t c) {
    const int ch = int(ch_of(c));
    mbar_arrive_expect_tx(&sm.bar_yqa, uint32_t(kTileYt + kTileQ + kTileAt - 4096));
#pragma unroll
    for (int s = 0; s < 2; ++s) tma_load_3d(sm.yt + s * 16384, &tm_yt, 32 * s, 0, ch, &sm.bar_yqa);
#pragma unroll
    for (int s = 0; s < 4; ++s) tma_load_3d(sm.q + s * 8192, &tm_q, 32 * s, 0, ch, &sm.bar_yqa);
    // At is zero for j >= 32, i < 32: three 32-row boxes, the fourth quadrant of the tile stays zero
    tma_load_3d(sm.at, &tm_at, 0, 0, ch, &sm.bar_yqa);
    tma_load_3d(sm.at + 8192, &tm_at, 32, 0, ch, &sm.bar_yqa);
    tma_load_3d(sm.at + 8192 + 4096, &tm_at, 32, 32, ch, &sm.bar_yqa);
  };
  auto load_ut = [&](int64_t c) {
    mbar_arrive_expect_tx(&sm.bar_ut, uint32_t(kTileU));
    tma_load_3d(sm.u, &tm_u, 0, 0, int(ch_of(c)), &sm.bar_ut);
  };
  auto load_kt = [&](int64_t c) {
    const int64_t ch = ch_of(c);
    mbar_arrive_expect_tx(&sm.bar_kt, uint32_t(kTileKn + kBlobD));
#pragma unroll
    for (int s = 0; s < 4; ++s) tma_load_3d(sm.kn + s * 8192, &tm_kn, 32 * s, 0, int(ch), &sm.bar_kt);
    bulk_g2s(sm.d, p.ws + ws.off_d() + ch * kBlobD, uint32_t(kBlobD), &sm.bar_kt);
  };

  // lines 32..63 of the first slab of At (j >= 32, i < 32) are never loaded: zero, once
  for (int e = tid; e < 4096 / 16; e += kScanThreads) {
    reinterpret_cast<float4*>(sm.at + 4096)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  fence_async_smem();
  if (tid == 0) {
    load_ut(0);
    load_yqa(0);
    load_kt(0);
  }

  // ---- S^T <- S_0^T : thread (v, part) gathers 32 key rows of column v of the key-major state ------
  {
    const float* src = (p.s_in != nullptr) ? p.s_in + bh * int64_t(kDim) * kDim + vrow : nullptr;
    uint32_t r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = (src != nullptr) ? __float_as_uint(src[(k0 + j) * kDim]) : 0u;
    tmem_st32(tmem_addr(tb, lane_base, kColS + k0), r);
    tmem_wait_st();
  }

  for (int64_t c = 0; c < p.n_chunks; ++c) {
    const uint32_t par = uint32_t(c & 1);
    const int64_t t0 = c * kChunk;
    if (c > 0) {
      // the previous state update must have finished reading R^T and the Kt buffer
      waiter.wait(&sm.bar_mma2, par ^ 1u);
      tc_fence_after();
      if (tid == 0) load_kt(c);
    }
    // ---- R^T <- U^T (16 token columns of row v of the U^T tile into TMEM) ---------------------------
    waiter.wait(&sm.bar_ut, par);
    {
      uint32_t r[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(sm.u[(i0 + j) * kDim + vrow]);
      tmem_st16(tmem_addr(tb, lane_base, kColR + i0), r);
      tmem_wait_st();
    }
    waiter.wait(&sm.bar_yqa, par);
    if (tid == 0) bulk_wait_read_all();  // the previous checkpoint has left its staging buffer
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      if (c + 1 < p.n_chunks) load_ut(c + 1);  // every thread has consumed the U^T tile
      const uint32_t y0 = smem_u32(sm.yt), q0 = smem_u32(sm.q), a0 = smem_u32(sm.at);
      const uint32_t id_neg_mn = idesc(128, 64, kFmtTF32, kMajorK, kMajorMN, 1, 0);
      const uint32_t id_pos_k = idesc(128, 64, kFmtTF32, kMajorK, kMajorK);
      const uint32_t id_pos_mn = idesc(128, 64, kFmtTF32, kMajorK, kMajorMN);
      // R^T -= S^T Y^T   (A = state columns, K = 128 keys; B = Yt[k][i] read MN-major)
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {
        mma_tf32_ts(tb + kColR, tb + kColS + ks * 8, smem_desc_sw128_mn(y0, 16384, ks), id_neg_mn, 1u);
      }
      // O^T = S^T Qg^T   (B = Q[i][k] read K-major)
#pragma unroll
      for (int ks = 0; ks < 16; ++ks) {
        mma_tf32_ts(tb + kColO, tb + kColS + ks * 8, smem_desc_sw128_k(q0, 8192, ks), id_pos_k, ks > 0 ? 1u : 0u);
      }
      // O^T += R^T Aqk^T  (A = residual columns, K = 64 tokens; B = At[j][i] read MN-major)
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        mma_tf32_ts(tb + kColO, tb + kColR + ks * 8, smem_desc_sw128_mn(a0, 8192, ks), id_pos_mn, 1u);
      }
      mma_commit(&sm.bar_mma1);
    }
    waiter.wait(&sm.bar_mma1, par);
    tc_fence_after();
    if (tid == 0 && c + 1 < p.n_chunks) load_yqa(c + 1);  // the three MMAs no longer read Y, Q, A

    // ---- training: keep the residual R = U - Y S_0 for backward -------------------------------------
    {
      uint32_t rr[16], ro[16];
      if (p.training) tmem_ld16(tmem_addr(tb, lane_base, kColR + i0), rr);
      tmem_ld16(tmem_addr(tb, lane_base, kColO + i0), ro);
      tmem_wait_ld();
      if (p.training) {
        // row-major R[j][v]: the 32 lanes of a warp fill one 128-byte line per token
        float* rn = reinterpret_cast<float*>(p.ws_out + ws.off_rn() + ch_of(c) * kBlobRn) + vrow;
#pragma unroll
        for (int j = 0; j < 16; ++j) rn[(i0 + j) * kDim] = to_tf32(__uint_as_float(rr[j]));
      }
      // ---- output rows of this chunk: o[t0 + i][v] ---------------------------------------------------
      T* out = static_cast<T*>(p.out);
      const bool failed = upstream_failed || waiter.dead;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (t0 + i0 + j < p.T) {  // the last chunk of a ragged sequence has fewer than 64 tokens
          out[((b * p.T + t0 + i0 + j) * p.H + h) * kDim + vrow] =
              from_float<T>(failed ? poison_nan() : __uint_as_float(ro[j]));
        }
      }
    }
    // ---- checkpoint the chunk-start state, then decay the accumulator: S^T <- S^T diag(d) ----------
    waiter.wait(&sm.bar_kt, par);
    {
      uint32_t r[32];
      tmem_ld32(tmem_addr(tb, lane_base, kColS + k0), r);
      tmem_wait_ld();
      if (p.bnd != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) sm.ck[(k0 + j) * kDim + vrow] = __uint_as_float(r[j]);
        fence_async_smem();
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * sm.d[k0 + j]);
      tmem_st32(tmem_addr(tb, lane_base, kColS + k0), r);
      tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      if (p.bnd != nullptr) {
        bulk_s2g(p.bnd + ((b * (p.n_chunks + 1) + c) * p.H + h) * int64_t(kDim) * kDim, sm.ck,
                 uint32_t(kDim * kDim * sizeof(float)));
        bulk_commit();
      }
      const uint32_t kn0 = smem_u32(sm.kn);
      const uint32_t id_s = idesc(128, 128, kFmtTF32, kMajorK, kMajorMN);
      // S^T += R^T Kt   (K = 64 tokens; B = Kn[j][k] read MN-major)
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        mma_tf32_ts(tb + kColS, tb + kColR + ks * 8, smem_desc_sw128_mn(kn0, 8192, ks), id_s, 1u);
      }
      mma_commit(&sm.bar_mma2);
    }
  }

  // ---- final state ---------------------------------------------------------------------------------
  if (p.n_chunks > 0) {
    waiter.wait(&sm.bar_mma2, uint32_t((p.n_chunks - 1) & 1));
    tc_fence_after();
  }
  {
    float* fin = (p.s_out != nullptr) ? p.s_out + bh * int64_t(kDim) * kDim + vrow : nullptr;
    float* ck = (p.bnd != nullptr)
                    ? p.bnd + ((b * (p.n_chunks + 1) + p.n_chunks) * p.H + h) * int64_t(kDim) * kDim + vrow
                    : nullptr;
    uint32_t r[32];
    tmem_ld32(tmem_addr(tb, lane_base, kColS + k0), r);
    tmem_wait_ld();
    const bool failed = upstream_failed || waiter.dead;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float x = failed ? poison_nan() : __uint_as_float(r[j]);
      if (fin != nullptr) fin[(k0 + j) * kDim] = x;
      if (ck != nullptr) ck[(k0 + j) * kDim] = x;
    }
  }
  if (tid == 0) bulk_wait_all();  // the last staged checkpoint is in global memory before the CTA retires
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 256);
}

// ---------------------------------------------------------------------------------------------
// test aid: a bounded wait that runs out
// ---------------------------------------------------------------------------------------------
// One CTA allocates tensor memory like the real kernels, waits with their BoundedWaiter on an
// mbarrier that nothing arms, and must come back by itself: status word set, tensor memory freed.
__global__ void __launch_bounds__(128, 1) debug_wait_expires_kernel(int* status, uint32_t max_polls) {
  __shared__ alignas(8) uint64_t bar;
  __shared__ uint32_t tmem_base;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    tmem_alloc(&tmem_base, 32);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  BoundedWaiter waiter(status, max_polls);
  waiter.wait(&bar, 0);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 32);
}

}  // namespace

int launch_debug_wait_expires(int* status, uint32_t max_polls, cudaStream_t stream) {
  debug_wait_expires_kernel<<<1, 128, 0, stream>>>(status, max_polls);
  return check_launch();
}

// ---- launcher ---------------------------------------------------------------------------------
int64_t chunk_workspace_bytes(int64_t batch, int64_t full_tokens, int64_t heads, int training) {
  const WsLayout ws{batch * (full_tokens / kChunk) * heads, training != 0};
  return ws.total();
}

// kind: 0 = forward of an inference call, 1 = backward, 2 = forward of a training call
int64_t chunk_scratch_bytes(int64_t batch, int64_t full_tokens, int64_t heads, int kind) {
  const ScratchLayout sc{batch * (full_tokens / kChunk) * heads};
  return kind == 1 ? sc.total_backward() : sc.total_forward(kind == 2);
}

int64_t chunk_status_offset(int64_t batch, int64_t full_tokens, int64_t heads) {
  const WsLayout ws{batch * (full_tokens / kChunk) * heads};
  return ws.off_status();
}

int launch_chunk_forward(const void* q, const void* k, const void* v, const void* g, const void* beta,
                         const void* w, const float* s_in, void* out, float* s_out, float* bnd,
                         uint8_t* workspace, uint8_t* scratch, int64_t B, int64_t T, int64_t H,
                         int64_t full_tokens, int training, int dtype, int g_dtype, float scale,
                         int prologue, cudaStream_t stream) {
  const int64_t n_chunks = full_tokens / kChunk;
  const int64_t n_ch = B * n_chunks * H;
  if (n_ch <= 0 || n_ch > int64_t(0x7fffffff)) return GDN2_ERR_TOO_LARGE;
  const WsLayout ws{n_ch, training != 0};
  int* status = reinterpret_cast<int*>(workspace + ws.off_status());
  cudaError_t err = cudaMemsetAsync(status, 0, kStatusBytes, stream);
  if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }

  // the prep kernel addresses its inputs through tensor maps: 16-byte aligned bases
  if (B * T > int64_t(0x7fffffff)) return GDN2_ERR_TOO_LARGE;
  const void* seq[6] = {g, k, q, beta, v, w};
  CUtensorMap tm[6];
  for (int i = 0; i < 6; ++i) {
    if ((reinterpret_cast<uintptr_t>(seq[i]) & 15u) != 0 ||
        !encode_sequence_map(&tm[i], seq[i], B, T, H, i == 0 ? g_dtype : dtype)) {
      return GDN2_ERR_LAUNCH;
    }
  }
  int device = 0, sm_count = 0;
  err = cudaGetDevice(&device);
  if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  if (err != cudaSuccess || sm_count <= 0) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
  const unsigned prep_grid = unsigned(n_ch < int64_t(sm_count) ? n_ch : int64_t(sm_count));

  profile_mark(0, stream);
  const ForwardTiles tiles = forward_tiles(workspace, scratch, n_ch, training != 0);
  PrepParams pp{q, k, v, g, beta, w, workspace, tiles, T, H, n_chunks, n_ch, scale, training, prologue};
  GDN2_DISPATCH_TYPES(dtype, g_dtype, {
    auto kernel = prologue != 0 ? chunk_prep_kernel<T, G, true> : chunk_prep_kernel<T, G, false>;
    const int smem = int(sizeof(PrepSmem));
    err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
    kernel<<<prep_grid, kPrepThreads, smem, stream>>>(pp, tm[0], tm[1], tm[2], tm[3], tm[4], tm[5]);
  });
  int st = check_launch();
  if (st != GDN2_OK) return st;
  profile_mark(1, stream);

  // the scan's operands: the same tiles, in the swizzle of the role the forward reads them in
  CUtensorMap tm_yt, tm_q, tm_kn, tm_at, tm_u;
  if (!encode_tile_map(&tm_yt, tiles.yt, n_ch, kDim, kChunk, true) ||
      !encode_tile_map(&tm_q, tiles.q, n_ch, kChunk, kDim, false) ||
      !encode_tile_map(&tm_kn, tiles.kn, n_ch, kChunk, kDim, true) ||
      !encode_tile_map(&tm_at, tiles.at, n_ch, kChunk, kChunk, true, 32) ||
      !encode_plain_tile_map(&tm_u, tiles.u, n_ch, kChunk, kDim)) {
    return GDN2_ERR_LAUNCH;
  }
  ScanParams sp{workspace, s_in, out, s_out, bnd, status, T, H, n_chunks, n_ch, workspace, training};
  const int smem = int(sizeof(ScanSmem));
  if (dtype == GDN2_BF16) {
    auto kernel = chunk_scan_kernel<__nv_bfloat16>;
    err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
    kernel<<<unsigned(B * H), kScanThreads, smem, stream>>>(sp, tm_yt, tm_q, tm_kn, tm_at, tm_u);
  } else {
    auto kernel = chunk_scan_kernel<__half>;
    err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
    kernel<<<unsigned(B * H), kScanThreads, smem, stream>>>(sp, tm_yt, tm_q, tm_kn, tm_at, tm_u);
  }
  st = check_launch();
  profile_mark(2, stream);
  return st;
}

}  // namespace gdn2
