// Token-path kernels: exact fp32 recurrence, one token at a time.
//
//   token_forward_kernel      decode / short-sequence forward, optional boundary stack
//   token_t1_zero_kernel      T == 1, zero initial state closed form (write-only state)
//   token_dstate_scan_kernel  reverse scan of the state cotangent
//   token_chunk_vjp_kernel    per-16-token-span recompute + reverse sweep -> all gradients
//
// These serve decode (the HBM-bound serving path), every sequence shorter than one
// tensor-core chunk, and the ragged tail after the last full chunk.  They follow the
// recurrence of src/gdn2_sm120/reference.py:80-93 of the reference literally; the
// thread mapping is this library's own (the reference's token kernel is
// src/gdn2_sm120/recurrent.py:108-243).
//
// State tile ownership in the forward / scan kernels: one CTA = (batch, head,
// 32 value columns), 128 threads.  Thread `tid` owns the float4 column group
// cg = tid & 7 of the key rows rg + 16*i, rg = tid >> 3, i = 0..7, so one warp
// touches four 128-byte row segments per i: fully coalesced 128-bit state I/O, 32
// fp32 state registers per thread, and every state element is read and written by
// exactly one thread (which is why an exact in-place state update is race-free).

#include "common.cuh"
#include "tc05.cuh"

namespace gdn2 {

namespace {

// Fewest (batch, head) pairs for which a decode step runs on the persistent ring kernel (below it
// the ring has too few heads per SM to overlap anything; measured equal to the plain kernel at 160-192)
#ifndef GDN2_DECODE_RING_MIN_HEADS
#define GDN2_DECODE_RING_MIN_HEADS 256
#endif

constexpr int kTokThreads = 128;
constexpr int kTokVT = 32;                     // value columns per CTA
constexpr int kTokTiles = kDim / kTokVT;       // 4 CTAs per (batch, head)
constexpr int kRowsPerThread = 8;              // 128 rows / 16 row groups
constexpr int64_t kStateElems = int64_t(kDim) * kDim;

struct TokenFwdParams {
  const void *q, *k, *v, *g, *beta, *w;
  const float* s_in;
  void* out;
  float* s_out;
  float* bnd;
  int64_t T, H, t_begin, t_end, n_slots;
  float scale;
  int prologue;  // kPrologueNorm | kPrologueGate: raw projections / gate pre-activations are activated here
};

__device__ __forceinline__ float4 ld_red4(const float (*red)[kTokVT], int col) {
  // sum of the four per-warp partial rows
  float4 s = *reinterpret_cast<const float4*>(&red[0][col]);
#pragma unroll
  for (int wv = 1; wv < 4; ++wv) {
    const float4 t = *reinterpret_cast<const float4*>(&red[wv][col]);
    s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
  }
  return s;
}

// kPro (here and in the two decode kernels below): the instantiation that can apply the layer prologue
// to raw inputs; the plain instantiation carries none of that code.
template <typename T, typename G, bool kPro = false>
__global__ void __launch_bounds__(kTokThreads) token_forward_kernel(const TokenFwdParams p) {
  __shared__ float s_a[2][kDim], s_e[2][kDim], s_k[2][kDim], s_q[2][kDim];
  __shared__ float s_z[2][kTokVT];
  __shared__ __align__(16) float s_red[2][2][4][kTokVT];  // [buffer][erase|output][warp][column]
  __shared__ float s_nrm[2][4][2];                        // fused prologue: per warp sums of q^2, k^2

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = tid & 7, rg = tid >> 3;
  const int vt = int(blockIdx.x % kTokTiles);
  const int64_t bh = blockIdx.x / kTokTiles;
  const int64_t b = bh / p.H, h = bh % p.H;
  const int col0 = vt * kTokVT + cg * 4;
  const bool pro_norm = kPro && (p.prologue & kPrologueNorm) != 0;
  const bool pro_gate = kPro && (p.prologue & kPrologueGate) != 0;

  auto stage = [&](int64_t t, int buf) {
    const int64_t idx = ((b * p.T + t) * p.H + h) * kDim;
    const float kv = ldf<T>(p.k, idx + tid);
    float gv = ldf<G>(p.g, idx + tid), bv = ldf<T>(p.beta, idx + tid);
    const float qv = ldf<T>(p.q, idx + tid);
    if (pro_gate) { gv = prologue_log_decay(gv); bv = prologue_sigmoid(bv); }
    s_a[buf][tid] = expf(gv);
    s_e[buf][tid] = bv * kv;
    s_k[buf][tid] = kv;
    s_q[buf][tid] = p.scale * qv;
    if (tid < kTokVT) {
      float wv = ldf<T>(p.w, idx + vt * kTokVT + tid);
      if (pro_gate) wv = prologue_sigmoid(wv);
      s_z[buf][tid] = wv * ldf<T>(p.v, idx + vt * kTokVT + tid);
    }
    if (pro_norm) {
      float sq = qv * qv, sk = kv * kv;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        sq += __shfl_xor_sync(0xffffffffu, sq, off);
        sk += __shfl_xor_sync(0xffffffffu, sk, off);
      }
      if (lane == 0) { s_nrm[buf][warp][0] = sq; s_nrm[buf][warp][1] = sk; }
    }
  };

  float S[kRowsPerThread][4];
  if (p.s_in != nullptr) {
    const float* src = p.s_in + bh * kStateElems;
    const bool vec = (reinterpret_cast<uintptr_t>(p.s_in) & 15) == 0;
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) load4(src + (rg + 16 * i) * kDim + col0, vec, S[i]);
  } else {
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) S[i][0] = S[i][1] = S[i][2] = S[i][3] = 0.f;
  }

  auto store_tile = [&](float* base) {
    const bool vec = (reinterpret_cast<uintptr_t>(base) & 15) == 0;
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) store4(base + (rg + 16 * i) * kDim + col0, vec, S[i]);
  };

  if (p.t_begin < p.t_end) {
    stage(p.t_begin, 0);
  }
  __syncthreads();

  for (int64_t t = p.t_begin; t < p.t_end; ++t) {
    const int64_t rel = t - p.t_begin;
    const int buf = int(rel & 1);
    if (p.bnd != nullptr && (rel % kTokenInterval) == 0) {
      store_tile(p.bnd + ((b * p.n_slots + rel / kTokenInterval) * p.H + h) * kStateElems);
    }
    // reciprocal norms of this token's raw q and k (1 when the inputs are already normalised)
    float iq = 1.f, ik = 1.f;
    if (pro_norm) {
      iq = rsqrtf(s_nrm[buf][0][0] + s_nrm[buf][1][0] + s_nrm[buf][2][0] + s_nrm[buf][3][0] + kPrologueEps);
      ik = rsqrtf(s_nrm[buf][0][1] + s_nrm[buf][1][1] + s_nrm[buf][2][1] + s_nrm[buf][3][1] + kPrologueEps);
    }
    // X = a * S ; partial r = X^T e over this thread's rows
    float r[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
      const float a = s_a[buf][rg + 16 * i], e = kPro ? s_e[buf][rg + 16 * i] * ik : s_e[buf][rg + 16 * i];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        S[i][c] *= a;
        r[c] = fmaf(S[i][c], e, r[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      r[c] += __shfl_xor_sync(0xffffffffu, r[c], 8);
      r[c] += __shfl_xor_sync(0xffffffffu, r[c], 16);
    }
    if (lane < 8) {
      *reinterpret_cast<float4*>(&s_red[buf][0][warp][cg * 4]) = make_float4(r[0], r[1], r[2], r[3]);
    }
    if (t + 1 < p.t_end) stage(t + 1, buf ^ 1);
    __syncthreads();

    const float4 rs = ld_red4(s_red[buf][0], cg * 4);
    const float u[4] = {s_z[buf][cg * 4 + 0] - rs.x, s_z[buf][cg * 4 + 1] - rs.y,
                        s_z[buf][cg * 4 + 2] - rs.z, s_z[buf][cg * 4 + 3] - rs.w};
    // S = X + k u^T ; partial o = S^T (scale q)
    float o[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
      const float kv = kPro ? s_k[buf][rg + 16 * i] * ik : s_k[buf][rg + 16 * i];
      const float qv = kPro ? s_q[buf][rg + 16 * i] * iq : s_q[buf][rg + 16 * i];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        S[i][c] = fmaf(kv, u[c], S[i][c]);
        o[c] = fmaf(S[i][c], qv, o[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      o[c] += __shfl_xor_sync(0xffffffffu, o[c], 8);
      o[c] += __shfl_xor_sync(0xffffffffu, o[c], 16);
    }
    if (lane < 8) {
      *reinterpret_cast<float4*>(&s_red[buf][1][warp][cg * 4]) = make_float4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();
    if (tid < kTokVT) {
      const float ov = s_red[buf][1][0][tid] + s_red[buf][1][1][tid] + s_red[buf][1][2][tid] +
                       s_red[buf][1][3][tid];
      stf<T>(p.out, ((b * p.T + t) * p.H + h) * kDim + vt * kTokVT + tid, ov);
    }
  }

  if (p.bnd != nullptr) {
    store_tile(p.bnd + ((b * p.n_slots + (p.n_slots - 1)) * p.H + h) * kStateElems);
  }
  if (p.s_out != nullptr) {
    store_tile(p.s_out + bh * kStateElems);
  }
}

// ---------------------------------------------------------------------------------
// Decode step (T == 1, 16-byte aligned states, many heads): persistent CTAs, one per SM, each
// walking over (batch, head) pairs.  A head's whole 64 KiB state travels global -> shared ->
// global as 1-D bulk asynchronous copies through a three-slot ring, so two loads and one store
// are in flight per SM while the current head is updated in place in shared memory.
// Thread = (value column v, key half): the sums over keys stay inside a thread except for one
// two-way combine, and shared-memory accesses to the state are conflict-free.
constexpr int kDecThreads = 256;
constexpr int kDecStages = 3;

struct DecodeSmem {
  alignas(128) float state[kDecStages][kDim * kDim];
  alignas(16) float ae[2][kDim], a[2][kDim], kk[2][kDim], qs[2][kDim], z[2][kDim];
  float red[2][2][kDim];   // [parity][key half][column]  erase partial sums
  float redo[2][2][kDim];  //                             output partial sums
  float nrm[2][4][2];      // fused prologue: [parity][warp of the key half][q | k] sums of squares
  alignas(8) uint64_t full[kDecStages];
};

struct DecodeParams {
  const void *q, *k, *v, *g, *beta, *w;
  const float* s_in;
  void* out;
  float* s_out;
  int64_t n_heads;  // batch * heads; T == 1 so sequence row index == head index
  float scale;
  int prologue;     // kPrologueNorm | kPrologueGate
};

template <typename T, typename G, bool kPro = false>
__global__ void __launch_bounds__(kDecThreads, 1) token_decode_ring_kernel(const DecodeParams p) {
  extern __shared__ __align__(128) unsigned char dec_smem_raw[];
  DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(dec_smem_raw);
  const int tid = threadIdx.x;
  const int col = tid & (kDim - 1), kh = tid >> 7;
  const int64_t first = blockIdx.x, stride = gridDim.x;
  const int64_t n_mine = (p.n_heads > first) ? (p.n_heads - first + stride - 1) / stride : 0;
  constexpr uint32_t kStateBytes = kDim * kDim * sizeof(float);

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < kDecStages; ++s) tc::mbar_init(&sm.full[s], 1);
    tc::fence_mbar_init();
  }
  __syncthreads();

  auto issue_load = [&](int64_t n) {  // thread 0 only
    const int s = int(n % kDecStages);
    tc::mbar_arrive_expect_tx(&sm.full[s], kStateBytes);
    tc::bulk_g2s(sm.state[s], p.s_in + (first + n * stride) * int64_t(kDim) * kDim, kStateBytes, &sm.full[s]);
  };
  // per-head vectors: threads 0..127 own a key channel, threads 128..255 a value channel
  float va = 0.f, vb = 0.f, vc = 0.f, vd = 0.f;
  auto fetch_vectors = [&](int64_t n) {
    const int64_t idx = (first + n * stride) * kDim + col;
    if (kh == 0) {
      va = ldf<G>(p.g, idx); vb = ldf<T>(p.beta, idx); vc = ldf<T>(p.k, idx); vd = ldf<T>(p.q, idx);
    } else {
      va = ldf<T>(p.w, idx); vb = ldf<T>(p.v, idx);
    }
  };
  const bool pro_norm = kPro && (p.prologue & kPrologueNorm) != 0;
  const bool pro_gate = kPro && (p.prologue & kPrologueGate) != 0;
  auto stage_vectors = [&](int buf) {
    if (kh == 0) {
      if (pro_gate) { va = prologue_log_decay(va); vb = prologue_sigmoid(vb); }
      const float av = expf(va);
      sm.a[buf][col] = av;
      sm.ae[buf][col] = av * (vb * vc);
      sm.kk[buf][col] = vc;
      sm.qs[buf][col] = p.scale * vd;
      if (pro_norm) {  // warps 0..3 hold the 128 key channels
        float sq = vd * vd, sk = vc * vc;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          sq += __shfl_xor_sync(0xffffffffu, sq, off);
          sk += __shfl_xor_sync(0xffffffffu, sk, off);
        }
        if ((tid & 31) == 0) { sm.nrm[buf][tid >> 5][0] = sq; sm.nrm[buf][tid >> 5][1] = sk; }
      }
    } else {
      if (pro_gate) va = prologue_sigmoid(va);
      sm.z[buf][col] = va * vb;
    }
  };

  if (n_mine > 0) {
    if (tid == 0) {
      issue_load(0);
      if (n_mine > 1) issue_load(1);
    }
    fetch_vectors(0);
    stage_vectors(0);
  }
  __syncthreads();

  bool dead = false;
  for (int64_t n = 0; n < n_mine; ++n) {
    const int s = int(n % kDecStages), buf = int(n & 1);
    const int64_t bh = first + n * stride;
    if (n + 1 < n_mine) fetch_vectors(n + 1);
    if (!dead && !tc::mbar_wait(&sm.full[s], uint32_t((n / kDecStages) & 1), 1u << 20)) dead = true;

    float* S = sm.state[s] + col;
    const int k0 = 64 * kh;
    // pass 1: r[v] = sum_k S[k][v] * (a[k] e[k])
    float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;  // four chains: the sum is latency-bound otherwise
#pragma unroll 4
    for (int kq = 0; kq < 64; kq += 4) {
      const float4 f = *reinterpret_cast<const float4*>(&sm.ae[buf][k0 + kq]);
      r0 = fmaf(S[(k0 + kq) * kDim], f.x, r0);
      r1 = fmaf(S[(k0 + kq + 1) * kDim], f.y, r1);
      r2 = fmaf(S[(k0 + kq + 2) * kDim], f.z, r2);
      r3 = fmaf(S[(k0 + kq + 3) * kDim], f.w, r3);
    }
    sm.red[buf][kh][col] = (r0 + r1) + (r2 + r3);
    if (tid == 0 && n + 2 < n_mine) {
      // The slot of head n + 2 was last used by head n - 1, whose store was issued at the end of the
      // previous iteration: by now it has normally finished reading the slot, so this wait does not
      // hold up the warp (at the top of the iteration it stalled every head by the store's read time).
      tc::bulk_wait_read_all();
      issue_load(n + 2);
    }
    // a copy that never arrived, for any thread: the head's results are marked invalid for all
    dead = __syncthreads_or(dead ? 1 : 0) != 0;
    // raw q / k: the erase sum is linear in k, the output in q, so the reciprocal norms scale the sums
    float iq = 1.f, ik = 1.f;
    if (pro_norm) {
      iq = rsqrtf(sm.nrm[buf][0][0] + sm.nrm[buf][1][0] + sm.nrm[buf][2][0] + sm.nrm[buf][3][0] + kPrologueEps);
      ik = rsqrtf(sm.nrm[buf][0][1] + sm.nrm[buf][1][1] + sm.nrm[buf][2][1] + sm.nrm[buf][3][1] + kPrologueEps);
    }
    const float r_sum = sm.red[buf][0][col] + sm.red[buf][1][col];
    const float u = kPro ? (sm.z[buf][col] - ik * r_sum) * ik  // u * ik: S += (k ik) u
                         : sm.z[buf][col] - r_sum;
    // pass 2: S <- a S + k u^T ; o[v] = sum_k S[k][v] (scale q[k])
    float o = 0.f;
#pragma unroll 4
    for (int kq = 0; kq < 64; kq += 4) {
      const float4 fa = *reinterpret_cast<const float4*>(&sm.a[buf][k0 + kq]);
      const float4 fk = *reinterpret_cast<const float4*>(&sm.kk[buf][k0 + kq]);
      const float4 fq = *reinterpret_cast<const float4*>(&sm.qs[buf][k0 + kq]);
      float x0 = fmaf(fk.x, u, fa.x * S[(k0 + kq) * kDim]);
      float x1 = fmaf(fk.y, u, fa.y * S[(k0 + kq + 1) * kDim]);
      float x2 = fmaf(fk.z, u, fa.z * S[(k0 + kq + 2) * kDim]);
      float x3 = fmaf(fk.w, u, fa.w * S[(k0 + kq + 3) * kDim]);
      S[(k0 + kq) * kDim] = x0; S[(k0 + kq + 1) * kDim] = x1;
      S[(k0 + kq + 2) * kDim] = x2; S[(k0 + kq + 3) * kDim] = x3;
      o = fmaf(x0, fq.x, o); o = fmaf(x1, fq.y, o); o = fmaf(x2, fq.z, o); o = fmaf(x3, fq.w, o);
    }
    sm.redo[buf][kh][col] = o;
    if (n + 1 < n_mine) stage_vectors(buf ^ 1);
    tc::fence_async_smem();
    __syncthreads();
    // A head whose state never arrived is not written back: the caller's state (which an in-place
    // update would otherwise overwrite with garbage) survives and the NaN output says so.
    if (tid == 0 && !dead) {
      tc::bulk_s2g(p.s_out + bh * int64_t(kDim) * kDim, sm.state[s], kStateBytes);
      tc::bulk_commit();
    }
    if (kh == 0) {
      float ov = sm.redo[buf][0][col] + sm.redo[buf][1][col];
      if (kPro) ov *= iq;
      if (dead) ov = __int_as_float(0x7fc00000);  // a bulk copy never arrived: make the failure visible
      stf<T>(p.out, bh * kDim + col, ov);
    }
  }
  if (tid == 0) tc::bulk_wait_all();
}

// ---------------------------------------------------------------------------------
struct T1ZeroParams {
  const void *q, *k, *v, *w;
  void* out;
  float* s_out;
  int64_t H;
  float scale;
  int prologue;
};

template <typename T, bool kPro = false>
__global__ void __launch_bounds__(kTokThreads) token_t1_zero_kernel(const T1ZeroParams p) {
  __shared__ float s_k[kDim];
  __shared__ float s_z[kTokVT];
  __shared__ float s_part[4];
  __shared__ float s_nrm[4][2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = tid & 7, rg = tid >> 3;
  const int vt = int(blockIdx.x % kTokTiles);
  const int64_t bh = blockIdx.x / kTokTiles;
  const int64_t idx = bh * kDim;  // T == 1: [B, 1, H, 128]

  const bool pro_norm = kPro && (p.prologue & kPrologueNorm) != 0;
  const bool pro_gate = kPro && (p.prologue & kPrologueGate) != 0;
  const float kv = ldf<T>(p.k, idx + tid);
  const float qv = ldf<T>(p.q, idx + tid);
  float qk = p.scale * qv * kv;
  if (tid < kTokVT) {
    float wv = ldf<T>(p.w, idx + vt * kTokVT + tid);
    if (pro_gate) wv = prologue_sigmoid(wv);
    s_z[tid] = wv * ldf<T>(p.v, idx + vt * kTokVT + tid);
  }
  float sq = qv * qv, sk = kv * kv;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    qk += __shfl_xor_sync(0xffffffffu, qk, off);
    if (pro_norm) {
      sq += __shfl_xor_sync(0xffffffffu, sq, off);
      sk += __shfl_xor_sync(0xffffffffu, sk, off);
    }
  }
  if (lane == 0) {
    s_part[warp] = qk;
    s_nrm[warp][0] = sq;
    s_nrm[warp][1] = sk;
  }
  if (!pro_norm) s_k[tid] = kv;
  __syncthreads();
  qk = s_part[0] + s_part[1] + s_part[2] + s_part[3];
  if (pro_norm) {  // raw q, k: scale by the reciprocal norms
    const float ik = rsqrtf(s_nrm[0][1] + s_nrm[1][1] + s_nrm[2][1] + s_nrm[3][1] + kPrologueEps);
    qk *= ik * rsqrtf(s_nrm[0][0] + s_nrm[1][0] + s_nrm[2][0] + s_nrm[3][0] + kPrologueEps);
    s_k[tid] = kv * ik;
    __syncthreads();
  }

  float z[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) z[c] = s_z[cg * 4 + c];
  float* dst = p.s_out + bh * kStateElems + vt * kTokVT + cg * 4;
  const bool vec = (reinterpret_cast<uintptr_t>(p.s_out) & 15) == 0;
#pragma unroll
  for (int i = 0; i < kRowsPerThread; ++i) {
    const float kr = s_k[rg + 16 * i];
    const float row[4] = {kr * z[0], kr * z[1], kr * z[2], kr * z[3]};
    store4(dst + (rg + 16 * i) * kDim, vec, row);
  }
  if (tid < kTokVT) stf<T>(p.out, idx + vt * kTokVT + tid, qk * s_z[tid]);
}

// ---------------------------------------------------------------------------------
struct DstateScanParams {
  const void *q, *k, *g, *beta, *d_out;
  const float* ds_final;
  float* d_bnd;
  float* ds_init;
  int64_t T, H, t_begin, t_end, n_slots;
  float scale;
};

template <typename T, typename G>
__global__ void __launch_bounds__(kTokThreads) token_dstate_scan_kernel(const DstateScanParams p) {
  __shared__ float s_a[2][kDim], s_e[2][kDim], s_k[2][kDim], s_q[2][kDim];
  __shared__ float s_do[2][kTokVT];
  __shared__ __align__(16) float s_red[2][4][kTokVT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = tid & 7, rg = tid >> 3;
  const int vt = int(blockIdx.x % kTokTiles);
  const int64_t bh = blockIdx.x / kTokTiles;
  const int64_t b = bh / p.H, h = bh % p.H;
  const int col0 = vt * kTokVT + cg * 4;

  auto stage = [&](int64_t t, int buf) {
    const int64_t idx = ((b * p.T + t) * p.H + h) * kDim;
    const float kv = ldf<T>(p.k, idx + tid);
    s_a[buf][tid] = expf(ldf<G>(p.g, idx + tid));
    s_e[buf][tid] = ldf<T>(p.beta, idx + tid) * kv;
    s_k[buf][tid] = kv;
    s_q[buf][tid] = p.scale * ldf<T>(p.q, idx + tid);
    if (tid < kTokVT) s_do[buf][tid] = ldf<T>(p.d_out, idx + vt * kTokVT + tid);
  };

  float dS[kRowsPerThread][4];
  if (p.ds_final != nullptr) {
    const float* src = p.ds_final + bh * kStateElems;
    const bool vec = (reinterpret_cast<uintptr_t>(p.ds_final) & 15) == 0;
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) load4(src + (rg + 16 * i) * kDim + col0, vec, dS[i]);
  } else {
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) dS[i][0] = dS[i][1] = dS[i][2] = dS[i][3] = 0.f;
  }
  auto store_tile = [&](float* base) {
    const bool vec = (reinterpret_cast<uintptr_t>(base) & 15) == 0;
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) store4(base + (rg + 16 * i) * kDim + col0, vec, dS[i]);
  };

  store_tile(p.d_bnd + ((b * p.n_slots + (p.n_slots - 1)) * p.H + h) * kStateElems);
  if (p.t_begin < p.t_end) stage(p.t_end - 1, 0);
  __syncthreads();

  int buf = 0;
  for (int64_t t = p.t_end - 1; t >= p.t_begin; --t, buf ^= 1) {
    // dS' = dS + (scale q) do^T ; partial du = dS'^T k
    float du[4] = {0.f, 0.f, 0.f, 0.f};
    float dov[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) dov[c] = s_do[buf][cg * 4 + c];
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
      const float kv = s_k[buf][rg + 16 * i], qv = s_q[buf][rg + 16 * i];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        dS[i][c] = fmaf(qv, dov[c], dS[i][c]);
        du[c] = fmaf(dS[i][c], kv, du[c]);
      }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      du[c] += __shfl_xor_sync(0xffffffffu, du[c], 8);
      du[c] += __shfl_xor_sync(0xffffffffu, du[c], 16);
    }
    if (lane < 8) {
      *reinterpret_cast<float4*>(&s_red[buf][warp][cg * 4]) = make_float4(du[0], du[1], du[2], du[3]);
    }
    if (t - 1 >= p.t_begin) stage(t - 1, buf ^ 1);
    __syncthreads();
    const float4 ds = ld_red4(s_red[buf], cg * 4);
    const float dus[4] = {ds.x, ds.y, ds.z, ds.w};
    // dS <- a * (dS' - e du^T)
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
      const float a = s_a[buf][rg + 16 * i], e = s_e[buf][rg + 16 * i];
#pragma unroll
      for (int c = 0; c < 4; ++c) dS[i][c] = a * fmaf(-e, dus[c], dS[i][c]);
    }
    const int64_t rel = t - p.t_begin;
    if ((rel % kTokenInterval) == 0) {
      store_tile(p.d_bnd + ((b * p.n_slots + rel / kTokenInterval) * p.H + h) * kStateElems);
    }
  }
  if (p.ds_init != nullptr) store_tile(p.ds_init + bh * kStateElems);
}

// ---------------------------------------------------------------------------------
// Chunk-local VJP.  One CTA = (batch, 16-token span, head), 128 threads, thread = key
// row.  The span is swept in 16 passes of 8 value columns: forward from the saved
// boundary keeping every decayed state X_t of the pass in shared memory (private to
// the owning thread), then in reverse with the cotangent tile in registers.  Sums over
// the value axis (dq, dk, d(beta k), dg) stay inside the thread and are accumulated
// across passes in registers, so no partial buffers, atomics or second kernel exist.
constexpr int kVjpThreads = 128;
constexpr int kVjpVT = 8;
constexpr int kVjpPasses = kDim / kVjpVT;

template <typename T>
struct VjpSmem {
  float hist[kTokenInterval][kVjpVT][kDim];  // X_t of the current pass      64 KiB
  float a[kTokenInterval][kDim];             // exp(g)                        8 KiB
  float du[kTokenInterval][kDim];            // d(u) for all value columns    8 KiB
  T q[kTokenInterval][kDim], k[kTokenInterval][kDim], beta[kTokenInterval][kDim];
  T v[kTokenInterval][kDim], w[kTokenInterval][kDim], dout[kTokenInterval][kDim];  // 24 KiB
  float u[kTokenInterval][kVjpVT];
  float red[2][4][kVjpVT];
};

struct ChunkVjpParams {
  const void *q, *k, *v, *g, *beta, *w, *d_out;
  const float *bnd, *d_bnd;
  void *dq, *dk, *dv, *dg, *dbeta, *dw;
  int64_t T, H, t_begin, t_end, n_slots;
  float scale;
};

// Sum eight per-thread values over the 128 threads of the CTA; every thread gets all
// eight totals.  Halving butterfly: 9 shuffles instead of 40.
__device__ __forceinline__ void block_sum8(float (&x)[8], float (*red)[4][kVjpVT], int& rb,
                                           int lane, int warp) {
  const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0, h4 = (lane & 4) != 0;
  float y[4], z[2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float recv = __shfl_xor_sync(0xffffffffu, h16 ? x[j] : x[j + 4], 16);
    y[j] = (h16 ? x[j + 4] : x[j]) + recv;  // column j + 4*h16
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float recv = __shfl_xor_sync(0xffffffffu, h8 ? y[j] : y[j + 2], 8);
    z[j] = (h8 ? y[j + 2] : y[j]) + recv;  // column j + 2*h8 + 4*h16
  }
  float s;
  {
    const float recv = __shfl_xor_sync(0xffffffffu, h4 ? z[0] : z[1], 4);
    s = (h4 ? z[1] : z[0]) + recv;  // column h4 + 2*h8 + 4*h16 == lane >> 2
  }
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if ((lane & 3) == 0) red[rb][warp][lane >> 2] = s;
  __syncthreads();
#pragma unroll
  for (int c = 0; c < 8; ++c) x[c] = red[rb][0][c] + red[rb][1][c] + red[rb][2][c] + red[rb][3][c];
  rb ^= 1;
}

template <typename T, typename G>
__global__ void __launch_bounds__(kVjpThreads) token_chunk_vjp_kernel(const ChunkVjpParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  VjpSmem<T>& sm = *reinterpret_cast<VjpSmem<T>*>(smem_raw);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t n_spans = p.n_slots - 1;
  const int64_t h = blockIdx.x % p.H;
  const int64_t j = (blockIdx.x / p.H) % n_spans;
  const int64_t b = blockIdx.x / (p.H * n_spans);
  const int64_t t0 = p.t_begin + j * kTokenInterval;
  const int n = int(min(int64_t(kTokenInterval), p.t_end - t0));

  for (int t = 0; t < n; ++t) {
    const int64_t idx = ((b * p.T + t0 + t) * p.H + h) * kDim + tid;
    sm.q[t][tid] = static_cast<const T*>(p.q)[idx];
    sm.k[t][tid] = static_cast<const T*>(p.k)[idx];
    sm.beta[t][tid] = static_cast<const T*>(p.beta)[idx];
    sm.v[t][tid] = static_cast<const T*>(p.v)[idx];
    sm.w[t][tid] = static_cast<const T*>(p.w)[idx];
    sm.dout[t][tid] = static_cast<const T*>(p.d_out)[idx];
    sm.a[t][tid] = expf(ldf<G>(p.g, idx));
  }
  __syncthreads();

  float adq[kTokenInterval], adk[kTokenInterval], ade[kTokenInterval], adg[kTokenInterval];
#pragma unroll
  for (int t = 0; t < kTokenInterval; ++t) adq[t] = adk[t] = ade[t] = adg[t] = 0.f;

  const float* s_src = p.bnd + ((b * p.n_slots + j) * p.H + h) * kStateElems + tid * kDim;
  const float* ds_src = p.d_bnd + ((b * p.n_slots + j + 1) * p.H + h) * kStateElems + tid * kDim;
  int rb = 0;

  for (int pass = 0; pass < kVjpPasses; ++pass) {
    const int cb = pass * kVjpVT;
    float S[kVjpVT];
    {
      const float4 lo = *reinterpret_cast<const float4*>(s_src + cb);
      const float4 hi = *reinterpret_cast<const float4*>(s_src + cb + 4);
      S[0] = lo.x; S[1] = lo.y; S[2] = lo.z; S[3] = lo.w;
      S[4] = hi.x; S[5] = hi.y; S[6] = hi.z; S[7] = hi.w;
    }
    // ---- forward recompute, keeping X_t ----
#pragma unroll
    for (int t = 0; t < kTokenInterval; ++t) {
      if (t < n) {
        const float a = sm.a[t][tid];
        const float kv = to_float(sm.k[t][tid]);
        const float e = to_float(sm.beta[t][tid]) * kv;
        float r[kVjpVT];
#pragma unroll
        for (int c = 0; c < kVjpVT; ++c) {
          S[c] *= a;
          sm.hist[t][c][tid] = S[c];
          r[c] = S[c] * e;
        }
        block_sum8(r, sm.red, rb, lane, warp);
#pragma unroll
        for (int c = 0; c < kVjpVT; ++c) {
          const float u = to_float(sm.w[t][cb + c]) * to_float(sm.v[t][cb + c]) - r[c];
          S[c] = fmaf(kv, u, S[c]);
          if (tid == c) sm.u[t][c] = u;
        }
      }
    }
    __syncthreads();  // sm.u of the last token visible to everyone

    float dS[kVjpVT];
    {
      const float4 lo = *reinterpret_cast<const float4*>(ds_src + cb);
      const float4 hi = *reinterpret_cast<const float4*>(ds_src + cb + 4);
      dS[0] = lo.x; dS[1] = lo.y; dS[2] = lo.z; dS[3] = lo.w;
      dS[4] = hi.x; dS[5] = hi.y; dS[6] = hi.z; dS[7] = hi.w;
    }
    // ---- reverse sweep ----
#pragma unroll
    for (int t = kTokenInterval - 1; t >= 0; --t) {
      if (t < n) {
        const float a = sm.a[t][tid];
        const float kv = to_float(sm.k[t][tid]);
        const float e = to_float(sm.beta[t][tid]) * kv;
        const float qs = p.scale * to_float(sm.q[t][tid]);
        float X[kVjpVT], du[kVjpVT];
        float acc_q = 0.f, acc_k = 0.f;
#pragma unroll
        for (int c = 0; c < kVjpVT; ++c) {
          X[c] = sm.hist[t][c][tid];
          const float u = sm.u[t][c];
          const float st = fmaf(kv, u, X[c]);            // S_t
          const float dov = to_float(sm.dout[t][cb + c]);
          acc_q = fmaf(st, dov, acc_q);
          dS[c] = fmaf(qs, dov, dS[c]);                  // dS'
          acc_k = fmaf(dS[c], u, acc_k);
          du[c] = dS[c] * kv;
        }
        adq[t] += acc_q;
        adk[t] += acc_k;
        block_sum8(du, sm.red, rb, lane, warp);
        float acc_e = 0.f, acc_g = 0.f;
#pragma unroll
        for (int c = 0; c < kVjpVT; ++c) {
          acc_e = fmaf(X[c], du[c], acc_e);
          const float dx = fmaf(-e, du[c], dS[c]);
          acc_g = fmaf(dx, X[c], acc_g);
          dS[c] = a * dx;
          if (tid == c) sm.du[t][cb + c] = du[c];
        }
        ade[t] -= acc_e;
        adg[t] += acc_g;
      }
    }
  }
  __syncthreads();  // sm.du complete

#pragma unroll
  for (int t = 0; t < kTokenInterval; ++t) {
    if (t < n) {
      const int64_t idx = ((b * p.T + t0 + t) * p.H + h) * kDim + tid;
      const float kv = to_float(sm.k[t][tid]);
      const float bv = to_float(sm.beta[t][tid]);
      stf<T>(p.dq, idx, p.scale * adq[t]);
      stf<T>(p.dk, idx, fmaf(ade[t], bv, adk[t]));
      stf<T>(p.dbeta, idx, ade[t] * kv);
      stf<G>(p.dg, idx, adg[t]);
      const float duv = sm.du[t][tid];
      stf<T>(p.dv, idx, duv * to_float(sm.w[t][tid]));
      stf<T>(p.dw, idx, duv * to_float(sm.v[t][tid]));
    }
  }
}

inline int64_t slots_for(int64_t t_begin, int64_t t_end) {
  return (t_end - t_begin + kTokenInterval - 1) / kTokenInterval + 1;
}

inline bool grid_fits(int64_t blocks) { return blocks > 0 && blocks <= int64_t(0x7fffffff); }

}  // namespace

// ---- launchers (called from api.cu) --------------------------------------------------
int launch_token_forward(const void* q, const void* k, const void* v, const void* g,
                         const void* beta, const void* w, const float* s_in, void* out,
                         float* s_out, float* bnd, int64_t B, int64_t T, int64_t H,
                         int64_t t_begin, int64_t t_end, int dtype, int g_dtype, float scale,
                         int prologue, cudaStream_t stream) {
  const int64_t blocks = B * H * kTokTiles;
  if (!grid_fits(blocks)) return GDN2_ERR_TOO_LARGE;
  // decode fast path: one token, state in and out, 16-byte aligned, enough heads to fill the GPU
  if (T == 1 && t_begin == 0 && t_end == 1 && s_in != nullptr && s_out != nullptr && bnd == nullptr &&
      B * H >= GDN2_DECODE_RING_MIN_HEADS &&
      ((reinterpret_cast<uintptr_t>(s_in) | reinterpret_cast<uintptr_t>(s_out)) & 15) == 0) {
    int dev = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
    DecodeParams dp{q, k, v, g, beta, w, s_in, out, s_out, B * H, scale, prologue};
    const int smem = int(sizeof(DecodeSmem));
    const unsigned grid = unsigned(B * H < sms ? B * H : sms);
    GDN2_DISPATCH_TYPES(dtype, g_dtype, {
      auto kernel = prologue != 0 ? token_decode_ring_kernel<T, G, true> : token_decode_ring_kernel<T, G, false>;
      err = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
      if (err != cudaSuccess) { record_cuda_error(err); return GDN2_ERR_LAUNCH; }
      kernel<<<grid, kDecThreads, smem, stream>>>(dp);
    });
    return check_launch();
  }
  TokenFwdParams p{q, k, v, g, beta, w, s_in, out, s_out, bnd,
                   T, H, t_begin, t_end, slots_for(t_begin, t_end), scale, prologue};
  GDN2_DISPATCH_TYPES(dtype, g_dtype, {
    if (prologue != 0) token_forward_kernel<T, G, true><<<unsigned(blocks), kTokThreads, 0, stream>>>(p);
    else token_forward_kernel<T, G, false><<<unsigned(blocks), kTokThreads, 0, stream>>>(p);
  });
  return check_launch();
}

int launch_token_t1_zero(const void* q, const void* k, const void* v, const void* w, void* out,
                         float* s_out, int64_t B, int64_t H, int dtype, float scale, int prologue,
                         cudaStream_t stream) {
  const int64_t blocks = B * H * kTokTiles;
  if (!grid_fits(blocks)) return GDN2_ERR_TOO_LARGE;
  T1ZeroParams p{q, k, v, w, out, s_out, H, scale, prologue};
  if (dtype == GDN2_BF16) {
    if (prologue != 0) token_t1_zero_kernel<__nv_bfloat16, true><<<unsigned(blocks), kTokThreads, 0, stream>>>(p);
    else token_t1_zero_kernel<__nv_bfloat16, false><<<unsigned(blocks), kTokThreads, 0, stream>>>(p);
  } else {
    if (prologue != 0) token_t1_zero_kernel<__half, true><<<unsigned(blocks), kTokThreads, 0, stream>>>(p);
    else token_t1_zero_kernel<__half, false><<<unsigned(blocks), kTokThreads, 0, stream>>>(p);
  }
  return check_launch();
}

int launch_token_dstate_scan(const void* q, const void* k, const void* g, const void* beta,
                             const void* d_out, const float* ds_final, float* d_bnd,
                             float* ds_init, int64_t B, int64_t T, int64_t H, int64_t t_begin,
                             int64_t t_end, int dtype, int g_dtype, float scale,
                             cudaStream_t stream) {
  const int64_t blocks = B * H * kTokTiles;
  if (!grid_fits(blocks)) return GDN2_ERR_TOO_LARGE;
  DstateScanParams p{q, k, g, beta, d_out, ds_final, d_bnd, ds_init,
                     T, H, t_begin, t_end, slots_for(t_begin, t_end), scale};
  GDN2_DISPATCH_TYPES(
      dtype, g_dtype,
      (token_dstate_scan_kernel<T, G><<<unsigned(blocks), kTokThreads, 0, stream>>>(p)));
  return check_launch();
}

int launch_token_chunk_vjp(const void* q, const void* k, const void* v, const void* g,
                           const void* beta, const void* w, const void* d_out, const float* bnd,
                           const float* d_bnd, void* dq, void* dk, void* dv, void* dg,
                           void* dbeta, void* dw, int64_t B, int64_t T, int64_t H,
                           int64_t t_begin, int64_t t_end, int dtype, int g_dtype, float scale,
                           cudaStream_t stream) {
  const int64_t n_slots = slots_for(t_begin, t_end);
  const int64_t blocks = B * (n_slots - 1) * H;
  if (!grid_fits(blocks)) return GDN2_ERR_TOO_LARGE;
  ChunkVjpParams p{q, k, v, g, beta, w, d_out, bnd, d_bnd, dq, dk, dv, dg, dbeta, dw,
                   T, H, t_begin, t_end, n_slots, scale};
  GDN2_DISPATCH_TYPES(dtype, g_dtype, {
    auto kernel = token_chunk_vjp_kernel<T, G>;
    const int smem = int(sizeof(VjpSmem<T>));
    cudaError_t err =
        ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem);
    if (err != cudaSuccess) {
      record_cuda_error(err);
      return GDN2_ERR_LAUNCH;
    }
    kernel<<<unsigned(blocks), kVjpThreads, smem, stream>>>(p);
  });
  return check_launch();
}

}  // namespace gdn2
