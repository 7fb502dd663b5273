// Inline-PTX wrappers for the sm_100a tensor-core path: tcgen05 MMA with TMEM accumulators,
// shared-memory matrix descriptors, mbarriers and bulk asynchronous copies.
//
// Two operand storage conventions are in use.
//
// "Blocked" tiles, no swizzle (tiles that threads build in shared memory, and dZ): a matrix X[r][c] of
// 4-byte (or 2-byte) elements is stored as 8-row x 16-byte core matrices,
//
//     offset(r, c) = (r / 8) * RS + (c / CH) * CS + (r % 8) * 16 + (c % CH) * ES,   CH = 16 / ES,
//
// RS = byte stride between 8-row groups, CS = byte stride between 16-byte column chunks.  Read as a
// K-major operand (MN index = r, K index = c): SBO = RS, LBO = CS, next K step = +2*CS.  (The same
// tile read MN-major works for 16-bit operands only; 32-bit operands have one MN-major form, below.)
//
// Swizzled slabs (tiles that arrive by tiled TMA loads from row-major global matrices): see
// smem_desc_sw128_k / smem_desc_sw128_mn.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gdn2 {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false (and the caller records an error and bails out) instead of
// spinning forever if the barrier never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t max_tries = (1u << 22)) {
  for (uint32_t i = 0; i < max_tries; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

// ---- proxies / bulk copies --------------------------------------------------------------
// Make generic-proxy shared-memory writes visible to the async proxy (MMA operand reads, bulk stores).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Ask for a 4-D box of a tensor map to be brought into L2 (no destination, no completion to wait for).
// Coordinates as for a load.
__device__ __forceinline__ void tma_prefetch_l2_4d(const void* tmap, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(tmap), "r"(c0),
               "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// 3-D tiled TMA load global -> shared; completion (bytes) on an mbarrier.  `tmap` points at a
// CUtensorMap in kernel-parameter space.  c0 must keep c0 * element size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
      : "memory");
}
// 4-D variants.  A load box that reaches past the end of a dimension is filled with zeros there, a store
// box is clipped.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tmap, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* tmap, int c0, int c1, int c2, int c3, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::"l"(tmap),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(smem_src))
               : "memory");
}
// 3-D tiled TMA store shared -> global (bulk async-group completion); same alignment rules.
__device__ __forceinline__ void tma_store_3d(const void* tmap, int c0, int c1, int c2, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(tmap),
               "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(smem_src))
               : "memory");
}

// 1-D bulk copy shared -> global (bulk async-group completion).
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- TMEM management ---------------------------------------------------------------------
// One full warp executes alloc / dealloc; ncols is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address: lane in bits [31:16], column in bits [15:0].
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// ---- descriptors --------------------------------------------------------------------------
// Shared-memory matrix descriptor, no swizzle, sm_100 descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Swizzled operands, fetched by tiled TMA loads from a row-major fp32 matrix X[rows][cols] in slabs of
// 32 columns: a slab is `rows` lines of 128 bytes, slab s of a tile starts s * rows * 128 bytes after
// the tile (which is 1024-byte aligned).
//   K-major operand (MN index = row, K index = column), TMA swizzle 128B: 8-line atoms, SBO = 1024;
//     the K step of 8 tf32 values is 32 bytes inside the line, then the next slab.
__device__ __forceinline__ uint64_t smem_desc_sw128_k(uint32_t tile, uint32_t slab_bytes, int kstep) {
  const uint32_t saddr = tile + uint32_t(kstep >> 2) * slab_bytes + uint32_t(kstep & 3) * 32u;
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024u >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;  // 128-byte swizzle
  return d;
}
//   MN-major operand (K index = row, MN index = column), TMA swizzle 128B with 32-byte atoms: 4-line
//     atoms, SBO = 512 (next 4 rows of K), LBO = slab stride (next 32 columns of MN); the K step of 8
//     rows is 1024 bytes.  32-bit operands have no other MN-major form.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t tile, uint32_t slab_bytes, int kstep) {
  const uint32_t saddr = tile + uint32_t(kstep) * 1024u;
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((slab_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(512u >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(1) << 61;  // 128-byte swizzle, 32-byte atoms
  return d;
}

enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2 };
enum : uint32_t { kMajorK = 0, kMajorMN = 1 };

// Instruction descriptor for kind::f16 / kind::tf32 with fp32 accumulation.
__host__ __device__ constexpr uint32_t idesc(uint32_t m, uint32_t n, uint32_t fmt, uint32_t a_major,
                                             uint32_t b_major, uint32_t a_neg = 0, uint32_t b_neg = 0) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (a_neg << 13) | (b_neg << 14) | (a_major << 15) |
         (b_major << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- MMA issue (one thread) ------------------------------------------------------------------
__device__ __forceinline__ void mma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t id,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t id,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(id), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// ---- TMEM <-> registers: each thread of a warp reads/writes N consecutive 32-bit columns of its lane
#define GDN2_R8(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])
#define GDN2_W8(r, o) "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]), "r"(r[o + 6]), "r"(r[o + 7])

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : GDN2_R8(r, 0)
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : GDN2_R8(r, 0), GDN2_R8(r, 8)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : GDN2_R8(r, 0), GDN2_R8(r, 8), GDN2_R8(r, 16), GDN2_R8(r, 24)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
          taddr),
      GDN2_W8(r, 0), GDN2_W8(r, 8)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      GDN2_W8(r, 0), GDN2_W8(r, 8), GDN2_W8(r, 16), GDN2_W8(r, 24)
      : "memory");
}

// ---- blocked tile addressing ---------------------------------------------------------------
template <int ES>
__device__ __forceinline__ uint32_t blk_off(int r, int c, int rs, int cs) {
  constexpr int CH = 16 / ES;
  return uint32_t((r >> 3) * rs + (c / CH) * cs + (r & 7) * 16 + (c % CH) * ES);
}

// 32-byte global store (sm_100: 256-bit vector access; the address must be 32-byte aligned).  Two
// neighbouring 16-byte chunks of a blocked tile leave in one instruction, which halves the cache lines
// a warp's store instructions touch in total.
__device__ __forceinline__ void store_global_32b(void* ptr, float4 lo, float4 hi) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "f"(lo.x), "f"(lo.y), "f"(lo.z),
               "f"(lo.w), "f"(hi.x), "f"(hi.y), "f"(hi.z), "f"(hi.w)
               : "memory");
}

// round-to-nearest (ties away from zero) fp32 -> tf32, kept in an fp32 container: the value
// cvt.rna.tf32.f32 gives for every finite input, formed with one integer add and one mask.  The
// conversion instruction shares the transcendental unit (16 results per clock and SM) with the
// exponentials; profiles of the chunk kernels showed that unit busy 75-90 % of the time with
// hundreds of roundings per thread, while the integer pipe was nearly idle.
__device__ __forceinline__ float to_tf32(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}
// The same rounding for a value that only the tensor cores will read (an operand tile in shared memory, a
// tile in the workspace): they ignore the 13 low bits of the container, so adding half a unit is all it
// takes and the mask can stay away.  Anything the CUDA cores multiply by as well needs to_tf32.
__device__ __forceinline__ float to_tf32_operand(float x) { return __uint_as_float(__float_as_uint(x) + 0x1000u); }

}  // namespace tc
}  // namespace gdn2
