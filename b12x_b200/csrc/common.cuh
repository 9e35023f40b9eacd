// Shared device helpers for the sm_100a MoE kernels: mbarrier, TMA, tcgen05/TMEM
// PTX wrappers and bounded waits.  Everything here is header-only.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/b200moe.h"

namespace b200moe {

// ---- status block (int32[16] at scratch + layout.status) ----------------------------------
// word 0: nonzero = a device-side bounded wait ran out; word 1: code of the wait site.
enum WaitSite : int {
  WAIT_NONE = 0,
  WAIT_SMEM_EMPTY = 1,   // producer waiting for a free pipeline stage
  WAIT_SMEM_FULL = 2,    // MMA issuer waiting for TMA data
  WAIT_TMEM_EMPTY = 3,   // MMA issuer waiting for the epilogue to drain the accumulator
  WAIT_TMEM_FULL = 4,    // epilogue waiting for the accumulator
  WAIT_DRAIN = 5,        // producer waiting for its own copies after an abort
  WAIT_CONVERT = 6,      // converter / MMA hand-off in the W4A16 kernel
  WAIT_SF_FULL = 7       // MMA issuer waiting for the scale atoms to reach TMEM
};

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait, then give up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}


// ---- per-role timeline (debug builds only: -DB200MOE_TIMELINE) -------------------------------
// One CTA's roles stamp the SM clock at every pipeline event of a window of k-blocks / tiles into
// a buffer the host registered with b200moe_debug_set_timeline: [kernel 2][cta 2][event 16][kTlN].
// The product build compiles none of this.
#ifdef B200MOE_TIMELINE
constexpr int kTlN = 96;          // k-blocks (or tiles) recorded per event
constexpr int kTlSkip = 160;      // k-blocks skipped first (steady state)
constexpr int kTlSkipTiles = 8;
enum TlEvent : int {
  TL_P_EMPTY = 0, TL_P_ISSUED = 1, TL_M_FULL = 2, TL_M_SF = 3, TL_M_COMMIT = 4, TL_S_LANDED = 5,
  TL_S_DONE = 6, TL_S_SLOTFREE = 7, TL_M_TMEM_EMPTY = 8, TL_E_FULL = 9, TL_E_RELEASED = 10, TL_E_DONE = 11,
  TL_M_MMA0 = 13, TL_M_ISSUED = 14, TL_M_PEEKED = 15,
  TL_O_LANDED = 12   // an otherwise idle lane that watches the stage's `full` barrier
};
static __device__ long long* g_timeline = nullptr;   // one per translation unit
__device__ __forceinline__ long long sm_clock() {
  long long t;
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
  return t;
}
// `buf` = this role's copy of the buffer pointer (null: this CTA is not recorded), read once at
// the top of the role so that a stamp costs one clock read and one store
__device__ __forceinline__ void tl_stamp(long long* buf, int kernel, int slot, int ev, int n, int skip) {
  if (buf == nullptr || n < skip || n >= skip + kTlN) return;
  buf[((kernel * 2 + slot) * 16 + ev) * kTlN + (n - skip)] = sm_clock();
}
#define TL_STAGE(kernel, slot, ev, n) tl_stamp(tl_buf, kernel, slot, ev, n, kTlSkip)
#define TL_TILE(kernel, slot, ev, n) tl_stamp(tl_buf, kernel, slot, ev, n, kTlSkipTiles)
#define TL_DECL(x) int x = 0
#define TL_INC(x) (++(x))
#else
#define TL_STAGE(kernel, slot, ev, n) ((void)0)
#define TL_TILE(kernel, slot, ev, n) ((void)0)
#define TL_DECL(x) ((void)0)
#define TL_INC(x) ((void)0)
#endif

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-suspending look at a barrier phase (try_wait may park the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false (and records the site) when the limit ran out or another
// role of this CTA already gave up; the caller must then leave its loop.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* cta_abort, int* status,
                                                  int site) {
  if (mbar_try_wait(bar, parity)) return true;
  // The limit is only looked at every 1024 failed polls, and the clock is first read then: a
  // wait that ends within a few polls never touches the (slow) global timer.
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3ffu) == 0) {
      if (*cta_abort) return false;
      const unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > kWaitLimitNs) {
        *cta_abort = 1;
        if (status != nullptr) {
          atomicCAS(status, 0, 1);
          atomicCAS(status + 1, 0, site);
        }
        return false;
      }
    }
  }
}

// ---- TMA --------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load, completes on an mbarrier of this CTA.  x = innermost coordinate (elements).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x),
      "r"(y)
      : "memory");
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes),
      "r"(smem_u32(bar))
      : "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------
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
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive (count 1) on an mbarrier of this CTA once all MMAs issued so far by this thread retire.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// 32 rows x 128 bit from shared memory -> 4 TMEM columns, replicated to the 4 sub-partitions.
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Each thread of the warp reads 16 consecutive fp32 columns of its own TMEM lane.
__device__ __forceinline__ void tc_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Each thread of the warp writes N consecutive 32-bit columns of its own TMEM lane.
__device__ __forceinline__ void tc_st_32x32b_x4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tc_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tc_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Scale atoms (512 bytes each, `natoms` of them back to back in shared memory) -> `4 * natoms`
// TMEM columns of this warp's sub-partition, atom j at columns [col_stride * j, +4): lane i takes
// the 16 bytes of atom row i, as tcgen05.cp.32x128b.warpx4 would place them.  Called by one warp
// per sub-partition; the tensor pipe is not involved.
template <int NATOMS>
__device__ __forceinline__ void sf_atoms_to_tmem(uint32_t taddr, const uint8_t* atoms, int lane, int col_stride) {
#pragma unroll
  for (int j = 0; j < NATOMS; ++j) {
    const uint4 v = *(reinterpret_cast<const uint4*>(atoms + 512 * j) + lane);
    const uint32_t r[4] = {v.x, v.y, v.z, v.w};
    tc_st_32x32b_x4(taddr + col_stride * j, r);
  }
}

// Shared-memory matrix descriptor (sm_100 "version 1"), K-major operand tile whose rows are
// 128 bytes long and stored with the 128-byte swizzle (what a SWIZZLE_128B TMA box writes).
// 8-row groups are 1024 bytes apart.  The tile base must be 1024-byte aligned; advancing along
// K inside the 128-byte row is done by adding (bytes >> 4) to the low word.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);  // start address
  d |= static_cast<uint64_t>(1) << 16;                    // leading byte offset (unused) = 1
  d |= static_cast<uint64_t>(1024 >> 4) << 32;            // stride byte offset: 8 rows * 128 B
  d |= static_cast<uint64_t>(1) << 46;                    // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                    // layout: SWIZZLE_128B
  return d;
}
// Un-swizzled descriptor for the scale-factor copy: 32 rows of 16 bytes, rows contiguous,
// 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t make_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>(128 >> 4) << 32;  // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Instruction descriptor, block-scaled kinds (mxf4nvf4 / mxf4 / mxf8f6f4), A and B K-major.
//   a_fmt/b_fmt: kind::mxf4nvf4 -> 1 (E2M1); kind::mxf8f6f4 -> 0 E4M3, 5 E2M1
//   sf_fmt: 0 = UE4M3, 1 = UE8M0;  sfa_id/sfb_id: byte offset of the scale inside the TMEM word
__host__ __device__ constexpr uint32_t make_idesc_block_scaled(int m, int n, int a_fmt, int b_fmt,
                                                               int sf_fmt, int sfa_id = 0,
                                                               int sfb_id = 0) {
  return (static_cast<uint32_t>(sfb_id & 3) << 4) | (static_cast<uint32_t>(a_fmt & 7) << 7) |
         (static_cast<uint32_t>(b_fmt & 7) << 10) | (static_cast<uint32_t>((n >> 3) & 63) << 17) |
         (static_cast<uint32_t>(sf_fmt & 1) << 23) | (static_cast<uint32_t>((m >> 4) & 31) << 24) |
         (static_cast<uint32_t>(sfa_id & 3) << 29);
}
// Instruction descriptor, kind::f16 with BF16 operands (K-major) and FP32 accumulation.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>((n >> 3) & 63) << 17) |
         (static_cast<uint32_t>((m >> 4) & 31) << 24);
}

// D[tmem] (+)= A[smem] * B[smem] with per-block scales read from TMEM.
__device__ __forceinline__ void mma_nvf4_4x(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
      "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void mma_mxf8f6f4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                             uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale "
      "[%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem),
      "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One 32-byte store (sm_100 has 256-bit global stores); `p` must be 32-byte aligned.
__device__ __forceinline__ void st_global_f32x8(float* p, const float (&v)[8]) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]),
               "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7])
               : "memory");
}

// ---- numeric helpers shared by the quantisers ---------------------------------
// 8 floats -> 8 E2M1 codes (round-to-nearest-even, saturating), v[0] in the low nibble.
// A negative zero result is stored as +0 (code 0), as the reference packer does.
__device__ __forceinline__ uint32_t pack_e2m1x8(const float (&v)[8]) {
  uint32_t p;
  asm volatile(
      "{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}\n"
      : "=r"(p)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  const uint32_t nz = (p | (p >> 1) | (p >> 2)) & 0x11111111u;  // magnitude != 0 per nibble
  return p & (0x77777777u | (nz << 3));
}
__device__ __forceinline__ uint8_t f32_to_e4m3_rn_sat(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(__half(h));
}

// Byte offset of scale (row m of a 128-row tile, scale column c) inside the chain of 512-byte
// atoms of that tile: atom = c / 4; inside the atom (m % 32) * 16 + (m / 32) * 4 + c % 4.
__device__ __forceinline__ uint32_t sf_atom_offset(uint32_t m, uint32_t c) {
  return (c >> 2) * 512u + (m & 31u) * 16u + (m >> 5) * 4u + (c & 3u);
}

__host__ __device__ constexpr int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

}  // namespace b200moe
