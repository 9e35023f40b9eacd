// Stages 4 and 5 for large batches (recipes nvfp4 and w4a8_mx) on CTA PAIRS: tcgen05 with cta_group::2.
//
// Two CTAs of a cluster share one 256 x 256 tile: each owns 128 token rows (its own row tile of the
// expert) and loads only HALF of the 256 weight rows; the pair's MMA (M = 256, N = 256, issued by
// one thread of the even CTA) reads the weight halves out of both CTAs' shared memory and writes a
// 128 x 256 accumulator into each CTA's tensor memory.  Per CTA and 256-value k-block that is
// 16 KiB of token rows + 16 KiB of weight rows + 6 KiB of scale atoms from L2 instead of 16 + 32 + 6:
// the wide single-CTA kernel is limited by exactly that operand stream.
//
// Roles per CTA (512 threads, four warp groups): warp 0 operand producer (the operand copies of
// either CTA complete on the EVEN CTA's stage barrier), warp 2 scale-atom producer (a ring of eight
// slots of its own, completing on barriers of the CTA itself), warps 4..7 move the CTA's scale atoms
// into its tensor memory (tcgen05.st) and arrive on the even CTA's stage barrier, warps 8..15
// epilogue of the CTA's own accumulator (drained into registers first, so that it overlaps the
// next tile's main loop; the other warp groups hand over registers for that).  Even CTA only:
// warp 1 issues the MMAs and commits (multicast) to both CTAs' barriers.  The odd CTA's epilogue warps release the
// accumulator with remote arrives on the even CTA's barrier.  Every wait is bounded; the two cluster-wide
// barriers (after set-up, before tear-down) are reached by both CTAs unconditionally.
#include <stdlib.h>

#include "cluster_pair.cuh"
#include "gemm_shared.cuh"

namespace b200moe {
namespace pair {

constexpr int kThreads = 512;                 // four warp groups
constexpr int kRegsSmall = 48;                // register allowance: producers, MMA, scale warps ...
constexpr int kRegsEpilogue = 208;            // ... and the epilogue warp groups
constexpr int kStages = 5;
constexpr int kRowBytes = 128;
constexpr int kSmemA = 128 * kRowBytes;       // this CTA's 128 token rows, one k-block
constexpr int kSmemB = 128 * kRowBytes;       // this CTA's half of the 256 weight rows
constexpr int kSmemSfa = 4 * 512;             // scale atoms of the token rows
constexpr int kSmemSfb = 2 * 4 * 512;         // scale atoms of all 256 weight rows (two chains)
constexpr int kStageBytes = kSmemA + kSmemB;                  // operand rows of one stage
constexpr int kSfSlots = 8;                   // ring of scale-atom slots, deeper than the stages
constexpr int kSfSlotBytes = kSmemSfa + kSmemSfb;
constexpr int kTmemCols = 512;
constexpr int kTmemSf = 256;                  // accumulator: columns 0..255
constexpr int kSfCols = 48;                   // per stage: 16 (tokens) + 32 (weights)
// bytes both CTAs' operand copies of one stage report to the barrier (the 4-bit unpacking TMA type of
// the MX kind counts the packed bytes it reads: half of what it writes)
__host__ __device__ constexpr uint32_t stage_tx_bytes(int kind) { return 2u * (kSmemA + (kind == KIND_MX ? kSmemB / 2 : kSmemB)); }

struct __align__(8) SmemTail {
  uint64_t full[kStages];       // used in the even CTA: all copies of the pair have landed
  uint64_t empty[kStages];      // per CTA: the MMAs that read the stage have retired
  uint64_t sf_landed[kSfSlots]; // per CTA: the slot's scale atoms are in this CTA's shared memory
  uint64_t sf_empty[kSfSlots];  // per CTA: the four scale warps have read the slot
  uint64_t tmem_full;           // per CTA: the accumulator is complete
  uint64_t tmem_empty;          // even CTA: all 16 epilogue warps of the pair have drained it
  uint32_t tmem_base;
  int abort_flag;
  int32_t tile_base[kMaxExperts + 1];
  int32_t pair_base[kMaxExperts + 1];
};
constexpr int kSmemBytes =
    1024 + kStages * kStageBytes + kSfSlots * kSfSlotBytes + static_cast<int>(sizeof(SmemTail));

__device__ __forceinline__ void mma_nvf4_4x_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X "
      "[%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

__device__ __forceinline__ void mma_mxf8f6f4_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                  uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale "
      "[%0], %1, %2, %3, [%5], [%6], p;\n\t}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Work item of a CTA pair: (expert, n-tile, pair of row tiles).  This CTA's row tile is
// first + rank; an expert with an odd number of row tiles leaves the odd CTA of its last pair
// without one (rows = 0: it multiplies the neighbour's rows again and stores nothing).
struct PairCoord {
  int e, nt, mt_load, mt, rows;
};
__device__ __forceinline__ PairCoord decode_pair(int w, const GemmParams& p, const SmemTail* tail, int rank) {
  const TileCoord c = decode_tile(w, p.n_tiles, tail->pair_base, p.E);
  PairCoord r;
  r.e = c.e;
  r.nt = c.nt;
  const int last = tail->tile_base[c.e + 1] - 1;
  r.mt = tail->tile_base[c.e] + 2 * (c.mt - tail->pair_base[c.e]) + rank;
  r.mt_load = r.mt <= last ? r.mt : last;
  r.rows = r.mt <= last ? p.mtile_rows[r.mt] : 0;
  return r;
}

// KIND_NVFP4: 256 values per stage, four MMAs of 64, one scale atom per MMA and 128 rows.
// KIND_MX: 128 values per stage (the weights' FP4 codes expanded to bytes by the TMA), four MMAs of
// 32, ONE scale atom per stage and 128 rows (its four bytes are the per-32 scales of the stage).
template <int KIND, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                               const GemmParams p) {
  constexpr bool kGated = epi_is_gated(EPI);
  constexpr int kPerStage = KIND == KIND_MX ? 128 : 256;   // reduction elements per stage
  constexpr int kPerMma = KIND == KIND_MX ? 32 : 64;
  constexpr uint32_t kAtomBytes = KIND == KIND_MX ? 512u : 2048u;   // scale bytes per stage and 128 rows
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + kStages * kSmemA;
  uint8_t* sSf = sB + kStages * kSmemB;          // [slot][token atoms 2 KiB | weight atoms 4 KiB]
  SmemTail* tail = reinterpret_cast<SmemTail*>(sSf + kSfSlots * kSfSlotBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());     // 0 = even CTA (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&tail->full[s], 1 + 8);   // the producer's arrive + the scale warps of both CTAs
      mbar_init(&tail->empty[s], 1);
    }
    for (int s = 0; s < kSfSlots; ++s) {
      mbar_init(&tail->sf_landed[s], 1);
      mbar_init(&tail->sf_empty[s], 4);
    }
    mbar_init(&tail->tmem_full, 1);
    mbar_init(&tail->tmem_empty, 16);
    tail->abort_flag = 0;
    fence_mbar_init();
    // row tiles and tile pairs per expert (prefix sums)
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      const int t0 = p.tile_base[e], t1 = p.tile_base[e + 1];
      tail->tile_base[e] = t0;
      tail->pair_base[e] = acc;
      acc += (t1 - t0 + (p.tile_mode == TILES_PAIRS ? 0 : 1)) >> 1;   // full pairs only, or the odd tile too
      if (e == p.E - 1) tail->tile_base[p.E] = t1;
    }
    tail->pair_base[p.E] = acc;
  }
  if (warp == 1) {
    tmem_alloc_pair(&tail->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after();

  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_flag = &tail->abort_flag;
  const int total_work = tail->pair_base[p.E] * p.n_tiles;
#ifdef B200MOE_TIMELINE
  const int tl_slot = cluster_id == 0 ? rank : -1;
  constexpr int tl_k = EPI == EPI_FC2 ? 1 : 0;
  long long* const tl_buf = tl_slot >= 0 ? g_timeline : nullptr;
#endif

  if (warp < 8) {
  regs_release_to<kRegsSmall>();
  if (warp == 0) {
    // ------------------------------ operand producer (both CTAs) -----------------
    // lane 0: (even CTA) arms the stage barrier; token rows.  lanes 1, 2: the two 64-row boxes
    // of this CTA's weight half.  All operand copies complete on the EVEN CTA's barrier.
    if (lane < 3) {
      if (lane == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TL_DECL(tl_n);
      for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
        const PairCoord c = decode_pair(w, p, tail, rank);
        int y;                          // row coordinate of this lane's copy
        if (lane == 0) {
          y = p.mtile_row0[c.mt_load];
        } else {
          const int b = lane - 1;
          int wrow;
          if (kGated) {
            int g = 2 * c.nt + rank;                               // pair group of this CTA
            if (g * 64 >= p.out_cols) g = 2 * c.nt;                // half-empty last tile
            wrow = (b ? p.sub1_base : p.sub0_base) + g * 64;       // 64 up rows / 64 gate rows
          } else {
            wrow = c.nt * 256 + rank * 128 + b * 64;
            if (wrow >= p.w_rows) wrow = c.nt * 256 + b * 64;
          }
          y = c.e * p.w_rows + wrow;
        }
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->empty[stage], phase ^ 1, abort_flag, p.status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (lane == 0) TL_STAGE(tl_k, tl_slot, TL_P_EMPTY, tl_n);
          const uint32_t bar = map_to_cta(smem_u32(&tail->full[stage]), 0);
          if (lane == 0) {
            if (rank == 0) mbar_expect_tx(&tail->full[stage], stage_tx_bytes(KIND));
            tma_load_2d_pair(sA + stage * kSmemA, &tmA, bar, kb * kRowBytes, y);
          } else {
            tma_load_2d_pair(sB + stage * kSmemB + (lane - 1) * 64 * kRowBytes, &tmB, bar, kb * kRowBytes, y);
          }
          if (lane == 0) TL_STAGE(tl_k, tl_slot, TL_P_ISSUED, tl_n);
          TL_INC(tl_n);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let copies in flight land
      }
    }
#ifdef B200MOE_TIMELINE
    else if (lane == 31 && tl_buf != nullptr && rank == 0) {
      int stage = 0, n = 0;
      uint32_t phase = 0;
      for (int w = cluster_id; w < total_work && n < kTlSkip + kTlN; w += num_clusters) {
        for (int kb = 0; kb < p.k_blocks; ++kb, ++n) {
          if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, nullptr, 0)) break;
          TL_STAGE(tl_k, tl_slot, TL_O_LANDED, n);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
#endif
  } else if (warp == 2) {
    // ------------------------------ scale-atom producer (both CTAs) --------------
    // The scale atoms travel through a ring of their own that is deeper than the operand stages:
    // they are in shared memory before the stage's tensor-memory columns are free again, so their
    // load is off the round trip that bounds the pipeline.  lane 0: token atoms, lanes 1, 2: the
    // two weight chains (both CTAs fetch both); they complete on this CTA's own barrier.
    if (lane < 3) {
      int slot = 0;
      uint32_t sphase = 0;
      bool ok = true;
      for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
        const PairCoord c = decode_pair(w, p, tail, rank);
        const uint8_t* my_sf;
        if (lane == 0) {
          my_sf = p.sfa + static_cast<size_t>(c.mt_load) * p.atoms_k * 512;
        } else {
          int rg = 2 * c.nt + (lane - 1);
          if (rg >= p.sfb_rowgroups) rg = 2 * c.nt;
          my_sf = p.sfb + (static_cast<size_t>(c.e) * p.sfb_rowgroups + rg) * p.atoms_k * 512;
        }
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->sf_empty[slot], sphase ^ 1, abort_flag, p.status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          const int ksteps = min(4, (p.kdim - kb * kPerStage) / kPerMma);
          // NVFP4: one scale atom per MMA step; MX: one atom covers the whole stage
          const uint32_t sf_bytes = KIND == KIND_MX ? 512u : static_cast<uint32_t>(ksteps) * 512u;
          const size_t sf_off = static_cast<size_t>(kb) * kAtomBytes;
          uint8_t* dst = sSf + slot * kSfSlotBytes;
          if (lane == 0) {
            mbar_expect_tx(&tail->sf_landed[slot], 3u * sf_bytes);
            bulk_load(dst, my_sf + sf_off, sf_bytes, &tail->sf_landed[slot]);
          } else {
            bulk_load(dst + kSmemSfa + (lane - 1) * 2048, my_sf + sf_off, sf_bytes, &tail->sf_landed[slot]);
          }
          if (++slot == kSfSlots) {
            slot = 0;
            sphase ^= 1;
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA) -------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc =
          KIND == KIND_MX ? make_idesc_block_scaled(256, 256, /*a e4m3*/ 0, /*b e2m1*/ 5, /*ue8m0*/ 1)
                          : make_idesc_block_scaled(256, 256, /*a*/ 1, /*b*/ 1, /*ue4m3*/ 0);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      const uint64_t adesc0 = make_desc_sw128(smem_u32(sA)), bdesc0 = make_desc_sw128(smem_u32(sB));
      const uint32_t sf0_t = tmem_base + kTmemSf;
      const int last_ksteps = min(4, (p.kdim - (p.k_blocks - 1) * kPerStage) / kPerMma);   // MMAs of a tile's last k-block
      TL_DECL(tl_n);
      TL_DECL(tl_t);
      for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
        if (!mbar_wait_bounded(&tail->tmem_empty, acc_phase ^ 1, abort_flag, p.status, WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        TL_TILE(tl_k, tl_slot, TL_M_TMEM_EMPTY, tl_t);
        TL_INC(tl_t);
        tc_fence_after();
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          // one barrier per stage: both CTAs' operand rows have landed (TMA byte count) and their
          // eight scale warps have put the scale atoms into tensor memory (their arrivals)
          if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, p.status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          TL_STAGE(tl_k, tl_slot, TL_M_SF, tl_n);
          tc_fence_after();
          // the stage's descriptors differ from stage 0's only in the start-address field (16-byte units)
          const uint32_t sfa_t = sf0_t + stage * kSfCols;
          const uint32_t sfb_t = sfa_t + 16;
          const uint64_t adesc = adesc0 + static_cast<uint32_t>(stage * (kSmemA >> 4));
          const uint64_t bdesc = bdesc0 + static_cast<uint32_t>(stage * (kSmemB >> 4));
          if (kb + 1 < p.k_blocks || last_ksteps == 4) {
            // this thread shares its scheduler with busy epilogue warps: the fewer instructions
            // between two MMAs, the shorter the tensor pipe waits for it
            if (KIND == KIND_MX) {
              // MMA step j uses byte j of each word of the stage's one scale atom
              mma_mxf8f6f4_pair(tmem_base, adesc, bdesc, idesc, sfa_t, sfb_t, kb > 0 ? 1u : 0u);
              TL_STAGE(tl_k, tl_slot, TL_M_MMA0, tl_n);
              mma_mxf8f6f4_pair(tmem_base, adesc + 2, bdesc + 2, idesc | (1u << 29) | (1u << 4), sfa_t + (1u << 30),
                                sfb_t + (1u << 30), 1u);
              mma_mxf8f6f4_pair(tmem_base, adesc + 4, bdesc + 4, idesc | (2u << 29) | (2u << 4), sfa_t + (2u << 30),
                                sfb_t + (2u << 30), 1u);
              mma_mxf8f6f4_pair(tmem_base, adesc + 6, bdesc + 6, idesc | (3u << 29) | (3u << 4), sfa_t + (3u << 30),
                                sfb_t + (3u << 30), 1u);
            } else {
              mma_nvf4_4x_pair(tmem_base, adesc, bdesc, idesc, sfa_t, sfb_t, kb > 0 ? 1u : 0u);
              TL_STAGE(tl_k, tl_slot, TL_M_MMA0, tl_n);
              mma_nvf4_4x_pair(tmem_base, adesc + 2, bdesc + 2, idesc, sfa_t + 4, sfb_t + 8, 1u);
              mma_nvf4_4x_pair(tmem_base, adesc + 4, bdesc + 4, idesc, sfa_t + 8, sfb_t + 16, 1u);
              mma_nvf4_4x_pair(tmem_base, adesc + 6, bdesc + 6, idesc, sfa_t + 12, sfb_t + 24, 1u);
            }
          } else {
            for (int j = 0; j < last_ksteps; ++j) {
              if (KIND == KIND_MX) {
                const uint32_t ju = static_cast<uint32_t>(j);
                mma_mxf8f6f4_pair(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc | (ju << 29) | (ju << 4),
                                  sfa_t + (ju << 30), sfb_t + (ju << 30), (kb > 0 || j > 0) ? 1u : 0u);
              } else {
                mma_nvf4_4x_pair(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, sfa_t + 4 * j, sfb_t + 8 * j,
                                 (kb > 0 || j > 0) ? 1u : 0u);
              }
            }
          }
          TL_STAGE(tl_k, tl_slot, TL_M_ISSUED, tl_n);
          tc_commit_pair_both(&tail->empty[stage]);
          TL_STAGE(tl_k, tl_slot, TL_M_COMMIT, tl_n);
          TL_INC(tl_n);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit_pair_both(&tail->tmem_full);
        acc_phase ^= 1;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------ scale atoms -> TMEM (both CTAs) ---------------
    // Four warps, one per TMEM sub-partition.  Per k-block: the slot's atoms have landed and the
    // stage's tensor-memory columns are free again (the MMAs of the stage's previous use have
    // retired: the same barrier the operand producer waits on); then shared memory -> registers
    // -> tensor memory (tcgen05.st), the slot is handed back, and the warp arrives on the even
    // CTA's scale barrier (8 arrivals: 4 warps of each CTA).
    const int sub = warp & 3;
    int stage = 0, slot = 0;
    uint32_t phase = 0, sphase = 0;
    bool ok = true;
    TL_DECL(tl_n);
    for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_bounded(&tail->sf_landed[slot], sphase, abort_flag, p.status, WAIT_SMEM_FULL)) {
          ok = false;
          break;
        }
        if (warp == 4 && lane == 0) TL_STAGE(tl_k, tl_slot, TL_S_LANDED, tl_n);
        if (!mbar_wait_bounded(&tail->empty[stage], phase ^ 1, abort_flag, p.status, WAIT_SMEM_EMPTY)) {
          ok = false;
          break;
        }
        if (warp == 4 && lane == 0) TL_STAGE(tl_k, tl_slot, TL_S_SLOTFREE, tl_n);
        tc_fence_after();
        const uint32_t sfa_t = tmem_base + kTmemSf + stage * kSfCols + (static_cast<uint32_t>(sub * 32) << 16);
        const uint32_t sfb_t = sfa_t + 16;
        const uint8_t* src = sSf + slot * kSfSlotBytes;
        if (KIND == KIND_MX) {
          sf_atoms_to_tmem<1>(sfa_t, src, lane, 4);
          sf_atoms_to_tmem<1>(sfb_t, src + kSmemSfa, lane, 4);
          sf_atoms_to_tmem<1>(sfb_t + 4, src + kSmemSfa + 2048, lane, 4);
        } else {
          sf_atoms_to_tmem<4>(sfa_t, src, lane, 4);
          sf_atoms_to_tmem<4>(sfb_t, src + kSmemSfa, lane, 8);
          sf_atoms_to_tmem<4>(sfb_t + 4, src + kSmemSfa + 2048, lane, 8);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&tail->sf_empty[slot]);
          mbar_arrive_cluster(map_to_cta(smem_u32(&tail->full[stage]), 0));
        }
        if (warp == 4 && lane == 0) TL_STAGE(tl_k, tl_slot, TL_S_DONE, tl_n);
        TL_INC(tl_n);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
        if (++slot == kSfSlots) {
          slot = 0;
          sphase ^= 1;
        }
      }
    }
  }
  } else {
    // ------------------------------ epilogue (both CTAs) --------------------------
    regs_raise_to<kRegsEpilogue>();
    const int sub = warp & 3;
    const int half = (warp - 8) >> 2;
    const int m = sub * 32 + lane;
    const uint32_t release_addr = map_to_cta(smem_u32(&tail->tmem_empty), 0);
    uint32_t acc_phase = 0;
    TL_DECL(tl_t);
    for (int w = cluster_id; w < total_work; w += num_clusters) {
      const PairCoord c = decode_pair(w, p, tail, rank);
      const int row0 = p.mtile_row0[c.mt_load];
      if (!mbar_wait_bounded(&tail->tmem_full, acc_phase, abort_flag, p.status, WAIT_TMEM_FULL)) break;
      if (warp == 8 && lane == 0) TL_TILE(tl_k, tl_slot, TL_E_FULL, tl_t);
      acc_phase ^= 1;
      tc_fence_after();
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(sub * 32) << 16);
      epilogue_tile<KIND, EPI, 256>(p, c.e, c.mt_load, c.nt, row0, c.rows, t_lane, m, half, lane, [&]() {
        if (lane == 0) mbar_arrive_cluster(release_addr);
        if (warp == 8 && lane == 0) TL_TILE(tl_k, tl_slot, TL_E_RELEASED, tl_t);
      });
      if (warp == 8 && lane == 0) TL_TILE(tl_k, tl_slot, TL_E_DONE, tl_t);
      TL_INC(tl_t);
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // nobody signals the other CTA's shared memory after this
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int KIND, int EPI>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int max_ctas,
                  cudaStream_t s) {
  auto kern = grouped_gemm_pair_kernel<KIND, EPI>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return B200MOE_ECUDA;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = s;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  // persistent grid: as many CTA pairs as can be resident at once
  cfg.gridDim = dim3(static_cast<unsigned>(max_ctas & ~1));
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) return B200MOE_ECUDA;
  if (2 * clusters < max_ctas) cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p) == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

}  // namespace pair

// The CTA-pair kernels serve nvfp4 and w4a8_mx plans with 128-row tiles and gated FC1 (or FC2).  A
// pair streams 38 KB per stage and CTA instead of 54 KB (nvfp4); they are the faster kernels once
// experts have several row tiles (C4: FC1 0.92 against 1.10 ms, FC2 0.41 against 0.52 ms).  Default:
// plans whose capacity averages at least two row tiles per expert; an expert with an odd number of
// row tiles leaves half a pair idle, so smaller plans stay on the single-CTA kernel.
// B200MOE_PAIR=1 / 0 forces them on (where the shape allows) / off.
// Whether the left-over row tile of an expert with an odd number of them goes to a single-CTA launch
// of its own (after the pair kernel) or into a half-empty pair.  The second launch has wave tails of
// its own, so it pays while experts hold few row tiles: 128 experts x 4 row tiles FC1 1.21 -> 1.15 ms,
// 128 x 2 (w4a16) 1.17 -> 1.10 ms, but 8 experts x 16 row tiles 0.915 -> 0.927 ms.  Default: plans
// that average fewer than eight row tiles per expert; B200MOE_TAIL_SPLIT=1 / 0 forces it on / off.
bool tail_split(const b200moe_gemm_args* a) {
  static int mode = -2;
  if (mode == -2) {
    const char* e = getenv("B200MOE_TAIL_SPLIT");
    mode = e == nullptr ? -1 : (atoi(e) != 0 ? 1 : 0);
  }
  if (mode >= 0) return mode == 1;
  return static_cast<int64_t>(a->layout->rows) < 1024ll * a->num_experts;
}

bool pair_ok(const b200moe_gemm_args* a, bool fc1) {
  static int mode = -2;
  if (mode == -2) {
    const char* e = getenv("B200MOE_PAIR");
    mode = e == nullptr ? -1 : (atoi(e) != 0 ? 1 : 0);
  }
  if (mode == 0 || a->layout->tile_rows != 128) return false;
  if (a->recipe != B200MOE_RECIPE_NVFP4 && a->recipe != B200MOE_RECIPE_W4A8_MX) return false;
  if (a->hidden_size % 64 != 0 || a->intermediate % 64 != 0 || a->num_experts > kMaxExperts) return false;
  if (fc1 && a->activation == B200MOE_ACT_RELU2) return false;
  if (mode == 1) return true;
  return static_cast<int64_t>(a->layout->rows) >= 256ll * a->num_experts;
}

template <int KIND>
static int pair_gemm1_any(const b200moe_gemm_args* a, cudaStream_t stream) {
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  constexpr bool mx = KIND == KIND_MX;
  if (a->w13_sf == nullptr || (!mx && a->a2_gscale == nullptr)) return B200MOE_EINVAL;
  char* base = static_cast<char*>(a->scratch);
  GemmParams p = {};
  fill_common(p, a, base);
  p.tile_mode = tail_split(a) ? TILES_PAIRS : TILES_ALL;
  p.atoms_k = ceil_div_i(K, mx ? 128 : 64);
  p.sfb_rowgroups = I / 64;              // pair atoms: 64 up rows + 64 gate rows
  CUtensorMap tmA, tmB;
  int rc = make_tmap_bytes_2d(&tmA, base + L.act_q, mx ? K : K / 2, L.rows, 128);
  if (rc != B200MOE_OK) return rc;
  rc = mx ? make_tmap_fp4_unpack_2d(&tmB, a->w13, K, static_cast<uint64_t>(E) * 2 * I, 64)
          : make_tmap_bytes_2d(&tmB, a->w13, K / 2, static_cast<uint64_t>(E) * 2 * I, 64);
  if (rc != B200MOE_OK) return rc;
  p.sfa = reinterpret_cast<const uint8_t*>(base + L.act_sf);
  p.sfb = a->w13_sf;
  p.alphas = a->w1_alphas;
  p.gscale2 = a->a2_gscale;
  p.out_q = reinterpret_cast<uint8_t*>(base + L.mid_q);
  p.out_sf = reinterpret_cast<uint8_t*>(base + L.mid_sf);
  p.tap = a->fc1_tap;
  p.kdim = K;
  p.k_blocks = ceil_div_i(K, mx ? 128 : 256);
  p.w_rows = 2 * I;
  p.sub0_base = a->gate_first ? I : 0;   // up rows
  p.sub1_base = a->gate_first ? 0 : I;   // gate rows
  p.n_step = 128;
  p.n_tiles = ceil_div_i(I, 128);
  p.out_cols = I;
  p.out_atoms = ceil_div_i(I, mx ? 128 : 64);
  const int ctas = a->num_sms > 0 ? a->num_sms : num_sms_cached();
  if (p.act_kind == 0 && !(p.limit > 0.f))
    return pair::launch<KIND, EPI_FC1_SILU>(tmA, tmB, p, ctas, stream);
  if (p.act_kind == 2) return pair::launch<KIND, EPI_FC1_SITU>(tmA, tmB, p, ctas, stream);
  return pair::launch<KIND, EPI_FC1_GATED>(tmA, tmB, p, ctas, stream);
}

template <int KIND>
static int pair_gemm2_any(const b200moe_gemm_args* a, cudaStream_t stream) {
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  constexpr bool mx = KIND == KIND_MX;
  if (a->w2_sf == nullptr) return B200MOE_EINVAL;
  char* base = static_cast<char*>(a->scratch);
  GemmParams p = {};
  fill_common(p, a, base);
  p.tile_mode = tail_split(a) ? TILES_PAIRS : TILES_ALL;
  p.atoms_k = ceil_div_i(I, mx ? 128 : 64);
  p.sfb_rowgroups = ceil_div_i(K, 128);
  CUtensorMap tmA, tmB;
  int rc = make_tmap_bytes_2d(&tmA, base + L.mid_q, mx ? I : I / 2, L.rows, 128);
  if (rc != B200MOE_OK) return rc;
  rc = mx ? make_tmap_fp4_unpack_2d(&tmB, a->w2, I, static_cast<uint64_t>(E) * K, 64)
          : make_tmap_bytes_2d(&tmB, a->w2, I / 2, static_cast<uint64_t>(E) * K, 64);
  if (rc != B200MOE_OK) return rc;
  p.sfa = reinterpret_cast<const uint8_t*>(base + L.mid_sf);
  p.sfb = a->w2_sf;
  p.alphas = a->w2_alphas;
  p.out_f32 = reinterpret_cast<float*>(base + L.routed);
  p.kdim = I;
  p.k_blocks = ceil_div_i(I, mx ? 128 : 256);
  p.w_rows = K;
  p.out_cols = K;
  p.n_step = 256;
  p.n_tiles = ceil_div_i(K, 256);
  const int ctas = a->num_sms > 0 ? a->num_sms : num_sms_cached();
  return pair::launch<KIND, EPI_FC2>(tmA, tmB, p, ctas, stream);
}

int nvfp4_pair_gemm1(const b200moe_gemm_args* a, cudaStream_t s) { return pair_gemm1_any<KIND_NVFP4>(a, s); }
int nvfp4_pair_gemm2(const b200moe_gemm_args* a, cudaStream_t s) { return pair_gemm2_any<KIND_NVFP4>(a, s); }
int mx_pair_gemm1(const b200moe_gemm_args* a, cudaStream_t s) { return pair_gemm1_any<KIND_MX>(a, s); }
int mx_pair_gemm2(const b200moe_gemm_args* a, cudaStream_t s) { return pair_gemm2_any<KIND_MX>(a, s); }

}  // namespace b200moe
