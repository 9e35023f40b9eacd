// Stages 4 and 5: grouped block-scaled expert GEMMs on tcgen05 (sm_100a), recipes nvfp4 and w4a8_mx.
//
//   FC1:  acc[128 x BN] = Xq[128 rows of one expert] . W13q[BN/2 up rows ; BN/2 gate rows]^T
//         epilogue: x alpha1 -> gated activation (fp32) -> (nvfp4: round to bf16) -> re-quantise
//         -> codes + scale atoms of the FC2 A operand
//   FC2:  acc[128 x BN] = Hq . W2q[BN rows]^T ; epilogue: x alpha2 -> float32 routed rows
//
// One persistent CTA per SM walks the (expert, n-tile, m-tile) work list that the sort kernel left
// in the scratch arena.  Four warp groups: warp 0 feeds a TMA pipeline (SWIZZLE_128B operand tiles +
// plain bulk copies of the 512-byte scale atoms) and warp 1 issues the block-scaled tcgen05.mma
// (warps 2, 3 idle); warps 4..7 move the scale atoms into TMEM with tcgen05.st; warps 8..15 are the
// epilogue.  Tile = 128 x 256 with one accumulator (two would leave no TMEM columns for the scale
// atoms): the epilogue warps drain it into registers first -- the first two warp groups hand most
// of their registers to them (setmaxnreg) -- and release it, so the arithmetic and the stores of a
// tile run under the main loop of the next.  Every wait is bounded; a wait that runs out marks the
// status block and every role leaves its loop.
#include <stdlib.h>

#include "gemm_shared.cuh"

namespace b200moe {

constexpr int kBM = 128;            // tile rows (MMA M)
constexpr int kRowBytes = 128;      // one swizzled operand row per stage
constexpr int kKPerStage = 256;     // nvfp4: reduction elements per stage
constexpr int kKPerMma = 64;
constexpr int kGemmThreads = 512;   // four warp groups: TMA + MMA (+2 idle), 4 scale warps, 2 x 4 epilogue warps
constexpr int kRegsSmall = 48;      // register allowance of the first two warp groups ...
constexpr int kRegsEpilogue = 208;  // ... and of the epilogue warp groups (2 x 128 x 48 + 2 x 128 x 208 = 64 Ki)
constexpr int kTmemCols = 512;
constexpr int kTmemSf = 256;        // first scale column (accumulators use columns 0..255)
constexpr int kMaxStages = 6;
constexpr int kSmemA = kBM * kRowBytes;        // 16 KiB
constexpr int kSmemSfa = 4 * 512;              // up to 4 scale atoms per stage

template <int BN>
struct TileCfg {
  static constexpr int kStages = 4;
  static constexpr int kBufs = 1;                       // accumulators in TMEM
  static constexpr int kSmemB = BN * kRowBytes;
  static constexpr int kSfbChains = BN / 128;           // scale-atom chains per stage for B
  static constexpr int kSmemSfb = kSfbChains * 4 * 512;
  static constexpr int kSfCols = 16 + 4 * (BN / 32);    // TMEM scale columns per stage
  static constexpr int kStageBytes = kSmemA + kSmemB + kSmemSfa + kSmemSfb;
};

struct __align__(8) GemmSmemTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sf_landed[kMaxStages]; // scale atoms of the stage are in shared memory
  uint32_t tmem_base;
  int abort_flag;
  int32_t tile_base[kMaxExperts + 1];
};
template <int BN>
constexpr int gemm_smem_bytes() {
  return 1024 + TileCfg<BN>::kStages * TileCfg<BN>::kStageBytes +
         static_cast<int>(sizeof(GemmSmemTail));
}


template <int KIND, int EPI, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap tmA,
                                const __grid_constant__ CUtensorMap tmA_small,
                                const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using Cfg = TileCfg<BN>;
  constexpr int kStages = Cfg::kStages;
  constexpr int kSmemB = Cfg::kSmemB;
  constexpr int kSmemSfb = Cfg::kSmemSfb;
  constexpr bool kGated = epi_is_gated(EPI);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + kStages * kSmemA;
  uint8_t* sSfa = sB + kStages * kSmemB;
  uint8_t* sSfb = sSfa + kStages * kSmemSfa;
  GemmSmemTail* tail = reinterpret_cast<GemmSmemTail*>(sSfb + kStages * kSmemSfb);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&tail->full[s], 1 + 4);   // the producer's arrive + the four scale warps
      mbar_init(&tail->empty[s], 1);
      mbar_init(&tail->sf_landed[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->tmem_full[b], 1);
      mbar_init(&tail->tmem_empty[b], 8);
    }
    tail->abort_flag = 0;
    fence_mbar_init();
  }
  build_tile_base(tail->tile_base, p.tile_base, p.E, p.tile_mode);
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  constexpr int kPerStage = KIND == KIND_MX ? 128 : kKPerStage;
  constexpr int kPerMma = KIND == KIND_MX ? 32 : kKPerMma;
  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_flag = &tail->abort_flag;
  const int total_work = tail->tile_base[p.E] * p.n_tiles;
#ifdef B200MOE_TIMELINE
  const int tl_slot = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x / 2 + 1 ? 1 : -1);
  constexpr int tl_k = EPI == EPI_FC2 ? 1 : 0;
  long long* const tl_buf = tl_slot >= 0 ? g_timeline : nullptr;
#endif

  if (warp < 8) {
  regs_release_to<kRegsSmall>();
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // A few lanes walk the same loop and each issues ONE of the stage's copies: lane 0 arms the
    // barrier and fetches A, lanes 1..kBoxes fetch the 64-row weight boxes, then one lane for the
    // activation scale atoms and one per weight scale chain.
    constexpr int kBoxes = BN / 64;
    constexpr int kLanes = 2 + kBoxes + Cfg::kSfbChains;
    if (lane < kLanes) {
      if (lane == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmA_small);
        tma_prefetch_desc(&tmB);
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TL_DECL(tl_n);
      // Where this lane's copy of tile `w` comes from.  Tiles of a decode batch hold a few rows:
      // they fetch 32 activation rows instead of 128 (the other rows of the shared-memory tile
      // keep stale data; MMA rows are independent).  A gated tile is BN/128 pair groups: box 2g =
      // 64 up rows, box 2g+1 = the 64 gate rows of the same columns; its scale chain g is the pair
      // atom of those columns.  A plain tile is BN consecutive rows.
      struct LaneSrc {
        const CUtensorMap* tm;   // operand lanes
        int y;                   // row coordinate
        const uint8_t* sf;       // scale lanes: atom chain
        uint32_t a_bytes;
      };
      auto locate = [&](int w) {
        const TileCoord c = decode_work(w, p, tail->tile_base);
        LaneSrc r;
        const bool small_a = p.mtile_rows[c.mt] <= 32;
        r.a_bytes = (small_a ? 32u : 128u) * kRowBytes;
        r.tm = &tmB;
        r.y = 0;
        r.sf = p.sfa + static_cast<size_t>(c.mt) * p.atoms_k * 512;
        if (lane == 0) {
          r.tm = small_a ? &tmA_small : &tmA;
          r.y = p.mtile_row0[c.mt];
        } else if (lane <= kBoxes) {
          const int b = lane - 1;
          int my_row;
          if (kGated) {
            int g = b >> 1;
            if (c.nt * p.n_step + g * 64 >= p.out_cols) g = 0;       // half-empty last tile
            my_row = ((b & 1) ? p.sub1_base : p.sub0_base) + c.nt * p.n_step + g * 64;
          } else {
            my_row = c.nt * p.n_step + b * 64;
            if (my_row >= p.w_rows) my_row = c.nt * p.n_step;
          }
          r.y = c.e * p.w_rows + my_row;
        } else if (lane > kBoxes + 1) {
          int rg = c.nt * Cfg::kSfbChains + (lane - kBoxes - 2);
          if (rg >= p.sfb_rowgroups) rg = c.nt * Cfg::kSfbChains;
          r.sf = p.sfb + (static_cast<size_t>(c.e) * p.sfb_rowgroups + rg) * p.atoms_k * 512;
        }
        return r;
      };
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const LaneSrc src = locate(w);
        const CUtensorMap* tma_a = src.tm;
        const uint32_t a_bytes = src.a_bytes;
        const int row0 = src.y;
        const int my_row_y = src.y;
        const uint8_t* my_sf = src.sf;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->empty[stage], phase ^ 1, abort_flag, p.status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (lane == 0) TL_STAGE(tl_k, tl_slot, TL_P_EMPTY, tl_n);
          const int ksteps = min(4, (p.kdim - kb * kPerStage) / kPerMma);
          // NVFP4: one scale atom per MMA step; MX: one atom covers the whole stage
          const uint32_t sf_bytes = KIND == KIND_MX ? 512u : static_cast<uint32_t>(ksteps) * 512u;
          const size_t sf_off = static_cast<size_t>(kb) * (KIND == KIND_MX ? 512 : 2048);
          // the unpacking TMA type counts the packed bytes it reads (64 per 128-value row)
          const uint32_t b_bytes = KIND == KIND_MX ? kSmemB / 2 : kSmemB;
          uint64_t* bar = &tail->full[stage];
          // the (small) scale atoms complete on a barrier of their own, so that their way into
          // TMEM starts before the operand rows of the stage have all landed
          uint64_t* sf_bar = &tail->sf_landed[stage];
          if (lane == 0) {
            mbar_expect_tx(bar, a_bytes + b_bytes);
            tma_load_2d(sA + stage * kSmemA, tma_a, bar, kb * kRowBytes, row0);
          } else if (lane <= kBoxes) {
            tma_load_2d(sB + stage * kSmemB + (lane - 1) * 64 * kRowBytes, &tmB, bar, kb * kRowBytes, my_row_y);
          } else if (lane == kBoxes + 1) {
            mbar_expect_tx(sf_bar, (1u + Cfg::kSfbChains) * sf_bytes);
            bulk_load(sSfa + stage * kSmemSfa, my_sf + sf_off, sf_bytes, sf_bar);
          } else {
            bulk_load(sSfb + stage * kSmemSfb + (lane - kBoxes - 2) * 2048, my_sf + sf_off, sf_bytes, sf_bar);
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
        // give copies that are still in flight time to land before the CTA leaves
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      }
    }
#ifdef B200MOE_TIMELINE
    else if (lane == 31 && tl_buf != nullptr) {
      // observer: when did the operand rows of each stage land?
      int stage = 0, n = 0;
      uint32_t phase = 0;
      for (int w = blockIdx.x; w < total_work && n < kTlSkip + kTlN; w += gridDim.x) {
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
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc =
          KIND == KIND_MX ? make_idesc_block_scaled(kBM, BN, /*a e4m3*/ 0, /*b e2m1*/ 5, /*ue8m0*/ 1)
                          : make_idesc_block_scaled(kBM, BN, /*a*/ 1, /*b*/ 1, /*ue4m3*/ 0);
      int stage = 0;
      constexpr int kSfbStep = 4 * (BN / 128);   // scale columns of B per MMA step
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      const uint64_t adesc0 = make_desc_sw128(smem_u32(sA)), bdesc0 = make_desc_sw128(smem_u32(sB));
      const uint32_t sf0_t = tmem_base + kTmemSf;
      // MMAs of a tile's last k-block (a K that is not a multiple of the stage leaves fewer)
      const int last_ksteps = min(4, (p.kdim - (p.k_blocks - 1) * kPerStage) / kPerMma);
      TL_DECL(tl_n);
      TL_DECL(tl_t);
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        if (!mbar_wait_bounded(&tail->tmem_empty[buf], acc_phase[buf] ^ 1, abort_flag, p.status,
                               WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        TL_TILE(tl_k, tl_slot, TL_M_TMEM_EMPTY, tl_t);
        TL_INC(tl_t);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          // one barrier per stage: the operand rows have landed (TMA byte count) and the four scale
          // warps have put the stage's scale atoms into TMEM (their arrivals)
          if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, p.status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          TL_STAGE(tl_k, tl_slot, TL_M_FULL, tl_n);
          TL_STAGE(tl_k, tl_slot, TL_M_SF, tl_n);
          tc_fence_after();
          // the stage's descriptors differ from stage 0's only in the start-address field (16-byte units)
          const uint32_t sfa_t = sf0_t + stage * Cfg::kSfCols;
          const uint32_t sfb_t = sfa_t + 16;
          const uint64_t adesc = adesc0 + static_cast<uint32_t>(stage * (kSmemA >> 4));
          const uint64_t bdesc = bdesc0 + static_cast<uint32_t>(stage * (kSmemB >> 4));
          // This thread shares its scheduler with busy epilogue warps: the fewer instructions between
          // two MMAs, the shorter the tensor pipe waits for it.  A full k-block is four MMAs, each 32
          // bytes further along the swizzled rows (+2 in 16-byte units): 64 FP4 values, or 32 bytes
          // of the MX kind, whose scale atom holds the four per-32 scales of the stage (MMA step j
          // uses byte j of each word).
          if (kb + 1 < p.k_blocks || last_ksteps == 4) {
            if (KIND == KIND_MX) {
              mma_mxf8f6f4(d_tmem, adesc, bdesc, idesc, sfa_t, sfb_t, kb > 0 ? 1u : 0u);
              mma_mxf8f6f4(d_tmem, adesc + 2, bdesc + 2, idesc | (1u << 29) | (1u << 4), sfa_t + (1u << 30),
                           sfb_t + (1u << 30), 1u);
              mma_mxf8f6f4(d_tmem, adesc + 4, bdesc + 4, idesc | (2u << 29) | (2u << 4), sfa_t + (2u << 30),
                           sfb_t + (2u << 30), 1u);
              mma_mxf8f6f4(d_tmem, adesc + 6, bdesc + 6, idesc | (3u << 29) | (3u << 4), sfa_t + (3u << 30),
                           sfb_t + (3u << 30), 1u);
            } else {
              mma_nvf4_4x(d_tmem, adesc, bdesc, idesc, sfa_t, sfb_t, kb > 0 ? 1u : 0u);
              mma_nvf4_4x(d_tmem, adesc + 2, bdesc + 2, idesc, sfa_t + 4, sfb_t + kSfbStep, 1u);
              mma_nvf4_4x(d_tmem, adesc + 4, bdesc + 4, idesc, sfa_t + 8, sfb_t + 2 * kSfbStep, 1u);
              mma_nvf4_4x(d_tmem, adesc + 6, bdesc + 6, idesc, sfa_t + 12, sfb_t + 3 * kSfbStep, 1u);
            }
          } else {
            for (int j = 0; j < last_ksteps; ++j) {
              if (KIND == KIND_MX) {
                const uint32_t ju = static_cast<uint32_t>(j);
                mma_mxf8f6f4(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc | (ju << 29) | (ju << 4),
                             sfa_t + (ju << 30), sfb_t + (ju << 30), (kb > 0 || j > 0) ? 1u : 0u);
              } else {
                mma_nvf4_4x(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, sfa_t + 4 * j,
                            sfb_t + kSfbStep * j, (kb > 0 || j > 0) ? 1u : 0u);
              }
            }
          }
          tc_commit(&tail->empty[stage]);
          TL_STAGE(tl_k, tl_slot, TL_M_COMMIT, tl_n);
          TL_INC(tl_n);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&tail->tmem_full[buf]);
        acc_phase[buf] ^= 1;
        if (Cfg::kBufs == 2) buf ^= 1;
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------ scale atoms -> TMEM ---------------------------
    // Four warps, one per TMEM sub-partition: every landed stage's scale atoms go from shared
    // memory through registers into the stage's TMEM columns (tcgen05.st), then the warp arrives
    // on the stage's scale barrier.  The tensor pipe sees only MMAs: a tcgen05.cp per scale atom
    // costs it about 70 ns (12 per stage at BN = 256 were the whole stage time, measured), and
    // an MMA issued right behind a tcgen05.cp by the same thread stalls on it.
    constexpr int kSfbStep = 4 * (BN / 128);   // scale columns of B per MMA step
    const int sub = warp & 3;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    TL_DECL(tl_n);
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_bounded(&tail->sf_landed[stage], phase, abort_flag, p.status, WAIT_SMEM_FULL)) {
          ok = false;
          break;
        }
        if (warp == 4 && lane == 0) TL_STAGE(tl_k, tl_slot, TL_S_LANDED, tl_n);
        const uint32_t sfa_t =
            tmem_base + kTmemSf + stage * Cfg::kSfCols + (static_cast<uint32_t>(sub * 32) << 16);
        const uint32_t sfb_t = sfa_t + 16;
        const uint8_t* sfa_s = sSfa + stage * kSmemSfa;
        const uint8_t* sfb_s = sSfb + stage * kSmemSfb;
        if (KIND == KIND_MX) {
          // one atom = the four per-32 scales of the stage
          sf_atoms_to_tmem<1>(sfa_t, sfa_s, lane, 4);
          sf_atoms_to_tmem<1>(sfb_t, sfb_s, lane, 4);
          if (Cfg::kSfbChains == 2) sf_atoms_to_tmem<1>(sfb_t + 4, sfb_s + 2048, lane, 4);
        } else {
          // one atom per MMA step (copied for all four steps; a short last stage leaves stale atoms unused)
          sf_atoms_to_tmem<4>(sfa_t, sfa_s, lane, 4);
          sf_atoms_to_tmem<4>(sfb_t, sfb_s, lane, kSfbStep);
          if (Cfg::kSfbChains == 2) sf_atoms_to_tmem<4>(sfb_t + 4, sfb_s + 2048, lane, kSfbStep);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->full[stage]);
        if (warp == 4 && lane == 0) TL_STAGE(tl_k, tl_slot, TL_S_DONE, tl_n);
        TL_INC(tl_n);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  }
  } else {
    // ------------------------------ epilogue ----------------------------------
    regs_raise_to<kRegsEpilogue>();
    // Eight warps.  Warp w may only read TMEM sub-partition (w & 3), i.e. tile rows
    // 32*(w&3) .. +31; the two warps that share a sub-partition split the tile's columns.
    const int sub = warp & 3;
    const int half = (warp - 8) >> 2;
    const int m = sub * 32 + lane;            // tile row = TMEM lane
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    TL_DECL(tl_t);
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      const TileCoord c = decode_work(w, p, tail->tile_base);
      const int row0 = p.mtile_row0[c.mt];
      const int nrows = p.mtile_rows[c.mt];
      if (!mbar_wait_bounded(&tail->tmem_full[buf], acc_phase[buf], abort_flag, p.status,
                          WAIT_TMEM_FULL))
        break;
      if (warp == 8 && lane == 0) TL_TILE(tl_k, tl_slot, TL_E_FULL, tl_t);
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const uint32_t t_lane = tmem_base + buf * BN + (static_cast<uint32_t>(sub * 32) << 16);
      epilogue_tile<KIND, EPI, BN>(p, c.e, c.mt, c.nt, row0, nrows, t_lane, m, half, lane, [&]() {
        if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);
        if (warp == 8 && lane == 0) TL_TILE(tl_k, tl_slot, TL_E_RELEASED, tl_t);
      });
      if (warp == 8 && lane == 0) TL_TILE(tl_k, tl_slot, TL_E_DONE, tl_t);
      TL_INC(tl_t);
      if (Cfg::kBufs == 2) buf ^= 1;
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------ host side ---------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D byte matrix [rows][row_bytes], box = box_rows x 128 bytes, 128-byte swizzle.
int make_tmap_bytes_2d(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                       uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return B200MOE_ECUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_bytes & 15) != 0) return B200MOE_EALIGN;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r =
      fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ECUDA;
}

int num_sms_cached() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    const char* e = getenv("B200MOE_NUM_SMS");   // persistent grid size override (experiments)
    if (e != nullptr && atoi(e) > 0 && atoi(e) < n) n = atoi(e);
  }
  return n;
}

// 2-D matrix of packed E2M1 values [rows][cols/2 bytes]; the TMA expands every 16 values (8 bytes)
// to a 16-byte slot, which is the operand form kind::mxf8f6f4 reads.  Box = box_rows x 128 values.
// The inner extent is declared rounded up to 128 values (a requirement of this TMA type); the
// columns beyond the real row are never multiplied (the K loop stops at the real K).
int make_tmap_fp4_unpack_2d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows,
                            uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return B200MOE_ECUDA;
  const uint64_t row_bytes = cols / 2;
  if ((reinterpret_cast<uintptr_t>(base) & 31) != 0 || (row_bytes & 31) != 0) return B200MOE_EALIGN;
  const cuuint64_t dims[2] = {(cols + 127) / 128 * 128, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ECUDA;
}

template <int KIND, int EPI, int BN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmA_small,
                       const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t s) {
  auto kern = grouped_gemm_blockscaled_kernel<KIND, EPI, BN>;
  constexpr int smem = gemm_smem_bytes<BN>();
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return B200MOE_ECUDA;
  kern<<<grid, kGemmThreads, smem, s>>>(tmA, tmA_small, tmB, p);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

void fill_common(GemmParams& p, const b200moe_gemm_args* a, char* base) {
  const b200moe_scratch_layout& L = *a->layout;
  p.tile_base = reinterpret_cast<const int32_t*>(base + L.tile_base);
  p.mtile_expert = reinterpret_cast<const int32_t*>(base + L.mtile_expert);
  p.mtile_row0 = reinterpret_cast<const int32_t*>(base + L.mtile_row0);
  p.mtile_rows = reinterpret_cast<const int32_t*>(base + L.mtile_rows);
  p.status = reinterpret_cast<int32_t*>(base + L.status);
  p.E = a->num_experts;
  p.gscale_len = a->gscale_len;
  p.limit = a->swiglu_limit;
  p.act_alpha = a->swiglu_alpha;
  p.act_beta = a->swiglu_beta;
  p.act_kind = a->activation == B200MOE_ACT_SWIGLUOAI ? 1 : (a->activation == B200MOE_ACT_SITU ? 2 : 0);
}

template <int KIND, int EPI>
static int launch_any(int /*bn*/, const CUtensorMap& tmA, const CUtensorMap& tmA_small,
                      const CUtensorMap& tmB, const GemmParams& p, int grid, cudaStream_t s) {
  return launch_gemm<KIND, EPI, 256>(tmA, tmA_small, tmB, p, grid, s);
}

// The first projection.  Gated activations: the weight scales are stored as PAIR atoms -- for every
// block of 64 intermediate columns one 128-row atom chain holding the 64 up rows followed by the 64
// gate rows (prepare_weights builds this from the checkpoint's scale tensor) -- so a tile is made of
// pair groups (64 up rows + 64 gate rows) whose scales are one atom per MMA step.  The weight codes
// are read where the checkpoint left them, with 64-row TMA boxes.
template <int KIND>
static int gemm1_any(const b200moe_gemm_args* a, cudaStream_t stream, int tile_mode) {
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  const bool gated = a->activation != B200MOE_ACT_RELU2;
  const bool mx = KIND == KIND_MX;
  if (K % 64 != 0 || I % 64 != 0 || E > kMaxExperts || a->w13_sf == nullptr) return B200MOE_EINVAL;
  if (!mx && a->a2_gscale == nullptr) return B200MOE_EINVAL;
  const int w_rows = gated ? 2 * I : I;
  char* base = static_cast<char*>(a->scratch);
  CUtensorMap tmA, tmA_small, tmB;
  const uint64_t a_row = mx ? K : K / 2;
  int rc = make_tmap_bytes_2d(&tmA, base + L.act_q, a_row, L.rows, 128);
  if (rc != B200MOE_OK) return rc;
  rc = make_tmap_bytes_2d(&tmA_small, base + L.act_q, a_row, L.rows, 32);
  if (rc != B200MOE_OK) return rc;
  rc = mx ? make_tmap_fp4_unpack_2d(&tmB, a->w13, K, static_cast<uint64_t>(E) * w_rows, 64)
          : make_tmap_bytes_2d(&tmB, a->w13, K / 2, static_cast<uint64_t>(E) * w_rows, 64);
  if (rc != B200MOE_OK) return rc;
  GemmParams p = {};
  fill_common(p, a, base);
  p.tile_mode = tile_mode;
  p.sfa = reinterpret_cast<const uint8_t*>(base + L.act_sf);
  p.sfb = a->w13_sf;
  p.alphas = a->w1_alphas;
  p.gscale2 = a->a2_gscale;
  p.out_q = reinterpret_cast<uint8_t*>(base + L.mid_q);
  p.out_sf = reinterpret_cast<uint8_t*>(base + L.mid_sf);
  p.tap = a->fc1_tap;
  p.kdim = K;
  p.k_blocks = ceil_div_i(K, mx ? 128 : 256);
  p.atoms_k = ceil_div_i(K, mx ? 128 : 64);
  p.w_rows = w_rows;
  p.out_cols = I;
  p.out_atoms = ceil_div_i(I, mx ? 128 : 64);
  const int grid = a->num_sms > 0 ? a->num_sms : num_sms_cached();
  const int bn = 256;
  if (gated) {
    p.sfb_rowgroups = I / 64;              // pair atoms
    p.n_step = bn / 2;                     // intermediate columns per tile
    p.n_tiles = ceil_div_i(I, p.n_step);
    p.sub0_base = a->gate_first ? I : 0;   // up rows
    p.sub1_base = a->gate_first ? 0 : I;   // gate rows
    if (p.act_kind == 0 && !(p.limit > 0.f))
      return launch_any<KIND, EPI_FC1_SILU>(bn, tmA, tmA_small, tmB, p, grid, stream);
    if (p.act_kind == 2) return launch_any<KIND, EPI_FC1_SITU>(bn, tmA, tmA_small, tmB, p, grid, stream);
    return launch_any<KIND, EPI_FC1_GATED>(bn, tmA, tmA_small, tmB, p, grid, stream);
  }
  p.sfb_rowgroups = ceil_div_i(I, 128);
  p.n_step = bn;
  p.n_tiles = ceil_div_i(I, bn);
  return launch_any<KIND, EPI_FC1_RELU2>(bn, tmA, tmA_small, tmB, p, grid, stream);
}

template <int KIND>
static int gemm2_any(const b200moe_gemm_args* a, cudaStream_t stream, int tile_mode) {
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  const bool mx = KIND == KIND_MX;
  if (I % 64 != 0 || K % 16 != 0 || E > kMaxExperts || a->w2_sf == nullptr) return B200MOE_EINVAL;
  char* base = static_cast<char*>(a->scratch);
  CUtensorMap tmA, tmA_small, tmB;
  const uint64_t a_row = mx ? I : I / 2;
  int rc = make_tmap_bytes_2d(&tmA, base + L.mid_q, a_row, L.rows, 128);
  if (rc != B200MOE_OK) return rc;
  rc = make_tmap_bytes_2d(&tmA_small, base + L.mid_q, a_row, L.rows, 32);
  if (rc != B200MOE_OK) return rc;
  rc = mx ? make_tmap_fp4_unpack_2d(&tmB, a->w2, I, static_cast<uint64_t>(E) * K, 64)
          : make_tmap_bytes_2d(&tmB, a->w2, I / 2, static_cast<uint64_t>(E) * K, 64);
  if (rc != B200MOE_OK) return rc;
  GemmParams p = {};
  fill_common(p, a, base);
  p.tile_mode = tile_mode;
  p.sfa = reinterpret_cast<const uint8_t*>(base + L.mid_sf);
  p.sfb = a->w2_sf;
  p.alphas = a->w2_alphas;
  p.out_f32 = reinterpret_cast<float*>(base + L.routed);
  p.kdim = I;
  p.k_blocks = ceil_div_i(I, mx ? 128 : 256);
  p.atoms_k = ceil_div_i(I, mx ? 128 : 64);
  p.w_rows = K;
  p.sfb_rowgroups = ceil_div_i(K, 128);
  p.out_cols = K;
  const int bn = 256;
  p.n_step = bn;
  p.n_tiles = ceil_div_i(K, bn);
  const int grid = a->num_sms > 0 ? a->num_sms : num_sms_cached();
  return launch_any<KIND, EPI_FC2>(bn, tmA, tmA_small, tmB, p, grid, stream);
}

int nvfp4_gemm1(const b200moe_gemm_args* a, cudaStream_t s, int tile_mode) { return gemm1_any<KIND_NVFP4>(a, s, tile_mode); }
int nvfp4_gemm2(const b200moe_gemm_args* a, cudaStream_t s, int tile_mode) { return gemm2_any<KIND_NVFP4>(a, s, tile_mode); }
int mx_gemm1(const b200moe_gemm_args* a, cudaStream_t s, int tile_mode) { return gemm1_any<KIND_MX>(a, s, tile_mode); }
int mx_gemm2(const b200moe_gemm_args* a, cudaStream_t s, int tile_mode) { return gemm2_any<KIND_MX>(a, s, tile_mode); }

}  // namespace b200moe

#ifdef B200MOE_TIMELINE
// Debug builds only: register the device buffer ([2][2][16][96] int64) the timeline stamps go to.
extern "C" int b200moe_debug_set_timeline(void* device_buffer) {
  long long* ptr = static_cast<long long*>(device_buffer);
  return cudaMemcpyToSymbol(b200moe::g_timeline, &ptr, sizeof(ptr)) == cudaSuccess ? 0 : -3;
}
#endif
