// Stages 4 and 5 for small batches (recipe nvfp4): the grouped block-scaled expert GEMMs with the
// operand roles swapped, so that the expert WEIGHTS fill the 128 rows of the tcgen05 tile and the
// few tokens of an expert are its columns.
//
//   tile = two 128-row weight sub-tiles x NT token columns (NT = 16, 32 or 64, chosen per tile
//          from the number of rows the expert received; plans for this kernel cut experts into
//          64-row tiles)
//   FC1 (gated):  sub-tile 0 = 128 up rows, sub-tile 1 = the 128 gate rows of the same columns
//                 acc0[i][t], acc1[i][t] -> x alpha1 -> activation -> bf16 -> NVFP4 re-quantise.
//                 A 16-value scale block runs along i, i.e. over 16 lanes: the block maximum is a
//                 warp shuffle reduction, two lanes share an output byte.
//   FC2:          sub-tiles = 256 consecutive output features; acc[h][t] x alpha2 -> float32 rows.
//
// Against the wide-tile kernel this reads the same weight bytes, but the accumulators take
// 2 x NT TMEM columns instead of 256 (double-buffered: the epilogue of a tile runs under the main
// loop of the next one), every epilogue warp has work when an expert holds two tokens, and the
// tensor pipe multiplies NT columns instead of 256 mostly empty rows.
//
// Warp roles: warp 0 TMA producer (six lanes, one copy each per stage), warp 1 MMA issue, warps
// 2..9 epilogue, warp 10 copies the scale atoms of every landed stage into TMEM (tcgen05.cp) and
// commits them to a barrier of their own.  An MMA that follows a tcgen05.cp in the SAME thread's
// instruction stream waits out the copy's latency in the tensor pipe (about 0.15 us per dependent
// MMA, measured); from a separate thread the copies run stages ahead.  Every wait is bounded.
#include <stdlib.h>

#include "gemm_shared.cuh"

namespace b200moe {
namespace small {

constexpr int kThreads = 352;                  // TMA, MMA, 8 epilogue warps, scale-copy warp
constexpr int kStages = 4;
constexpr int kMaxTok = 64;                    // token columns of a tile (MMA N)
constexpr int kRowBytes = 128;                 // one swizzled operand row per stage = 256 values
constexpr int kSmemW = 128 * kRowBytes;        // one weight sub-tile per stage (16 KiB)
constexpr int kSmemX = kMaxTok * kRowBytes;    // token rows per stage (8 KiB)
constexpr int kSmemSf = 4 * 512;               // four scale atoms per operand and stage
constexpr int kTmemCols = 512;
constexpr int kAccCols = 2 * kMaxTok;          // one accumulator buffer: two sub-tiles
constexpr int kTmemSf = 2 * kAccCols;          // first scale column (two accumulator buffers)
constexpr int kSfCols = 48;                    // per stage: sub-tile 0, sub-tile 1, tokens (16 each)

struct __align__(8) SmemTail {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t sf_full[kStages];     // scale atoms of the stage are in TMEM
  uint32_t tmem_base;
  int abort_flag;
  int32_t tile_base[kMaxExperts + 1];
};
constexpr int kSmemBytes =
    1024 + kStages * (2 * kSmemW + kSmemX + 3 * kSmemSf) + static_cast<int>(sizeof(SmemTail));

__device__ __forceinline__ int token_cols(int nrows) { return nrows <= 16 ? 16 : (nrows <= 32 ? 32 : 64); }

// Maximum over the 16 lanes that hold one scale block.
__device__ __forceinline__ float block16_max(float a) {
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
  a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 8));
  return a;
}

// NVFP4 re-quantisation of 16 token columns held by one lane (lane = intermediate column); the
// arithmetic per value is that of requant_block16.  codes[0] = tokens 0..7, codes[1] = 8..15 (one
// nibble per token), sfw[k] = the scale bytes of tokens 4k..4k+3.
__device__ __forceinline__ void requant_lane16(const float (&h)[16], float gs, float rgs,
                                               uint32_t (&codes)[2], uint32_t (&sfw)[4]) {
  float lo[16], hi[16], denom[16];
  sfw[0] = sfw[1] = sfw[2] = sfw[3] = 0u;
#pragma unroll
  for (int t = 0; t < 16; ++t) {
    const float amax = block16_max(fabsf(h[t]));
    const float raw =
        fminf(div_rn_normal(__fmul_rn(amax, gs), 6.0f, 0.16666667163372039794921875f), 448.0f);
    const uint8_t sfb = f32_to_e4m3_rn_sat(raw);
    sfw[t >> 2] |= static_cast<uint32_t>(sfb) << (8 * (t & 3));
    const float sf = e4m3_to_f32(sfb);
    denom[t] = fmaxf(div_rn_normal(sf, gs, rgs), 1e-30f);
    const float q = __fmul_rn(h[t], rcp_approx(denom[t]));
    lo[t] = __fmul_rn(q, 1.0f - 4.76837158e-7f);
    hi[t] = __fmul_rn(q, 1.0f + 4.76837158e-7f);
  }
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    float a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = lo[8 * w + i];
      b[i] = hi[8 * w + i];
    }
    codes[w] = pack_e2m1x8(a);
    if (codes[w] != pack_e2m1x8(b)) {
      // a quotient within 2^-21 of a rounding boundary: take the correctly rounded division
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = __fdiv_rn(h[8 * w + i], denom[8 * w + i]);
      codes[w] = pack_e2m1x8(a);
    }
  }
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_nvfp4_small_kernel(const __grid_constant__ CUtensorMap tmW,
                                const __grid_constant__ CUtensorMap tmX16,
                                const __grid_constant__ CUtensorMap tmX32,
                                const __grid_constant__ CUtensorMap tmX64, const GemmParams p) {
  constexpr bool kGated = epi_is_gated(EPI);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sW = smem;                              // [stage][sub-tile][16 KiB]
  uint8_t* sX = sW + kStages * 2 * kSmemW;         // [stage][8 KiB]
  uint8_t* sSf = sX + kStages * kSmemX;            // [stage][sub0, sub1, tokens][2 KiB]
  SmemTail* tail = reinterpret_cast<SmemTail*>(sSf + kStages * 3 * kSmemSf);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
      mbar_init(&tail->sf_full[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->tmem_full[b], 1);
      mbar_init(&tail->tmem_empty[b], 8);
    }
    tail->abort_flag = 0;
    fence_mbar_init();
  }
  for (int i = threadIdx.x; i <= p.E; i += blockDim.x) tail->tile_base[i] = p.tile_base[i];
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_flag = &tail->abort_flag;
  const int total_work = tail->tile_base[p.E] * p.n_tiles;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // lane 0: arms the barrier, token rows; lanes 1, 2: the two weight sub-tiles; lane 3: token
    // scale atoms; lanes 4, 5: weight scale atoms.
    if (lane < 6) {
      if (lane == 0) {
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmX16);
        tma_prefetch_desc(&tmX32);
        tma_prefetch_desc(&tmX64);
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int sub = (lane == 2 || lane == 5) ? 1 : 0;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const TileCoord c = decode_tile(w, p.n_tiles, tail->tile_base, p.E);
        const int row0 = p.mtile_row0[c.mt];
        const int ntok = token_cols(p.mtile_rows[c.mt]);
        const CUtensorMap* tmx = ntok == 16 ? &tmX16 : (ntok == 32 ? &tmX32 : &tmX64);
        // first weight row (inside the expert) of this lane's sub-tile, and its scale atom chain
        int wrow = (sub ? p.sub1_base : p.sub0_base) + c.nt * p.n_step;
        if (wrow >= p.w_rows) wrow = p.sub0_base + c.nt * p.n_step;   // half-empty last tile
        const uint8_t* my_sf =
            lane == 3 ? p.sfa + static_cast<size_t>(c.mt) * p.atoms_k * 512
                      : p.sfb + (static_cast<size_t>(c.e) * p.sfb_rowgroups + (wrow >> 7)) * p.atoms_k * 512;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->empty[stage], phase ^ 1, abort_flag, p.status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          const int ksteps = min(4, (p.kdim - kb * 256) / 64);
          const uint32_t sf_bytes = static_cast<uint32_t>(ksteps) * 512u;
          const size_t sf_off = static_cast<size_t>(kb) * 2048;
          uint64_t* bar = &tail->full[stage];
          if (lane == 0) {
            mbar_expect_tx(bar, static_cast<uint32_t>(ntok) * kRowBytes + 2u * kSmemW + 3u * sf_bytes);
            tma_load_2d(sX + stage * kSmemX, tmx, bar, kb * kRowBytes, row0);
          } else if (lane <= 2) {
            tma_load_2d(sW + (stage * 2 + sub) * kSmemW, &tmW, bar, kb * kRowBytes, c.e * p.w_rows + wrow);
          } else {
            const int slot = lane == 3 ? 2 : sub;
            bulk_load(sSf + (stage * 3 + slot) * kSmemSf, my_sf + sf_off, sf_bytes, bar);
          }
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
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const TileCoord c = decode_tile(w, p.n_tiles, tail->tile_base, p.E);
        const int ntok = token_cols(p.mtile_rows[c.mt]);
        const uint32_t idesc = make_idesc_block_scaled(128, ntok, /*a*/ 1, /*b*/ 1, /*ue4m3*/ 0);
        if (!mbar_wait_bounded(&tail->tmem_empty[buf], acc_phase[buf] ^ 1, abort_flag, p.status,
                               WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + buf * kAccCols;
        const uint32_t d1 = d0 + kMaxTok;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, p.status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int ksteps = min(4, (p.kdim - kb * 256) / 64);
          const uint32_t sf_t = tmem_base + kTmemSf + stage * kSfCols;   // sub0 | sub1 | tokens
          const uint32_t sf_s = smem_u32(sSf + stage * 3 * kSmemSf);
          const uint64_t w0 = make_desc_sw128(smem_u32(sW + (stage * 2) * kSmemW));
          const uint64_t w1 = make_desc_sw128(smem_u32(sW + (stage * 2 + 1) * kSmemW));
          const uint64_t xd = make_desc_sw128(smem_u32(sX + stage * kSmemX));
          // the scale-copy warp has put this stage's scale atoms into TMEM
          if (!mbar_wait_bounded(&tail->sf_full[stage], phase, abort_flag, p.status, WAIT_SF_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          for (int j = 0; j < ksteps; ++j) {
            // 64 FP4 values = 32 bytes further along the swizzled row -> +2 in 16-byte units
            const uint32_t accum = (kb > 0 || j > 0) ? 1u : 0u;
            mma_nvf4_4x(d0, w0 + 2 * j, xd + 2 * j, idesc, sf_t + 4 * j, sf_t + 32 + 4 * j, accum);
            mma_nvf4_4x(d1, w1 + 2 * j, xd + 2 * j, idesc, sf_t + 16 + 4 * j, sf_t + 32 + 4 * j, accum);
          }
          tc_commit(&tail->empty[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&tail->tmem_full[buf]);
        acc_phase[buf] ^= 1;
        buf ^= 1;
      }
    }
  } else if (warp == 10) {
    // ------------------------------ scale copies -------------------------------
    // One thread moves the scale atoms of every landed stage from shared memory into TMEM and
    // signals their completion on a barrier of its own, so that the MMA issuer never has a
    // tensor-memory copy in front of a dependent MMA in its instruction stream.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, p.status, WAIT_SMEM_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int ksteps = min(4, (p.kdim - kb * 256) / 64);
          const uint32_t sf_t = tmem_base + kTmemSf + stage * kSfCols;
          const uint32_t sf_s = smem_u32(sSf + stage * 3 * kSmemSf);
          for (int j = 0; j < ksteps; ++j) {
            tc_cp_32x128b_warpx4(sf_t + 4 * j, make_desc_sf(sf_s + 512 * j));
            tc_cp_32x128b_warpx4(sf_t + 16 + 4 * j, make_desc_sf(sf_s + kSmemSf + 512 * j));
            tc_cp_32x128b_warpx4(sf_t + 32 + 4 * j, make_desc_sf(sf_s + 2 * kSmemSf + 512 * j));
          }
          tc_commit(&tail->sf_full[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // Warp w reads TMEM sub-partition (w & 3): weight rows 32*(w&3) .. +31 of a sub-tile.  The two
    // warps of a sub-partition split the token chunks (gated FC1: a lane needs the up and the gate
    // value of its column) or the two sub-tiles (FC2).
    const int sub = warp & 3;
    const int half = (warp - 2) >> 2;
    const int lrow = sub * 32 + lane;          // weight row inside the sub-tile = TMEM lane
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      const TileCoord c = decode_tile(w, p.n_tiles, tail->tile_base, p.E);
      const int row0 = p.mtile_row0[c.mt];
      const int nrows = p.mtile_rows[c.mt];
      const int chunks = token_cols(nrows) >> 4;
      const float alpha = p.alphas[c.e];
      if (!mbar_wait_bounded(&tail->tmem_full[buf], acc_phase[buf], abort_flag, p.status, WAIT_TMEM_FULL))
        break;
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const uint32_t t_lane = tmem_base + buf * kAccCols + (static_cast<uint32_t>(sub * 32) << 16);

      if (kGated) {
        // this warp's token chunks: half, half + 2 (at most two)
        uint32_t ru[2][16], rg[2][16];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int ch = half + 2 * k;
          if (ch < chunks) {
            tc_ld_32x32b_x16(t_lane + ch * 16, ru[k]);
            tc_ld_32x32b_x16(t_lane + kMaxTok + ch * 16, rg[k]);
          }
        }
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);

        const float gs2 = p.gscale2[p.gscale_len > 1 ? c.e : 0];
        const float rgs2 = __frcp_rn(gs2);
        const int icol = c.nt * 128 + lrow;                    // intermediate column of this lane
        uint8_t* sft = p.out_sf + static_cast<size_t>(c.mt) * p.out_atoms * 512;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int ch = half + 2 * k;
          if (ch < chunks) {
            float h[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              const float up = __fmul_rn(__uint_as_float(ru[k][t]), alpha);
              const float gate = __fmul_rn(__uint_as_float(rg[k][t]), alpha);
              if (p.tap != nullptr && ch * 16 + t < nrows) {
                float* trow = p.tap + static_cast<size_t>(row0 + ch * 16 + t) * p.w_rows + icol;
                trow[p.sub0_base] = up;
                trow[p.sub1_base] = gate;
              }
              h[t] = round_bf16(act_gated<EPI>(gate, up, p));
            }
            uint32_t codes[2], sfw[4];
            requant_lane16(h, gs2, rgs2, codes, sfw);
            // Two lanes (columns 2j, 2j+1) share a byte: the even lane writes tokens 0..7 of the
            // chunk, the odd lane tokens 8..15.
            const bool odd = lane & 1;
            const uint32_t got = __shfl_xor_sync(0xffffffffu, odd ? codes[0] : codes[1], 1);
            const uint32_t even_nib = odd ? got : codes[0];      // column 2j   -> low nibble
            const uint32_t odd_nib = odd ? codes[1] : got;       // column 2j+1 -> high nibble
            const int tok0 = ch * 16 + (odd ? 8 : 0);
            uint8_t* qcol = p.out_q + (icol >> 1);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (tok0 + i < nrows) {
                const uint32_t byte = ((even_nib >> (4 * i)) & 0xfu) | (((odd_nib >> (4 * i)) & 0xfu) << 4);
                qcol[static_cast<size_t>(row0 + tok0 + i) * (p.out_cols >> 1)] = static_cast<uint8_t>(byte);
              }
            }
            // scale bytes: lane j of a 16-lane block writes the byte of token j of the chunk
            const int j = lane & 15;
            const uint32_t word = (j >> 2) == 0 ? sfw[0] : ((j >> 2) == 1 ? sfw[1] : ((j >> 2) == 2 ? sfw[2] : sfw[3]));
            if (ch * 16 + j < nrows)
              sft[sf_atom_offset(static_cast<uint32_t>(ch * 16 + j), static_cast<uint32_t>(icol >> 4))] =
                  static_cast<uint8_t>(word >> (8 * (j & 3)));
          }
        }
      } else {
        // FC2: this warp drains sub-tile `half`, all token chunks (at most four)
        uint32_t rr[4][16];
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          if (ch < chunks) tc_ld_32x32b_x16(t_lane + half * kMaxTok + ch * 16, rr[ch]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);
        const int f = c.nt * p.n_step + half * 128 + lrow;       // output feature of this lane
        if (f < p.out_cols) {
          float* ocol = p.out_f32 + f;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            if (ch < chunks) {
#pragma unroll
              for (int t = 0; t < 16; ++t)
                if (ch * 16 + t < nrows)
                  ocol[static_cast<size_t>(row0 + ch * 16 + t) * p.out_cols] =
                      __fmul_rn(__uint_as_float(rr[ch][t]), alpha);
            }
          }
        }
      }
      buf ^= 1;
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

template <int EPI>
static int launch(const CUtensorMap& tmW, const CUtensorMap (&tmX)[3], const GemmParams& p, int grid,
                  cudaStream_t s) {
  auto kern = grouped_gemm_nvfp4_small_kernel<EPI>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return B200MOE_ECUDA;
  kern<<<grid, kThreads, kSmemBytes, s>>>(tmW, tmX[0], tmX[1], tmX[2], p);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

static int token_maps(CUtensorMap (&tmX)[3], const void* base, uint64_t row_bytes, uint64_t rows) {
  const uint32_t boxes[3] = {16, 32, 64};
  for (int i = 0; i < 3; ++i) {
    const int rc = make_tmap_bytes_2d(&tmX[i], base, row_bytes, rows, boxes[i]);
    if (rc != B200MOE_OK) return rc;
  }
  return B200MOE_OK;
}

}  // namespace small

// The small-batch kernels serve plans cut into 64-row tiles.  B200MOE_SMALL_BATCH=0 keeps the
// wide-tile kernels on such plans (comparison runs).
bool nvfp4_small_batch_ok(const b200moe_gemm_args* a, bool fc1) {
  static int enabled = -1;
  if (enabled < 0) {
    const char* e = getenv("B200MOE_SMALL_BATCH");
    enabled = (e != nullptr && atoi(e) == 0) ? 0 : 1;
  }
  if (!enabled || a->layout->tile_rows != 64) return false;
  if (a->hidden_size % 64 != 0 || a->intermediate % 128 != 0 || a->num_experts > kMaxExperts) return false;
  if (fc1 && (a->activation == B200MOE_ACT_RELU2 || a->w13_sf_rows == nullptr)) return false;
  return true;
}

int nvfp4_small_gemm1(const b200moe_gemm_args* a, cudaStream_t stream) {
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  if (a->a2_gscale == nullptr) return B200MOE_EINVAL;
  char* base = static_cast<char*>(a->scratch);
  CUtensorMap tmW, tmX[3];
  int rc = make_tmap_bytes_2d(&tmW, a->w13, K / 2, static_cast<uint64_t>(E) * 2 * I, 128);
  if (rc != B200MOE_OK) return rc;
  rc = small::token_maps(tmX, base + L.act_q, K / 2, L.rows);
  if (rc != B200MOE_OK) return rc;
  GemmParams p = {};
  fill_common(p, a, base);
  p.sfa = reinterpret_cast<const uint8_t*>(base + L.act_sf);
  p.sfb = a->w13_sf_rows;
  p.alphas = a->w1_alphas;
  p.gscale2 = a->a2_gscale;
  p.out_q = reinterpret_cast<uint8_t*>(base + L.mid_q);
  p.out_sf = reinterpret_cast<uint8_t*>(base + L.mid_sf);
  p.tap = a->fc1_tap;
  p.kdim = K;
  p.k_blocks = ceil_div_i(K, 256);
  p.atoms_k = K / 64;
  p.w_rows = 2 * I;
  p.sfb_rowgroups = 2 * I / 128;
  p.sub0_base = a->gate_first ? I : 0;   // up rows
  p.sub1_base = a->gate_first ? 0 : I;   // gate rows
  p.n_step = 128;
  p.n_tiles = I / 128;
  p.out_cols = I;
  p.out_atoms = I / 64;
  const int grid = a->num_sms > 0 ? a->num_sms : num_sms_cached();
  if (p.act_kind == 0 && !(p.limit > 0.f)) return small::launch<EPI_FC1_SILU>(tmW, tmX, p, grid, stream);
  if (p.act_kind == 2) return small::launch<EPI_FC1_SITU>(tmW, tmX, p, grid, stream);
  return small::launch<EPI_FC1_GATED>(tmW, tmX, p, grid, stream);
}

int nvfp4_small_gemm2(const b200moe_gemm_args* a, cudaStream_t stream) {
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  char* base = static_cast<char*>(a->scratch);
  CUtensorMap tmW, tmX[3];
  int rc = make_tmap_bytes_2d(&tmW, a->w2, I / 2, static_cast<uint64_t>(E) * K, 128);
  if (rc != B200MOE_OK) return rc;
  rc = small::token_maps(tmX, base + L.mid_q, I / 2, L.rows);
  if (rc != B200MOE_OK) return rc;
  GemmParams p = {};
  fill_common(p, a, base);
  p.sfa = reinterpret_cast<const uint8_t*>(base + L.mid_sf);
  p.sfb = a->w2_sf;
  p.alphas = a->w2_alphas;
  p.out_f32 = reinterpret_cast<float*>(base + L.routed);
  p.kdim = I;
  p.k_blocks = ceil_div_i(I, 256);
  p.atoms_k = I / 64;
  p.w_rows = K;
  p.sfb_rowgroups = ceil_div_i(K, 128);
  p.sub0_base = 0;
  p.sub1_base = 128;
  p.n_step = 256;
  p.n_tiles = ceil_div_i(K, 256);
  p.out_cols = K;
  const int grid = a->num_sms > 0 ? a->num_sms : num_sms_cached();
  return small::launch<EPI_FC2>(tmW, tmX, p, grid, stream);
}

}  // namespace b200moe
