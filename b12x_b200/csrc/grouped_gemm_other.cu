// Grouped expert GEMMs of the w4a16 recipe: BF16 activations x NVFP4 weights that are expanded to
// a 16-bit float on the fly, on tcgen05.mma.kind::f16 with FP32 accumulation in TMEM.
//
// The tensor core cannot read 4-bit operands next to 16-bit ones, so the main loop has a conversion
// step.  Three rings in shared memory: (1) per k-block of 64, the token rows (16 KiB) and the scale
// atoms (2 KiB); (2) the packed codes of FOUR k-blocks, one TMA box of 128 rows x 128 bytes per
// sub-tile (the path from L2 takes about as long for a 32-byte row as for a 128-byte one, so a box of
// 32-byte rows per k-block cost four times the requests; 128-byte swizzle, so the converters'
// 16-byte reads, one row per thread, spread over the banks); (3) two converted weight tiles of
// 32 KiB, 128-byte-swizzled as the MMA reads them.  Eight converter warps expand a k-block's codes
// into a converted tile and hand it to the MMA warp through an mbarrier; tcgen05.commit gives the
// tile and the load stage back.  The accumulator is double buffered in TMEM (2 x 256 columns), so
// the epilogue of one tile overlaps the main loop of the next.
//
// Conversion (E4M3 block scales).  The hardware conversion cvt.rn.f16x2.e2m1x2 turns a byte into
// two FP16 code values, a half2 multiply applies the block scale (2 + 4 significant bits, between
// 2^-10 and 2688: exact in FP16 as in BF16), and FP16 -> FP32 -> BF16 re-encodes the pair.  The
// integer pipe issues at half rate, and the byte-permute look-up used before (about ten integer
// instructions per two values) held this kernel at 0.28 of the BF16 peak.  Both operands stay
// BF16: a launch whose instruction descriptor named BF16 tokens and FP16 weights, which would
// save the re-encoding, ended with a CUDA error on B200, and with both BF16 the same code runs.
// Power-of-two (E8M0) scales exceed the FP16 range; for them the code values are re-encoded first and
// multiplied by the scale in BF16.
//
// Where the time goes (timing-only builds of the CTA-pair kernel below, FC1 of the Qwen3 shape,
// 1.17 ms): without the MMAs 1.06 ms, without the conversion 1.02 ms, with the converters copying
// instead of converting 1.07 ms, without the epilogue 1.11 ms.  So neither the tensor pipe nor the
// conversion arithmetic bounds it: the load -> convert -> hand-over chain and the load -> MMA ->
// commit chain each take about 950 clocks per k-block on their own (four MMAs are 512 clocks at the
// nominal rate, 690 at the rate a library BF16 GEMM reaches here).  For the single-CTA kernel,
// earlier: ring depths (3 / 4 / 6 load stages, 2 / 3 / 4 converted tiles), sixteen converter warps
// on alternate k-blocks, and an FC2 variant with the expanded weights as the tensor-memory operand
// of the MMA (no shared-memory round trip for them) all changed nothing and were removed.
//
// Numerics follow the reference's W4A16 oracle (tests/_reference/w4a16_reference.py:266-359):
// weights de-quantised then held in BF16, x in BF16, FP32 accumulation, activation in FP32, BF16
// intermediate.
#include <stdlib.h>

#include "cluster_pair.cuh"

namespace b200moe {

int make_tmap_bytes_2d(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                       uint32_t box_rows);
bool tail_split(const b200moe_gemm_args* a);

namespace w4a16 {

#ifndef W4A16_LOAD_STAGES
#define W4A16_LOAD_STAGES 4
#endif
constexpr int kStages = W4A16_LOAD_STAGES;  // load ring: token rows and scale atoms of one k-block
constexpr int kRawStages = 2;               // ring of packed codes, kKBlocksPerRaw k-blocks each
constexpr int kKBlocksPerRaw = 4;
#ifndef W4A16_B_STAGES
#define W4A16_B_STAGES 2
#endif
constexpr int kBStages = W4A16_B_STAGES;    // converted weight tiles
constexpr int kKPerStage = 64;              // BF16 elements per 128-byte operand row
#ifndef W4A16_CONV_GROUPS
#define W4A16_CONV_GROUPS 1
#endif
constexpr int kConvGroups = W4A16_CONV_GROUPS;   // groups of 8 converter warps; group g takes stages g, g + groups, ...
constexpr int kConvWarps = 8 * kConvGroups;
constexpr int kThreads = (2 + kConvWarps + 8) * 32;   // TMA, MMA, converter warps, 8 epilogue warps
constexpr int kSmemA = 128 * 128;           // 16 KiB
constexpr int kSmemB = 256 * 128;           // 32 KiB
constexpr int kSmemRaw = 2 * 128 * 128;     // packed codes of the two sub-tiles, 128 bytes = 4 k-blocks per row
constexpr int kSmemSf = 4 * 512;            // two scale atoms per sub-tile (a sub-tile may straddle)
constexpr int kStageBytes = kSmemA + kSmemSf;
constexpr int kMaxExperts = 1024;

struct __align__(8) SmemTail {
  uint64_t full[kStages];        // load stage landed (TMA transaction bytes)
  uint64_t empty[kStages];       // load stage free: 8 converter warps + the MMAs that read its rows
  uint64_t rfull[kRawStages];    // packed codes landed
  uint64_t rempty[kRawStages];   // packed codes read by every converter warp
  uint64_t bfull[kBStages];      // converted tile written (8 converter warps)
  uint64_t bempty[kBStages];     // converted tile read by its MMAs
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int32_t tile_base[kMaxExperts + 1];
};
constexpr int kSmemBytes =
    1024 + kStages * kStageBytes + kRawStages * kSmemRaw + kBStages * kSmemB +
    static_cast<int>(sizeof(SmemTail));
static_assert(kSmemBytes <= 227 * 1024, "shared memory of the W4A16 kernel");

enum { EPI_FC1_GATED = 0, EPI_FC1_RELU2 = 1, EPI_FC2 = 2 };

struct Params {
  const uint8_t* sf;             // weight scale storage, 128x4-swizzled [E][sf_rowgroups][atoms_k][512]
  const int32_t* tile_base;
  const int32_t* mtile_row0;
  const int32_t* mtile_rows;
  int32_t* status;
  const float* alphas;
  __nv_bfloat16* out_bf16;       // FC1: intermediate [rows][out_cols]
  float* out_f32;                // FC2: routed rows [rows][out_cols]
  float* tap;
  const float* row_scale;        // FC1, optional: per sorted position, multiplies the row with its alpha
  int E, n_tiles, kdim, k_blocks, atoms_k, sf_rowgroups, w_rows;
  int sub0_base, sub1_base, n_step, out_cols;
  float limit, act_alpha, act_beta;
  int swigluoai;
  int sf_e8m0;                   // scale bytes are E8M0 (2^(b-127)) instead of E4M3
  int tile_mode;                 // 0 all row tiles; 1 only the left-over row tile of experts with an odd
                                 // number of them (after the CTA-pair kernel); 2 full pairs only
};

struct TileCoord {
  int e, mt, nt;
};
__device__ __forceinline__ TileCoord decode_tile(int w, int n_tiles, const int32_t* tb, int E) {
  const int q = w / n_tiles;
  int lo = 0, hi = E;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (tb[mid + 1] <= q) lo = mid + 1; else hi = mid;
  }
  TileCoord c;
  c.e = lo;
  const int me = tb[lo + 1] - tb[lo];
  const int local = w - tb[lo] * n_tiles;
  c.nt = local / me;
  c.mt = tb[lo] + local % me;
  return c;
}

// through the single-CTA kernel's shared-memory work list `tb`: the row-tile prefix sums, or (tile
// mode 1) the prefix sums of "has a left-over row tile"
__device__ __forceinline__ TileCoord decode_work(int w, const Params& p, const int32_t* tb) {
  TileCoord c = decode_tile(w, p.n_tiles, tb, p.E);
  if (p.tile_mode == 1) c.mt = p.tile_base[c.e + 1] - 1;
  return c;
}

__device__ __forceinline__ float act_gated(float gate, float up, const Params& p) {
  if (p.limit > 0.f) {
    gate = fminf(gate, p.limit);
    up = fminf(fmaxf(up, -p.limit), p.limit);
  }
  if (p.swigluoai) {
    const float s = __frcp_rn(1.0f + expf(-(p.act_alpha * gate)));
    return (gate * s) * (up + p.act_beta);
  }
  const float s = __frcp_rn(1.0f + expf(-gate));
  return (gate * s) * up;
}

// Four bytes of E2M1 codes (element 0 in the low nibble) -> four f16x2 words of code values: the
// hardware conversion takes a byte (two codes, low nibble -> low half).
__device__ __forceinline__ void cvt_e2m1x8_f16(uint32_t w, uint32_t (&v)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}\n"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
      : "r"(w));
}

// Eight E2M1 codes -> four bf16x2 words, each value multiplied in BF16 by the bf16 scale pair `sc`
// (power-of-two scales: the product is exact unless it leaves the BF16 range).
__device__ __forceinline__ void cvt_e2m1x8_bf16(uint32_t w, __nv_bfloat162 sc, uint32_t (&out)[4]) {
  uint32_t v[4];
  cvt_e2m1x8_f16(w, v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v[j]));
    const __nv_bfloat162 x = __hmul2(__floats2bfloat162_rn(f.x, f.y), sc);
    out[j] = *reinterpret_cast<const uint32_t*>(&x);
  }
}

// Eight E2M1 codes times an E4M3 block scale -> four bf16x2 words.  `sc` = the scale as an f16x2
// pair.  The product is exact in FP16 (2 + 4 significant bits, between 2^-10 and 2688), so
// FP16 -> FP32 -> BF16 rounds nothing.  (Re-labelling the FP16 code value as a BF16 number by a
// shift and two masks and multiplying in BF16 by 2^112 x scale is exact too and saves the three
// conversions, but measured slower: FC1 of the Qwen3 shape 1.38 against 1.29 ms.)
__device__ __forceinline__ void cvt_e2m1x8_scaled(uint32_t w, uint32_t sc, uint32_t (&out)[4]) {
  uint32_t v[4];
  cvt_e2m1x8_f16(w, v);
  const __half2 s2 = *reinterpret_cast<const __half2*>(&sc);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(__hmul2(*reinterpret_cast<const __half2*>(&v[j]), s2));
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    out[j] = *reinterpret_cast<const uint32_t*>(&b);
  }
}
// Four E4M3 scale bytes -> two f16x2 words (bytes 0,1 and 2,3; low byte -> low half).
__device__ __forceinline__ void cvt_e4m3x4_f16(uint32_t w, uint32_t& s01, uint32_t& s23) {
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %2;\n\t"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}\n"
      : "=r"(s01), "=r"(s23)
      : "r"(w));
}

// Epilogue of one 128-row x 256-column accumulator for the rows of one warp (lane = token row `m`
// of the tile, `half` = which half of the columns this warp takes): FC1 applies the expert's alpha
// and the activation and stores BF16, FC2 applies alpha and stores the fp32 routed rows.
template <int EPI>
__device__ __forceinline__ void epilogue_rows(const Params& p, float alpha, int nt, size_t pos, bool valid,
                                              uint32_t t_lane, int half) {
  if (EPI != EPI_FC2 && p.row_scale != nullptr && valid) alpha = __fmul_rn(alpha, p.row_scale[pos]);
  if (EPI == EPI_FC1_GATED) {
    const int col0 = nt * 128 + half * 64;
    __nv_bfloat16* orow = p.out_bf16 + pos * p.out_cols + col0;
#pragma unroll 1
    for (int ch = 0; ch < 4; ++ch) {
      uint32_t ru[16], rg[16];
      tc_ld_32x32b_x16(t_lane + half * 64 + ch * 16, ru);
      tc_ld_32x32b_x16(t_lane + 128 + half * 64 + ch * 16, rg);
      tc_wait_ld();
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        float h2[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const float up = __fmul_rn(__uint_as_float(ru[i + q]), alpha);
          const float gate = __fmul_rn(__uint_as_float(rg[i + q]), alpha);
          if (p.tap != nullptr && valid && col0 + ch * 16 < p.out_cols) {
            float* trow = p.tap + pos * p.w_rows;
            trow[p.sub0_base + col0 + ch * 16 + i + q] = up;
            trow[p.sub1_base + col0 + ch * 16 + i + q] = gate;
          }
          h2[q] = act_gated(gate, up, p);
        }
        const __nv_bfloat162 b2 = __floats2bfloat162_rn(h2[0], h2[1]);
        o[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
      }
      if (valid && col0 + ch * 16 < p.out_cols) {
        uint4* dst = reinterpret_cast<uint4*>(orow + ch * 16);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  } else if (EPI == EPI_FC1_RELU2) {
    const int col0 = nt * 256 + half * 128;
    __nv_bfloat16* orow = p.out_bf16 + pos * p.out_cols + col0;
#pragma unroll 1
    for (int ch = 0; ch < 8; ++ch) {
      uint32_t rr2[16];
      tc_ld_32x32b_x16(t_lane + half * 128 + ch * 16, rr2);
      tc_wait_ld();
      uint32_t o[8];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        float h2[2];
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const float v = __fmul_rn(__uint_as_float(rr2[i + q]), alpha);
          if (p.tap != nullptr && valid && col0 + ch * 16 < p.out_cols)
            p.tap[pos * p.w_rows + col0 + ch * 16 + i + q] = v;
          const float r = fmaxf(v, 0.f);
          h2[q] = __fmul_rn(r, r);
        }
        const __nv_bfloat162 b2 = __floats2bfloat162_rn(h2[0], h2[1]);
        o[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
      }
      if (valid && col0 + ch * 16 < p.out_cols) {
        uint4* dst = reinterpret_cast<uint4*>(orow + ch * 16);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
    }
  } else {
    const int col0 = nt * 256 + half * 128;
    float* orow = p.out_f32 + pos * p.out_cols + col0;
#pragma unroll 1
    for (int ch = 0; ch < 8; ++ch) {
      uint32_t rr2[16];
      tc_ld_32x32b_x16(t_lane + half * 128 + ch * 16, rr2);
      tc_wait_ld();
      if (valid && col0 + ch * 16 < p.out_cols) {
        // 32 bytes per lane and instruction: half as many store instructions as with 16-byte
        // stores, and the converter warps need the load/store unit too
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__uint_as_float(rr2[8 * q + i]), alpha);
          st_global_f32x8(orow + ch * 16 + 8 * q, v);
        }
      }
    }
  }
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_w4a16_kernel(const __grid_constant__ CUtensorMap tmA,
                          const __grid_constant__ CUtensorMap tmW, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + kStages * kSmemA;
  uint8_t* sRaw = sB + kBStages * kSmemB;
  uint8_t* sSf = sRaw + kRawStages * kSmemRaw;
  SmemTail* tail = reinterpret_cast<SmemTail*>(sSf + kStages * kSmemSf);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 9);
    }
    for (int r = 0; r < kRawStages; ++r) {
      mbar_init(&tail->rfull[r], 1);
      mbar_init(&tail->rempty[r], kConvWarps);
    }
    for (int b = 0; b < kBStages; ++b) {
      mbar_init(&tail->bfull[b], 8);
      mbar_init(&tail->bempty[b], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->tmem_full[b], 1);
      mbar_init(&tail->tmem_empty[b], 8);
    }
    tail->abort_flag = 0;
    fence_mbar_init();
  }
  if (p.tile_mode == 1) {
    if (threadIdx.x == 0) {
      int acc = 0;
      for (int e = 0; e < p.E; ++e) {
        tail->tile_base[e] = acc;
        acc += (p.tile_base[e + 1] - p.tile_base[e]) & 1;
      }
      tail->tile_base[p.E] = acc;
    }
  } else {
    for (int i = threadIdx.x; i <= p.E; i += blockDim.x) tail->tile_base[i] = p.tile_base[i];
  }
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, 512);
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
    // seven lanes walk the same loop, each issues one of the stage's seven copies
    if (lane < 7) {
      if (lane == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
      }
      int stage = 0, rs = 0;
      uint32_t phase = 0, rphase = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        const TileCoord c = decode_work(w, p, tail->tile_base);
        const int row0 = p.mtile_row0[c.mt];
        const int r0 = p.sub0_base + c.nt * p.n_step;
        int r1 = p.sub1_base + c.nt * p.n_step;
        if (r1 >= p.w_rows) r1 = r0;
        const uint8_t* sf_e = p.sf + static_cast<size_t>(c.e) * p.sf_rowgroups * p.atoms_k * 512;
        // a 128-row sub-tile starting at row r touches scale row-groups r/128 and (r+127)/128
        const int g[4] = {r0 >> 7, min((r0 + 127) >> 7, p.sf_rowgroups - 1), r1 >> 7,
                          min((r1 + 127) >> 7, p.sf_rowgroups - 1)};
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if ((kb & (kKBlocksPerRaw - 1)) == 0 && (lane == 1 || lane == 2)) {
            // the codes of four k-blocks in one box of 128-byte rows: the path from L2 takes
            // about as long for a 32-byte row as for a 128-byte one
            if (!mbar_wait_bounded(&tail->rempty[rs], rphase ^ 1, abort_flag, p.status,
                                   WAIT_SMEM_EMPTY)) {
              ok = false;
              break;
            }
            uint64_t* rbar = &tail->rfull[rs];
            if (lane == 1) {
              mbar_expect_tx(rbar, kSmemRaw);
              tma_load_2d(sRaw + rs * kSmemRaw, &tmW, rbar, kb * 32, c.e * p.w_rows + r0);
            } else {
              tma_load_2d(sRaw + rs * kSmemRaw + 128 * 128, &tmW, rbar, kb * 32, c.e * p.w_rows + r1);
            }
          }
          if ((kb & (kKBlocksPerRaw - 1)) == kKBlocksPerRaw - 1 || kb == p.k_blocks - 1) {
            if (++rs == kRawStages) {
              rs = 0;
              rphase ^= 1;
            }
          }
          if (!mbar_wait_bounded(&tail->empty[stage], phase ^ 1, abort_flag, p.status,
                                 WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          uint64_t* bar = &tail->full[stage];
          if (lane == 0) {
            mbar_expect_tx(bar, kSmemA + kSmemSf);
            tma_load_2d(sA + stage * kSmemA, &tmA, bar, kb * kKPerStage, row0);
          } else if (lane >= 3) {
            const int q = lane - 3;
            bulk_load(sSf + stage * kSmemSf + q * 512,
                      sf_e + (static_cast<size_t>(g[q]) * p.atoms_k + kb) * 512, 512, bar);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, 256);
      int stage = 0, bstage = 0;
      uint32_t phase = 0, bphase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int buf = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
        if (!mbar_wait_bounded(&tail->tmem_empty[buf], acc_phase[buf] ^ 1, abort_flag, p.status,
                               WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, p.status, WAIT_SMEM_FULL) ||
              !mbar_wait_bounded(&tail->bfull[bstage], bphase, abort_flag, p.status, WAIT_CONVERT)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = make_desc_sw128(smem_u32(sA + stage * kSmemA));
          const uint64_t bdesc = make_desc_sw128(smem_u32(sB + bstage * kSmemB));
#pragma unroll
          for (int j = 0; j < 4; ++j)   // 16 bf16 = 32 bytes per MMA step
            mma_bf16(d_tmem, adesc + 2 * j, bdesc + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          tc_commit(&tail->empty[stage]);
          tc_commit(&tail->bempty[bstage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
          if (++bstage == kBStages) {
            bstage = 0;
            bphase ^= 1;
          }
        }
        if (ok) tc_commit(&tail->tmem_full[buf]);
        acc_phase[buf] ^= 1;
        buf ^= 1;
      }
    }
  } else if (warp < 2 + kConvWarps) {
    // ------------------------------ converters --------------------------------
    // thread t of a group expands weight row t of the 256-row operand tile: 64 codes -> 64 bf16
    // = 128 bytes.  The groups take alternate stages, so the fixed latencies of a stage (barrier
    // wake-up, shared-memory loads, the proxy fence) of one group lie under the arithmetic of the other.
    const int group = (threadIdx.x - 64) >> 8;
    const int t = (threadIdx.x - 64) & 255;
    const int sub_tile = t >> 7, rr = t & 127;
    int it = 0;
    int stage = 0, bstage = 0, rs = 0;
    uint32_t phase = 0, bphase = 0, rphase = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < total_work; w += gridDim.x) {
      const TileCoord c = decode_work(w, p, tail->tile_base);
      const int r0 = p.sub0_base + c.nt * p.n_step;
      int r1 = p.sub1_base + c.nt * p.n_step;
      if (r1 >= p.w_rows) r1 = r0;
      const int wrow = (sub_tile ? r1 : r0) + rr;          // weight row inside the expert
      const int first_group = (sub_tile ? r1 : r0) >> 7;
      // scale bytes of this row inside the two staged atoms of its sub-tile
      const int atom_sel = (wrow >> 7) - first_group;       // 0 or 1
      const uint32_t sf_off = sub_tile * 1024 + atom_sel * 512 + (wrow & 31) * 16 + ((wrow >> 5) & 3) * 4;
      for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
        if (kConvGroups == 1 || it % kConvGroups == group) {
        if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, p.status, WAIT_CONVERT) ||
            !mbar_wait_bounded(&tail->rfull[rs], rphase, abort_flag, p.status, WAIT_CONVERT) ||
            !mbar_wait_bounded(&tail->bempty[bstage], bphase ^ 1, abort_flag, p.status,
                               WAIT_CONVERT)) {
          ok = false;
          break;
        }
        tc_fence_after();
        // 128-byte rows, 16-byte chunks swizzled by the row (as the TMA wrote them); this k-block
        // owns chunks 2q and 2q + 1
        const uint8_t* raw = sRaw + rs * kSmemRaw + t * 128;
        const int q2 = (kb & (kKBlocksPerRaw - 1)) * 2;
        const uint4 c0 = *reinterpret_cast<const uint4*>(raw + ((q2 ^ (t & 7)) << 4));
        const uint4 c1 = *reinterpret_cast<const uint4*>(raw + (((q2 + 1) ^ (t & 7)) << 4));
        const uint32_t sfw = *reinterpret_cast<const uint32_t*>(sSf + stage * kSmemSf + sf_off);
        const uint32_t words[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        uint8_t* brow = sB + bstage * kSmemB + t * 128;
        if (!p.sf_e8m0) {
          uint32_t s01, s23;
          cvt_e4m3x4_f16(sfw, s01, s23);
#pragma unroll
          for (int blk = 0; blk < 4; ++blk) {               // 16 values per scale
            const uint32_t sc = __byte_perm(blk < 2 ? s01 : s23, 0u, (blk & 1) ? 0x3232u : 0x1010u);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t o[4];
              cvt_e2m1x8_scaled(words[blk * 2 + h], sc, o);
              const int chunk = blk * 2 + h;                 // 16-byte chunk of the 128-byte row
              *reinterpret_cast<uint4*>(brow + ((chunk ^ (t & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        } else {
#pragma unroll
          for (int blk = 0; blk < 4; ++blk) {               // 16 values per scale
            const uint32_t sb = (sfw >> (8 * blk)) & 0xffu;
            // E8M0: 2^(b-127) is the f32 with exponent field b (b = 0: the subnormal 2^-127)
            const float sv = __uint_as_float(sb != 0u ? sb << 23 : 0x00400000u);
            const __nv_bfloat16 s = __float2bfloat16_rn(sv);
            const __nv_bfloat162 sc = __halves2bfloat162(s, s);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t o[4];
              cvt_e2m1x8_bf16(words[blk * 2 + h], sc, o);
              const int chunk = blk * 2 + h;
              *reinterpret_cast<uint4*>(brow + ((chunk ^ (t & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
        fence_proxy_async_smem();                            // generic writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&tail->bfull[bstage]);
          mbar_arrive(&tail->empty[stage]);
        }
        }
        if ((kb & (kKBlocksPerRaw - 1)) == kKBlocksPerRaw - 1 || kb == p.k_blocks - 1) {
          // this warp has read all it needs of the packed codes
          __syncwarp();
          if (lane == 0) mbar_arrive(&tail->rempty[rs]);
          if (++rs == kRawStages) {
            rs = 0;
            rphase ^= 1;
          }
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
        if (++bstage == kBStages) {
          bstage = 0;
          bphase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int sub = warp & 3;
    const int half = (warp - 2 - kConvWarps) >> 2;
    const int m = sub * 32 + lane;
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      const TileCoord c = decode_work(w, p, tail->tile_base);
      const int row0 = p.mtile_row0[c.mt];
      const int nrows = p.mtile_rows[c.mt];
      const float alpha = p.alphas[c.e];
      if (!mbar_wait_bounded(&tail->tmem_full[buf], acc_phase[buf], abort_flag, p.status,
                             WAIT_TMEM_FULL))
        break;
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const uint32_t t_lane = tmem_base + buf * 256 + (static_cast<uint32_t>(sub * 32) << 16);
      const bool valid = m < nrows;
      const size_t pos = static_cast<size_t>(row0 + m);
      epilogue_rows<EPI>(p, alpha, c.nt, pos, valid, t_lane, half);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);
      buf ^= 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// The same GEMMs on CTA PAIRS (clusters of two, tcgen05 cta_group::2), for plans with several row
// tiles per expert.
//
// A pair shares one 256 x 256 tile: each CTA owns 128 token rows (its own row tile of the expert)
// and expands only ITS HALF of the 256 weight rows (FC1, gated: the even CTA the 128 "up" rows, the
// odd CTA the 128 "gate" rows); the pair's MMA (M = 256, N = 256, issued by one thread of the even
// CTA) reads the halves out of both CTAs' shared memory and writes a 128 x 256 accumulator into each
// CTA's tensor memory.  Per CTA and k-block of 64 that halves the conversion work (two threads per
// weight row) and the shared-memory traffic that bounds the single-CTA kernel: the MMAs read
// 16 + 16 KiB of operands instead of 16 + 32, the converters write 16 KiB instead of 32.
//
// Roles per CTA (640 threads): warp 0 token-row producer (the copies of both CTAs complete on the
// EVEN CTA's stage barrier), warp 2 producer of packed codes and scale atoms (four k-blocks per
// stage, own ring), warps 4..11 converters (arrive on the even CTA's "tile converted" barrier, 16
// arrivals per k-block), warps 12..19 epilogue of the CTA's own accumulator (double buffered:
// 2 x 256 columns).  Even CTA only: warp 1 issues the MMAs and commits (multicast) to both CTAs'
// barriers.  Every wait is bounded; the two cluster-wide barriers (after set-up, before tear-down)
// are reached by both CTAs unconditionally.
namespace pr {

using namespace ::b200moe::pair;

// ring depths: 7/2/3, 6/3/3, 8/2/2 and 3/3/2 (token rows / converted tiles / code boxes) are all slower
constexpr int kAStages = 5;                  // token rows of one k-block
constexpr int kBStagesP = 4;                 // converted weight rows of one k-block (this CTA's half)
constexpr int kRawStagesP = 3;               // packed codes + scale atoms of four k-blocks
constexpr int kSmemAP = 128 * 128;           // 16 KiB
constexpr int kSmemBP = 128 * 128;           // 16 KiB
constexpr int kSmemCodes = 128 * 128;        // 128 weight rows x 128 bytes (four k-blocks)
constexpr int kSmemAtoms = 2 * 4 * 512;      // two scale row-groups (the rows may straddle) x four k-blocks
constexpr int kRawBytes = kSmemCodes + kSmemAtoms;
constexpr int kConvWarpsP = 8;
constexpr int kThreadsP = (4 + kConvWarpsP + 8) * 32;

struct __align__(8) SmemTailP {
  uint64_t afull[kAStages];      // even CTA: the token rows of both CTAs have landed
  uint64_t aempty[kAStages];     // per CTA: the MMAs that read the stage have retired
  uint64_t rfull[kRawStagesP];   // per CTA: codes and scale atoms have landed
  uint64_t rempty[kRawStagesP];  // per CTA: the eight converter warps have read them
  uint64_t bfull[kBStagesP];     // even CTA: the 16 converter warps of the pair have written the tile
  uint64_t bempty[kBStagesP];    // per CTA: the MMAs that read the tile have retired
  uint64_t tmem_full[2];         // per CTA: accumulator complete
  uint64_t tmem_empty[2];        // even CTA: the 16 epilogue warps of the pair have drained it
  uint32_t tmem_base;
  int abort_flag;
  int32_t tile_base[kMaxExperts + 1];
  int32_t pair_base[kMaxExperts + 1];
};
constexpr int kSmemBytesP = 1024 + kAStages * kSmemAP + kBStagesP * kSmemBP + kRawStagesP * kRawBytes +
                            static_cast<int>(sizeof(SmemTailP));
static_assert(kSmemBytesP <= 227 * 1024, "shared memory of the W4A16 CTA-pair kernel");

// Work item of a pair: (expert, n-tile, pair of row tiles).  This CTA's row tile is first + rank;
// an expert with an odd number of row tiles leaves the odd CTA of its last pair without one
// (rows = 0: it multiplies the neighbour's rows again and stores nothing).
struct PairCoord {
  int e, nt, mt_load, rows;
};
__device__ __forceinline__ PairCoord decode_pair(int w, const Params& p, const SmemTailP* tail, int rank) {
  const TileCoord c = decode_tile(w, p.n_tiles, tail->pair_base, p.E);
  PairCoord r;
  r.e = c.e;
  r.nt = c.nt;
  const int last = tail->tile_base[c.e + 1] - 1;
  const int mt = tail->tile_base[c.e] + 2 * (c.mt - tail->pair_base[c.e]) + rank;
  r.mt_load = mt <= last ? mt : last;
  r.rows = mt <= last ? p.mtile_rows[mt] : 0;
  return r;
}
// first weight row (inside the expert) of the 128 rows this CTA expands for n-tile `nt`
__device__ __forceinline__ int weight_row0(const Params& p, int nt, int rank) {
  const int r0 = p.sub0_base + nt * p.n_step;
  if (rank == 0) return r0;
  const int r1 = p.sub1_base + nt * p.n_step;
  return r1 >= p.w_rows ? r0 : r1;
}

template <int EPI>
__global__ void __launch_bounds__(kThreadsP, 1)
grouped_gemm_w4a16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                               const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + kAStages * kSmemAP;
  uint8_t* sRaw = sB + kBStagesP * kSmemBP;       // [stage][codes 16 KiB | atoms 4 KiB]
  SmemTailP* tail = reinterpret_cast<SmemTailP*>(sRaw + kRawStagesP * kRawBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());     // 0 = even CTA (issues the MMAs)
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) {
      mbar_init(&tail->afull[s], 1);
      mbar_init(&tail->aempty[s], 1);
    }
    for (int s = 0; s < kRawStagesP; ++s) {
      mbar_init(&tail->rfull[s], 1);
      mbar_init(&tail->rempty[s], kConvWarpsP);
    }
    for (int s = 0; s < kBStagesP; ++s) {
      mbar_init(&tail->bfull[s], 2 * kConvWarpsP);
      mbar_init(&tail->bempty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->tmem_full[b], 1);
      mbar_init(&tail->tmem_empty[b], 16);
    }
    tail->abort_flag = 0;
    fence_mbar_init();
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      const int t0 = p.tile_base[e], t1 = p.tile_base[e + 1];
      tail->tile_base[e] = t0;
      tail->pair_base[e] = acc;
      acc += (t1 - t0 + (p.tile_mode == 2 ? 0 : 1)) >> 1;   // full pairs only, or the odd tile too
      if (e == p.E - 1) tail->tile_base[p.E] = t1;
    }
    tail->pair_base[p.E] = acc;
  }
  if (warp == 1) {
    tmem_alloc_pair(&tail->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after();

  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_flag = &tail->abort_flag;
  const int total_work = tail->pair_base[p.E] * p.n_tiles;

  if (warp == 0) {
    // ------------------------------ token-row producer (both CTAs) -----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
        const PairCoord c = decode_pair(w, p, tail, rank);
        const int row0 = p.mtile_row0[c.mt_load];
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->aempty[stage], phase ^ 1, abort_flag, p.status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          if (rank == 0) mbar_expect_tx(&tail->afull[stage], 2u * kSmemAP);
          tma_load_2d_pair(sA + stage * kSmemAP, &tmA, map_to_cta(smem_u32(&tail->afull[stage]), 0),
                           kb * kKPerStage, row0);
          if (++stage == kAStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let copies in flight land
      }
    }
  } else if (warp == 2) {
    // ------------------------------ codes + scale atoms (both CTAs) ----------------
    // lane 0: the packed codes of this CTA's 128 weight rows, four k-blocks per box; lanes 1, 2: the
    // scale atoms of the (up to) two row-groups those rows touch, four k-blocks = 2 KiB contiguous
    if (lane < 3) {
      if (lane == 0) tma_prefetch_desc(&tmW);
      int rs = 0;
      uint32_t rphase = 0;
      bool ok = true;
      for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
        const PairCoord c = decode_pair(w, p, tail, rank);
        const int r = weight_row0(p, c.nt, rank);
        const uint8_t* sf_e = p.sf + static_cast<size_t>(c.e) * p.sf_rowgroups * p.atoms_k * 512;
        const int g = lane == 2 ? min((r + 127) >> 7, p.sf_rowgroups - 1) : (r >> 7);
        for (int kb = 0; kb < p.k_blocks; kb += kKBlocksPerRaw) {
          if (!mbar_wait_bounded(&tail->rempty[rs], rphase ^ 1, abort_flag, p.status, WAIT_SMEM_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t atom_bytes = static_cast<uint32_t>(min(kKBlocksPerRaw, p.atoms_k - kb)) * 512u;
          uint8_t* dst = sRaw + rs * kRawBytes;
          if (lane == 0) {
            mbar_expect_tx(&tail->rfull[rs], kSmemCodes + 2u * atom_bytes);
            tma_load_2d(dst, &tmW, &tail->rfull[rs], kb * 32, c.e * p.w_rows + r);
          } else {
            bulk_load(dst + kSmemCodes + (lane - 1) * 2048,
                      sf_e + (static_cast<size_t>(g) * p.atoms_k + kb) * 512, atom_bytes, &tail->rfull[rs]);
          }
          if (++rs == kRawStagesP) {
            rs = 0;
            rphase ^= 1;
          }
        }
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA) --------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, 256);
      int stage = 0, bstage = 0, buf = 0;
      uint32_t phase = 0, bphase = 0;
      uint32_t acc_phase[2] = {0, 0};
      bool ok = true;
      const uint64_t adesc0 = make_desc_sw128(smem_u32(sA)), bdesc0 = make_desc_sw128(smem_u32(sB));
      for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
        if (!mbar_wait_bounded(&tail->tmem_empty[buf], acc_phase[buf] ^ 1, abort_flag, p.status,
                               WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait_bounded(&tail->afull[stage], phase, abort_flag, p.status, WAIT_SMEM_FULL) ||
              !mbar_wait_bounded(&tail->bfull[bstage], bphase, abort_flag, p.status, WAIT_CONVERT)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = adesc0 + static_cast<uint32_t>(stage * (kSmemAP >> 4));
          const uint64_t bdesc = bdesc0 + static_cast<uint32_t>(bstage * (kSmemBP >> 4));
          mma_bf16_pair(d_tmem, adesc, bdesc, idesc, kb > 0 ? 1u : 0u);     // 16 bf16 = 32 bytes per MMA
          mma_bf16_pair(d_tmem, adesc + 2, bdesc + 2, idesc, 1u);
          mma_bf16_pair(d_tmem, adesc + 4, bdesc + 4, idesc, 1u);
          mma_bf16_pair(d_tmem, adesc + 6, bdesc + 6, idesc, 1u);
          tc_commit_pair_both(&tail->aempty[stage]);
          tc_commit_pair_both(&tail->bempty[bstage]);
          if (++stage == kAStages) {
            stage = 0;
            phase ^= 1;
          }
          if (++bstage == kBStagesP) {
            bstage = 0;
            bphase ^= 1;
          }
        }
        if (ok) tc_commit_pair_both(&tail->tmem_full[buf]);
        acc_phase[buf] ^= 1;
        buf ^= 1;
      }
    }
  } else if (warp >= 4 && warp < 4 + kConvWarpsP) {
    // ------------------------------ converters (both CTAs) -------------------------
    // Two threads per weight row, 32 codes (16 bytes) -> 32 bf16 (64 bytes) each.  Warps 4..7 take
    // the first half of the k-block, warps 8..11 the second: a warp touches 32 different rows, so
    // its 16-byte accesses to the 128-byte-swizzled rows spread over all banks.
    const int t = threadIdx.x - 128;
    const int khalf = t >> 7, rr = t & 127;
    const uint32_t bfull_base = map_to_cta(smem_u32(&tail->bfull[0]), 0);
    int bstage = 0, rs = 0;
    uint32_t bphase = 0, rphase = 0;
    bool ok = true;
    for (int w = cluster_id; ok && w < total_work; w += num_clusters) {
      const PairCoord c = decode_pair(w, p, tail, rank);
      const int r = weight_row0(p, c.nt, rank);
      const int wrow = r + rr;                               // weight row inside the expert
      const int atom_sel = (wrow >> 7) - (r >> 7);           // 0 or 1: which staged row-group
      const uint32_t sf_off = kSmemCodes + atom_sel * 2048 + (wrow & 31) * 16 + ((wrow >> 5) & 3) * 4;
      for (int kb = 0; kb < p.k_blocks; ++kb) {
        if (!mbar_wait_bounded(&tail->rfull[rs], rphase, abort_flag, p.status, WAIT_CONVERT) ||
            !mbar_wait_bounded(&tail->bempty[bstage], bphase ^ 1, abort_flag, p.status, WAIT_CONVERT)) {
          ok = false;
          break;
        }
        const int kq = kb & (kKBlocksPerRaw - 1);
        const uint8_t* raw = sRaw + rs * kRawBytes;
        const int chunk = kq * 2 + khalf;                    // 16-byte chunk of the 128-byte code row
        const uint4 cw = *reinterpret_cast<const uint4*>(raw + rr * 128 + ((chunk ^ (rr & 7)) << 4));
        const uint32_t sfw = *reinterpret_cast<const uint32_t*>(raw + sf_off + kq * 512);
        const uint32_t sf2 = (sfw >> (16 * khalf)) & 0xffffu;            // this half's two scale bytes
        const uint32_t words[4] = {cw.x, cw.y, cw.z, cw.w};
        uint8_t* brow = sB + bstage * kSmemBP + rr * 128;
        if (!p.sf_e8m0) {
          uint32_t s01, s23;
          cvt_e4m3x4_f16(sf2, s01, s23);
#pragma unroll
          for (int j = 0; j < 4; ++j) {                      // 8 values per word, 16 per scale
            const uint32_t sc = __byte_perm(s01, 0u, j < 2 ? 0x1010u : 0x3232u);
            uint32_t o[4];
            cvt_e2m1x8_scaled(words[j], sc, o);
            *reinterpret_cast<uint4*>(brow + (((khalf * 4 + j) ^ (rr & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t sb = (sf2 >> (j < 2 ? 0 : 8)) & 0xffu;
            // E8M0: 2^(b-127) is the f32 with exponent field b (b = 0: the subnormal 2^-127)
            const float sv = __uint_as_float(sb != 0u ? sb << 23 : 0x00400000u);
            const __nv_bfloat16 s1 = __float2bfloat16_rn(sv);
            uint32_t o[4];
            cvt_e2m1x8_bf16(words[j], __halves2bfloat162(s1, s1), o);
            *reinterpret_cast<uint4*>(brow + (((khalf * 4 + j) ^ (rr & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        fence_proxy_async_smem();                            // generic writes -> tensor-core reads
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(bfull_base + static_cast<uint32_t>(bstage * sizeof(uint64_t)));
        if (kq == kKBlocksPerRaw - 1 || kb == p.k_blocks - 1) {
          // this warp has read all it needs of the stage's codes and atoms
          if (lane == 0) mbar_arrive(&tail->rempty[rs]);
          if (++rs == kRawStagesP) {
            rs = 0;
            rphase ^= 1;
          }
        }
        if (++bstage == kBStagesP) {
          bstage = 0;
          bphase ^= 1;
        }
      }
    }
  } else if (warp >= 4 + kConvWarpsP) {
    // ------------------------------ epilogue (both CTAs) ---------------------------
    const int sub = warp & 3;
    const int half = (warp - 4 - kConvWarpsP) >> 2;
    const int m = sub * 32 + lane;
    const uint32_t release_base = map_to_cta(smem_u32(&tail->tmem_empty[0]), 0);
    uint32_t acc_phase[2] = {0, 0};
    int buf = 0;
    for (int w = cluster_id; w < total_work; w += num_clusters) {
      const PairCoord c = decode_pair(w, p, tail, rank);
      const int row0 = p.mtile_row0[c.mt_load];
      const float alpha = p.alphas[c.e];
      if (!mbar_wait_bounded(&tail->tmem_full[buf], acc_phase[buf], abort_flag, p.status, WAIT_TMEM_FULL)) break;
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const uint32_t t_lane = tmem_base + buf * 256 + (static_cast<uint32_t>(sub * 32) << 16);
      epilogue_rows<EPI>(p, alpha, c.nt, static_cast<size_t>(row0 + m), m < c.rows, t_lane, half);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(release_base + static_cast<uint32_t>(buf * sizeof(uint64_t)));
      buf ^= 1;
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // nobody signals the other CTA's shared memory after this
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace pr

// Calibration side channel of the w4a16 recipe (reference W4A16FusedMoeKernel._collect_activation_amax_epilogue,
// b12x/moe/_shared/kernels/w4a16/kernel.py:7288-7365): amax[layer][expert][0] = max(old, max |x| over the
// rows routed to the expert), [..][1] the same over its activated BF16 intermediate rows.  One CTA per
// row tile and operand (blockIdx.y: 0 = FC1 input rows, 1 = FC2 input rows); non-negative floats
// order like their bit patterns, so the running maximum is an integer atomicMax.
__global__ void __launch_bounds__(256) activation_amax_kernel(
    const __nv_bfloat16* __restrict__ rows_fc1, const __nv_bfloat16* __restrict__ rows_fc2, int K, int I,
    const int32_t* __restrict__ tile_base, int E, const int32_t* __restrict__ mtile_expert,
    const int32_t* __restrict__ mtile_row0, const int32_t* __restrict__ mtile_rows, float* __restrict__ amax,
    int layer_idx) {
  const int mt = blockIdx.x;
  if (mt >= tile_base[E]) return;
  const int which = blockIdx.y;
  const int len = which == 0 ? K : I;
  const __nv_bfloat16* base = (which == 0 ? rows_fc1 : rows_fc2) + static_cast<size_t>(mtile_row0[mt]) * len;
  const int nvec = (mtile_rows[mt] * len) >> 3;                 // 8 values per 16-byte load; rows are contiguous
  float m = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 p = reinterpret_cast<const uint4*>(base)[i];
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      m = fmaxf(m, fabsf(__uint_as_float(w[j] << 16)));
      m = fmaxf(m, fabsf(__uint_as_float(w[j] & 0xffff0000u)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int wgt = 1; wgt < 8; ++wgt) m = fmaxf(m, part[wgt]);
    if (!(m != m)) {      // a NaN row leaves the record alone
      int* dst = reinterpret_cast<int*>(amax + (static_cast<size_t>(layer_idx) * E + mtile_expert[mt]) * 2 + which);
      atomicMax(dst, __float_as_int(m));
    }
  }
}

// x rows -> sorted-position order (the A operand of FC1), one warp per row
__global__ void __launch_bounds__(256) permute_rows_bf16_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, const int32_t* __restrict__ expert_offsets,
    int E, const int32_t* __restrict__ sorted_route_ids, int num_topk, int K,
    __nv_bfloat16* __restrict__ out, const float* __restrict__ route_weights, float* __restrict__ row_scale) {
  const int total = expert_offsets[E];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int pos = blockIdx.x * 8 + warp; pos < total; pos += gridDim.x * 8) {
    const int route = sorted_route_ids[pos];
    const int tkn = route / num_topk;
    if (route_weights != nullptr && lane == 0) row_scale[pos] = route_weights[route];
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(tkn) * x_row_stride);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(pos) * K);
    for (int j = lane; j < (K >> 3); j += 32) dst[j] = __ldg(src + j);
  }
}

// 2-D bf16 matrix [rows][cols], box = box_rows x 64 elements (128 bytes), 128-byte swizzle
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
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
static int make_tmap_bf16(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows,
                          uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return B200MOE_ECUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || ((cols * 2) & 15) != 0) return B200MOE_EALIGN;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ECUDA;
}
// packed weight codes [rows][row_bytes], box = 128 rows x 128 bytes (four k-blocks), 128-byte
// swizzle so that the converters' 16-byte reads, one row per thread, spread over the banks
static int make_tmap_codes(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return B200MOE_ECUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_bytes & 15) != 0) return B200MOE_EALIGN;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, 128};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ECUDA;
}

static int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int EPI>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmW, const Params& p, int grid,
                  cudaStream_t s) {
  auto kern = grouped_gemm_w4a16_kernel<EPI>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
    return B200MOE_ECUDA;
  kern<<<grid, kThreads, kSmemBytes, s>>>(tmA, tmW, p);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

template <int EPI>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmW, const Params& p, int max_ctas,
                       cudaStream_t s) {
  auto kern = pr::grouped_gemm_w4a16_pair_kernel<EPI>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pr::kSmemBytesP) != cudaSuccess)
    return B200MOE_ECUDA;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.blockDim = dim3(pr::kThreadsP);
  cfg.dynamicSmemBytes = pr::kSmemBytesP;
  cfg.stream = s;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  // persistent grid: as many CTA pairs as can be resident at once
  cfg.gridDim = dim3(static_cast<unsigned>(max_ctas & ~1));
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) != cudaSuccess || clusters < 1) return B200MOE_ECUDA;
  if (2 * clusters < max_ctas) cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
  return cudaLaunchKernelEx(&cfg, kern, tmA, tmW, p) == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

// CTA pairs once the plan averages two row tiles per expert (an expert with an odd number of row
// tiles leaves half a pair idle); B200MOE_W4A16_PAIR=1 / 0 forces them on / off.
static bool use_pair(const b200moe_gemm_args* a) {
  static int mode = -2;
  if (mode == -2) {
    const char* e = getenv("B200MOE_W4A16_PAIR");
    mode = e == nullptr ? -1 : (atoi(e) != 0 ? 1 : 0);
  }
  if (mode == 0 || a->layout->tile_rows != 128) return false;
  if (mode == 1) return true;
  return static_cast<int64_t>(a->layout->rows) >= 256ll * a->num_experts;
}

// Plans for CTA pairs: full pairs of row tiles on the pair kernel, then the left-over row tile of
// experts with an odd number of them on the single-CTA kernel (plans with few row tiles per expert;
// otherwise, or with B200MOE_TAIL_SPLIT=0, the pair kernel takes those too, as half-empty pairs).  Other plans: the single-CTA kernel on every row tile.
template <int EPI>
static int launch_split(const b200moe_gemm_args* a, const CUtensorMap& tmA, const CUtensorMap& tmW, Params p,
                        int grid, cudaStream_t s) {
  if (!use_pair(a)) {
    p.tile_mode = 0;
    return launch<EPI>(tmA, tmW, p, grid, s);
  }
  const bool split = ::b200moe::tail_split(a);
  p.tile_mode = split ? 2 : 0;
  const int rc = launch_pair<EPI>(tmA, tmW, p, grid, s);
  if (rc != B200MOE_OK || !split) return rc;
  p.tile_mode = 1;
  return launch<EPI>(tmA, tmW, p, grid, s);
}

static void fill_common(Params& p, const b200moe_gemm_args* a, char* base) {
  const b200moe_scratch_layout& L = *a->layout;
  p.tile_base = reinterpret_cast<const int32_t*>(base + L.tile_base);
  p.mtile_row0 = reinterpret_cast<const int32_t*>(base + L.mtile_row0);
  p.mtile_rows = reinterpret_cast<const int32_t*>(base + L.mtile_rows);
  p.status = reinterpret_cast<int32_t*>(base + L.status);
  p.E = a->num_experts;
  p.limit = a->swiglu_limit;
  p.act_alpha = a->swiglu_alpha;
  p.act_beta = a->swiglu_beta;
  p.swigluoai = a->activation == B200MOE_ACT_SWIGLUOAI;
}

}  // namespace w4a16

int w4a16_gemm1(const b200moe_gemm_args* a, cudaStream_t stream) {
  if (a->activation == B200MOE_ACT_SITU) return B200MOE_EUNSUPPORTED;   // no W4A16 oracle for it
  using namespace w4a16;
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  const bool gated = a->activation != B200MOE_ACT_RELU2;
  if (K % 64 != 0 || I % 16 != 0 || E > kMaxExperts || a->w13_sf == nullptr || a->x == nullptr)
    return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) != 0 || (a->x_row_stride % 8) != 0) return B200MOE_EALIGN;
  const int w_rows = gated ? 2 * I : I;
  char* base = static_cast<char*>(a->scratch);
  const int rows = a->num_tokens * a->num_topk;
  int ggrid = (rows + 7) / 8;
  if (ggrid > 148 * 8) ggrid = 148 * 8;
  permute_rows_bf16_kernel<<<ggrid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a->x), a->x_row_stride,
      reinterpret_cast<const int32_t*>(base + L.expert_offsets), E,
      reinterpret_cast<const int32_t*>(base + L.sorted_route_ids), a->num_topk, K,
      reinterpret_cast<__nv_bfloat16*>(base + L.act_q), a->fc1_route_weights,
      reinterpret_cast<float*>(base + L.act_sf));   // w4a16 has no activation scales: the region holds the row weights
  CUtensorMap tmA, tmW;
  int rc = make_tmap_bf16(&tmA, base + L.act_q, K, L.rows, 128);
  if (rc != B200MOE_OK) return rc;
  rc = make_tmap_codes(&tmW, a->w13, K / 2, static_cast<uint64_t>(E) * w_rows);
  if (rc != B200MOE_OK) return rc;
  Params p = {};
  fill_common(p, a, base);
  p.sf = a->w13_sf;
  p.sf_e8m0 = a->sf_e8m0;
  p.alphas = a->w1_alphas;
  p.out_bf16 = reinterpret_cast<__nv_bfloat16*>(base + L.mid_q);
  p.tap = a->fc1_tap;
  p.row_scale = a->fc1_route_weights != nullptr ? reinterpret_cast<const float*>(base + L.act_sf) : nullptr;
  p.kdim = K;
  p.k_blocks = K / kKPerStage;
  p.atoms_k = ceil_div_i(K, 64);
  p.sf_rowgroups = ceil_div_i(w_rows, 128);
  p.w_rows = w_rows;
  p.out_cols = I;
  const int grid = a->num_sms > 0 ? a->num_sms : sm_count();
  if (gated) {
    p.n_tiles = ceil_div_i(I, 128);
    p.n_step = 128;
    p.sub0_base = a->gate_first ? I : 0;
    p.sub1_base = a->gate_first ? 0 : I;
    return launch_split<EPI_FC1_GATED>(a, tmA, tmW, p, grid, stream);
  }
  p.n_tiles = ceil_div_i(I, 256);
  p.n_step = 256;
  p.sub0_base = 0;
  p.sub1_base = 128;
  return launch_split<EPI_FC1_RELU2>(a, tmA, tmW, p, grid, stream);
}

int w4a16_gemm2(const b200moe_gemm_args* a, cudaStream_t stream) {
  using namespace w4a16;
  const b200moe_scratch_layout& L = *a->layout;
  const int K = a->hidden_size, I = a->intermediate, E = a->num_experts;
  if (I % 64 != 0 || K % 16 != 0 || E > kMaxExperts || a->w2_sf == nullptr) return B200MOE_EINVAL;
  char* base = static_cast<char*>(a->scratch);
  CUtensorMap tmA, tmW;
  int rc = make_tmap_bf16(&tmA, base + L.mid_q, I, L.rows, 128);
  if (rc != B200MOE_OK) return rc;
  rc = make_tmap_codes(&tmW, a->w2, I / 2, static_cast<uint64_t>(E) * K);
  if (rc != B200MOE_OK) return rc;
  Params p = {};
  fill_common(p, a, base);
  p.sf = a->w2_sf;
  p.sf_e8m0 = a->sf_e8m0;
  p.alphas = a->w2_alphas;
  p.out_f32 = reinterpret_cast<float*>(base + L.routed);
  p.kdim = I;
  p.k_blocks = I / kKPerStage;
  p.atoms_k = ceil_div_i(I, 64);
  p.sf_rowgroups = ceil_div_i(K, 128);
  p.w_rows = K;
  p.out_cols = K;
  p.n_tiles = ceil_div_i(K, 256);
  p.n_step = 256;
  p.sub0_base = 0;
  p.sub1_base = 128;
  const int grid = a->num_sms > 0 ? a->num_sms : sm_count();
  return launch_split<EPI_FC2>(a, tmA, tmW, p, grid, stream);
}

int w4a16_activation_amax(const b200moe_amax_args* a, cudaStream_t stream) {
  const b200moe_scratch_layout& L = *a->layout;
  char* base = static_cast<char*>(a->scratch);
  const int tr = L.tile_rows == 64 ? 64 : 128;
  const int rows = a->num_rows;
  const int mtiles = (rows + tr - 1) / tr + (a->num_experts < rows ? a->num_experts : rows);
  const int gx = mtiles < L.mtile_cap ? mtiles : L.mtile_cap;
  w4a16::activation_amax_kernel<<<dim3(gx, 2), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(base + L.act_q), reinterpret_cast<const __nv_bfloat16*>(base + L.mid_q),
      a->hidden_size, a->intermediate, reinterpret_cast<const int32_t*>(base + L.tile_base), a->num_experts,
      reinterpret_cast<const int32_t*>(base + L.mtile_expert), reinterpret_cast<const int32_t*>(base + L.mtile_row0),
      reinterpret_cast<const int32_t*>(base + L.mtile_rows), a->amax, a->layer_idx);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

}  // namespace b200moe
