// Pieces shared by the grouped GEMM kernels of this library: launch parameters, the work-list
// decoder, the epilogue arithmetic and the host-side tensor-map helpers.
#pragma once

#include "quant_shared.cuh"

namespace b200moe {

constexpr int kMaxExperts = 1024;

// FC1 epilogues: GATED = SwiGLU with a clamp and/or the SwiGLU-OAI form (chosen at run time), SILU = plain
// SwiGLU, SITU = the SiTU form; each is its own instantiation so that none carries the others' code.
enum { EPI_FC1_GATED = 0, EPI_FC1_RELU2 = 1, EPI_FC2 = 2, EPI_FC1_SILU = 3, EPI_FC1_SITU = 4 };
__host__ __device__ constexpr bool epi_is_gated(int epi) { return epi == EPI_FC1_GATED || epi == EPI_FC1_SILU || epi == EPI_FC1_SITU; }
// KIND_NVFP4: A and B packed E2M1, E4M3 scale per 16, kind::mxf4nvf4 (K = 64 per MMA, 256 per stage).
// KIND_MX:    A E4M3 bytes, B E2M1 expanded by TMA to one value per byte slot, E8M0 scale per 32,
//             kind::mxf8f6f4 (K = 32 per MMA, 128 per stage; one scale atom per stage).
enum { KIND_NVFP4 = 0, KIND_MX = 1 };

// Which row tiles a launch works on.  Plans with several row tiles per expert run the CTA-pair kernel
// on every FULL pair of row tiles (TILES_PAIRS) and a single-CTA kernel on the row tile that is left
// over in experts with an odd number of them (TILES_TAIL): a pair with one empty half costs a whole
// pair's loads and MMAs, the single tile a little more than half of that on one SM instead of two.
enum { TILES_ALL = 0, TILES_TAIL = 1, TILES_PAIRS = 2 };

struct GemmParams {
  const uint8_t* sfa;            // activation scale atoms [mtile][atoms_k][512]
  const uint8_t* sfb;            // weight scale atoms [E][rowgroups][atoms_k][512]
  const int32_t* tile_base;      // [E+1]
  const int32_t* mtile_expert;
  const int32_t* mtile_row0;
  const int32_t* mtile_rows;
  int32_t* status;
  const float* alphas;           // [E]
  const float* gscale2;          // FC1 epilogue: reciprocal FC2-input scale
  uint8_t* out_q;                // FC1: codes [rows][out_cols/2]
  uint8_t* out_sf;               // FC1: scale atoms [mtile][out_atoms][512]
  float* out_f32;                // FC2: routed rows [rows][out_cols]
  float* tap;                    // FC1 debug tap [rows][w_rows] or null
  int E, n_tiles, kdim, k_blocks, atoms_k;
  int sfb_rowgroups;             // per expert
  int w_rows;                    // weight rows per expert
  int sub0_base, sub1_base;      // first weight row of the two sub-tiles at n-tile 0
  int n_step;                    // weight rows advanced per n-tile
  int out_cols;                  // I (FC1) or K (FC2)
  int out_atoms;                 // FC1: scale atoms per tile of the output
  int gscale_len;
  float limit, act_alpha, act_beta;
  int act_kind;                  // gated FC1: 0 SwiGLU, 1 SwiGLU-OAI, 2 SiTU
  int tile_mode;                 // TILES_ALL / TILES_TAIL / TILES_PAIRS
};

struct TileCoord {
  int e, mt, nt;
};
// work id -> (expert, m-tile, n-tile); expert-major, then n-tile, m-tile fastest, so that the CTAs
// running at the same time share weight tiles through L2.  (Bands of 4 / 8 / 16 n-tiles with the
// n-tile fastest inside a band were measured too: 0 to 6 % slower on the large-batch shapes.)
__device__ __forceinline__ TileCoord decode_tile(int w, int n_tiles, const int32_t* tb, int E) {
  const int q = w / n_tiles;
  int lo = 0, hi = E;  // e = number of i in [1,E] with tb[i] <= q
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
// the same through the kernel's shared-memory work list `tb` (see build_tile_base)
__device__ __forceinline__ TileCoord decode_work(int w, const GemmParams& p, const int32_t* tb) {
  TileCoord c = decode_tile(w, p.n_tiles, tb, p.E);
  if (p.tile_mode == TILES_TAIL) c.mt = p.tile_base[c.e + 1] - 1;   // the expert's last row tile
  return c;
}

// Shared-memory work list of a single-CTA kernel (all threads call it before the set-up barrier):
// the row-tile prefix sums as they are, or the prefix sums of "has a left-over row tile".
__device__ __forceinline__ void build_tile_base(int32_t* dst, const int32_t* __restrict__ src, int E, int tile_mode) {
  if (tile_mode == TILES_TAIL) {
    if (threadIdx.x == 0) {
      int acc = 0;
      for (int e = 0; e < E; ++e) {
        dst[e] = acc;
        acc += (src[e + 1] - src[e]) & 1;
      }
      dst[E] = acc;
    }
  } else {
    for (int i = threadIdx.x; i <= E; i += blockDim.x) dst[i] = src[i];
  }
}

// SiTU (b12x/moe/_shared/kernels/reference.py:160-172): 4 tanh(g / 4) sigmoid(g) * 25 tanh(u / 25)
constexpr float kSituBeta = 4.0f, kSituLinearBeta = 25.0f;

// EPI selects the form: EPI_FC1_SILU plain SwiGLU (no clamp); EPI_FC1_GATED clamp and/or SwiGLU-OAI, chosen
// at run time; EPI_FC1_SITU the SiTU form.
template <int EPI>
__device__ __forceinline__ float act_gated(float gate, float up, const GemmParams& p) {
  if (EPI == EPI_FC1_SITU) {
    const float s = rcp_newton(1.0f + expf(fminf(-gate, 80.0f)));
    const float sg = __fmul_rn(__fmul_rn(kSituBeta, tanhf(__fdiv_rn(gate, kSituBeta))), s);
    const float su = __fmul_rn(kSituLinearBeta, tanhf(__fdiv_rn(up, kSituLinearBeta)));
    return __fmul_rn(sg, su);
  }
  if (EPI == EPI_FC1_GATED) {
    if (p.limit > 0.f) {
      gate = fminf(gate, p.limit);
      up = fminf(fmaxf(up, -p.limit), p.limit);
    }
    if (p.act_kind == 1) {
      const float s = rcp_newton(1.0f + expf(fminf(-(p.act_alpha * gate), 80.0f)));
      return (gate * s) * (up + p.act_beta);
    }
  }
  // the exponent is capped so that 1 + e stays finite (sigmoid below 2e-35 instead of 0)
  const float s = rcp_newton(1.0f + expf(fminf(-gate, 80.0f)));
  return (gate * s) * up;
}

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// MXFP8 quantisation of 32 values (b12x/_lib/intrinsics.py:223-265): E8M0 byte = exponent of
// pow2_ceil(amax / 448), payload = e4m3_rn_sat(x * 2^(127 - byte)).
__device__ __forceinline__ void requant_block32_mx(const float (&v)[32], uint32_t (&o)[8],
                                                   uint8_t& sf_byte) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  uint32_t bits = __float_as_uint(__fmul_rn(amax, static_cast<float>(1.0 / 448.0)));
  if (bits & 0x007fffffu) bits = (bits + 0x00800000u) & 0x7f800000u;
  sf_byte = static_cast<uint8_t>((bits >> 23) & 0xffu);
  const int ex = 254 - static_cast<int>(sf_byte);
  const float inv = sf_byte == 0 ? 0.f : __uint_as_float(static_cast<uint32_t>(ex < 0 ? 0 : ex) << 23);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t acc = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float q = fminf(fmaxf(__fmul_rn(v[4 * j + k], inv), -448.f), 448.f);
      acc |= static_cast<uint32_t>(f32_to_e4m3_rn_sat(q)) << (8 * k);
    }
    o[j] = acc;
  }
}

// n scale bytes (n = 1, 2 or 4, packed in `word`) -> the tile's atom chain at scale column `col`
template <int N>
__device__ __forceinline__ void store_sf(uint8_t* sf_tile, uint32_t m, uint32_t col, uint32_t word) {
  uint8_t* dst = sf_tile + sf_atom_offset(m, col);
  if (N == 4) *reinterpret_cast<uint32_t*>(dst) = word;
  else if (N == 2) *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(word);
  else *dst = static_cast<uint8_t>(word);
}

// Epilogue of one 128 x 256 accumulator tile, run by each of the eight epilogue warps: warp w may
// only read TMEM sub-partition (w & 3), i.e. tile rows 32*(w&3) .. +31 (m = that row, t_lane =
// the accumulator's TMEM address with the sub-partition's lane in the upper half); the two warps
// that share a sub-partition split the tile's columns (half = 0 / 1: columns [128*half, +128)).
//
// The warp first drains its 32 x 128 share of the accumulator into registers (128 per thread: the
// kernels raise the epilogue warps' register allowance with setmaxnreg for this) and calls
// release() -- the MMA thread may then start the next tile -- and only then does the arithmetic
// and the stores, under the next tile's main loop.  nrows == 0 (a tile that does not exist)
// stores nothing.
template <int KIND, int EPI, int BN, class Release>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, int e, int mt, int nt, int row0, int nrows,
                                              uint32_t t_lane, int m, int half, int lane, Release release) {
  static_assert(BN == 256, "the epilogue is written for 256-column tiles");
  constexpr bool kGated = epi_is_gated(EPI);
  uint32_t acc[128];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint32_t r[16];
    tc_ld_32x32b_x16(t_lane + half * 128 + c * 16, r);
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[c * 16 + i] = r[i];
  }
  tc_wait_ld();
  tc_fence_before();
  __syncwarp();
  release();

  const float alpha = p.alphas[e];
  const bool valid = m < nrows;
  const size_t pos = static_cast<size_t>(row0 + m);
  uint8_t* sft = p.out_sf + static_cast<size_t>(mt) * p.out_atoms * 512;
  if (kGated) {
    // a gated tile is two pair groups; this warp's group: acc[0..63] = up, acc[64..127] = gate of
    // the intermediate columns col0 .. col0 + 63
    const int col0 = nt * 128 + half * 64;
    const bool cols_ok = col0 < p.out_cols;
    if (KIND == KIND_MX) {
      // w4a8_mx: the activation output goes straight into the MXFP8 quantiser (no bf16 staging)
      uint8_t* qrow = p.out_q + pos * p.out_cols + col0;
      uint32_t sfw = 0u;
#pragma unroll
      for (int blk = 0; blk < 2; ++blk) {
        float h[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float up = __fmul_rn(__uint_as_float(acc[blk * 32 + i]), alpha);
          const float gate = __fmul_rn(__uint_as_float(acc[64 + blk * 32 + i]), alpha);
          if (p.tap != nullptr && valid && cols_ok) {
            float* trow = p.tap + pos * p.w_rows + col0 + blk * 32 + i;
            trow[p.sub0_base] = up;
            trow[p.sub1_base] = gate;
          }
          h[i] = act_gated<EPI>(gate, up, p);
        }
        uint32_t o[8];
        uint8_t sfb;
        requant_block32_mx(h, o, sfb);
        if (valid && cols_ok) {
          uint4* dst = reinterpret_cast<uint4*>(qrow + blk * 32);
          dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
          dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
        sfw |= static_cast<uint32_t>(sfb) << (8 * blk);
      }
      if (cols_ok && nrows > 0) store_sf<2>(sft, m, col0 >> 5, sfw);
    } else {
      const float gs2 = p.gscale2[p.gscale_len > 1 ? e : 0];
      const float rgs2 = __frcp_rn(gs2);
      uint8_t* qrow = p.out_q + pos * (p.out_cols >> 1) + (col0 >> 1);
      uint32_t sfw = 0u;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float h[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float up = __fmul_rn(__uint_as_float(acc[ch * 16 + i]), alpha);
          const float gate = __fmul_rn(__uint_as_float(acc[64 + ch * 16 + i]), alpha);
          if (p.tap != nullptr && valid && cols_ok) {
            float* trow = p.tap + pos * p.w_rows + col0 + ch * 16 + i;
            trow[p.sub0_base] = up;
            trow[p.sub1_base] = gate;
          }
          h[i] = round_bf16(act_gated<EPI>(gate, up, p));
        }
        uint32_t lo, hi;
        uint8_t sfb;
        quant_block16(h, gs2, rgs2, lo, hi, sfb);
        if (valid && cols_ok) *reinterpret_cast<uint2*>(qrow + ch * 8) = make_uint2(lo, hi);
        sfw |= static_cast<uint32_t>(sfb) << (8 * ch);
      }
      // scale atoms are per tile: padding rows are written too (their values are never used)
      if (cols_ok && nrows > 0) store_sf<4>(sft, m, col0 >> 4, sfw);
    }
  } else if (EPI == EPI_FC1_RELU2) {
    const int col0 = nt * 256 + half * 128;
    if (col0 < p.out_cols) {
      if (KIND == KIND_MX) {
        uint8_t* qrow = p.out_q + pos * p.out_cols + col0;
        uint32_t sfw = 0u;
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          float h[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = __fmul_rn(__uint_as_float(acc[blk * 32 + i]), alpha);
            if (p.tap != nullptr && valid && col0 + blk * 32 < p.out_cols)
              p.tap[pos * p.w_rows + col0 + blk * 32 + i] = v;
            const float r = fmaxf(v, 0.f);
            h[i] = __fmul_rn(r, r);
          }
          uint32_t o[8];
          uint8_t sfb;
          requant_block32_mx(h, o, sfb);
          if (valid && col0 + blk * 32 < p.out_cols) {
            uint4* dst = reinterpret_cast<uint4*>(qrow + blk * 32);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
          sfw |= static_cast<uint32_t>(sfb) << (8 * blk);
        }
        if (nrows > 0) store_sf<4>(sft, m, col0 >> 5, sfw);
      } else {
        const float gs2 = p.gscale2[p.gscale_len > 1 ? e : 0];
        const float rgs2 = __frcp_rn(gs2);
        uint8_t* qrow = p.out_q + pos * (p.out_cols >> 1) + (col0 >> 1);
        uint32_t sfw[2] = {0u, 0u};
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float h[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float v = __fmul_rn(__uint_as_float(acc[ch * 16 + i]), alpha);
            if (p.tap != nullptr && valid && col0 + ch * 16 < p.out_cols)
              p.tap[pos * p.w_rows + col0 + ch * 16 + i] = v;
            const float r = fmaxf(v, 0.f);
            h[i] = round_bf16(__fmul_rn(r, r));
          }
          uint32_t lo, hi;
          uint8_t sfb;
          quant_block16(h, gs2, rgs2, lo, hi, sfb);
          if (valid && col0 + ch * 16 < p.out_cols)
            *reinterpret_cast<uint2*>(qrow + ch * 8) = make_uint2(lo, hi);
          sfw[ch >> 2] |= static_cast<uint32_t>(sfb) << (8 * (ch & 3));
        }
        if (nrows > 0) store_sf<4>(sft, m, col0 >> 4, sfw[0]);
        if (nrows > 0 && col0 + 64 < p.out_cols) store_sf<4>(sft, m, (col0 >> 4) + 4, sfw[1]);
      }
    }
  } else {
    const int col0 = nt * 256 + half * 128;
    float* orow = p.out_f32 + pos * p.out_cols + col0;
    // 32-byte stores: a lane writes whole sectors of its own row (rows are 32-byte aligned: the row
    // length is a multiple of 16 floats and the arena's views start on 1 KiB boundaries)
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      if (valid && col0 + ch * 16 < p.out_cols) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          float v[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__uint_as_float(acc[ch * 16 + 8 * q + i]), alpha);
          st_global_f32x8(orow + ch * 16 + 8 * q, v);
        }
      }
    }
  }
}

// Register allowance per warp group (the four warps of a group execute this together).
template <int N>
__device__ __forceinline__ void regs_release_to() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void regs_raise_to() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// ---- host helpers (defined in grouped_gemm_bs.cu) ------------------------------------------
// 2-D byte matrix [rows][row_bytes], box = box_rows x 128 bytes, 128-byte swizzle.
int make_tmap_bytes_2d(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                       uint32_t box_rows);
// 2-D matrix of packed E2M1 values; the TMA expands every 16 values to a 16-byte slot (kind::mxf8f6f4)
int make_tmap_fp4_unpack_2d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint32_t box_rows);
int num_sms_cached();
void fill_common(GemmParams& p, const b200moe_gemm_args* a, char* base);

}  // namespace b200moe
