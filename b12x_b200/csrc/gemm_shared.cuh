// Pieces shared by the grouped GEMM kernels of this library: launch parameters, the work-list
// decoder, the epilogue arithmetic and the host-side tensor-map helpers.
#pragma once

#include "common.cuh"

namespace b200moe {

constexpr int kMaxExperts = 1024;

enum { EPI_FC1_GATED = 0, EPI_FC1_RELU2 = 1, EPI_FC2 = 2, EPI_FC1_SILU = 3 };
// KIND_NVFP4: A and B packed E2M1, E4M3 scale per 16, kind::mxf4nvf4 (K = 64 per MMA, 256 per stage).
// KIND_MX:    A E4M3 bytes, B E2M1 expanded by TMA to one value per byte slot, E8M0 scale per 32,
//             kind::mxf8f6f4 (K = 32 per MMA, 128 per stage; one scale atom per stage).
enum { KIND_NVFP4 = 0, KIND_MX = 1 };

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
  int swigluoai;
};

struct TileCoord {
  int e, mt, nt;
};
// work id -> (expert, m-tile, n-tile); expert-major, then n-tile, m-tile fastest, so that the CTAs
// running at the same time share weight tiles through L2.
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

// Branch-free reciprocal and division for the epilogues (a call with a slow-path branch per
// element keeps the compiler from interleaving the 16 independent element chains of a chunk).
__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// 1/x for normal x: hardware approximation + one Newton step (error <= 0.5 ulp + 2^-46)
__device__ __forceinline__ float rcp_newton(float x) {
  const float r = rcp_approx(x);
  return __fmaf_rn(r, __fmaf_rn(-x, r, 1.0f), r);
}
// a / b, correctly rounded when the quotient is a normal number or zero; rb = RN(1 / b).
// Two residual corrections with exact fma residuals (Markstein).
__device__ __forceinline__ float div_rn_normal(float a, float b, float rb) {
  float q = __fmul_rn(a, rb);
  q = __fmaf_rn(__fmaf_rn(-b, q, a), rb, q);
  q = __fmaf_rn(__fmaf_rn(-b, q, a), rb, q);
  return q;
}

// GENERIC = false: plain SwiGLU (no clamp); true: clamp and/or the SwiGLU-OAI form, chosen at run time.
template <bool GENERIC>
__device__ __forceinline__ float act_gated(float gate, float up, const GemmParams& p) {
  if (GENERIC) {
    if (p.limit > 0.f) {
      gate = fminf(gate, p.limit);
      up = fminf(fmaxf(up, -p.limit), p.limit);
    }
    if (p.swigluoai) {
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

// ---- host helpers (defined in grouped_gemm_bs.cu) ------------------------------------------
// 2-D byte matrix [rows][row_bytes], box = box_rows x 128 bytes, 128-byte swizzle.
int make_tmap_bytes_2d(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t rows,
                       uint32_t box_rows);
int num_sms_cached();
void fill_common(GemmParams& p, const b200moe_gemm_args* a, char* base);

}  // namespace b200moe
