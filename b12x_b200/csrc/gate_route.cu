// The step in front of the layer: router gate GEMM  logits[T][E] = hidden[T][K] . gate_weight[E][K]^T
// (+ bias), folded with the top-k router into ONE launch.  Two kernels:
//
//   gate_route_simt_kernel  any operand types (bf16 / f32), any K, E <= 1024.  A CTA multiplies
//       4 tokens x 32 experts on the CUDA cores; the last CTA of a token group to finish (a
//       counter per group, no waiting) routes that group's tokens.  Decode batches: the grid
//       spreads the gate matrix over many SMs.
//   gate_route_tc_kernel    bf16 x bf16, E a multiple of 16 and <= 256.  One CTA per 128 tokens:
//       TMA-fed tcgen05.mma (kind::f16) with the E logits of a token in one TMEM lane; the epilogue
//       writes the logits and routes its 32 tokens per warp.  Prefill batches.
//
// The logits are produced as the reference does (b12x/moe/fused_moe/_impl.py:11461-11468: a matrix
// product written in the operands' common type, then the bias added in that type): fp32
// accumulation, one rounding to bf16 when both operands are bf16, the bias added with one more
// rounding.  The router then works on the stored logits (same routine as b200moe_route_topk).
#include "gemm_shared.cuh"
#include "route_shared.cuh"

namespace b200moe {

constexpr int kGateTok = 4;       // tokens per CTA (SIMT kernel)
constexpr int kGateExp = 32;      // experts per CTA (SIMT kernel): 8 warps x 4

__device__ __forceinline__ float ld_elem(const void* p, int64_t i, int dt) {
  return dt == B200MOE_DT_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                               : reinterpret_cast<const float*>(p)[i];
}
// 8 consecutive elements starting at element i (i a multiple of 8, storage 16-byte aligned)
__device__ __forceinline__ void ld8(const void* p, int64_t i, int dt, float (&v)[8]) {
  if (dt == B200MOE_DT_BF16) {
    const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __uint_as_float(w[j] << 16);
      v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
    }
  } else {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    const float4 b = *(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}

// logit as stored: the fp32 sum rounded to the logits' type, then the bias added in that type
__device__ __forceinline__ float finish_logit(float acc, const void* bias, int e, int bias_dt, bool bf16_out) {
  float v = bf16_out ? round_bf16(acc) : acc;
  if (bias != nullptr) {
    float b = ld_elem(bias, e, bias_dt);
    if (bf16_out) b = round_bf16(b);
    v = __fadd_rn(v, b);
    if (bf16_out) v = round_bf16(v);
  }
  return v;
}

template <int MODE>
__device__ __forceinline__ void route_rows(const b200moe_route_args& r, int t0, int n, int warp_in_group,
                                           int warps_in_group, int lane) {
  for (int i = warp_in_group; i < n; i += warps_in_group) route_topk_token<MODE, true>(r, t0 + i, lane);
}

__device__ __forceinline__ void route_rows_any(const b200moe_route_args& r, int t0, int n, int wig, int nw, int lane) {
  if (r.mode == B200MOE_ROUTE_SOFTMAX_TOPK) route_rows<B200MOE_ROUTE_SOFTMAX_TOPK>(r, t0, n, wig, nw, lane);
  else if (r.mode == B200MOE_ROUTE_RAW) route_rows<B200MOE_ROUTE_RAW>(r, t0, n, wig, nw, lane);
  else route_rows<B200MOE_ROUTE_SIGMOID>(r, t0, n, wig, nw, lane);
}

__global__ void __launch_bounds__(256) gate_route_simt_kernel(b200moe_gate_route_args g, b200moe_route_args r,
                                                              int vec_ok) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * kGateTok;
  const int e0 = blockIdx.y * kGateExp + warp * 4;
  const int K = g.hidden_size, E = g.num_experts, T = g.num_tokens;
  const bool bf16_out = g.hidden_dtype == B200MOE_DT_BF16 && g.weight_dtype == B200MOE_DT_BF16;
  float acc[kGateTok][4];
#pragma unroll
  for (int i = 0; i < kGateTok; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int k_vec = vec_ok ? (K & ~7) : 0;
  for (int k = lane * 8; k < k_vec; k += 256) {
    float xv[kGateTok][8];
#pragma unroll
    for (int i = 0; i < kGateTok; ++i) {
      if (t0 + i < T) ld8(g.hidden, static_cast<int64_t>(t0 + i) * g.hidden_row_stride + k, g.hidden_dtype, xv[i]);
      else {
#pragma unroll
        for (int q = 0; q < 8; ++q) xv[i][q] = 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (e0 + j < E) {
        float wv[8];
        ld8(g.gate_weight, static_cast<int64_t>(e0 + j) * K + k, g.weight_dtype, wv);
#pragma unroll
        for (int i = 0; i < kGateTok; ++i)
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(xv[i][q], wv[q]));
      }
    }
  }
  for (int k = k_vec + lane; k < K; k += 32) {   // tail, or everything when the rows are not 16-byte aligned
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (e0 + j < E) {
        const float wv = ld_elem(g.gate_weight, static_cast<int64_t>(e0 + j) * K + k, g.weight_dtype);
#pragma unroll
        for (int i = 0; i < kGateTok; ++i)
          if (t0 + i < T)
            acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(
                ld_elem(g.hidden, static_cast<int64_t>(t0 + i) * g.hidden_row_stride + k, g.hidden_dtype), wv));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kGateTok; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc[i][j] += __shfl_xor_sync(0xffffffffu, acc[i][j], off);
  if (lane < kGateTok * 4) {
    const int i = lane >> 2, j = lane & 3;
    float v = 0.f;
#pragma unroll
    for (int a = 0; a < kGateTok; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b)
        if (a == i && b == j) v = acc[a][b];
    if (t0 + i < T && e0 + j < E) {
      v = finish_logit(v, g.gate_bias, e0 + j, g.bias_dtype, bf16_out);
      const int64_t o = static_cast<int64_t>(t0 + i) * E + e0 + j;
      if (bf16_out) reinterpret_cast<__nv_bfloat16*>(g.logits_out)[o] = __float2bfloat16_rn(v);
      else reinterpret_cast<float*>(g.logits_out)[o] = v;
    }
  }
  // the last CTA of this token group to get here routes the group's tokens (nobody waits)
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(g.tile_counters + blockIdx.x, 1);
    is_last = prev == static_cast<int>(gridDim.y) - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int n = min(kGateTok, T - t0);
  if (warp < n) route_rows_any(r, t0, n, warp, 8, lane);
}

// ---------------------------------------------------------------------------------------------
constexpr int kTcThreads = 192;       // TMA warp, MMA warp, four epilogue warps
constexpr int kTcStages = 4;
struct __align__(8) GateTail {
  uint64_t full[kTcStages];
  uint64_t empty[kTcStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kTcThreads, 1)
gate_route_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                     b200moe_gate_route_args g, b200moe_route_args r, int tmem_cols) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int E = g.num_experts, K = g.hidden_size, T = g.num_tokens;
  const int smem_w = E * 128;                        // one k-block of the gate matrix
  uint8_t* sX = smem;                                // [stage][128 rows][128 bytes]
  uint8_t* sW = sX + kTcStages * 16384;              // [stage][E rows][128 bytes]
  GateTail* tail = reinterpret_cast<GateTail*>(sW + kTcStages * ((smem_w + 1023) & ~1023));
  const int w_stage = (smem_w + 1023) & ~1023;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (K + 63) / 64;                // 64 bf16 = one 128-byte swizzled row

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    mbar_init(&tail->acc_full, 1);
    tail->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, static_cast<uint32_t>(tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_flag = &tail->abort_flag;
  const int t0 = blockIdx.x * 128;

  if (warp == 0) {
    if (lane < 2) {
      if (lane == 0) {
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmW);
      }
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait_bounded(&tail->empty[stage], phase ^ 1, abort_flag, g.status, WAIT_SMEM_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          // rows beyond T and bytes beyond a row's end arrive as zeros
          mbar_expect_tx(&tail->full[stage], 16384u + static_cast<uint32_t>(smem_w));
          tma_load_2d(sX + stage * 16384, &tmX, &tail->full[stage], kb * 128, t0);
        } else {
          tma_load_2d(sW + stage * w_stage, &tmW, &tail->full[stage], kb * 128, 0);
        }
        if (++stage == kTcStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let copies in flight land
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, E);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait_bounded(&tail->full[stage], phase, abort_flag, g.status, WAIT_SMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint64_t adesc = make_desc_sw128(smem_u32(sX + stage * 16384));
        const uint64_t bdesc = make_desc_sw128(smem_u32(sW + stage * w_stage));
        // four MMAs of 16 elements; the zero-filled tail of the last k-block adds nothing
#pragma unroll
        for (int j = 0; j < 4; ++j)
          mma_bf16(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, (kb > 0 || j > 0) ? 1u : 0u);
        tc_commit(&tail->empty[stage]);
        if (++stage == kTcStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) tc_commit(&tail->acc_full);
    }
  } else {
    // epilogue: warp w reads TMEM sub-partition w & 3 = tokens t0 + 32 * (w & 3) + lane
    const int sub = warp & 3;
    const int t = t0 + sub * 32 + lane;
    if (mbar_wait_bounded(&tail->acc_full, 0, abort_flag, g.status, WAIT_TMEM_FULL)) {
      tc_fence_after();
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(sub * 32) << 16);
      __nv_bfloat16* row = reinterpret_cast<__nv_bfloat16*>(g.logits_out) + static_cast<int64_t>(t) * E;
      for (int c = 0; c < E; c += 16) {
        uint32_t v[16];
        tc_ld_32x32b_x16(t_lane + c, v);
        tc_wait_ld();
        if (t < T) {
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float a = finish_logit(__uint_as_float(v[2 * i]), g.gate_bias, c + 2 * i, g.bias_dtype, true);
            const float b = finish_logit(__uint_as_float(v[2 * i + 1]), g.gate_bias, c + 2 * i + 1, g.bias_dtype, true);
            pk[i] = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(a))) |
                    (static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(b))) << 16);
          }
          uint4* dst = reinterpret_cast<uint4*>(row + c);
          dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
      }
      // this warp's 32 rows are in global memory: route them
      __threadfence();
      __syncwarp();
      const int n = min(32, T - (t0 + sub * 32));
      if (n > 0) route_rows_any(r, t0 + sub * 32, n, 0, 1, lane);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(tmem_cols));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [rows][row_bytes] bytes with `stride_bytes` between rows; box = box_rows x 128 bytes, 128-byte swizzle
static int tmap_rows(CUtensorMap* out, const void* base, uint64_t row_bytes, uint64_t stride_bytes, uint64_t rows,
                     uint32_t box_rows) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return B200MOE_ECUDA;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {stride_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ECUDA;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_gate_route(const b200moe_gate_route_args* g, void* stream) {
  if (g == nullptr || g->hidden == nullptr || g->gate_weight == nullptr || g->logits_out == nullptr ||
      g->topk_ids == nullptr || g->topk_weights == nullptr || g->tile_counters == nullptr)
    return B200MOE_EINVAL;
  const int T = g->num_tokens, E = g->num_experts, K = g->hidden_size;
  if (E <= 0 || E > 1024 || K <= 0 || T < 0) return B200MOE_EINVAL;
  if (g->num_topk <= 0 || g->num_topk > E || g->num_topk > 32) return B200MOE_EINVAL;
  if (g->mode < B200MOE_ROUTE_SOFTMAX_TOPK || g->mode > B200MOE_ROUTE_SIGMOID) return B200MOE_EINVAL;
  for (int dt : {g->hidden_dtype, g->weight_dtype, g->bias_dtype})
    if (dt != B200MOE_DT_F32 && dt != B200MOE_DT_BF16) return B200MOE_EINVAL;
  if (g->hidden_row_stride < K) return B200MOE_EINVAL;
  if (T == 0) return B200MOE_OK;
  const bool both_bf16 = g->hidden_dtype == B200MOE_DT_BF16 && g->weight_dtype == B200MOE_DT_BF16;
  b200moe_route_args r = {};
  r.logits = g->logits_out;
  r.bias = g->selection_bias;
  r.topk_logits = g->topk_logits;
  r.topk_ids = g->topk_ids;
  r.topk_weights = g->topk_weights;
  r.logits_row_stride = E;
  r.num_tokens = T;
  r.num_experts = E;
  r.num_topk = g->num_topk;
  r.logits_dtype = both_bf16 ? B200MOE_DT_BF16 : B200MOE_DT_F32;
  r.mode = g->mode;
  r.renormalize = g->renormalize;
  r.route_scale = g->route_scale;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool tc_ok = both_bf16 && E % 16 == 0 && E >= 16 && E <= 256 && K % 8 == 0 &&
                     g->hidden_row_stride % 8 == 0 && aligned16(g->hidden) && aligned16(g->gate_weight) &&
                     aligned16(g->logits_out);
  int kernel = g->kernel;
  if (kernel == B200MOE_GATE_AUTO) kernel = (tc_ok && T >= 128) ? B200MOE_GATE_TC : B200MOE_GATE_SIMT;
  if (kernel == B200MOE_GATE_TC) {
    if (!tc_ok) return B200MOE_EUNSUPPORTED;
    CUtensorMap tmX, tmW;
    int rc = tmap_rows(&tmX, g->hidden, static_cast<uint64_t>(K) * 2, static_cast<uint64_t>(g->hidden_row_stride) * 2,
                       static_cast<uint64_t>(T), 128);
    if (rc != B200MOE_OK) return rc;
    rc = tmap_rows(&tmW, g->gate_weight, static_cast<uint64_t>(K) * 2, static_cast<uint64_t>(K) * 2,
                   static_cast<uint64_t>(E), static_cast<uint32_t>(E));
    if (rc != B200MOE_OK) return rc;
    int cols = 32;
    while (cols < E) cols <<= 1;
    const int smem = 1024 + kTcStages * (16384 + ((E * 128 + 1023) & ~1023)) + static_cast<int>(sizeof(GateTail));
    if (cudaFuncSetAttribute(gate_route_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return B200MOE_ECUDA;
    gate_route_tc_kernel<<<(T + 127) / 128, kTcThreads, smem, s>>>(tmX, tmW, *g, r, cols);
    return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
  }
  if (kernel != B200MOE_GATE_SIMT) return B200MOE_EINVAL;
  const size_t he = g->hidden_dtype == B200MOE_DT_BF16 ? 2 : 4, we = g->weight_dtype == B200MOE_DT_BF16 ? 2 : 4;
  // the 8-element loads need 16-byte aligned rows (32 bytes per load for f32 operands)
  const int vec_ok = aligned16(g->hidden) && aligned16(g->gate_weight) &&
                     (g->hidden_row_stride * he) % (he * 8) == 0 && (static_cast<size_t>(K) * we) % (we * 8) == 0;
  const dim3 grid((T + kGateTok - 1) / kGateTok, (E + kGateExp - 1) / kGateExp);
  // the per-group arrival counters start at zero (a memset node when the call is captured)
  if (cudaMemsetAsync(g->tile_counters, 0, sizeof(int32_t) * grid.x, s) != cudaSuccess) return B200MOE_ECUDA;
  gate_route_simt_kernel<<<grid, 256, 0, s>>>(*g, r, vec_ok);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}
