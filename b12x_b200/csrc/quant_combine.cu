// Stage 3 (permute + activation quantisation) and stage 6 (top-k weighted combine).
// Both are HBM-bound streaming kernels: 16-byte vector accesses, one warp per row.
#include "quant_shared.cuh"

namespace b200moe {

__global__ void __launch_bounds__(256) permute_quant_nvfp4_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, const float* __restrict__ gscale,
    int gscale_len, int num_topk, int K, const int32_t* __restrict__ tile_base, int E,
    const int32_t* __restrict__ mtile_expert, const int32_t* __restrict__ mtile_row0,
    const int32_t* __restrict__ mtile_rows, const int32_t* __restrict__ sorted_route_ids,
    uint8_t* __restrict__ act_q, uint8_t* __restrict__ act_sf, int wpr_cap) {
  const int mt = blockIdx.x;
  if (mt >= tile_base[E]) return;
  const int e = mtile_expert[mt];
  const int row0 = mtile_row0[mt];
  const int nrows = mtile_rows[mt];
  const float gs = gscale[gscale_len > 1 ? e : 0];
  const float rgs = __frcp_rn(gs);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = K >> 4;                    // 16-element blocks per row
  const int atoms = (nblk + 3) >> 2;          // 512-byte scale atoms per tile
  uint8_t* sf_tile = act_sf + static_cast<size_t>(mt) * atoms * 512;

  // All eight warps work on the same row (a decode tile holds two or three rows: one warp per
  // row would leave the others idle and walk the row in 14 dependent steps).
  // (a short row takes only some of the warps; the others start on the next row)
  const int wpr = min(wpr_cap, (nblk + 31) >> 5);     // warps per row
  const int rows_par = 8 / wpr;                 // rows in flight per CTA
  const int wrow = warp / wpr, wchunk = warp - wrow * wpr;
  for (int i = blockIdx.y * rows_par + wrow; wrow < rows_par && i < nrows; i += gridDim.y * rows_par) {
    const int pos = row0 + i;
    const int r = sorted_route_ids[pos];
    const int t = r / num_topk;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t) * x_row_stride);
    uint2* dst = reinterpret_cast<uint2*>(act_q + static_cast<size_t>(pos) * (K >> 1));
    for (int b0 = wchunk * 32; b0 < nblk; b0 += wpr * 32) {
      const int b = b0 + lane;
      uint8_t sfb = 0;
      if (b < nblk) {
        const uint4 p0 = __ldg(src + 2 * b), p1 = __ldg(src + 2 * b + 1);
        const uint32_t w[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        float v[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[2 * j] = __uint_as_float(w[j] << 16);
          v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
        uint32_t lo, hi;
        quant_block16(v, gs, rgs, lo, hi, sfb);
        dst[b] = make_uint2(lo, hi);
      }
      // four neighbouring lanes hold the four scales of one 32-bit word of the atom
      uint32_t word = sfb;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 1) << 8;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 2) << 16;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 3) << 24;
      if ((lane & 3) == 0 && b < nblk) {
        *reinterpret_cast<uint32_t*>(sf_tile + sf_atom_offset(i, b)) = word;
      }
    }
  }
}

__global__ void __launch_bounds__(256) permute_quant_mxfp8_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, int num_topk, int K,
    const int32_t* __restrict__ tile_base, int E, const int32_t* __restrict__ mtile_row0,
    const int32_t* __restrict__ mtile_rows, const int32_t* __restrict__ sorted_route_ids,
    uint8_t* __restrict__ act_q, uint8_t* __restrict__ act_sf, int wpr_cap) {
  const int mt = blockIdx.x;
  if (mt >= tile_base[E]) return;
  const int row0 = mtile_row0[mt];
  const int nrows = mtile_rows[mt];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nblk = K >> 5;            // 32-element blocks per row
  const int atoms = (nblk + 3) >> 2;
  uint8_t* sf_tile = act_sf + static_cast<size_t>(mt) * atoms * 512;

  const int wpr = min(wpr_cap, (nblk + 31) >> 5);     // warps per row
  const int rows_par = 8 / wpr;                 // rows in flight per CTA
  const int wrow = warp / wpr, wchunk = warp - wrow * wpr;
  for (int i = blockIdx.y * rows_par + wrow; wrow < rows_par && i < nrows; i += gridDim.y * rows_par) {
    const int pos = row0 + i;
    const int r = sorted_route_ids[pos];
    const int t = r / num_topk;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t) * x_row_stride);
    uint4* dst = reinterpret_cast<uint4*>(act_q + static_cast<size_t>(pos) * K);
    for (int b0 = wchunk * 32; b0 < nblk; b0 += wpr * 32) {
      const int b = b0 + lane;
      uint8_t sfb = 0;
      if (b < nblk) {
        float v[32];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 p = __ldg(src + 4 * b + q);
          const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            v[q * 8 + 2 * j] = __uint_as_float(w[j] << 16);
            v[q * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
          }
        }
        uint32_t o[8];
        quant_block32_mx(v, o, sfb);
        dst[2 * b] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[2 * b + 1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
      uint32_t word = sfb;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 1) << 8;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 2) << 16;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 3) << 24;
      if ((lane & 3) == 0 && b < nblk) {
        *reinterpret_cast<uint32_t*>(sf_tile + sf_atom_offset(i, b)) = word;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// combine: out[t] = sum over slots (slot order) of w[t,slot] * routed[pos(t,slot)], each product
// and each sum rounded to fp32 separately (no fused multiply-add), one final rounding to bf16.
// This is the accumulation of the reference oracle (reference.py:408-411, 988-990).
// ------------------------------------------------------------------------------------------
template <int BATCH>
__global__ void __launch_bounds__(256) combine_kernel(
    const float* __restrict__ routed, const int32_t* __restrict__ inv_perm,
    const float* __restrict__ topk_weights, void* __restrict__ out, int64_t out_row_stride,
    int num_topk, int K, int out_f32, float output_scale) {
  const int t = blockIdx.x;
  extern __shared__ int32_t sm[];
  int32_t* pos = sm;
  float* w = reinterpret_cast<float*>(sm + num_topk);
  for (int s = threadIdx.x; s < num_topk; s += blockDim.x) {
    pos[s] = inv_perm[static_cast<int64_t>(t) * num_topk + s];
    w[s] = topk_weights != nullptr ? topk_weights[static_cast<int64_t>(t) * num_topk + s] : 1.0f;
  }
  __syncthreads();
  const int nvec = K >> 2;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < nvec; j += gridDim.y * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    // slots in order, BATCH at a time: the loads of a batch are issued before the first add
    for (int s0 = 0; s0 < num_topk; s0 += BATCH) {
      float4 v[BATCH];
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        const int p = s0 + q < num_topk ? pos[s0 + q] : -1;
        v[q] = p >= 0 ? __ldg(reinterpret_cast<const float4*>(routed + static_cast<size_t>(p) * K) + j)
                      : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int q = 0; q < BATCH; ++q) {
        if (s0 + q < num_topk && pos[s0 + q] >= 0) {
          const float ws = w[s0 + q];
          acc.x = __fadd_rn(acc.x, __fmul_rn(ws, v[q].x));
          acc.y = __fadd_rn(acc.y, __fmul_rn(ws, v[q].y));
          acc.z = __fadd_rn(acc.z, __fmul_rn(ws, v[q].z));
          acc.w = __fadd_rn(acc.w, __fmul_rn(ws, v[q].w));
        }
      }
    }
    if (out_f32) {
      float* o = reinterpret_cast<float*>(out) + static_cast<int64_t>(t) * out_row_stride;
      if (output_scale != 1.0f) {
        acc.x = __fmul_rn(acc.x, output_scale);
        acc.y = __fmul_rn(acc.y, output_scale);
        acc.z = __fmul_rn(acc.z, output_scale);
        acc.w = __fmul_rn(acc.w, output_scale);
      }
      reinterpret_cast<float4*>(o)[j] = acc;
    } else {
      __nv_bfloat16 b[4] = {__float2bfloat16_rn(acc.x), __float2bfloat16_rn(acc.y),
                            __float2bfloat16_rn(acc.z), __float2bfloat16_rn(acc.w)};
      if (output_scale != 1.0f) {
        // the caller-visible scaling is an in-place multiply of the bf16 output
#pragma unroll
        for (int q = 0; q < 4; ++q)
          b[q] = __float2bfloat16_rn(__fmul_rn(__bfloat162float(b[q]), output_scale));
      }
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + static_cast<int64_t>(t) * out_row_stride;
      uint2 pk;
      pk.x = static_cast<uint32_t>(__bfloat16_as_ushort(b[0])) |
             (static_cast<uint32_t>(__bfloat16_as_ushort(b[1])) << 16);
      pk.y = static_cast<uint32_t>(__bfloat16_as_ushort(b[2])) |
             (static_cast<uint32_t>(__bfloat16_as_ushort(b[3])) << 16);
      reinterpret_cast<uint2*>(o)[j] = pk;
    }
  }
}

// ------------------------------------------------------------------------------------------
// Standalone row quantisers (the reference's quantization.nvfp4 / quantization.mxfp8 ops): a
// dense [M, K] bf16 matrix, no permutation; codes row-major, scales as 128-row atom chains
// ([row group][k atom][512 bytes], the 128x4-swizzled layout) and, for MXFP8, also row-major.
//
// NVFP4 here is the "reciprocal" arithmetic of the reference's grouped quantiser
// (b12x/_lib/intrinsics.py:149-193), which differs from the MoE path's direct division:
//   sf   = e4m3_rn(gs * (amax / 6))
//   out  = 1 / (sf * (1 / gs))          (a zero factor gives zero, not infinity)
//   code = e2m1_rte(clamp(x * out, -6, 6))
// A scale beyond the E4M3 range saturates to 448 (torch yields NaN there; the op's contract
// gs = 448 * 6 / amax(tensor) keeps scales in range).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float recip_or_zero(float v) { return v == 0.f ? 0.f : __fdiv_rn(1.0f, v); }

__global__ void __launch_bounds__(256) quantize_rows_nvfp4_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, int M, int K, const float* __restrict__ gscale,
    uint8_t* __restrict__ out_q, uint8_t* __restrict__ out_sf) {
  const int nblk = K >> 4;
  const int atoms = (nblk + 3) >> 2;
  const float gs = gscale[0];
  const float rgs = recip_or_zero(gs);
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * x_row_stride);
    uint2* dst = reinterpret_cast<uint2*>(out_q + static_cast<size_t>(row) * (K >> 1));
    uint8_t* sf_tile = out_sf + static_cast<size_t>(row >> 7) * atoms * 512;
    for (int b0 = (threadIdx.x >> 5) * 32; b0 < nblk; b0 += 256) {
      const int b = b0 + lane;
      uint8_t sfb = 0;
      if (b < nblk) {
        const uint4 p0 = __ldg(src + 2 * b), p1 = __ldg(src + 2 * b + 1);
        const uint32_t w[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        float v[16];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[2 * j] = __uint_as_float(w[j] << 16);
          v[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
          amax = fmaxf(amax, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
        }
        sfb = f32_to_e4m3_rn_sat(__fmul_rn(gs, __fdiv_rn(amax, 6.0f)));
        const float out = recip_or_zero(__fmul_rn(e4m3_to_f32(sfb), rgs));
        float q0[8], q1[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          q0[i] = fminf(fmaxf(__fmul_rn(v[i], out), -6.0f), 6.0f);
          q1[i] = fminf(fmaxf(__fmul_rn(v[8 + i], out), -6.0f), 6.0f);
        }
        dst[b] = make_uint2(pack_e2m1x8(q0), pack_e2m1x8(q1));
      }
      uint32_t word = sfb;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 1) << 8;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 2) << 16;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 3) << 24;
      if ((lane & 3) == 0 && b < nblk)
        *reinterpret_cast<uint32_t*>(sf_tile + sf_atom_offset(row & 127, b)) = word;
    }
  }
}

// MXFP8 rows (b12x/_lib/intrinsics.py:223-312): the arithmetic of permute_quant_mxfp8_kernel.
// Scale bytes go row-major to `scale_rows` and / or swizzled to `scale_mma` (either may be null);
// only the bytes of live rows and real columns are written.
__global__ void __launch_bounds__(256) quantize_rows_mxfp8_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, int M, int K, uint8_t* __restrict__ values,
    uint8_t* __restrict__ scale_rows, uint8_t* __restrict__ scale_mma) {
  const int nblk = K >> 5;
  const int atoms = (nblk + 3) >> 2;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * x_row_stride);
    uint4* dst = reinterpret_cast<uint4*>(values + static_cast<size_t>(row) * K);
    for (int b = threadIdx.x; b < nblk; b += blockDim.x) {
      float v[32];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 p = __ldg(src + 4 * b + q);
        const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[q * 8 + 2 * j] = __uint_as_float(w[j] << 16);
          v[q * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
      }
      uint32_t o[8];
      uint8_t sfb;
      quant_block32_mx(v, o, sfb);
      dst[2 * b] = make_uint4(o[0], o[1], o[2], o[3]);
      dst[2 * b + 1] = make_uint4(o[4], o[5], o[6], o[7]);
      if (scale_rows != nullptr) scale_rows[static_cast<size_t>(row) * nblk + b] = sfb;
      if (scale_mma != nullptr)
        scale_mma[static_cast<size_t>(row >> 7) * atoms * 512 + sf_atom_offset(row & 127, b)] = sfb;
    }
  }
}

// ------------------------------------------------------------------------------------------
// gather_rows: send-side packing of the expert-parallel dispatch (one warp per row, 16-byte
// vectors).  Rows are ordered by the preceding sort (destination rank, then flat route id).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_rows_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, const int32_t* __restrict__ topk_ids,
    const int32_t* __restrict__ expert_offsets, int num_groups,
    const int32_t* __restrict__ sorted_route_ids, int num_topk, int K, int local_modulus,
    __nv_bfloat16* __restrict__ out_rows, int32_t* __restrict__ out_ids) {
  const int total = expert_offsets[num_groups];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int pos = blockIdx.x * 8 + warp; pos < total; pos += gridDim.x * 8) {
    const int r = sorted_route_ids[pos];
    const int t = r / num_topk;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t) * x_row_stride);
    uint4* dst = reinterpret_cast<uint4*>(out_rows + static_cast<size_t>(pos) * K);
    for (int j = lane; j < (K >> 3); j += 32) dst[j] = __ldg(src + j);
    if (lane == 0) out_ids[pos] = topk_ids[r] % local_modulus;
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_gather_rows(const b200moe_gather_args* a, void* stream) {
  if (a == nullptr || a->x == nullptr || a->topk_ids == nullptr || a->out_rows == nullptr ||
      a->out_ids == nullptr || a->scratch == nullptr || a->layout == nullptr)
    return B200MOE_EINVAL;
  if (a->hidden_size <= 0 || a->hidden_size % 8 != 0 || a->local_modulus <= 0 || a->num_groups <= 0)
    return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) != 0 || (a->x_row_stride % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(a->out_rows) & 15) != 0)
    return B200MOE_EALIGN;
  const int rows = a->num_tokens * a->num_topk;
  if (rows > a->layout->rows) return B200MOE_ECAPACITY;
  if (rows == 0) return B200MOE_OK;
  const b200moe_scratch_layout& L = *a->layout;
  char* base = static_cast<char*>(a->scratch);
  int grid = (rows + 7) / 8;
  if (grid > 148 * 8) grid = 148 * 8;
  gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a->x), a->x_row_stride, a->topk_ids,
      reinterpret_cast<const int32_t*>(base + L.expert_offsets), a->num_groups,
      reinterpret_cast<const int32_t*>(base + L.sorted_route_ids), a->num_topk, a->hidden_size,
      a->local_modulus, static_cast<__nv_bfloat16*>(a->out_rows), a->out_ids);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

static int check_quant_args(const b200moe_quant_args* a, int block) {
  if (a == nullptr || a->x == nullptr || a->scratch == nullptr || a->layout == nullptr)
    return B200MOE_EINVAL;
  if (a->hidden_size <= 0 || a->hidden_size % block != 0 || a->hidden_size % 8 != 0)
    return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) != 0 || (a->x_row_stride % 8) != 0)
    return B200MOE_EALIGN;
  if (a->num_tokens * a->num_topk > a->layout->rows) return B200MOE_ECAPACITY;
  return B200MOE_OK;
}

extern "C" int b200moe_permute_quant_nvfp4(const b200moe_quant_args* a, void* stream) {
  const int rc = check_quant_args(a, 16);
  if (rc != B200MOE_OK) return rc;
  if (a->a1_gscale == nullptr || (a->gscale_len != 1 && a->gscale_len != a->num_experts))
    return B200MOE_EINVAL;
  if (a->num_tokens == 0) return B200MOE_OK;
  const b200moe_scratch_layout& L = *a->layout;
  char* base = static_cast<char*>(a->scratch);
  const int rows = a->num_tokens * a->num_topk;
  const int tr = L.tile_rows == 64 ? 64 : 128;
  const int mtiles = (rows + tr - 1) / tr + (a->num_experts < rows ? a->num_experts : rows);
  // tiles of a decode batch hold few rows: one CTA per tile; large batches: 4 CTAs per tile
  // Small batches: the eight warps of a CTA share a row and a tile's rows are spread over enough
  // CTAs to fill the GPU about four times.  Large batches: one warp per row, sixteen CTAs per tile.
  const int gx = mtiles < L.mtile_cap ? mtiles : L.mtile_cap;
  const bool large = rows >= 2048 && L.tile_rows != 64;   // a 64-row plan expects few rows per expert
  // (large: 16 CTAs per tile keep enough loads in flight; 4 ran the Mixtral shape at 0.064 ms, 16 at 0.051 ms)
  int gy = large ? 16 : (4 * 148 + gx - 1) / gx;
  gy = gy < 1 ? 1 : (gy > 16 ? 16 : gy);
  const int wpr_cap = large ? 1 : 8;
  const dim3 grid(gx, gy);
  permute_quant_nvfp4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a->x), a->x_row_stride, a->a1_gscale, a->gscale_len,
      a->num_topk, a->hidden_size, reinterpret_cast<const int32_t*>(base + L.tile_base),
      a->num_experts, reinterpret_cast<const int32_t*>(base + L.mtile_expert),
      reinterpret_cast<const int32_t*>(base + L.mtile_row0),
      reinterpret_cast<const int32_t*>(base + L.mtile_rows),
      reinterpret_cast<const int32_t*>(base + L.sorted_route_ids),
      reinterpret_cast<uint8_t*>(base + L.act_q), reinterpret_cast<uint8_t*>(base + L.act_sf), wpr_cap);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_permute_quant_mxfp8(const b200moe_quant_args* a, void* stream) {
  const int rc = check_quant_args(a, 32);
  if (rc != B200MOE_OK) return rc;
  if (a->num_tokens == 0) return B200MOE_OK;
  const b200moe_scratch_layout& L = *a->layout;
  char* base = static_cast<char*>(a->scratch);
  const int rows = a->num_tokens * a->num_topk;
  const int tr = L.tile_rows == 64 ? 64 : 128;
  const int mtiles = (rows + tr - 1) / tr + (a->num_experts < rows ? a->num_experts : rows);
  // Small batches: the eight warps of a CTA share a row and a tile's rows are spread over enough
  // CTAs to fill the GPU about four times.  Large batches: one warp per row, four CTAs per tile.
  const int gx = mtiles < L.mtile_cap ? mtiles : L.mtile_cap;
  const bool large = rows >= 2048 && L.tile_rows != 64;   // a 64-row plan expects few rows per expert
  int gy = large ? 4 : (4 * 148 + gx - 1) / gx;
  gy = gy < 1 ? 1 : (gy > 16 ? 16 : gy);
  const int wpr_cap = large ? 1 : 8;
  const dim3 grid(gx, gy);
  permute_quant_mxfp8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a->x), a->x_row_stride, a->num_topk, a->hidden_size,
      reinterpret_cast<const int32_t*>(base + L.tile_base), a->num_experts,
      reinterpret_cast<const int32_t*>(base + L.mtile_row0),
      reinterpret_cast<const int32_t*>(base + L.mtile_rows),
      reinterpret_cast<const int32_t*>(base + L.sorted_route_ids),
      reinterpret_cast<uint8_t*>(base + L.act_q), reinterpret_cast<uint8_t*>(base + L.act_sf), wpr_cap);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

// fp32 -> bf16 (round to nearest even), 8 values per thread: the last step of the tensor-parallel
// layer, after the fp32 partial outputs of the ranks have been summed
__global__ void __launch_bounds__(256) round_rows_bf16_kernel(const float* __restrict__ in,
                                                              __nv_bfloat16* __restrict__ out, int64_t n8) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(in)[2 * i], b = reinterpret_cast<const float4*>(in)[2 * i + 1];
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x, a.y), p1 = __floats2bfloat162_rn(a.z, a.w);
    const __nv_bfloat162 p2 = __floats2bfloat162_rn(b.x, b.y), p3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 o;
    o.x = *reinterpret_cast<const uint32_t*>(&p0);
    o.y = *reinterpret_cast<const uint32_t*>(&p1);
    o.z = *reinterpret_cast<const uint32_t*>(&p2);
    o.w = *reinterpret_cast<const uint32_t*>(&p3);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

extern "C" int b200moe_round_rows_bf16(const float* in, void* out, int64_t count, void* stream) {
  if (in == nullptr || out == nullptr || count < 0 || (count & 7) != 0) return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(in) & 15) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0) return B200MOE_EALIGN;
  if (count == 0) return B200MOE_OK;
  const int64_t n8 = count >> 3;
  int64_t grid = (n8 + 255) / 256;
  grid = grid > 148 * 16 ? 148 * 16 : grid;
  round_rows_bf16_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      in, static_cast<__nv_bfloat16*>(out), n8);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_combine(const b200moe_combine_args* a, void* stream) {
  if (a == nullptr || a->topk_weights == nullptr || a->out == nullptr || a->scratch == nullptr ||
      a->layout == nullptr)
    return B200MOE_EINVAL;
  if (a->hidden_size <= 0 || a->hidden_size % 4 != 0 || a->num_topk <= 0) return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a->out) & 15) != 0 || (a->out_row_stride % 4) != 0)
    return B200MOE_EALIGN;
  if (a->num_tokens * a->num_topk > a->layout->rows) return B200MOE_ECAPACITY;
  if (a->num_tokens == 0) return B200MOE_OK;
  const b200moe_scratch_layout& L = *a->layout;
  char* base = static_cast<char*>(a->scratch);
  // small batches: several CTAs per token (slices of K), so that the grid fills the GPU
  int ysplit = (2 * 148 + a->num_tokens - 1) / a->num_tokens;
  const int ymax = (a->hidden_size / 4 + 255) / 256;
  ysplit = ysplit < 1 ? 1 : (ysplit > ymax ? ymax : ysplit);
  const dim3 grid(a->num_tokens, ysplit);
  const size_t smem = a->num_topk * 8;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
#define B200MOE_COMBINE_ARGS \
  reinterpret_cast<const float*>(base + L.routed), reinterpret_cast<const int32_t*>(base + L.inv_perm), \
      (a->unit_weights ? nullptr : a->topk_weights), a->out, a->out_row_stride, a->num_topk, a->hidden_size, a->out_f32, \
      a->output_scale
  if (a->num_topk <= 2) combine_kernel<2><<<grid, 256, smem, cs>>>(B200MOE_COMBINE_ARGS);
  else if (a->num_topk <= 4) combine_kernel<4><<<grid, 256, smem, cs>>>(B200MOE_COMBINE_ARGS);
  else combine_kernel<8><<<grid, 256, smem, cs>>>(B200MOE_COMBINE_ARGS);
#undef B200MOE_COMBINE_ARGS
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_quantize_rows_nvfp4(const void* x, int64_t x_row_stride, int32_t m, int32_t k,
                                           const float* global_scale, uint8_t* out_q, uint8_t* out_sf,
                                           void* stream) {
  if (x == nullptr || global_scale == nullptr || out_q == nullptr || out_sf == nullptr) return B200MOE_EINVAL;
  if (m < 0 || k <= 0 || k % 16 != 0) return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (x_row_stride % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(out_q) & 7) != 0 || (reinterpret_cast<uintptr_t>(out_sf) & 3) != 0)
    return B200MOE_EALIGN;
  if (m == 0) return B200MOE_OK;
  const int grid = m < 148 * 8 ? m : 148 * 8;
  quantize_rows_nvfp4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), x_row_stride, m, k, global_scale, out_q, out_sf);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_quantize_rows_mxfp8(const void* x, int64_t x_row_stride, int32_t m, int32_t k,
                                           uint8_t* values, uint8_t* scale_rows, uint8_t* scale_mma,
                                           void* stream) {
  if (x == nullptr || values == nullptr) return B200MOE_EINVAL;
  if (m < 0 || k <= 0 || k % 32 != 0) return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (x_row_stride % 8) != 0 ||
      (reinterpret_cast<uintptr_t>(values) & 15) != 0)
    return B200MOE_EALIGN;
  if (m == 0) return B200MOE_OK;
  const int grid = m < 148 * 8 ? m : 148 * 8;
  const int threads = k / 32 >= 256 ? 256 : (k / 32 >= 128 ? 128 : 64);
  quantize_rows_mxfp8_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), x_row_stride, m, k, values, scale_rows, scale_mma);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}
