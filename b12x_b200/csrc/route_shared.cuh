// The per-token router shared by the stand-alone top-k kernel and the fused gate kernels.
#pragma once

#include "common.cuh"

namespace b200moe {

// ------------------------------------------------------------------------------------------
// route_topk: one warp per token.  Lane l holds experts l, l+32, ... (E <= 1024 -> 32 values).
// Selection repeats "max, ties to the LARGEST expert index" k times, which is the tie rule of
// the reference router (b12x/moe/_shared/routing.py:38-46).
// ------------------------------------------------------------------------------------------
constexpr int kRouteMaxPerLane = 32;  // 1024 experts

// One warp routes token `warp`.  PAST_L1: the logits were written by other CTAs of the same launch
// (read them with ld.global.cg).
template <int MODE, bool PAST_L1 = false>
__device__ __forceinline__ void route_topk_token(const b200moe_route_args& a, int warp, int lane) {
  const int E = a.num_experts;
  const int per_lane = (E + 31) >> 5;
  const float NEG_INF = __int_as_float(0xff800000);

  float raw[kRouteMaxPerLane];  // raw logit
  float sel[kRouteMaxPerLane];  // value used for selection
#pragma unroll
  for (int i = 0; i < kRouteMaxPerLane; ++i) {
    raw[i] = NEG_INF;
    sel[i] = NEG_INF;
    if (i < per_lane) {
      const int e = i * 32 + lane;
      if (e < E) {
        float v;
        if (a.logits_dtype == B200MOE_DT_BF16) {
          const unsigned short* p16 = reinterpret_cast<const unsigned short*>(a.logits) + warp * a.logits_row_stride + e;
          v = __bfloat162float(__ushort_as_bfloat16(PAST_L1 ? __ldcg(p16) : *p16));
        } else {
          const float* p32 = reinterpret_cast<const float*>(a.logits) + warp * a.logits_row_stride + e;
          v = PAST_L1 ? __ldcg(p32) : *p32;
        }
        raw[i] = v;
        if (MODE == B200MOE_ROUTE_SIGMOID) {
          const float s = 1.0f / (1.0f + expf(-v));
          raw[i] = s;  // "original score"
          sel[i] = a.bias ? s + a.bias[e] : s;
        } else {
          sel[i] = v;
        }
      }
    }
  }

  float my_val = 0.f;   // lane `slot` keeps the slot's weight source (k <= 32 per pass)
  float my_logit = 0.f;
  int my_id = 0;
  for (int slot = 0; slot < a.num_topk; ++slot) {
    // lane-local best (ties -> larger index: scan ascending with >=)
    float best = NEG_INF;
    int best_e = -1;
#pragma unroll
    for (int i = 0; i < kRouteMaxPerLane; ++i) {
      if (i < per_lane) {
        const int e = i * 32 + lane;
        if (e < E && sel[i] >= best) {
          best = sel[i];
          best_e = e;
        }
      }
    }
    // warp arg-max with the same tie rule
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, off);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, off);
      if (ob > best || (ob == best && oe > best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    // fetch the weight source of the winner and retire it
    float win_raw = 0.f;
    if (best_e >= 0 && (best_e & 31) == lane) {
      const int i = best_e >> 5;
#pragma unroll
      for (int j = 0; j < kRouteMaxPerLane; ++j) {
        if (j == i) {
          win_raw = raw[j];
          sel[j] = NEG_INF;
          raw[j] = NEG_INF;
        }
      }
    }
    win_raw = __shfl_sync(0xffffffffu, win_raw, best_e >= 0 ? (best_e & 31) : 0);
    if ((slot & 31) == lane) {
      my_val = win_raw;
      my_logit = (MODE == B200MOE_ROUTE_SIGMOID) ? win_raw : best;
      my_id = best_e < 0 ? 0 : best_e;
    }
    // write out (k <= 32, so this runs once, after the last slot)
    if ((slot & 31) == 31 || slot == a.num_topk - 1) {
      const int base = slot & ~31;
      const int n_here = slot - base + 1;
      const bool active = lane < n_here;
      float w = my_val;
      if (MODE == B200MOE_ROUTE_SOFTMAX_TOPK) {
        // softmax over the selected logits, max-shifted (slot 0 holds the maximum)
        const float mx = __shfl_sync(0xffffffffu, my_val, 0);
        float ex = active ? expf(my_val - mx) : 0.f;
        float sum = ex;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        w = ex / sum;
      } else if (MODE == B200MOE_ROUTE_SIGMOID) {
        float sum = active ? my_val : 0.f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (a.renormalize) w = my_val / fmaxf(sum, 1e-20f);
        w = w * a.route_scale;
      }
      if (active) {
        const int64_t o = static_cast<int64_t>(warp) * a.num_topk + base + lane;
        a.topk_ids[o] = my_id;
        a.topk_weights[o] = w;
        if (a.topk_logits) a.topk_logits[o] = my_logit;
      }
    }
  }
}

}  // namespace b200moe
