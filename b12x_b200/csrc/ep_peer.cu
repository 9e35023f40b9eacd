// Expert-parallel dispatch and combine over NVLink peer memory (one process per GPU, buffers in
// symmetric memory so that every rank holds a device pointer to every peer's copy).
//
//   dispatch : each rank copies its routed rows straight into the destination ranks' receive
//              buffers (plain peer stores), in the order of the preceding sort by destination rank;
//              rank `r` owns the slots [r*cap, (r+1)*cap) of every receive buffer, writes the
//              destination-local expert id of each row next to it and -1 into its unused slots,
//              and finally raises flag[r] = epoch on every peer.
//   wait     : a one-warp kernel that polls this rank's flags until all peers have reached `epoch`.
//              The poll is bounded (2 s); on expiry it records an error in the status block and
//              returns, so a missing peer never hangs the GPU.
//   combine  : the home rank pulls the per-route FC2 rows (fp32) of its tokens from the experts'
//              ranks with plain peer loads and sums them in slot order, exactly as the single-GPU
//              combine does -- the return all-to-all and the weighted sum are one kernel.
//
// No kernel here uses multimem or cluster features; peers are only touched with ld/st.global.
// The reference library has no counterpart (its ep_moe replicates the input and lets the caller
// sum partial outputs, b12x/moe/ep_moe/_impl.py:1-14).
#include "quant_shared.cuh"

namespace b200moe {

__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int32_t* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct PeerPtrs {
  void* p[B200MOE_MAX_RANKS];
};

// Scale bytes of one warp item (32 blocks): lanes 0, 4, .., 28 hold one 32-bit word each.  A link
// packet per 4-byte word would double the packets of a row, so with 16-byte-aligned scale rows
// lanes 0 and 16 collect four words each and store 16 bytes (bytes past the row's last block are
// zero and lie inside the padded row); otherwise the words go out one by one.
__device__ __forceinline__ void store_scale_words(uint8_t* dsf, int b, int nblk, uint32_t word, int lane,
                                                  int sf_row_stride) {
  if ((sf_row_stride & 15) == 0) {
    uint4 q;
    q.x = word;
    q.y = __shfl_down_sync(0xffffffffu, word, 4);
    q.z = __shfl_down_sync(0xffffffffu, word, 8);
    q.w = __shfl_down_sync(0xffffffffu, word, 12);
    if ((lane & 15) == 0 && b < nblk) *reinterpret_cast<uint4*>(dsf + b) = q;
  } else if ((lane & 3) == 0 && b < nblk) {
    *reinterpret_cast<uint32_t*>(dsf + b) = word;
  }
}

// PAYLOAD 0: bf16 rows as they are.  1: NVFP4 codes + E4M3 scale bytes, quantised here with the
// destination expert's input scale (the bytes the expert rank's own quantiser would have made, so
// 9K/16 bytes cross the link per route instead of 2K).  2: MXFP8 values + E8M0 scale bytes (K + K/32).
// Scale bytes travel row-major, `sf_row_stride` (a multiple of 4) per slot; the expert rank files them
// into scale atoms when it puts the rows in expert order (permute_packed_kernel).
template <int PAYLOAD>
__global__ void __launch_bounds__(256) ep_dispatch_kernel(
    const __nv_bfloat16* __restrict__ x, int64_t x_row_stride, const int32_t* __restrict__ topk_ids,
    const int32_t* __restrict__ group_offsets, const int32_t* __restrict__ sorted_route_ids,
    PeerPtrs rows, PeerPtrs sfs, PeerPtrs ids, PeerPtrs flags, const float* __restrict__ a1_gscale,
    const int32_t* __restrict__ local_ids, int gscale_len, int sf_row_stride, int32_t* done_counter,
    int32_t* __restrict__ status, int world,
    int rank, int num_topk, int K, int local_modulus, int cap, int epoch_arg, int32_t* epoch_dev) {
  // Epoch kept on the device (a captured CUDA graph replays with fixed arguments): this step is
  // *epoch_dev + 1.  Every block reads it on entry; the last block out stores it back after all
  // others have left, and the later kernels of the step read the stored value.
  const int epoch = epoch_dev != nullptr ? *static_cast<volatile int32_t*>(epoch_dev) + 1 : epoch_arg;
  __shared__ int offs[B200MOE_MAX_RANKS + 1];
  if (threadIdx.x <= world) offs[threadIdx.x] = group_offsets[threadIdx.x];
  __syncthreads();
  const int total = offs[world];
  const int lane = threadIdx.x & 31;
  // Work item of a WARP: 32 consecutive blocks of one row (512 NVFP4 / 1024 MXFP8 values, or 32
  // 16-byte pieces of a bf16 row).  Every warp of the grid is busy whatever the row length, and a
  // warp's loads and (peer) stores of one item are independent of its next item's.
  const int nblk = PAYLOAD == 0 ? K >> 3 : (PAYLOAD == 1 ? K >> 4 : K >> 5);
  const int cpr = (nblk + 31) >> 5;                       // items per row
  const int warps = static_cast<int>(gridDim.x) * (blockDim.x >> 5);
  for (int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < total * cpr; item += warps) {
    const int pos = item / cpr;
    const int b = (item - pos * cpr) * 32 + lane;
    int d = 0;
    while (d + 1 < world && pos >= offs[d + 1]) ++d;
    const int j = pos - offs[d];
    if (j >= cap) {
      // more rows for rank d than its receive region holds: the row is not sent, the step is invalid
      if (lane == 0 && status != nullptr) {
        atomicCAS(status, 0, 1);
        atomicCAS(status + 1, 0, 48 + d);     // 48 + destination rank: receive capacity exceeded
      }
      continue;
    }
    const int slot = rank * cap + j;
    const int r = sorted_route_ids[pos];
    const int t = r / num_topk;
    const int expert = topk_ids[r];
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(t) * x_row_stride);
    if constexpr (PAYLOAD == 0) {
      uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(rows.p[d]) +
                                            static_cast<size_t>(slot) * K);
      if (b < nblk) dst[b] = __ldg(src + b);
    } else if constexpr (PAYLOAD == 1) {
      const float gs = a1_gscale[gscale_len == 1 ? 0 : expert];
      const float rgs = __frcp_rn(gs);
      uint2* dst = reinterpret_cast<uint2*>(static_cast<uint8_t*>(rows.p[d]) + static_cast<size_t>(slot) * (K >> 1));
      uint8_t* dsf = static_cast<uint8_t*>(sfs.p[d]) + static_cast<size_t>(slot) * sf_row_stride;
      uint8_t sfb = 0;
      if (b < nblk) {
        float v[16];
        bf16x8_to_f32(__ldg(src + 2 * b), v);
        bf16x8_to_f32(__ldg(src + 2 * b + 1), v + 8);
        uint32_t lo, hi;
        quant_block16(v, gs, rgs, lo, hi, sfb);
        dst[b] = make_uint2(lo, hi);
      }
      // four neighbouring lanes hold the four scale bytes of one 32-bit word
      uint32_t word = sfb;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 1) << 8;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 2) << 16;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 3) << 24;
      store_scale_words(dsf, b, nblk, word, lane, sf_row_stride);
    } else {
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(rows.p[d]) + static_cast<size_t>(slot) * K);
      uint8_t* dsf = static_cast<uint8_t*>(sfs.p[d]) + static_cast<size_t>(slot) * sf_row_stride;
      uint8_t sfb = 0;
      if (b < nblk) {
        float v[32];
#pragma unroll
        for (int q = 0; q < 4; ++q) bf16x8_to_f32(__ldg(src + 4 * b + q), v + 8 * q);
        uint32_t o[8];
        quant_block32_mx(v, o, sfb);
        dst[2 * b] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[2 * b + 1] = make_uint4(o[4], o[5], o[6], o[7]);
      }
      uint32_t word = sfb;      // lanes past the row's end contribute 0: the padding bytes are defined
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 1) << 8;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 2) << 16;
      word |= __shfl_down_sync(0xffffffffu, static_cast<uint32_t>(sfb), 3) << 24;
      store_scale_words(dsf, b, nblk, word, lane, sf_row_stride);
    }
    if (lane == 0 && b == 0)
      static_cast<int32_t*>(ids.p[d])[slot] = local_ids != nullptr ? local_ids[r] : expert % local_modulus;
  }
  // unused slots of this rank's region on every peer: no route
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < world * cap; i += gridDim.x * blockDim.x) {
    const int d = i / cap, j = i - d * cap;
    if (j >= offs[d + 1] - offs[d]) static_cast<int32_t*>(ids.p[d])[rank * cap + j] = -1;
  }
  // last block out raises the flags: every block publishes its peer stores first
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(done_counter, 1);
    is_last = prev == static_cast<int>(gridDim.x) - 1;
    if (is_last) {
      *done_counter = 0;
      if (epoch_dev != nullptr) *epoch_dev = epoch;
    }
  }
  __syncthreads();
  // one thread per peer: the release stores (a system-scope fence each, i.e. a link round trip)
  // go out side by side instead of one after the other
  if (is_last && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<int32_t*>(flags.p[threadIdx.x]) + rank, epoch);
  }
}

// Replicated experts: route i to expert e goes to holder pattern[e][i % 16] of that expert -- a
// (rank, local expert slot) pair.  An expert held by one rank has sixteen equal entries; a hot
// expert copied to other ranks spreads its routes over its holders in sixteenths.
__global__ void ep_place_routes_kernel(const int32_t* __restrict__ topk_ids, int n, int num_experts,
                                       const int32_t* __restrict__ pattern_rank,
                                       const int32_t* __restrict__ pattern_local,
                                       int32_t* __restrict__ dest_rank, int32_t* __restrict__ dest_local) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int e = topk_ids[i];
    const bool ok = e >= 0 && e < num_experts;
    const int j = e * 16 + (i & 15);
    dest_rank[i] = ok ? pattern_rank[j] : -1;
    dest_local[i] = ok ? pattern_local[j] : -1;
  }
}

// Expert side of the quantised dispatch: rows arrive in slot order, already quantised; copy each
// into its place in expert order and file its scale bytes into the tile's 128x4 scale atoms --
// what the permute + quantise kernel leaves behind, without the arithmetic.
template <int PAYLOAD>
__global__ void __launch_bounds__(256) permute_packed_kernel(
    const uint8_t* __restrict__ q_rows, const uint8_t* __restrict__ sf_rows, int sf_row_stride, int K,
    const int32_t* __restrict__ tile_base, int E, const int32_t* __restrict__ mtile_row0,
    const int32_t* __restrict__ mtile_rows, const int32_t* __restrict__ sorted_route_ids,
    uint8_t* __restrict__ act_q, uint8_t* __restrict__ act_sf) {
  const int mt = blockIdx.x;
  if (mt >= tile_base[E]) return;
  const int row0 = mtile_row0[mt];
  const int nrows = mtile_rows[mt];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_bytes = PAYLOAD == 1 ? K >> 1 : K;
  const int nblk = PAYLOAD == 1 ? K >> 4 : K >> 5;
  const int nwords = (nblk + 3) >> 2;          // one word = the four scale bytes of one atom column group
  uint8_t* sf_tile = act_sf + static_cast<size_t>(mt) * nwords * 512;
  for (int i = blockIdx.y * 8 + warp; i < nrows; i += gridDim.y * 8) {
    const int pos = row0 + i;
    const int r = sorted_route_ids[pos];
    const uint4* src = reinterpret_cast<const uint4*>(q_rows + static_cast<size_t>(r) * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(act_q + static_cast<size_t>(pos) * row_bytes);
    for (int q = lane; q < (row_bytes >> 4); q += 32) dst[q] = __ldcg(src + q);
    const uint32_t* ssrc = reinterpret_cast<const uint32_t*>(sf_rows + static_cast<size_t>(r) * sf_row_stride);
    for (int w = lane; w < nwords; w += 32)
      *reinterpret_cast<uint32_t*>(sf_tile + sf_atom_offset(i, 4 * w)) = __ldcg(ssrc + w);
  }
}

__global__ void ep_signal_kernel(PeerPtrs flags, int world, int rank, int epoch_arg,
                                 const int32_t* epoch_dev) {
  const int epoch = epoch_dev != nullptr ? *epoch_dev : epoch_arg;
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<int32_t*>(flags.p[threadIdx.x]) + rank, epoch);
  }
}

__global__ void ep_wait_kernel(const int32_t* __restrict__ flags, int world, int epoch_arg,
                               const int32_t* epoch_dev, int32_t* __restrict__ status,
                               unsigned long long limit_ns) {
  const int epoch = epoch_dev != nullptr ? *epoch_dev : epoch_arg;
  const int r = threadIdx.x;
  if (r >= world) return;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (ld_acquire_sys(flags + r) < epoch) {
    if ((++spins & 0x3ffu) == 0) {
      const unsigned long long now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > limit_ns) {
        if (status != nullptr) {
          atomicCAS(status, 0, 1);
          atomicCAS(status + 1, 0, 16 + r);   // 16 + peer rank: that peer never arrived
        }
        return;
      }
    }
  }
}

__global__ void __launch_bounds__(256) ep_combine_pull_kernel(
    const int32_t* __restrict__ group_offsets, const int32_t* __restrict__ inv_perm,
    const float* __restrict__ topk_weights, PeerPtrs arenas, int64_t peer_inv_perm_off,
    int64_t peer_routed_off, __nv_bfloat16* __restrict__ out, int64_t out_row_stride, int world,
    int rank, int num_topk, int K, int cap, float output_scale, PeerPtrs signal_flags,
    const int32_t* __restrict__ wait_flags, const int32_t* epoch_dev, int32_t* __restrict__ status,
    unsigned long long limit_ns) {
  extern __shared__ unsigned char sm_raw[];
  // Optional hand-shake folded into this kernel (saves two launches per step).  Block (0,0) tells
  // every peer that this rank's FC2 rows are complete (the FC2 kernel ended before this one began)
  // and then waits for ALL peers: the kernel cannot end before every rank has finished the step's
  // FC2, which is what allows the next step's dispatch to overwrite the peers' receive buffers.
  // Every other block waits only for the ranks that hold ITS token's rows, so rows of ranks that are
  // done are pulled while a slower rank still computes.  All waits are bounded.
  const bool fold = wait_flags != nullptr;
  const int epoch = fold ? *epoch_dev : 0;
  auto wait_for = [&](int peer) -> bool {
    unsigned long long t0 = 0;
    uint32_t spins = 0;
    while (ld_acquire_sys(wait_flags + peer) < epoch) {
      if ((++spins & 0x3ffu) == 0) {
        const unsigned long long now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > limit_ns) {
          if (status != nullptr) {
            atomicCAS(status, 0, 1);
            atomicCAS(status + 1, 0, 16 + peer);
          }
          return false;
        }
      }
    }
    return true;
  };
  if (fold && blockIdx.x == 0 && blockIdx.y == 0) {
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(static_cast<int32_t*>(signal_flags.p[threadIdx.x]) + rank, epoch);
      wait_for(static_cast<int>(threadIdx.x));
    }
    __syncthreads();
  }
  const float** rowp = reinterpret_cast<const float**>(sm_raw);
  float* w = reinterpret_cast<float*>(sm_raw + num_topk * sizeof(float*));
  const int t = blockIdx.x;
  for (int s = threadIdx.x; s < num_topk; s += blockDim.x) {
    const int pos = inv_perm[static_cast<int64_t>(t) * num_topk + s];
    const float* rp = nullptr;
    if (pos >= 0) {
      int d = 0;
      while (d + 1 < world && pos >= group_offsets[d + 1]) ++d;
      const int j = pos - group_offsets[d];
      const int slot = rank * cap + j;
      const char* arena = static_cast<const char*>(arenas.p[d]);
      // a route beyond the receive capacity was never sent (the dispatch raised the status word);
      // the rows of rank d are read only after rank d has said that they are complete
      if (j < cap && (!fold || wait_for(d))) {
        const int p = reinterpret_cast<const int32_t*>(arena + peer_inv_perm_off)[slot];
        if (p >= 0) rp = reinterpret_cast<const float*>(arena + peer_routed_off) + static_cast<size_t>(p) * K;
      }
    }
    rowp[s] = rp;
    w[s] = topk_weights[static_cast<int64_t>(t) * num_topk + s];
  }
  __syncthreads();
  const int nvec = K >> 2;
  for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < nvec; j += gridDim.y * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    // slots in order, eight at a time: the (peer) loads of a batch are issued before the first add
    for (int s0 = 0; s0 < num_topk; s0 += 8) {
      float4 v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float* rp = s0 + q < num_topk ? rowp[s0 + q] : nullptr;
        v[q] = rp != nullptr ? *(reinterpret_cast<const float4*>(rp) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (s0 + q < num_topk && rowp[s0 + q] != nullptr) {
          const float ws = w[s0 + q];
          acc.x = __fadd_rn(acc.x, __fmul_rn(ws, v[q].x));
          acc.y = __fadd_rn(acc.y, __fmul_rn(ws, v[q].y));
          acc.z = __fadd_rn(acc.z, __fmul_rn(ws, v[q].z));
          acc.w = __fadd_rn(acc.w, __fmul_rn(ws, v[q].w));
        }
      }
    }
    __nv_bfloat16 b[4] = {__float2bfloat16_rn(acc.x), __float2bfloat16_rn(acc.y),
                          __float2bfloat16_rn(acc.z), __float2bfloat16_rn(acc.w)};
    if (output_scale != 1.0f) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        b[q] = __float2bfloat16_rn(__fmul_rn(__bfloat162float(b[q]), output_scale));
    }
    uint2 pk;
    pk.x = static_cast<uint32_t>(__bfloat16_as_ushort(b[0])) |
           (static_cast<uint32_t>(__bfloat16_as_ushort(b[1])) << 16);
    pk.y = static_cast<uint32_t>(__bfloat16_as_ushort(b[2])) |
           (static_cast<uint32_t>(__bfloat16_as_ushort(b[3])) << 16);
    reinterpret_cast<uint2*>(out + static_cast<int64_t>(t) * out_row_stride)[j] = pk;
  }
}

}  // namespace b200moe

using namespace b200moe;

static bool fill_peers(PeerPtrs& dst, void* const* src, int world) {
  for (int i = 0; i < B200MOE_MAX_RANKS; ++i) dst.p[i] = i < world ? src[i] : nullptr;
  for (int i = 0; i < world; ++i)
    if (dst.p[i] == nullptr) return false;
  return true;
}

template <int PAYLOAD>
static void launch_dispatch(const b200moe_ep_dispatch_args* a, const PeerPtrs& rows_p, const PeerPtrs& sf_p,
                            const PeerPtrs& ids_p, const PeerPtrs& flags_p, int grid, cudaStream_t stream) {
  const b200moe_scratch_layout& L = *a->layout;
  char* base = static_cast<char*>(a->scratch);
  ep_dispatch_kernel<PAYLOAD><<<grid, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(a->x), a->x_row_stride, a->topk_ids,
      reinterpret_cast<const int32_t*>(base + L.expert_offsets),
      reinterpret_cast<const int32_t*>(base + L.sorted_route_ids), rows_p, sf_p, ids_p, flags_p,
      a->a1_gscale, a->local_ids, a->gscale_len, a->sf_row_stride, a->done_counter, a->status, a->world, a->rank,
      a->num_topk, a->hidden_size, a->local_modulus, a->cap_rows, a->epoch, a->epoch_dev);
}

extern "C" int b200moe_ep_dispatch(const b200moe_ep_dispatch_args* a, void* stream) {
  if (a == nullptr || a->x == nullptr || a->topk_ids == nullptr || a->scratch == nullptr ||
      a->layout == nullptr || a->done_counter == nullptr)
    return B200MOE_EINVAL;
  if (a->world < 1 || a->world > B200MOE_MAX_RANKS || a->rank < 0 || a->rank >= a->world ||
      a->hidden_size <= 0 || a->hidden_size % 8 != 0 || a->local_modulus <= 0 || a->cap_rows <= 0)
    return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a->x) & 15) != 0 || (a->x_row_stride % 8) != 0) return B200MOE_EALIGN;
  const int rows = a->num_tokens * a->num_topk;
  if (rows > a->layout->rows) return B200MOE_ECAPACITY;
  // fewer slots per source rank than its routes: allowed only with a status word for the overflow
  if (rows > a->cap_rows && a->status == nullptr) return B200MOE_ECAPACITY;
  PeerPtrs rows_p, ids_p, flags_p, sf_p = {};
  if (!fill_peers(rows_p, a->peer_rows, a->world) || !fill_peers(ids_p, a->peer_ids, a->world) ||
      !fill_peers(flags_p, a->peer_flags, a->world))
    return B200MOE_EINVAL;
  if (a->payload != B200MOE_EP_PAYLOAD_BF16) {
    const int blk = a->payload == B200MOE_EP_PAYLOAD_NVFP4 ? 64 : 32;   // values per scale word / per block
    if (a->payload != B200MOE_EP_PAYLOAD_NVFP4 && a->payload != B200MOE_EP_PAYLOAD_MXFP8) return B200MOE_EINVAL;
    if (a->hidden_size % blk != 0 || !fill_peers(sf_p, a->peer_sf, a->world)) return B200MOE_EINVAL;
    const int nsf = a->hidden_size / (a->payload == B200MOE_EP_PAYLOAD_NVFP4 ? 16 : 32);
    if (a->sf_row_stride % 4 != 0 || a->sf_row_stride < ((nsf + 3) & ~3)) return B200MOE_EALIGN;
    if (a->payload == B200MOE_EP_PAYLOAD_NVFP4 && (a->a1_gscale == nullptr || a->gscale_len < 1))
      return B200MOE_EINVAL;
  }
  // one warp per 32 blocks of a row; eight warps per CTA, at most eight CTAs per SM
  const int per = a->payload == B200MOE_EP_PAYLOAD_BF16 ? 8 : (a->payload == B200MOE_EP_PAYLOAD_NVFP4 ? 16 : 32);
  const int64_t items = static_cast<int64_t>(rows) * ((a->hidden_size / per + 31) / 32);
  int grid = static_cast<int>((items + 7) / 8 < 148 * 8 ? (items + 7) / 8 : 148 * 8);
  grid = grid < 1 ? 1 : grid;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->payload == B200MOE_EP_PAYLOAD_NVFP4) launch_dispatch<1>(a, rows_p, sf_p, ids_p, flags_p, grid, st);
  else if (a->payload == B200MOE_EP_PAYLOAD_MXFP8) launch_dispatch<2>(a, rows_p, sf_p, ids_p, flags_p, grid, st);
  else launch_dispatch<0>(a, rows_p, sf_p, ids_p, flags_p, grid, st);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_ep_place_routes(const int32_t* topk_ids, int32_t num_routes, int32_t num_experts,
                                       const int32_t* pattern_rank, const int32_t* pattern_local,
                                       int32_t* dest_rank, int32_t* dest_local, void* stream) {
  if (topk_ids == nullptr || pattern_rank == nullptr || pattern_local == nullptr || dest_rank == nullptr ||
      dest_local == nullptr || num_routes < 0 || num_experts <= 0)
    return B200MOE_EINVAL;
  if (num_routes == 0) return B200MOE_OK;
  int grid = (num_routes + 255) / 256;
  grid = grid > 148 * 4 ? 148 * 4 : grid;
  ep_place_routes_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, num_routes, num_experts, pattern_rank, pattern_local, dest_rank, dest_local);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_permute_packed(const b200moe_packed_args* a, void* stream) {
  if (a == nullptr || a->q_rows == nullptr || a->sf_rows == nullptr || a->scratch == nullptr ||
      a->layout == nullptr)
    return B200MOE_EINVAL;
  if (a->payload != B200MOE_EP_PAYLOAD_NVFP4 && a->payload != B200MOE_EP_PAYLOAD_MXFP8) return B200MOE_EINVAL;
  const int blk = a->payload == B200MOE_EP_PAYLOAD_NVFP4 ? 64 : 32;
  if (a->num_rows < 0 || a->num_experts <= 0 || a->hidden_size <= 0 || a->hidden_size % blk != 0)
    return B200MOE_EINVAL;
  const int nsf = a->hidden_size / (a->payload == B200MOE_EP_PAYLOAD_NVFP4 ? 16 : 32);
  if (a->sf_row_stride % 4 != 0 || a->sf_row_stride < ((nsf + 3) & ~3) ||
      (reinterpret_cast<uintptr_t>(a->q_rows) & 15) != 0 || (reinterpret_cast<uintptr_t>(a->sf_rows) & 3) != 0)
    return B200MOE_EALIGN;
  const b200moe_scratch_layout& L = *a->layout;
  if (a->num_rows > L.rows) return B200MOE_ECAPACITY;
  if (a->num_rows == 0) return B200MOE_OK;
  char* base = static_cast<char*>(a->scratch);
  const int tr = L.tile_rows == 64 ? 64 : 128;
  const int mtiles = (a->num_rows + tr - 1) / tr + (a->num_experts < a->num_rows ? a->num_experts : a->num_rows);
  const int gx = mtiles < L.mtile_cap ? mtiles : L.mtile_cap;
  int gy = (4 * 148 + gx - 1) / gx;
  gy = gy < 2 ? 2 : (gy > 16 ? 16 : gy);
  const dim3 grid(gx, gy);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int32_t* tile_base = reinterpret_cast<const int32_t*>(base + L.tile_base);
  const int32_t* row0 = reinterpret_cast<const int32_t*>(base + L.mtile_row0);
  const int32_t* nrows = reinterpret_cast<const int32_t*>(base + L.mtile_rows);
  const int32_t* sorted = reinterpret_cast<const int32_t*>(base + L.sorted_route_ids);
  uint8_t* q = reinterpret_cast<uint8_t*>(base + L.act_q);
  uint8_t* sf = reinterpret_cast<uint8_t*>(base + L.act_sf);
  if (a->payload == B200MOE_EP_PAYLOAD_NVFP4)
    permute_packed_kernel<1><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(a->q_rows),
        static_cast<const uint8_t*>(a->sf_rows), a->sf_row_stride, a->hidden_size, tile_base, a->num_experts,
        row0, nrows, sorted, q, sf);
  else
    permute_packed_kernel<2><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(a->q_rows),
        static_cast<const uint8_t*>(a->sf_rows), a->sf_row_stride, a->hidden_size, tile_base, a->num_experts,
        row0, nrows, sorted, q, sf);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_ep_signal(void* const* peer_flags, int32_t world, int32_t rank, int32_t epoch,
                                 const int32_t* epoch_dev, void* stream) {
  if (peer_flags == nullptr || world < 1 || world > B200MOE_MAX_RANKS || rank < 0 || rank >= world)
    return B200MOE_EINVAL;
  PeerPtrs flags_p;
  if (!fill_peers(flags_p, peer_flags, world)) return B200MOE_EINVAL;
  ep_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags_p, world, rank, epoch, epoch_dev);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_ep_wait(const int32_t* flags, int32_t world, int32_t epoch,
                               const int32_t* epoch_dev, int32_t* status, int32_t timeout_ms,
                               void* stream) {
  if (flags == nullptr || world < 1 || world > B200MOE_MAX_RANKS || timeout_ms < 0 || timeout_ms > 10000)
    return B200MOE_EINVAL;
  const unsigned long long limit_ns =
      timeout_ms > 0 ? static_cast<unsigned long long>(timeout_ms) * 1000000ull : kWaitLimitNs;
  ep_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, epoch, epoch_dev, status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_ep_combine(const b200moe_ep_combine_args* a, void* stream) {
  if (a == nullptr || a->topk_weights == nullptr || a->out == nullptr || a->scratch == nullptr ||
      a->layout == nullptr)
    return B200MOE_EINVAL;
  if (a->world < 1 || a->world > B200MOE_MAX_RANKS || a->rank < 0 || a->rank >= a->world ||
      a->hidden_size <= 0 || a->hidden_size % 4 != 0 || a->num_topk <= 0 || a->cap_rows <= 0)
    return B200MOE_EINVAL;
  if ((reinterpret_cast<uintptr_t>(a->out) & 7) != 0 || (a->out_row_stride % 4) != 0) return B200MOE_EALIGN;
  if (a->num_tokens * a->num_topk > a->layout->rows) return B200MOE_ECAPACITY;
  PeerPtrs arenas, sig = {};
  if (!fill_peers(arenas, a->peer_scratch, a->world)) return B200MOE_EINVAL;
  if (a->wait_flags != nullptr) {
    if (a->epoch_dev == nullptr || a->timeout_ms < 0 || a->timeout_ms > 10000 ||
        !fill_peers(sig, a->signal_flags, a->world))
      return B200MOE_EINVAL;
  }
  if (a->num_tokens == 0) {
    // a rank without tokens of its own still owes its peers the "my FC2 rows are complete" signal
    // when the hand-shake rides in this call (they would otherwise wait out their limit)
    if (a->wait_flags != nullptr) {
      ep_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(sig, a->world, a->rank, 0, a->epoch_dev);
      return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
    }
    return B200MOE_OK;
  }
  const unsigned long long limit_ns =
      a->timeout_ms > 0 ? static_cast<unsigned long long>(a->timeout_ms) * 1000000ull : kWaitLimitNs;
  const b200moe_scratch_layout& L = *a->layout;
  char* base = static_cast<char*>(a->scratch);
  int ysplit = (2 * 148 + a->num_tokens - 1) / a->num_tokens;
  const int ymax = (a->hidden_size / 4 + 255) / 256;
  ysplit = ysplit < 1 ? 1 : (ysplit > ymax ? ymax : ysplit);
  ep_combine_pull_kernel<<<dim3(a->num_tokens, ysplit), 256, a->num_topk * 16,
                           static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const int32_t*>(base + L.expert_offsets),
      reinterpret_cast<const int32_t*>(base + L.inv_perm), a->topk_weights, arenas,
      a->peer_inv_perm_off, a->peer_routed_off, static_cast<__nv_bfloat16*>(a->out), a->out_row_stride,
      a->world, a->rank, a->num_topk, a->hidden_size, a->cap_rows, a->output_scale, sig, a->wait_flags,
      a->epoch_dev, a->status, limit_ns);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}
