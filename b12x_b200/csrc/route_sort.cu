// Stage 1 (top-k routing) and stage 2 (stable expert sort) of the fused MoE layer.
// Both are tiny integer/compare kernels; the sort is a single-CTA stable counting sort so that
// the permutation is canonical: positions ordered by (expert asc, flat route id asc).
#include "route_shared.cuh"

namespace b200moe {

template <int MODE>
__global__ void __launch_bounds__(128) route_topk_kernel(b200moe_route_args a) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (warp >= a.num_tokens) return;
  route_topk_token<MODE>(a, warp, threadIdx.x & 31);
}

// ------------------------------------------------------------------------------------------
// expert_sort: one CTA, up to 32 warps.  The first `count_warps` warps each own the contiguous
// route range [w*chunk, (w+1)*chunk).  Pass 1 counts per (warp, expert) in shared memory, a scan
// over warps then experts gives every (warp, expert) its first position, pass 2 walks the range
// again 32 routes at a time and ranks equal experts inside the step with match_any, which
// keeps the order of flat route ids.  The block has at least 256 threads whatever the number of
// routes, so that the per-expert tables of a small batch are not walked by a single warp.
// ------------------------------------------------------------------------------------------
constexpr int kSortThreads = 1024;

__global__ void __launch_bounds__(kSortThreads) expert_sort_kernel(
    const int32_t* topk_ids, const int32_t* __restrict__ expert_map,
    int expert_map_len, int rows, int E, int32_t* __restrict__ status,
    int32_t* __restrict__ expert_counts, int32_t* __restrict__ expert_offsets,
    int32_t* __restrict__ tile_base, int32_t* __restrict__ mtile_expert,
    int32_t* __restrict__ mtile_row0, int32_t* __restrict__ mtile_rows,
    int32_t* __restrict__ sorted_route_ids, int32_t* __restrict__ inv_perm, int mtile_cap,
    int tile_rows, int count_warps, const int32_t* wait_flags, const int32_t* wait_epoch_dev, int32_t* wait_status,
    int wait_world, unsigned long long wait_limit_ns) {
  extern __shared__ int32_t smem[];
  if (wait_flags != nullptr) {
    // the ids come from peers: wait (bounded) until every peer has flagged this step
    const int epoch = *wait_epoch_dev;
    if (static_cast<int>(threadIdx.x) < wait_world) {
      unsigned long long t0 = 0;
      uint32_t spins = 0;
      int v;
      while (true) {
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(wait_flags + threadIdx.x) : "memory");
        if (v >= epoch) break;
        if ((++spins & 0x3ffu) == 0) {
          const unsigned long long now = global_timer_ns();
          if (t0 == 0) t0 = now;
          if (now - t0 > wait_limit_ns) {
            if (wait_status != nullptr) {
              atomicCAS(wait_status, 0, 1);
              atomicCAS(wait_status + 1, 0, 16 + static_cast<int>(threadIdx.x));
            }
            break;
          }
        }
      }
    }
    __syncthreads();
  }
  const int nwarps = count_warps;
  int32_t* wcount = smem;                 // [nwarps][E]
  int32_t* etotal = smem + nwarps * E;    // [E]
  int32_t* eoffs = etotal + E;            // [E+1]
  int32_t* tbase = eoffs + (E + 1);       // [E+1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_shift = tile_rows == 64 ? 6 : 7;   // tile_rows is 64 or 128

  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) wcount[i] = 0;
  if (threadIdx.x < 16) status[threadIdx.x] = 0;  // the sort opens every layer call
  __syncthreads();

  // routes per warp, a multiple of 32 so that steps never straddle two warps
  const int chunk = ((rows + nwarps - 1) / nwarps + 31) & ~31;
  const int r_begin = warp < nwarps ? warp * chunk : rows;   // the other warps own no routes
  const int r_end = min(rows, r_begin + chunk);

  // The ids may have been stored by peer GPUs while this kernel was already resident (it then
  // spun on their flags above): they are read past L1 and never through the read-only path.
  auto local_expert = [&](int r) -> int {
    int e = __ldcg(topk_ids + r);
    if (expert_map != nullptr) e = (e >= 0 && e < expert_map_len) ? expert_map[e] : -1;
    return (e >= 0 && e < E) ? e : -1;
  };

  for (int r0 = r_begin; r0 < r_end; r0 += 32) {
    const int r = r0 + lane;
    const int e = (r < r_end) ? local_expert(r) : -1;
    if (e >= 0) atomicAdd(&wcount[warp * E + e], 1);
  }
  __syncthreads();

  // per expert: exclusive scan over warps (turn counts into within-expert bases)
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nwarps; ++w) {
      const int c = wcount[w * E + e];
      wcount[w * E + e] = run;
      run += c;
    }
    etotal[e] = run;
  }
  __syncthreads();
  // scan over experts by one warp: every lane sums a contiguous span, a shuffle scan over the
  // lanes gives each span its base
  if (warp == 0) {
    const int per = (E + 31) >> 5;
    const int e0 = min(E, lane * per), e1 = min(E, e0 + per);
    int cnt = 0, tl = 0;
    for (int e = e0; e < e1; ++e) {
      cnt += etotal[e];
      tl += (etotal[e] + tile_rows - 1) >> tile_shift;
    }
    int pc = cnt, pt = tl;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, pc, d), b = __shfl_up_sync(0xffffffffu, pt, d);
      if (lane >= d) {
        pc += a;
        pt += b;
      }
    }
    int pos = pc - cnt, tiles = pt - tl;
    for (int e = e0; e < e1; ++e) {
      eoffs[e] = pos;
      tbase[e] = tiles;
      pos += etotal[e];
      tiles += (etotal[e] + tile_rows - 1) >> tile_shift;
    }
    if (lane == 31) {
      eoffs[E] = pc;
      tbase[E] = pt;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    expert_offsets[e] = eoffs[e];
    tile_base[e] = tbase[e];
    if (e < E) {
      expert_counts[e] = etotal[e];
      const int nt = (etotal[e] + tile_rows - 1) >> tile_shift;
      for (int t = 0; t < nt; ++t) {
        const int mt = tbase[e] + t;
        if (mt < mtile_cap) {
          mtile_expert[mt] = e;
          mtile_row0[mt] = eoffs[e] + t * tile_rows;
          mtile_rows[mt] = min(tile_rows, etotal[e] - t * tile_rows);
        }
      }
    }
  }

  // pass 2: stable positions
  for (int r0 = r_begin; r0 < r_end; r0 += 32) {
    const int r = r0 + lane;
    const int e = (r < r_end) ? local_expert(r) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (r < r_end) {
      if (e >= 0) {
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int base = wcount[warp * E + e];  // read before the leader bumps it
        const int pos = eoffs[e] + base + rank;
        sorted_route_ids[pos] = r;
        inv_perm[r] = pos;
      } else {
        inv_perm[r] = -1;
      }
    }
    __syncwarp();
    if (e >= 0 && r < r_end && (peers & ((1u << lane) - 1u)) == 0) {
      wcount[warp * E + e] += __popc(peers);
    }
    __syncwarp();
  }
}


// ------------------------------------------------------------------------------------------
// The same stable sort for many routes (tens of thousands and more: prefill batches, the expert
// side of expert parallelism), spread over many CTAs in three launches:
//   count   : CTA c owns routes [c * kChunk, (c + 1) * kChunk); per-expert counts of the chunk go
//             to chunk_counts[c][E] (it also waits for the peers' flags and clears the status block
//             where the single-CTA kernel would)
//   scan    : one CTA turns the chunk counts into per-chunk bases (exclusive over chunks, per
//             expert) and builds the per-expert offsets and the row-tile tables
//   scatter : CTA c walks its chunk again, warp by warp and 32 routes at a time, exactly as the
//             single-CTA kernel does, so that positions keep the order of flat route ids
// ------------------------------------------------------------------------------------------
constexpr int kChunk = 2048;          // routes per CTA
constexpr int kMultiCtaSortRows = 16384;   // from this many routes on the three-launch sort is used
constexpr int kChunkThreads = 256;    // 8 warps x 256 routes

__device__ __forceinline__ int sort_local_expert(const int32_t* topk_ids, const int32_t* expert_map,
                                                 int expert_map_len, int E, int r) {
  int e = __ldcg(topk_ids + r);       // may have been stored by peer GPUs: never the read-only path
  if (expert_map != nullptr) e = (e >= 0 && e < expert_map_len) ? expert_map[e] : -1;
  return (e >= 0 && e < E) ? e : -1;
}

__global__ void __launch_bounds__(kChunkThreads) sort_count_kernel(
    const int32_t* topk_ids, const int32_t* __restrict__ expert_map, int expert_map_len, int rows, int E,
    int32_t* __restrict__ status, int32_t* __restrict__ chunk_counts, const int32_t* wait_flags,
    const int32_t* wait_epoch_dev, int32_t* wait_status, int wait_world, unsigned long long wait_limit_ns) {
  extern __shared__ int32_t smem[];   // [E]
  if (wait_flags != nullptr) {
    const int epoch = *wait_epoch_dev;
    if (static_cast<int>(threadIdx.x) < wait_world) {
      unsigned long long t0 = 0;
      uint32_t spins = 0;
      int v;
      while (true) {
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(wait_flags + threadIdx.x) : "memory");
        if (v >= epoch) break;
        if ((++spins & 0x3ffu) == 0) {
          const unsigned long long now = global_timer_ns();
          if (t0 == 0) t0 = now;
          if (now - t0 > wait_limit_ns) {
            if (wait_status != nullptr) {
              atomicCAS(wait_status, 0, 1);
              atomicCAS(wait_status + 1, 0, 16 + static_cast<int>(threadIdx.x));
            }
            break;
          }
        }
      }
    }
    __syncthreads();
  }
  if (blockIdx.x == 0 && threadIdx.x < 16) status[threadIdx.x] = 0;   // the sort opens every layer call
  for (int i = threadIdx.x; i < E; i += blockDim.x) smem[i] = 0;
  __syncthreads();
  const int r0 = blockIdx.x * kChunk, r1 = min(rows, r0 + kChunk);
  for (int r = r0 + threadIdx.x; r < r1; r += blockDim.x) {
    const int e = sort_local_expert(topk_ids, expert_map, expert_map_len, E, r);
    if (e >= 0) atomicAdd(&smem[e], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) chunk_counts[static_cast<size_t>(blockIdx.x) * E + i] = smem[i];
}

__global__ void __launch_bounds__(1024) sort_scan_kernel(
    int chunks, int E, int32_t* __restrict__ chunk_counts, int32_t* __restrict__ expert_counts,
    int32_t* __restrict__ expert_offsets, int32_t* __restrict__ tile_base, int32_t* __restrict__ mtile_expert,
    int32_t* __restrict__ mtile_row0, int32_t* __restrict__ mtile_rows, int mtile_cap, int tile_rows) {
  extern __shared__ int32_t smem[];
  int32_t* etotal = smem;             // [E]
  int32_t* eoffs = etotal + E;        // [E+1]
  int32_t* tbase = eoffs + (E + 1);   // [E+1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_shift = tile_rows == 64 ? 6 : 7;
  // per expert: exclusive scan over the chunks (counts become the chunk's first position inside the expert)
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      const size_t i = static_cast<size_t>(c) * E + e;
      const int n = chunk_counts[i];
      chunk_counts[i] = run;
      run += n;
    }
    etotal[e] = run;
  }
  __syncthreads();
  if (warp == 0) {
    const int per = (E + 31) >> 5;
    const int e0 = min(E, lane * per), e1 = min(E, e0 + per);
    int cnt = 0, tl = 0;
    for (int e = e0; e < e1; ++e) {
      cnt += etotal[e];
      tl += (etotal[e] + tile_rows - 1) >> tile_shift;
    }
    int pc = cnt, pt = tl;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, pc, d), b = __shfl_up_sync(0xffffffffu, pt, d);
      if (lane >= d) {
        pc += a;
        pt += b;
      }
    }
    int pos = pc - cnt, tiles = pt - tl;
    for (int e = e0; e < e1; ++e) {
      eoffs[e] = pos;
      tbase[e] = tiles;
      pos += etotal[e];
      tiles += (etotal[e] + tile_rows - 1) >> tile_shift;
    }
    if (lane == 31) {
      eoffs[E] = pc;
      tbase[E] = pt;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    expert_offsets[e] = eoffs[e];
    tile_base[e] = tbase[e];
    if (e < E) expert_counts[e] = etotal[e];
  }
  // row tiles: one warp per expert at a time (an expert of a large batch has many tiles)
  for (int e = warp; e < E; e += (blockDim.x >> 5)) {
    const int nt = (etotal[e] + tile_rows - 1) >> tile_shift;
    for (int t = lane; t < nt; t += 32) {
      const int mt = tbase[e] + t;
      if (mt < mtile_cap) {
        mtile_expert[mt] = e;
        mtile_row0[mt] = eoffs[e] + t * tile_rows;
        mtile_rows[mt] = min(tile_rows, etotal[e] - t * tile_rows);
      }
    }
  }
}

__global__ void __launch_bounds__(kChunkThreads) sort_scatter_kernel(
    const int32_t* topk_ids, const int32_t* __restrict__ expert_map, int expert_map_len, int rows, int E,
    const int32_t* __restrict__ chunk_base, const int32_t* __restrict__ expert_offsets,
    int32_t* __restrict__ sorted_route_ids, int32_t* __restrict__ inv_perm) {
  extern __shared__ int32_t smem[];   // [8 warps][E] counts -> bases
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kWarps = kChunkThreads / 32, kPerWarp = kChunk / kWarps;
  for (int i = threadIdx.x; i < kWarps * E; i += blockDim.x) smem[i] = 0;
  __syncthreads();
  const int c0 = blockIdx.x * kChunk;
  const int r_begin = min(rows, c0 + warp * kPerWarp), r_end = min(rows, r_begin + kPerWarp);
  for (int r0 = r_begin; r0 < r_end; r0 += 32) {
    const int r = r0 + lane;
    const int e = r < r_end ? sort_local_expert(topk_ids, expert_map, expert_map_len, E, r) : -1;
    if (e >= 0) atomicAdd(&smem[warp * E + e], 1);
  }
  __syncthreads();
  // per expert: exclusive scan over this CTA's warps, on top of the chunk's base and the expert's offset
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = expert_offsets[e] + chunk_base[static_cast<size_t>(blockIdx.x) * E + e];
    for (int w = 0; w < kWarps; ++w) {
      const int n = smem[w * E + e];
      smem[w * E + e] = run;
      run += n;
    }
  }
  __syncthreads();
  for (int r0 = r_begin; r0 < r_end; r0 += 32) {
    const int r = r0 + lane;
    const int e = r < r_end ? sort_local_expert(topk_ids, expert_map, expert_map_len, E, r) : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    if (r < r_end) {
      if (e >= 0) {
        const int pos = smem[warp * E + e] + __popc(peers & ((1u << lane) - 1u));   // read before the leader bumps it
        sorted_route_ids[pos] = r;
        inv_perm[r] = pos;
      } else {
        inv_perm[r] = -1;
      }
    }
    __syncwarp();
    if (e >= 0 && r < r_end && (peers & ((1u << lane) - 1u)) == 0) smem[warp * E + e] += __popc(peers);
    __syncwarp();
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_route_topk(const b200moe_route_args* a, void* stream) {
  if (a == nullptr || a->logits == nullptr || a->topk_ids == nullptr || a->topk_weights == nullptr)
    return B200MOE_EINVAL;
  if (a->num_experts <= 0 || a->num_experts > 1024) return B200MOE_EINVAL;
  if (a->num_topk <= 0 || a->num_topk > a->num_experts || a->num_topk > 32) return B200MOE_EINVAL;
  if (a->num_tokens < 0) return B200MOE_EINVAL;
  if (a->num_tokens == 0) return B200MOE_OK;
  const int warps_per_block = 4;
  const dim3 grid((a->num_tokens + warps_per_block - 1) / warps_per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (a->mode) {
    case B200MOE_ROUTE_SOFTMAX_TOPK:
      route_topk_kernel<B200MOE_ROUTE_SOFTMAX_TOPK><<<grid, 128, 0, s>>>(*a);
      break;
    case B200MOE_ROUTE_RAW:
      route_topk_kernel<B200MOE_ROUTE_RAW><<<grid, 128, 0, s>>>(*a);
      break;
    case B200MOE_ROUTE_SIGMOID:
      route_topk_kernel<B200MOE_ROUTE_SIGMOID><<<grid, 128, 0, s>>>(*a);
      break;
    default:
      return B200MOE_EINVAL;
  }
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

extern "C" int b200moe_expert_sort(const b200moe_sort_args* a, void* stream) {
  if (a == nullptr || a->topk_ids == nullptr || a->scratch == nullptr || a->layout == nullptr)
    return B200MOE_EINVAL;
  const b200moe_scratch_layout& L = *a->layout;
  const int rows = a->num_tokens * a->num_topk;
  const int E = a->num_experts;
  if (E <= 0 || E > 1024 || rows < 0) return B200MOE_EINVAL;
  if (a->wait_flags != nullptr && (a->wait_epoch_dev == nullptr || a->wait_world < 1 ||
                                   a->wait_world > B200MOE_MAX_RANKS || a->wait_timeout_ms < 0 ||
                                   a->wait_timeout_ms > 10000))
    return B200MOE_EINVAL;
  if (rows > L.rows) return B200MOE_ECAPACITY;
  char* base = static_cast<char*>(a->scratch);
  const unsigned long long limit_ns =
      a->wait_timeout_ms > 0 ? static_cast<unsigned long long>(a->wait_timeout_ms) * 1000000ull : kWaitLimitNs;
  if (rows >= kMultiCtaSortRows) {
    // many routes: count per chunk, scan, scatter (three launches over many CTAs)
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int chunks = (rows + kChunk - 1) / kChunk;
    int32_t* chunk_counts = reinterpret_cast<int32_t*>(base + L.sort_tmp);
    sort_count_kernel<<<chunks, kChunkThreads, static_cast<size_t>(E) * 4, s>>>(
        a->topk_ids, a->expert_map, a->expert_map_len, rows, E, reinterpret_cast<int32_t*>(base + L.status),
        chunk_counts, a->wait_flags, a->wait_epoch_dev, a->wait_status, a->wait_world, limit_ns);
    sort_scan_kernel<<<1, 1024, (3 * static_cast<size_t>(E) + 2) * 4, s>>>(
        chunks, E, chunk_counts, reinterpret_cast<int32_t*>(base + L.expert_counts),
        reinterpret_cast<int32_t*>(base + L.expert_offsets), reinterpret_cast<int32_t*>(base + L.tile_base),
        reinterpret_cast<int32_t*>(base + L.mtile_expert), reinterpret_cast<int32_t*>(base + L.mtile_row0),
        reinterpret_cast<int32_t*>(base + L.mtile_rows), L.mtile_cap, L.tile_rows == 64 ? 64 : 128);
    sort_scatter_kernel<<<chunks, kChunkThreads, static_cast<size_t>(kChunkThreads / 32) * E * 4, s>>>(
        a->topk_ids, a->expert_map, a->expert_map_len, rows, E, chunk_counts,
        reinterpret_cast<const int32_t*>(base + L.expert_offsets), reinterpret_cast<int32_t*>(base + L.sorted_route_ids),
        reinterpret_cast<int32_t*>(base + L.inv_perm));
    return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
  }
  // fewer warps for small problems keeps the shared-memory clear short
  int nwarps = (rows + 31) / 32;
  nwarps = nwarps < 1 ? 1 : (nwarps > 32 ? 32 : nwarps);
  const size_t smem = (static_cast<size_t>(nwarps) * E + 3 * static_cast<size_t>(E) + 2) * 4;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(expert_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (32 * 1024 + 3 * 1024 + 2) * 4) != cudaSuccess)
    return B200MOE_ECUDA;
  expert_sort_kernel<<<1, (nwarps < 8 ? 8 : nwarps) * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      a->topk_ids, a->expert_map, a->expert_map_len, rows, E,
      reinterpret_cast<int32_t*>(base + L.status),
      reinterpret_cast<int32_t*>(base + L.expert_counts),
      reinterpret_cast<int32_t*>(base + L.expert_offsets),
      reinterpret_cast<int32_t*>(base + L.tile_base),
      reinterpret_cast<int32_t*>(base + L.mtile_expert),
      reinterpret_cast<int32_t*>(base + L.mtile_row0),
      reinterpret_cast<int32_t*>(base + L.mtile_rows),
      reinterpret_cast<int32_t*>(base + L.sorted_route_ids),
      reinterpret_cast<int32_t*>(base + L.inv_perm), L.mtile_cap,
      L.tile_rows == 64 ? 64 : 128, nwarps, a->wait_flags, a->wait_epoch_dev, a->wait_status, a->wait_world, limit_ns);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}

// ------------------------------------------------------------------------------------------
// b200moe_expert_sort_static: the same sort kernel, but the tables it needs besides its inputs
// and outputs (status words, per-expert counts, tile tables) live in a fixed array that is part
// of the library image instead of in memory the caller had to allocate.
//
// Who needs this: callers that must not, or cannot, obtain device memory at the point of the
// call -- a serving process that handed the whole GPU to its own pool at start-up, code running
// between a graph capture's begin and end, or a latency-critical loop that has to stay clear of
// the allocator's device-wide synchronisation.  They pass only the routes in and the three
// result arrays out.
//
// The array is one per GPU and shared by every call on that GPU: it still holds what the
// previous call left there (the kernel rewrites everything it later reads, including the status
// words, so nothing has to be cleared by the caller), and two calls whose kernels overlap on the
// GPU -- different streams, no ordering between them -- race on it.  Every GPU on which the
// library is loaded keeps these 32 KiB reserved until the process exits.
//
// The array's name is only a host-side handle, not an address a kernel could use; the device
// address is looked up with cudaGetSymbolAddress the first time the entry point runs on a device
// (with that device current) and cached per device.  Make that first call outside any stream
// capture.  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
// ------------------------------------------------------------------------------------------
namespace b200moe {
constexpr int kStaticSortMaxRoutes = 65536;
constexpr int kStaticSortMaxExperts = 1024;
constexpr int kStaticSortMtileCap = kStaticSortMaxRoutes / 128 + kStaticSortMaxExperts;  // 1536
constexpr int kStaticOffStatus = 0;                                        // int32 words
constexpr int kStaticOffCounts = 16;
constexpr int kStaticOffTileBase = kStaticOffCounts + kStaticSortMaxExperts;
constexpr int kStaticOffMtileExpert = kStaticOffTileBase + kStaticSortMaxExperts + 8;
constexpr int kStaticOffMtileRow0 = kStaticOffMtileExpert + kStaticSortMtileCap;
constexpr int kStaticOffMtileRows = kStaticOffMtileRow0 + kStaticSortMtileCap;
constexpr int kStaticSortWords = kStaticOffMtileRows + kStaticSortMtileCap;
constexpr int kStaticSortBytes = 32 * 1024;
static_assert(kStaticSortWords * 4 <= kStaticSortBytes, "static sort scratch too small");
constexpr int kMaxDevices = 64;
}  // namespace b200moe

static __device__ __align__(256) unsigned char g_static_sort_scratch[b200moe::kStaticSortBytes];
static int32_t* g_static_sort_ptr[b200moe::kMaxDevices] = {};

extern "C" int b200moe_expert_sort_static(const int32_t* topk_ids, const int32_t* expert_map,
                                          int32_t expert_map_len, int32_t num_tokens,
                                          int32_t num_topk, int32_t num_experts,
                                          int32_t* expert_offsets, int32_t* sorted_route_ids,
                                          int32_t* inv_perm, void* stream) {
  if (topk_ids == nullptr || expert_offsets == nullptr || sorted_route_ids == nullptr ||
      inv_perm == nullptr || num_tokens < 0 || num_topk <= 0 || num_experts <= 0)
    return B200MOE_EINVAL;
  const long long rows64 = static_cast<long long>(num_tokens) * num_topk;
  if (rows64 > kStaticSortMaxRoutes || num_experts > kStaticSortMaxExperts)
    return B200MOE_ECAPACITY;  // beyond the fixed size of the built-in array
  const int rows = static_cast<int>(rows64);
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200MOE_ECUDA;
  if (g_static_sort_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_sort_scratch) != cudaSuccess || p == nullptr)
      return B200MOE_ECUDA;
    g_static_sort_ptr[dev] = static_cast<int32_t*>(p);
  }
  int32_t* w = g_static_sort_ptr[dev];
  int nwarps = (rows + 31) / 32;
  nwarps = nwarps < 1 ? 1 : (nwarps > 32 ? 32 : nwarps);
  const size_t smem = (static_cast<size_t>(nwarps) * num_experts + 3 * static_cast<size_t>(num_experts) + 2) * 4;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(expert_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (32 * 1024 + 3 * 1024 + 2) * 4) != cudaSuccess)
    return B200MOE_ECUDA;
  expert_sort_kernel<<<1, (nwarps < 8 ? 8 : nwarps) * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, expert_map, expert_map_len, rows, num_experts, w + kStaticOffStatus,
      w + kStaticOffCounts, expert_offsets, w + kStaticOffTileBase, w + kStaticOffMtileExpert,
      w + kStaticOffMtileRow0, w + kStaticOffMtileRows, sorted_route_ids, inv_perm,
      kStaticSortMtileCap, 128, nwarps, nullptr, nullptr, nullptr, 0, 0ull);
  return cudaGetLastError() == cudaSuccess ? B200MOE_OK : B200MOE_ECUDA;
}
