// Host-only part of the C ABI: scratch layout, device query, error strings and the recipe
// dispatch of the two GEMM entry points.
#include "common.cuh"

namespace b200moe {
int nvfp4_gemm1(const b200moe_gemm_args* a, cudaStream_t stream, int tile_mode);
int nvfp4_gemm2(const b200moe_gemm_args* a, cudaStream_t stream, int tile_mode);
bool tail_split(const b200moe_gemm_args* a);
bool nvfp4_small_batch_ok(const b200moe_gemm_args* a, bool fc1);
int nvfp4_small_gemm1(const b200moe_gemm_args* a, cudaStream_t stream);
int nvfp4_small_gemm2(const b200moe_gemm_args* a, cudaStream_t stream);
bool pair_ok(const b200moe_gemm_args* a, bool fc1);
int nvfp4_pair_gemm1(const b200moe_gemm_args* a, cudaStream_t stream);
int nvfp4_pair_gemm2(const b200moe_gemm_args* a, cudaStream_t stream);
int mx_pair_gemm1(const b200moe_gemm_args* a, cudaStream_t stream);
int mx_pair_gemm2(const b200moe_gemm_args* a, cudaStream_t stream);
int mx_gemm1(const b200moe_gemm_args* a, cudaStream_t stream, int tile_mode);
int mx_gemm2(const b200moe_gemm_args* a, cudaStream_t stream, int tile_mode);
int w4a16_gemm1(const b200moe_gemm_args* a, cudaStream_t stream);
int w4a16_gemm2(const b200moe_gemm_args* a, cudaStream_t stream);
int w4a16_activation_amax(const b200moe_amax_args* a, cudaStream_t stream);
}  // namespace b200moe

static inline int64_t align_up64(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

extern "C" int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }

extern "C" const char* b200moe_strerror(int code) {
  switch (code) {
    case B200MOE_OK: return "ok";
    case B200MOE_EINVAL: return "invalid argument or unsupported shape";
    case B200MOE_ECAPACITY: return "problem exceeds the planned scratch capacity";
    case B200MOE_ECUDA: return "CUDA runtime or driver call failed";
    case B200MOE_EUNSUPPORTED: return "recipe/activation combination not implemented";
    case B200MOE_EALIGN: return "pointer or stride not aligned for TMA / vector access";
    default: return "unknown b200moe status";
  }
}

extern "C" int b200moe_query_device(int device, b200moe_device_info* out) {
  if (out == nullptr) return B200MOE_EINVAL;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return B200MOE_ECUDA;
  out->sm_major = prop.major;
  out->sm_minor = prop.minor;
  out->num_sms = prop.multiProcessorCount;
  out->max_smem_optin = static_cast<int32_t>(prop.sharedMemPerBlockOptin);
  out->total_mem = static_cast<int64_t>(prop.totalGlobalMem);
  return B200MOE_OK;
}

extern "C" int b200moe_scratch_nbytes(const b200moe_caps* c, b200moe_scratch_layout* L) {
  if (c == nullptr || L == nullptr) return B200MOE_EINVAL;
  if (c->max_tokens <= 0 || c->num_topk <= 0 || c->num_experts <= 0 || c->num_experts > 1024 ||
      c->hidden_size <= 0 || c->intermediate <= 0)
    return B200MOE_EINVAL;
  const int64_t T = c->max_tokens, k = c->num_topk, E = c->num_experts;
  const int64_t K = c->hidden_size, I = c->intermediate;
  const int64_t rows64 = T * k;
  if (rows64 > (1 << 30)) return B200MOE_EINVAL;
  if (c->tile_rows != 0 && c->tile_rows != 64 && c->tile_rows != 128) return B200MOE_EINVAL;
  // 64-row tiles go with the small-batch kernel (nvfp4, I a multiple of 128): chosen when the plan
  // averages at most 48 routed rows per expert, or asked for by the caller
  const bool small_ok = c->recipe == B200MOE_RECIPE_NVFP4 && I % 128 == 0 && K % 64 == 0;
  int64_t tile_rows = c->tile_rows;
  if (tile_rows == 0) tile_rows = (small_ok && rows64 <= 48 * E) ? 64 : 128;
  if (tile_rows == 64 && !small_ok) tile_rows = 128;
  const int64_t mtile_cap = (rows64 + tile_rows - 1) / tile_rows + (E < rows64 ? E : rows64);
  int64_t act_row = 0, mid_row = 0, act_atoms = 0, mid_atoms = 0;
  switch (c->recipe) {
    case B200MOE_RECIPE_NVFP4:
      if (K % 64 != 0 || I % 64 != 0) return B200MOE_EINVAL;
      act_row = K / 2; mid_row = I / 2;
      act_atoms = (K + 63) / 64; mid_atoms = (I + 63) / 64;
      break;
    case B200MOE_RECIPE_W4A8_MX:
      if (K % 32 != 0 || I % 32 != 0) return B200MOE_EINVAL;
      act_row = K; mid_row = I;
      act_atoms = (K + 127) / 128; mid_atoms = (I + 127) / 128;
      break;
    case B200MOE_RECIPE_W4A16:
      if (K % 32 != 0 || I % 32 != 0) return B200MOE_EINVAL;
      act_row = K * 2; mid_row = I * 2;   // bf16 rows in sorted order, bf16 intermediate
      break;
    default:
      return B200MOE_EINVAL;
  }
  int64_t off = 0;
  auto take = [&](int64_t nbytes) {
    const int64_t o = off;
    off = align_up64(off + nbytes, 1024);
    return o;
  };
  L->status = take(16 * 4);
  L->expert_counts = take(E * 4);
  L->expert_offsets = take((E + 1) * 4);
  L->tile_base = take((E + 1) * 4);
  L->mtile_expert = take(mtile_cap * 4);
  L->mtile_row0 = take(mtile_cap * 4);
  L->mtile_rows = take(mtile_cap * 4);
  L->sorted_route_ids = take(rows64 * 4);
  L->inv_perm = take(rows64 * 4);
  L->act_q = take(rows64 * act_row);
  L->act_sf = take(mtile_cap * act_atoms * 512);
  L->mid_q = take(rows64 * mid_row);
  L->mid_sf = take(mtile_cap * mid_atoms * 512);
  L->routed = take(rows64 * K * 4);
  L->sort_tmp = take(((rows64 + 2047) / 2048) * E * 4);
  L->total_nbytes = off;
  L->rows = static_cast<int32_t>(rows64);
  L->mtile_cap = static_cast<int32_t>(mtile_cap);
  L->tile_rows = static_cast<int32_t>(tile_rows);
  L->reserved = 0;
  return B200MOE_OK;
}

static int check_gemm_args(const b200moe_gemm_args* a) {
  if (a == nullptr || a->scratch == nullptr || a->layout == nullptr || a->w13 == nullptr ||
      a->w2 == nullptr || a->w1_alphas == nullptr || a->w2_alphas == nullptr)
    return B200MOE_EINVAL;
  if (a->num_tokens < 0 || a->num_topk <= 0 || a->num_experts <= 0) return B200MOE_EINVAL;
  if (a->num_tokens * a->num_topk > a->layout->rows) return B200MOE_ECAPACITY;
  if (a->activation < B200MOE_ACT_SILU || a->activation > B200MOE_ACT_SITU)
    return B200MOE_EINVAL;
  return B200MOE_OK;
}

extern "C" int b200moe_grouped_gemm1_act(const b200moe_gemm_args* a, void* stream) {
  const int rc = check_gemm_args(a);
  if (rc != B200MOE_OK) return rc;
  if (a->num_tokens == 0) return B200MOE_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (a->recipe) {
    case B200MOE_RECIPE_NVFP4:
      if (a->w13_sf == nullptr || a->a2_gscale == nullptr) return B200MOE_EINVAL;
      if (b200moe::nvfp4_small_batch_ok(a, /*fc1=*/true)) return b200moe::nvfp4_small_gemm1(a, s);
      if (b200moe::pair_ok(a, /*fc1=*/true)) {
        // full pairs of row tiles on CTA pairs, then the left-over row tiles on single CTAs
        const int rc1 = b200moe::nvfp4_pair_gemm1(a, s);
        return (rc1 != B200MOE_OK || !b200moe::tail_split(a)) ? rc1 : b200moe::nvfp4_gemm1(a, s, 1);
      }
      return b200moe::nvfp4_gemm1(a, s, 0);
    case B200MOE_RECIPE_W4A8_MX:
      if (b200moe::pair_ok(a, /*fc1=*/true)) {
        const int rc1 = b200moe::mx_pair_gemm1(a, s);
        return (rc1 != B200MOE_OK || !b200moe::tail_split(a)) ? rc1 : b200moe::mx_gemm1(a, s, 1);
      }
      return b200moe::mx_gemm1(a, s, 0);
    case B200MOE_RECIPE_W4A16:
      return b200moe::w4a16_gemm1(a, s);
    default:
      return B200MOE_EINVAL;
  }
}

extern "C" int b200moe_grouped_gemm2(const b200moe_gemm_args* a, void* stream) {
  const int rc = check_gemm_args(a);
  if (rc != B200MOE_OK) return rc;
  if (a->num_tokens == 0) return B200MOE_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (a->recipe) {
    case B200MOE_RECIPE_NVFP4:
      if (a->w2_sf == nullptr) return B200MOE_EINVAL;
      if (b200moe::nvfp4_small_batch_ok(a, /*fc1=*/false)) return b200moe::nvfp4_small_gemm2(a, s);
      if (b200moe::pair_ok(a, /*fc1=*/false)) {
        const int rc1 = b200moe::nvfp4_pair_gemm2(a, s);
        return (rc1 != B200MOE_OK || !b200moe::tail_split(a)) ? rc1 : b200moe::nvfp4_gemm2(a, s, 1);
      }
      return b200moe::nvfp4_gemm2(a, s, 0);
    case B200MOE_RECIPE_W4A8_MX:
      if (b200moe::pair_ok(a, /*fc1=*/false)) {
        const int rc1 = b200moe::mx_pair_gemm2(a, s);
        return (rc1 != B200MOE_OK || !b200moe::tail_split(a)) ? rc1 : b200moe::mx_gemm2(a, s, 1);
      }
      return b200moe::mx_gemm2(a, s, 0);
    case B200MOE_RECIPE_W4A16:
      return b200moe::w4a16_gemm2(a, s);
    default:
      return B200MOE_EINVAL;
  }
}

extern "C" int b200moe_activation_amax(const b200moe_amax_args* a, void* stream) {
  if (a == nullptr || a->scratch == nullptr || a->layout == nullptr || a->amax == nullptr) return B200MOE_EINVAL;
  if (a->recipe != B200MOE_RECIPE_W4A16) return B200MOE_EUNSUPPORTED;
  if (a->num_rows < 0 || a->num_experts <= 0 || a->layer_idx < 0 || a->hidden_size <= 0 || a->intermediate <= 0 ||
      a->hidden_size % 8 != 0 || a->intermediate % 8 != 0)
    return B200MOE_EINVAL;
  if (a->num_rows > a->layout->rows) return B200MOE_ECAPACITY;
  if (a->num_rows == 0) return B200MOE_OK;
  return b200moe::w4a16_activation_amax(a, static_cast<cudaStream_t>(stream));
}
