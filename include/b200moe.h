/*
 * b200moe.h -- C ABI of the B200 (sm_100a) fused mixture-of-experts layer.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, launches on
 * the stream it is given, never allocates, never synchronises, and returns 0 or
 * a negative B200MOE_E* code (see b200moe_strerror).  All data pointers are
 * DEVICE pointers unless a comment says otherwise.  Problems that only the
 * device can see (a bounded wait that ran out) are written to the int32
 * status block at the start of the scratch arena (word 0 != 0).
 *
 * The Python facade `b12x_b200.moe.fused_moe` binds these with ctypes; each
 * comment names the routine of the reference library (b12x 1.2.6, paths
 * relative to its repository root) whose role the entry point takes over.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 4

/* ---- status codes ------------------------------------------------------ */
#define B200MOE_OK            0
#define B200MOE_EINVAL       -1   /* bad argument / unsupported shape          */
#define B200MOE_ECAPACITY    -2   /* problem larger than the planned scratch   */
#define B200MOE_ECUDA        -3   /* a CUDA runtime / driver call failed       */
#define B200MOE_EUNSUPPORTED -4   /* recipe x activation not implemented       */
#define B200MOE_EALIGN       -5   /* pointer or stride not aligned for TMA     */

/* ---- enums (int32 in the structs) --------------------------------------- */
enum { B200MOE_RECIPE_NVFP4 = 0, B200MOE_RECIPE_W4A8_MX = 1, B200MOE_RECIPE_W4A16 = 2 };
enum { B200MOE_ACT_SILU = 0, B200MOE_ACT_RELU2 = 1, B200MOE_ACT_SWIGLUOAI = 2, B200MOE_ACT_SITU = 3 };
/* score function of the router */
enum {
  B200MOE_ROUTE_SOFTMAX_TOPK = 0, /* top-k on raw logits, softmax over the k selected */
  B200MOE_ROUTE_RAW          = 1, /* top-k on raw logits, weights = the logits        */
  B200MOE_ROUTE_SIGMOID      = 2  /* sigmoid scores (+bias for selection), renorm, scale */
};
enum { B200MOE_DT_F32 = 0, B200MOE_DT_BF16 = 1 };

/* ---- device / scratch planning ----------------------------------------- */
typedef struct {
  int32_t sm_major, sm_minor, num_sms, max_smem_optin;
  int64_t total_mem;
} b200moe_device_info;

/* Capacity of one plan.  Mirrors the tensor-free part of the reference's
 * TPMoEScratchCaps (b12x/moe/fused_moe/_impl.py:747-860). */
typedef struct {
  int32_t max_tokens;    /* T capacity                                        */
  int32_t num_topk;      /* k                                                 */
  int32_t num_experts;   /* E (weights held by this rank)                     */
  int32_t hidden_size;   /* K                                                 */
  int32_t intermediate;  /* I                                                 */
  int32_t recipe;        /* B200MOE_RECIPE_*                                  */
  int32_t activation;    /* B200MOE_ACT_*                                     */
  int32_t tile_rows;     /* rows per expert tile: 0 = choose (64 when the plan
                            averages <= 48 routed rows per expert and the
                            recipe has the small-batch kernel, else 128)      */
} b200moe_caps;

/* Byte offsets of every view inside the single uint8 scratch arena.  The
 * reference prices the same kind of layout in _plan_core_workspace
 * (b12x/moe/fused_moe/_impl.py:2525-3090). */
typedef struct {
  int64_t total_nbytes;
  int64_t status;            /* int32[16]; word 0: device error, word 1: where  */
  int64_t expert_counts;     /* int32[E]                                        */
  int64_t expert_offsets;    /* int32[E+1]  first sorted position per expert    */
  int64_t tile_base;         /* int32[E+1]  first row tile per expert           */
  int64_t mtile_expert;      /* int32[mtile_cap]                                */
  int64_t mtile_row0;        /* int32[mtile_cap] sorted position of tile row 0  */
  int64_t mtile_rows;        /* int32[mtile_cap] valid rows (1..tile_rows)      */
  int64_t sorted_route_ids;  /* int32[rows]  flat route id (t*k+slot) per position */
  int64_t inv_perm;          /* int32[rows]  position per flat route id, -1 = dropped */
  int64_t act_q;             /* FC1 input: codes [rows][K/2] (nvfp4) / [rows][K] (mxfp8) / bf16 [rows][K] (w4a16) */
  int64_t act_sf;            /* FC1 input scales, 512-byte atoms [mtile_cap][ceil(K/64|128)]  */
  int64_t mid_q;             /* FC2 input codes  [rows][I/2] / [rows][I] / bf16 [rows][I]     */
  int64_t mid_sf;            /* FC2 input scales atoms                                         */
  int64_t routed;            /* float32 [rows][K] per-route FC2 output (alpha applied)         */
  int64_t sort_tmp;          /* int32 [ceil(rows/2048)][E] per-chunk counts of the multi-CTA sort */
  int32_t rows;              /* T*k                                             */
  int32_t mtile_cap;         /* ceil(rows/tile_rows) + min(E, rows)             */
  int32_t tile_rows;         /* 64 or 128: rows per expert tile of this plan    */
  int32_t reserved;
} b200moe_scratch_layout;

int b200moe_abi_version(void);
const char* b200moe_strerror(int code);
/* HOST pointer out. */
int b200moe_query_device(int device, b200moe_device_info* out);
/* HOST pointers.  Replaces tp_moe_required_nbytes / plan_tp_moe_scratch sizing
 * (b12x/moe/fused_moe/_impl.py:6781-6863). */
int b200moe_scratch_nbytes(const b200moe_caps* caps, b200moe_scratch_layout* out);

/* ---- stage 1: top-k routing -------------------------------------------- */
/* Replaces route_topk / _route_topk_kernel (b12x/moe/_shared/routing.py:8-134)
 * and, for B200MOE_ROUTE_SIGMOID, the host-side scoring of
 * compute_model_gate_routing (benchmarks/benchmark_moe.py:1282-1322).
 * Ties go to the larger expert index; slot order = descending score. */
typedef struct {
  const void* logits;        /* [T][row_stride] f32 or bf16                     */
  const float* bias;         /* [E] added to scores for SELECTION only, or NULL */
  float* topk_logits;        /* [T][k] selected raw logits (may be NULL)        */
  int32_t* topk_ids;         /* [T][k]                                          */
  float* topk_weights;       /* [T][k]                                          */
  int64_t logits_row_stride; /* elements                                        */
  int32_t num_tokens, num_experts, num_topk;
  int32_t logits_dtype;      /* B200MOE_DT_*                                    */
  int32_t mode;              /* B200MOE_ROUTE_*                                 */
  int32_t renormalize;       /* SIGMOID mode: divide by the sum of the k scores */
  float route_scale;         /* SIGMOID mode: final multiplier                  */
  int32_t reserved;
} b200moe_route_args;
int b200moe_route_topk(const b200moe_route_args* a, void* stream);

/* ---- the step in front of stage 1: router gate GEMM + top-k in one launch ---- */
/* Replaces the gate projection and routing of b12x_route_experts_fast
 * (b12x/moe/fused_moe/_impl.py:11356-11490: torch.mm into the route workspace,
 * bias add, then the top-k kernel).  logits_out receives hidden . gate_weight^T
 * (+ gate_bias) in the operands' common type: bf16 when both are bf16, else f32
 * (fp32 accumulation; one rounding for the product, one more for the bias).
 * The router then runs on the stored logits with the semantics of
 * b200moe_route_topk.  `kernel` picks the implementation: AUTO = tensor cores for
 * bf16 operands with E % 16 == 0, E <= 256, K % 8 == 0 and at least 128 tokens,
 * else the CUDA-core kernel. */
enum { B200MOE_GATE_AUTO = 0, B200MOE_GATE_SIMT = 1, B200MOE_GATE_TC = 2 };
typedef struct {
  const void* hidden;        /* [T][hidden_row_stride] bf16 or f32                */
  const void* gate_weight;   /* [E][K] contiguous, bf16 or f32                    */
  const void* gate_bias;     /* [E] bf16 or f32, or NULL                          */
  void* logits_out;          /* [T][E] contiguous, bf16 or f32 (see above)        */
  int32_t* tile_counters;    /* int32[ceil(T/4)] work space (cleared by the call on its stream)  */
  const float* selection_bias; /* SIGMOID mode, [E] or NULL                      */
  float* topk_logits;        /* [T][k] or NULL                                    */
  int32_t* topk_ids;         /* [T][k]                                            */
  float* topk_weights;       /* [T][k]                                            */
  int32_t* status;           /* int32[16] status block for bounded waits, or NULL */
  int64_t hidden_row_stride; /* elements                                          */
  int32_t num_tokens, num_experts, hidden_size, num_topk;
  int32_t hidden_dtype, weight_dtype, bias_dtype; /* B200MOE_DT_*                  */
  int32_t mode;              /* B200MOE_ROUTE_*                                   */
  int32_t renormalize;
  float route_scale;
  int32_t kernel;            /* B200MOE_GATE_*                                    */
  int32_t reserved;
} b200moe_gate_route_args;
int b200moe_gate_route(const b200moe_gate_route_args* a, void* stream);

/* ---- stage 2: expert sort / permutation -------------------------------- */
/* Replaces the histogram / prefix / route-pack phases of the reference's
 * dynamic kernel (b12x/moe/_shared/kernels/dynamic.py:2881-3160) and the W4A16
 * route pack (b12x/moe/_shared/kernels/w4a16/route_pack.py:288-523) with a
 * STABLE counting sort: position order = (expert asc, flat route id asc).
 * Ids outside [0,E) are dropped (inv_perm = -1), like ep_moe's -1 map entries. */
typedef struct {
  const int32_t* topk_ids;   /* [T*k] flat                                      */
  const int32_t* expert_map; /* optional [global E] -> local id or -1, or NULL  */
  void* scratch;             /* arena base                                      */
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  int32_t num_tokens, num_topk, num_experts, expert_map_len;
  /* Optional (expert parallelism over peer memory): before reading topk_ids, wait (bounded) until
   * wait_flags[r] >= *wait_epoch_dev for every r < wait_world -- the ids were stored by peers.
   * On expiry wait_status[0] = 1, wait_status[1] = 16 + r, and the sort goes on. */
  const int32_t* wait_flags; /* or NULL                                         */
  const int32_t* wait_epoch_dev;
  int32_t* wait_status;
  int32_t wait_world, wait_timeout_ms;
} b200moe_sort_args;
int b200moe_expert_sort(const b200moe_sort_args* a, void* stream);

/* The same sort for callers that cannot hand over scratch memory.  It has no counterpart in the
 * reference.  Inputs are the routes (and the optional expert map); outputs are the three arrays
 * the caller passes: expert_offsets [num_experts + 1], sorted_route_ids [num_tokens * num_topk],
 * inv_perm [num_tokens * num_topk].  Everything else the kernel needs sits in a 32 KiB array built
 * into the library (held by every GPU that loads it, until exit), so the call allocates nothing.
 * Limits: num_tokens * num_topk <= 65536 and num_experts <= 1024, otherwise B200MOE_ECAPACITY.
 * The built-in array is shared by all calls on a GPU and keeps the previous call's contents; the
 * kernel rewrites what it reads, but calls whose kernels can overlap on the GPU race on it.
 * The first call on each device looks up the array's device address: make it before any stream
 * capture, with the device current.  The address is cached per device and stays valid for the
 * lifetime of that device's primary context: after cudaDeviceReset (or once the context is
 * destroyed some other way) the library must be reloaded before the next call. */
int b200moe_expert_sort_static(const int32_t* topk_ids, const int32_t* expert_map,
                               int32_t expert_map_len, int32_t num_tokens, int32_t num_topk,
                               int32_t num_experts, int32_t* expert_offsets,
                               int32_t* sorted_route_ids, int32_t* inv_perm, void* stream);

/* ---- stage 3: permute + activation quantisation ------------------------ */
/* Replaces quantize_block_fp4 / quantize_block_fp8_mx as used by the dynamic
 * kernel's route/pack phase (b12x/moe/_shared/kernels/dynamic.py:3059-3850;
 * b12x/_lib/intrinsics.py:5846-5890, 5973-6005), exact ("direct division")
 * variant.  Output rows are in sorted-position order. */
typedef struct {
  const void* x;             /* bf16 [T][x_row_stride]                          */
  const float* a1_gscale;    /* [E] or [1] reciprocal input scale (nvfp4 only)  */
  void* scratch;
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  int64_t x_row_stride;      /* elements                                        */
  int32_t num_tokens, num_topk, num_experts, hidden_size;
  int32_t gscale_len;        /* 1 or E                                          */
  int32_t reserved;
} b200moe_quant_args;
int b200moe_permute_quant_nvfp4(const b200moe_quant_args* a, void* stream);
int b200moe_permute_quant_mxfp8(const b200moe_quant_args* a, void* stream);

/* Expert-parallel dispatch helper: copies the bf16 rows of x into sorted-position order
 * (out_rows[pos] = x[route / k]) and emits each route's destination-local expert id
 * (topk_ids[route] % local_modulus).  The sort that precedes it ranks routes by destination rank.
 * The reference has no token all-to-all (b12x/moe/ep_moe/_impl.py:1-14 replicates the input);
 * this is the send-side packing of the NCCL dispatch that replaces it. */
typedef struct {
  const void* x;             /* bf16 [T][x_row_stride]                          */
  const int32_t* topk_ids;   /* [T*k]                                           */
  void* out_rows;            /* bf16 [rows][hidden]                             */
  int32_t* out_ids;          /* [rows]                                          */
  void* scratch;
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  int64_t x_row_stride;
  int32_t num_tokens, num_topk, num_groups, hidden_size;
  int32_t local_modulus;     /* experts per rank                                */
  int32_t reserved;
} b200moe_gather_args;
int b200moe_gather_rows(const b200moe_gather_args* a, void* stream);

/* ---- stage 4/5: grouped expert GEMMs ----------------------------------- */
/* Weights in the checkpoint layout the reference consumes
 * (b12x/moe/fused_moe/_impl.py:407-431): w13 [E][w1_rows][K/2] u8, two E2M1 per
 * byte (low nibble = even k); block scales 128x4-swizzled
 * [E][pad128(rows)][pad4(cols/16)] E4M3 (nvfp4, w4a16) or plain row-major
 * [E][rows][cols/32] E8M0 (w4a8_mx, converted once at prepare time into the
 * swizzled form); per-expert alphas.  Replaces the FC1 mainloop + activation +
 * requantisation epilogue (dynamic.py:1112-1160, 1467-1497, 6700-6905) and the
 * FC2 mainloop (dynamic.py:6905-7760) of the reference's dynamic kernel, and the
 * W4A16 fused kernel (w4a16/kernel.py:5514). */
typedef struct {
  const uint8_t* w13;        /* FC1 weights                                     */
  const uint8_t* w13_sf;     /* FC1 block scales (swizzled atoms)               */
  const uint8_t* w13_sf_rows;/* nvfp4, gated: the same scales as 128-row atoms in the
                                checkpoint's row order [E][2I/128][K/64][512] (what the
                                small-batch kernel reads), or NULL                 */
  const float* w1_alphas;    /* [E]                                             */
  const uint8_t* w2;         /* FC2 weights [E][K][I/2]                         */
  const uint8_t* w2_sf;
  const float* w2_alphas;    /* [E]                                             */
  const float* a2_gscale;    /* [E] or [1] reciprocal FC2-input scale (nvfp4)   */
  const void* x;             /* bf16 [T][K] (w4a16 only: A operand gathers rows)*/
  void* scratch;
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  float* fc1_tap;            /* optional f32 [rows][w1_rows] alpha-scaled FC1 output (debug tap), or NULL */
  int64_t x_row_stride;
  int32_t num_tokens, num_topk, num_experts, hidden_size, intermediate;
  int32_t recipe, activation;
  int32_t gate_first;        /* 1: FC1 rows [gate;up] (SwiGLU-OAI), 0: [up;gate] */
  int32_t gscale_len;
  float swiglu_limit;        /* <=0: none                                       */
  float swiglu_alpha, swiglu_beta;
  int32_t num_sms;           /* persistent grid size, 0 = all SMs               */
  int32_t sf_e8m0;           /* w4a16 only: 1 = the per-16 block-scale bytes are E8M0
                                (an fp4_e8m0_k32 source, each per-32 scale written twice;
                                b12x/moe/_shared/kernels/w4a16/prepare.py:1289-1325), 0 = E4M3 */
  /* w4a16 only (reference apply_router_weight_on_input, b12x/moe/fused_moe/_impl.py:10631-10634,
   * w4a16/kernel.py:5773): [T*k] router weights; FC1 multiplies every route's rows by its weight
   * before the activation, and the combine must then be called with unit_weights = 1.  NULL = off. */
  const float* fc1_route_weights;
} b200moe_gemm_args;
int b200moe_grouped_gemm1_act(const b200moe_gemm_args* a, void* stream);
int b200moe_grouped_gemm2(const b200moe_gemm_args* a, void* stream);

/* Calibration side channel (w4a16 only, as in the reference: b12x/moe/fused_moe/_impl.py:10601-10604,
 * w4a16/kernel.py:7288-7365).  After b200moe_grouped_gemm1_act of the same arguments:
 * amax[layer_idx][e][0] = max(old, max |x| over the rows routed to local expert e),
 * amax[layer_idx][e][1] = the same over the expert's activated BF16 intermediate rows.
 * amax is a device float32 [layers][num_experts][2] that the caller zeroes once. */
typedef struct {
  void* scratch;
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  float* amax;
  int32_t num_rows;          /* tokens * top_k of the call                      */
  int32_t num_experts, hidden_size, intermediate, layer_idx, recipe;
} b200moe_amax_args;
int b200moe_activation_amax(const b200moe_amax_args* a, void* stream);

/* ---- stage 6: top-k weighted combine ----------------------------------- */
/* Replaces the bf16 atomic scatter / deterministic top-k sum of the reference
 * (dynamic.py:7737-7750; w4a16/kernel.py:7733-7790): out[t] = sum over slots
 * in slot order of w[t,slot] * routed[pos(t,slot)], fp32, one rounding. */
typedef struct {
  const float* topk_weights; /* [T][k]                                          */
  void* out;                 /* bf16 [T][out_row_stride] or f32 when out_f32    */
  void* scratch;
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  int64_t out_row_stride;
  int32_t num_tokens, num_topk, hidden_size;
  int32_t out_f32;           /* 1: write un-rounded float32 (parity tap)        */
  float output_scale;        /* multiplies the sum (routed_scaling_factor), 1.0 = none */
  int32_t unit_weights;      /* 1: every route weighs 1 (the router weights went into FC1) */
} b200moe_combine_args;
int b200moe_combine(const b200moe_combine_args* a, void* stream);
/* out[i] = bf16_rn(in[i]) for `count` contiguous values (count % 8 == 0, both pointers 16-byte
 * aligned): the rounding step of the tensor-parallel layer after the ranks' fp32 partial outputs
 * have been summed (the reference leaves that sum to its caller, b12x/moe/__init__.py:3-8). */
int b200moe_round_rows_bf16(const float* in, void* out, int64_t count, void* stream);

/* ---- expert parallelism over NVLink peer memory --------------------------- */
/* No counterpart in the reference (b12x/moe/ep_moe/_impl.py:1-14 replicates the input on every
 * rank and leaves the sum of partial outputs to the caller).  One process per GPU; the buffers
 * named peer_* live in symmetric memory, i.e. the caller holds a device pointer to every rank's
 * copy.  Rank r owns slots [r*cap_rows, (r+1)*cap_rows) of every receive buffer.  Flags are int32
 * arrays of B200MOE_MAX_RANKS entries per rank, zero before the first step; `epoch` must grow by
 * one per step.  With `epoch_dev` (a device int32, zero before the first step) the epoch lives on
 * the device instead: the dispatch advances it, the signal and the waits read it, and the whole
 * step can be captured once in a CUDA graph and replayed.  The only device-side wait (b200moe_ep_wait) is bounded: after 2 s it writes
 * status[0] = 1, status[1] = 16 + the missing peer, and returns. */
#define B200MOE_MAX_RANKS 16
typedef struct {
  const void* x;             /* bf16 [T][x_row_stride]                          */
  const int32_t* topk_ids;   /* [T*k] global expert ids                         */
  void* peer_rows[B200MOE_MAX_RANKS];   /* bf16 [world*cap_rows][hidden] on each rank   */
  void* peer_ids[B200MOE_MAX_RANKS];    /* int32 [world*cap_rows] on each rank          */
  void* peer_flags[B200MOE_MAX_RANKS];  /* int32 [B200MOE_MAX_RANKS] on each rank       */
  int32_t* done_counter;     /* local int32, zero; the kernel leaves it zero    */
  int32_t* epoch_dev;        /* device epoch counter, or NULL to use `epoch`    */
  void* scratch;             /* home arena, already sorted by destination rank  */
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  int64_t x_row_stride;
  int32_t num_tokens, num_topk, world, rank;
  int32_t hidden_size, local_modulus, cap_rows, epoch;
  /* What crosses the link per route.  BF16: the row as it is (2K bytes; peer_rows is bf16).
   * NVFP4 / MXFP8: the row quantised HERE, with the destination expert's input scale
   * a1_gscale[global expert id] for NVFP4 -- the same bytes the expert rank's permute + quantise
   * stage would produce -- so that 9K/16 resp. K + K/32 bytes cross instead: peer_rows is then
   * u8 [world*cap_rows][K/2 | K], peer_sf u8 [world*cap_rows][sf_row_stride] (row-major scale
   * bytes, zero padded to a multiple of 4), and the expert rank runs b200moe_permute_packed
   * where it would have run b200moe_permute_quant_*. */
  int32_t payload;           /* B200MOE_EP_PAYLOAD_*                            */
  int32_t sf_row_stride;     /* bytes, multiple of 4, >= K/16 resp. K/32        */
  int32_t gscale_len;        /* 1 or the GLOBAL expert count (nvfp4 payload)    */
  int32_t reserved;
  void* peer_sf[B200MOE_MAX_RANKS];
  const float* a1_gscale;    /* reciprocal input scales of ALL experts, global numbering */
  /* cap_rows may be smaller than T*k (a capacity factor).  A route beyond the destination's
   * region is not sent; the kernel then writes status[0] = 1, status[1] = 48 + destination rank.
   * Required when cap_rows < T*k. */
  int32_t* status;
  /* Optional [T*k]: the destination-local expert id of every route (replicated experts, see
   * b200moe_ep_place_routes); NULL = topk_ids[route] % local_modulus. */
  const int32_t* local_ids;
} b200moe_ep_dispatch_args;
enum { B200MOE_EP_PAYLOAD_BF16 = 0, B200MOE_EP_PAYLOAD_NVFP4 = 1, B200MOE_EP_PAYLOAD_MXFP8 = 2 };
/* Pack rows by destination rank, store them and their local expert ids into the peers' receive
 * buffers, mark this rank's unused slots with -1, then raise peer_flags[d][rank] = epoch. */
int b200moe_ep_dispatch(const b200moe_ep_dispatch_args* a, void* stream);

/* Expert replication against skewed routing: a hot expert's weights are also held by other ranks,
 * and its routes are spread over the holders.  pattern_rank / pattern_local are [num_experts][16]:
 * route i (flat index) to expert e goes to rank pattern_rank[e][i % 16], where the expert is local
 * id pattern_local[e][i % 16].  Writes dest_rank[i] (the key of the sort by destination; -1 for an
 * id outside [0, num_experts)) and dest_local[i] (b200moe_ep_dispatch_args.local_ids).  Every copy
 * of an expert computes the same bytes, so the layer's result does not depend on the placement. */
int b200moe_ep_place_routes(const int32_t* topk_ids, int32_t num_routes, int32_t num_experts,
                            const int32_t* pattern_rank, const int32_t* pattern_local,
                            int32_t* dest_rank, int32_t* dest_local, void* stream);

/* Expert side of a quantised dispatch: act_q[pos] = q_rows[sorted_route_ids[pos]] and the scale
 * bytes of that slot filed into the 128x4 scale atoms of the row's tile -- exactly what
 * b200moe_permute_quant_nvfp4 / _mxfp8 leave in the arena, for rows that arrive quantised.
 * Runs after b200moe_expert_sort over the received ids (top-1: route id = slot). */
typedef struct {
  const void* q_rows;        /* u8 [num_rows][K/2 | K], 16-byte aligned         */
  const void* sf_rows;       /* u8 [num_rows][sf_row_stride]                    */
  void* scratch;
  const b200moe_scratch_layout* layout; /* HOST pointer                        */
  int32_t num_rows, num_experts, hidden_size, payload;
  int32_t sf_row_stride, reserved;
} b200moe_packed_args;
int b200moe_permute_packed(const b200moe_packed_args* a, void* stream);
/* Raise peer_flags[d][rank] = epoch on every rank once the stream's earlier work is done. */
int b200moe_ep_signal(void* const* peer_flags /* HOST array */, int32_t world, int32_t rank,
                      int32_t epoch, const int32_t* epoch_dev /* or NULL */, void* stream);
/* Return (on the stream) when flags[r] >= epoch for every r < world, or after the time limit
 * (timeout_ms, 0 = the default 2000, at most 10000). */
int b200moe_ep_wait(const int32_t* flags, int32_t world, int32_t epoch,
                    const int32_t* epoch_dev /* or NULL */, int32_t* status, int32_t timeout_ms,
                    void* stream);

typedef struct {
  const float* topk_weights; /* [T][k]                                          */
  void* out;                 /* bf16 [T][out_row_stride]                        */
  void* peer_scratch[B200MOE_MAX_RANKS]; /* the experts' arenas (all ranks share one layout) */
  void* scratch;             /* home arena                                      */
  const b200moe_scratch_layout* layout; /* HOST pointer, home arena             */
  int64_t peer_inv_perm_off, peer_routed_off;  /* offsets inside an expert arena */
  int64_t out_row_stride;
  int32_t num_tokens, num_topk, world, rank;
  int32_t hidden_size, cap_rows;
  float output_scale;
  int32_t timeout_ms;        /* of the folded wait, 0 = default                 */
  /* Optional: fold "signal + wait" into this launch.  With wait_flags set, the kernel first raises
   * signal_flags[d][rank] = *epoch_dev on every rank d (this rank's FC2 rows are complete), then
   * waits (bounded, status as for b200moe_ep_wait) until wait_flags[r] >= *epoch_dev for all r. */
  void* signal_flags[B200MOE_MAX_RANKS];
  const int32_t* wait_flags; /* this rank's flags, or NULL for no hand-shake    */
  const int32_t* epoch_dev;
  int32_t* status;
} b200moe_ep_combine_args;
/* out[t] = sum over slots of w[t,slot] * (FC2 row of that route, read from the rank that computed
 * it), fp32, slot order, one bf16 rounding: the return all-to-all and the combine in one kernel. */
int b200moe_ep_combine(const b200moe_ep_combine_args* a, void* stream);

/* ---- standalone activation quantisers ------------------------------------- */
/* Replace the reference's quantization.nvfp4 op (b12x/quantization/nvfp4/api.py:24-62; numerics of
 * quantize_grouped_nvfp4_torch, b12x/_lib/intrinsics.py:149-193: sf = e4m3(gs * (amax / 6)),
 * code = e2m1_rte(clamp(x / (sf / gs), +-6)) evaluated with reciprocals) and quantization.mxfp8
 * (b12x/quantization/mxfp8/api.py:5-18; b12x/_lib/intrinsics.py:223-312).  x: bf16 [m][k], row
 * stride in elements.  out_q: [m][k/2] (two E2M1 per byte) resp. values [m][k] E4M3.  Scales: 128x4
 * swizzled atoms [ceil(m/128)][ceil(k/64 | k/128)][512] (out_sf, scale_mma) and row-major UE8M0
 * [m][k/32] (scale_rows); scale_rows / scale_mma may be NULL.  Only bytes of live rows are written. */
int b200moe_quantize_rows_nvfp4(const void* x, int64_t x_row_stride, int32_t m, int32_t k,
                                const float* global_scale /* device, 1 value */, uint8_t* out_q,
                                uint8_t* out_sf, void* stream);
int b200moe_quantize_rows_mxfp8(const void* x, int64_t x_row_stride, int32_t m, int32_t k, uint8_t* values,
                                uint8_t* scale_rows, uint8_t* scale_mma, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
