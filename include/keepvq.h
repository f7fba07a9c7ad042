/*
 * keepvq.h - C ABI of libkeepvq.so: KEEP's E8P lattice codes decoded and applied on an
 * NVIDIA B200 (sm_100a) for RAMP's routed expert path.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its comment says "host".  Callers own all
 *     memory; no entry point allocates, frees or synchronises.  Work is enqueued on `stream`
 *     (a cudaStream_t passed as void*; NULL is the legacy default stream).
 *   - Every entry point returns KEEPVQ_OK (0) or a negative keepvq_status.  Bad shapes, dtypes
 *     or alignment are reported that way; nothing aborts.  keepvq_status_string() names a code.
 *   - Tensors are dense and row-major.  `codes` is [experts, out_dim, in_dim/8]: uint16 for
 *     16-bit E8P codes, uint8 for the 8-bit E8 residual.  `scales` is
 *     [experts, out_dim, groups]; scale g of a row covers in_dim/groups consecutive inputs.
 *   - A codebook is the 256-word packed table of the reference (src/keep/vq/e8.py:127-139
 *     for E8P, :165-174 for the residual).  It is read on every call; nothing is cached
 *     between calls, so a caller may overwrite codes, scales or tables between calls.
 *
 * Citations (file:line) name the interface of the reference (jackmaxwil/keep) that an entry
 * point stands in for.
 */
#ifndef KEEPVQ_H
#define KEEPVQ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KEEPVQ_ABI_VERSION 3

typedef enum keepvq_status {
  KEEPVQ_OK = 0,
  KEEPVQ_ERR_NULL = -1,        /* a required pointer is NULL */
  KEEPVQ_ERR_SHAPE = -2,       /* sizes are inconsistent (in_dim % 8, in_dim % groups, ...) */
  KEEPVQ_ERR_DTYPE = -3,       /* unknown dtype tag or code width */
  KEEPVQ_ERR_ALIGN = -4,       /* a pointer or row pitch misses the alignment the kernel needs */
  KEEPVQ_ERR_UNSUPPORTED = -5, /* valid, but no kernel serves this combination */
  KEEPVQ_ERR_LAUNCH = -6,      /* the CUDA runtime refused the launch; see keepvq_last_cuda_error */
  KEEPVQ_ERR_CAPACITY = -7     /* a fixed-size buffer is too small for the request */
} keepvq_status;

typedef enum keepvq_dtype {
  KEEPVQ_F32 = 0,
  KEEPVQ_F16 = 1,
  KEEPVQ_BF16 = 2
} keepvq_dtype;

/* Layout of the 8-bit residual's table argument. */
typedef enum keepvq_table_layout {
  KEEPVQ_TABLE_PACKED = 0,      /* uint32[256], nibble d = dim d        (e8.py:165-174)          */
  KEEPVQ_TABLE_PAIR_PACKED = 1, /* uint32[256], nibbles k,k+4 = dims 2k,2k+1 (e8_1bit_m1.py:25-33) */
  KEEPVQ_TABLE_HALF2_PAIRS = 2  /* uint32[256][4], fp16 bits of dims 2k|2k+1 (e8p_nested_m1.py:29-36) */
} keepvq_table_layout;

/* Route index that means "this route has no residual" (e8_1bit_m1.py:22). */
#define KEEPVQ_NO_RESIDUAL 0xFFFFFFFFu

int keepvq_abi_version(void);
const char* keepvq_status_string(int status);
/* Text of the last CUDA runtime error an entry point saw on this host thread ("" if none). */
const char* keepvq_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * Code-to-weight decode.  Stands in for keep.vq.e8.decode_weight_matrix
 * (src/keep/vq/e8.py:542-571): out[r, 8c+d] = decode(codes[r, c])[d] * scales[r, c / (cw/groups)].
 * The product is exact in fp32, so an fp32 output is bit-identical to the reference.
 * ------------------------------------------------------------------------------------------ */
typedef struct keepvq_decode_args {
  const void* codes;        /* [rows, codewords] uint16 (code_bits 16) or uint8 (8) */
  int32_t code_bits;        /* 8 or 16 */
  const void* scales;       /* [rows, groups], or NULL for unit scales */
  int32_t scales_dtype;     /* keepvq_dtype */
  const uint32_t* codebook; /* uint32[256], KEEPVQ_TABLE_PACKED */
  int64_t rows;
  int64_t codewords;        /* in_dim / 8 */
  int64_t groups;
  void* out;                /* [rows, codewords*8] */
  int32_t out_dtype;        /* keepvq_dtype */
} keepvq_decode_args;

int keepvq_decode_weights(const keepvq_decode_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Routed matrix-vector products, few activation rows.  One entry point behind
 *   vq_qmv                  src/ramp/kernels/vq_qmv.py:163-232    (experts=1, routes=1)
 *   vq_qmm                  src/ramp/kernels/vq_qmm.py:93-152     (experts=1, rhs=0, lhs=row)
 *   gather_vqmm (direct)    src/ramp/ops/vq_switch.py:916-932, kernels/gather_vqmm.py:473-594
 *   e8p_m1_token_layout / e8p_m1_per_route          src/ramp/kernels/e8p_m1.py:134-183
 *   e8_1bit_m1_token_layout / _per_route            src/ramp/kernels/e8_1bit_m1.py:76-97
 *   e8p_nested_m1_token_layout / _per_route         src/ramp/kernels/e8p_nested_m1.py:90-112
 *
 * out[r, n] = sum_k W[rhs[r]][n, k] * x[row(r), k], one rounding to out_dtype.
 * row(r) = lhs[r] if lhs != NULL else r / x_div.  With a residual,
 * W = base + residual[hot_of_slot[rhs[r]]] for slots whose entry is not KEEPVQ_NO_RESIDUAL;
 * base and residual are accumulated apart and added once in fp32.  A route whose rhs is
 * KEEPVQ_NO_RESIDUAL, or any other value >= experts, writes zeros (the 8-bit kernels of the
 * reference do the same for NO_RESIDUAL, e8_1bit_m1.metal:25-32; here it holds for every code
 * width, so a masked router pick is safe).  Activation row indices are not range-checked
 * (vq_switch.py:637,646-648).
 * Arithmetic: every weight is a multiple of 1/4, so the kernel works on the integers 4w and on
 * activations quantised per row to fixed point with a power-of-two step: 16 bits for fp16 / bf16
 * rows (error at most 2^-16 of the row's largest magnitude per element), 24 bits for fp32 rows
 * (2^-24).  The integer sums are exact; scales are applied in fp32 per scale group.  Any table is
 * accepted: one whose nibbles are all odd (the E8P table) takes a faster decode.
 * ------------------------------------------------------------------------------------------ */
typedef struct keepvq_matvec_args {
  const void* x;            /* [x_rows, in_dim] */
  int32_t x_dtype;          /* keepvq_dtype */
  int64_t x_rows;
  const void* codes;        /* [experts, out_dim, in_dim/8] */
  int32_t code_bits;        /* 8 or 16 */
  const void* scales;       /* [experts, out_dim, groups] */
  int32_t scales_dtype;
  int64_t experts;
  int64_t out_dim;
  int64_t in_dim;
  int64_t groups;
  const uint32_t* codebook; /* table of `codes` */
  int32_t codebook_layout;  /* keepvq_table_layout; 16-bit codes take KEEPVQ_TABLE_PACKED only */
  const uint32_t* rhs;      /* [routes] first-axis index into codes per route */
  const int32_t* lhs;       /* [routes] activation row per route, or NULL */
  int32_t x_div;            /* used when lhs == NULL: top_k (token layout) or 1 (per route) */
  int64_t routes;
  /* optional nested residual; res_codes == NULL turns it off */
  const uint8_t* res_codes;    /* [res_rows, out_dim, in_dim/8] */
  const void* res_scales;      /* [res_rows, out_dim, res_groups] */
  int32_t res_scales_dtype;
  int64_t res_rows;
  int64_t res_groups;
  const uint32_t* res_table;   /* KEEPVQ_TABLE_HALF2_PAIRS */
  const uint32_t* hot_of_slot; /* [experts] */
  void* out;                /* [routes, out_dim] */
  int32_t out_dtype;
} keepvq_matvec_args;

int keepvq_routed_matvec(const keepvq_matvec_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Router with routed residency.  Two launches that together stand in for
 *   Gate.forward           tests/fixtures/v41_reference/model.py:811-829
 *   gate_masked            scripts/runpod/v41_reap/local_eval.py:69-90
 *   the fused dual top-k   scripts/v41_build/omlx_lattice.py:77-104,333-338
 *   the admission test     scripts/v41_build/omlx_routed.py:184-203
 * ------------------------------------------------------------------------------------------ */
typedef enum keepvq_score_func {
  KEEPVQ_SCORE_SOFTMAX = 0,
  KEEPVQ_SCORE_SIGMOID = 1,
  KEEPVQ_SCORE_SQRT_SOFTPLUS = 2
} keepvq_score_func;

/* logits[t, e] = (x[t] . router_w[e]) / gate_temp in fp32. */
typedef struct keepvq_router_logits_args {
  const void* x;        /* [tokens, hidden] */
  int32_t x_dtype;
  const void* router_w; /* [pool, hidden] */
  int32_t router_dtype;
  int64_t tokens;
  int64_t pool;
  int64_t hidden;       /* multiple of 8 */
  float gate_temp;
  float* logits;        /* [tokens, pool] */
} keepvq_router_logits_args;

int keepvq_router_logits(const keepvq_router_logits_args* args, void* stream);

/* One router evaluation, two selections.
 *   scores = f(logits)
 *   served = top_k(scores + served_bias);  demand = top_k(scores + pool_bias)
 * served_bias[e] <= -1e29 (or -inf) marks expert e absent: it is never served while a resident
 * remains, and a pick that lands on one anyway (fewer residents than top_k) gets weight 0 and
 * slot KEEPVQ_NO_RESIDUAL.  Served weights are raw scores, renormalised over the served picks
 * when norm_topk_prob != 0, times route_scale.  Demand keeps raw scores.  admit[t, j] is the
 * demanded expert when it is absent and its demand weight, renormalised over the k demanded
 * scores and times route_scale, is >= tau; otherwise -1.  Ties go to the lowest expert id;
 * picks are in descending biased score. */
typedef struct keepvq_routed_topk_args {
  const float* logits;       /* [tokens, pool] */
  int64_t tokens;
  int64_t pool;
  int32_t top_k;             /* <= 16 */
  int32_t score_func;        /* keepvq_score_func */
  int32_t norm_topk_prob;
  float route_scale;
  float tau;
  const float* served_bias;  /* [pool] or NULL (all resident, zero bias) */
  const float* pool_bias;    /* [pool] or NULL (zero) */
  const uint32_t* slot_of;   /* [pool] expert -> slot, or NULL (slot = expert) */
  float* scores;             /* [tokens, pool] optional output, may be NULL */
  uint32_t* served_expert;   /* [tokens, top_k] */
  uint32_t* served_slot;     /* [tokens, top_k] */
  float* served_weight;      /* [tokens, top_k] */
  uint32_t* want;            /* [tokens, top_k] */
  float* want_score;         /* [tokens, top_k] */
  int32_t* admit;            /* [tokens, top_k] optional, may be NULL */
} keepvq_routed_topk_args;

int keepvq_routed_topk(const keepvq_routed_topk_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * One routed MoE layer at decode, as a single launch sequence with no host round trip:
 * router logits -> dual top-k -> gate/up projections + SwiGLU * gate weight -> down projection
 * -> fp32 sum over the k served experts.  Stands in for the decode step
 *   scripts/v41_build/omlx_lattice.py:327-371   (served path, rounding points)
 *   scripts/runpod/v41_reap/local_eval.py:508-585, tests/fixtures/v41_reference/model.py:843-853
 *   src/ramp/models/glm4_moe_adapter.py:367-372 (QuantizedVQSwitchGLU) + the weighted sum
 *
 * Per token t and served pick j (slot s, weight g):
 *   G = round(W1[s] x_t), U = round(W3[s] x_t)       rounded to the activation dtype
 *   h = round(silu(G) * U * g)                        (optional clamp: G <= limit, |U| <= limit)
 *   y_t += float(round(W2[s] h))                      fp32 sum in pick order
 *   out_t = round(y_t)
 * W = base codes (+ the 8-bit residual of slots that hot_of_slot marks, when given).
 * ------------------------------------------------------------------------------------------ */
typedef struct keepvq_expert_weights {
  const uint16_t* codes;    /* [slots, out_dim, in_dim/8] */
  const void* scales;       /* [slots, out_dim, groups] */
  int64_t groups;
  const uint8_t* res_codes; /* [res_rows, out_dim, in_dim/8] or NULL */
  const void* res_scales;   /* [res_rows, out_dim, res_groups] */
  int64_t res_groups;
} keepvq_expert_weights;

typedef struct keepvq_moe_layer_args {
  const void* x;             /* [tokens, hidden] */
  int32_t x_dtype;           /* keepvq_dtype; also the dtype of `out` */
  int64_t tokens;
  int64_t hidden;
  int64_t inter;
  /* router */
  const void* router_w;      /* [pool, hidden] */
  int32_t router_dtype;
  int64_t pool;
  int32_t top_k;
  int32_t score_func;
  int32_t norm_topk_prob;
  float gate_temp;
  float route_scale;
  float tau;
  const float* served_bias;  /* see keepvq_routed_topk_args */
  const float* pool_bias;
  const uint32_t* slot_of;
  /* experts, indexed by slot */
  int64_t slots;
  keepvq_expert_weights w1;  /* gate  [slots, inter, hidden/8]  */
  keepvq_expert_weights w3;  /* up    [slots, inter, hidden/8]  */
  keepvq_expert_weights w2;  /* down  [slots, hidden, inter/8]  */
  int32_t scales_dtype;      /* dtype of every scales / res_scales array */
  const uint32_t* codebook;  /* E8P packed abs grid */
  int64_t res_rows;          /* 0 when no residual tier */
  const uint32_t* res_table; /* KEEPVQ_TABLE_HALF2_PAIRS */
  const uint32_t* hot_of_slot; /* [slots] */
  float swiglu_limit;        /* 0 = plain SwiGLU */
  int32_t codebook_all_odd;  /* caller vouches that every nibble of `codebook` is odd (the E8P table
                                is); allows the int8 tensor-core kernels.  0 = general kernels */
  /* outputs */
  void* out;                 /* [tokens, hidden] */
  uint32_t* served_expert;   /* [tokens, top_k] */
  uint32_t* served_slot;     /* [tokens, top_k] */
  float* served_weight;      /* [tokens, top_k] */
  uint32_t* want;            /* [tokens, top_k] */
  float* want_score;         /* [tokens, top_k] */
  int32_t* admit;            /* [tokens, top_k] or NULL */
  /* scratch, at least keepvq_moe_layer_workspace_bytes(), 256-byte aligned */
  void* workspace;
  int64_t workspace_bytes;
  /* Live routes the caller expects among tokens * top_k, or 0 for "all of them".  A caller whose
     rows are mostly dead (the fixed-capacity blocks of an expert-parallel exchange) says so here;
     it only picks between kernel families (few or many routes per expert), never the result. */
  int64_t expected_routes;
  /* [tokens, hidden] fp32, 16-byte aligned, or NULL: the shared expert's output before rounding.
     The pick sum adds it in fp32 after the picks and rounds once,
     out[t] = round(sum_j down[t, j] + shared[t]), which is what the reference's shared down kernel
     does from the other side (it adds the routed sum to its own dot and rounds to bf16,
     scripts/v41_build/omlx_lattice.py:372-389). */
  const float* shared;
} keepvq_moe_layer_args;

/* Bytes of scratch keepvq_moe_decode_layer needs for these sizes (host arithmetic only). */
int64_t keepvq_moe_layer_workspace_bytes(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k);
int keepvq_moe_decode_layer(const keepvq_moe_layer_args* args, void* stream);
/* Byte offset, inside the scratch, of an int32 the tcgen05 kernels set to 1 when one of their
 * bounded waits expires (they then stop, free their tensor memory and return; the call's outputs
 * are invalid).  The library clears it at the start of a call that can set it and never reads it
 * back itself: a host that wants to know copies the word out after the call.  No counterpart in
 * the reference. */
int64_t keepvq_moe_layer_status_offset(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k);

/* Byte offset, inside the scratch, of the per-route outputs [tokens * top_k, hidden] (activation
 * dtype) that the pick sum adds up: after the DOWN stage, row t * top_k + j holds round(W2 h) of
 * token t's pick j (rows of picks without a slot are not written).  A caller that wants the
 * routes' outputs unsummed, as QuantizedVQSwitchGLU returns them
 * (src/ramp/models/glm4_moe_adapter.py:367-372), runs the stages up to DOWN and reads them here. */
int64_t keepvq_moe_layer_route_output_offset(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k);
/* Likewise the routes' hidden rows h = round(silu(G) * U * g), [tokens * top_k, inter], that the
 * GATE_UP stage leaves for the DOWN stage (the activation step of the reference's switch MLP,
 * glm4_moe_adapter.py:363-364, with the gate weight applied as omlx_lattice.py:368 does). */
int64_t keepvq_moe_layer_route_hidden_offset(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k);

/* The same sequence, cut into stages: run the stages named in `stages` (a mask) on the same
 * arguments and scratch.  A later stage reads what earlier ones left in the outputs and the
 * scratch, so a profiler or benchmark can replay one stage after a full run.  No counterpart in
 * the reference; its stages are separate MLX ops (scripts/v41_build/omlx_lattice.py:332-371). */
typedef enum keepvq_moe_stage {
  KEEPVQ_STAGE_ROUTER = 1,   /* logits + dual top-k */
  KEEPVQ_STAGE_PREPARE = 2,  /* route grouping + activation quantisation (tensor-core kernels only) */
  KEEPVQ_STAGE_GATE_UP = 4,  /* gate, up, SwiGLU * weight */
  KEEPVQ_STAGE_DOWN = 8,     /* down projection */
  KEEPVQ_STAGE_COMBINE = 16, /* sum over the k picks */
  KEEPVQ_STAGE_ALL = 31
} keepvq_moe_stage;
int keepvq_moe_decode_stages(const keepvq_moe_layer_args* args, int32_t stages, void* stream);

/* ------------------------------------------------------------------------------------------
 * Residency bookkeeping for one layer, on the device: admission of strongly demanded absent
 * experts, routing of experts whose bytes have landed, least-recently-strongly-demanded eviction.
 * Stands in for Cache.begin / harvest / install / evict (scripts/v41_build/omlx_routed.py:167-247),
 * which the reference runs in host Python; here the router tables (served_bias, slot_of) are
 * updated in place on the stream, so the next decode call sees them with no host round trip.
 *
 * One tick consumes the demand (want, want_score) of call `call` while call `step` is being built
 * (step - call = the reference's lag):
 *   g = want_score / (sum over the k picks + 1e-20) * route_scale, in double;  strong = g >= tau
 *   wanted[e] = max g over strong picks;   stats.resident += demanded picks that are resident
 *   install: every reading expert whose `landed` flag is set is routed (served_bias <- pool_bias,
 *            slot_of, slot_expert, last_use[slot] = step)
 *   wanted and resident -> last_use[slot] = call;  wanted, absent, not reading -> candidate
 *   cooling slots whose stamp <= call move to the end of the free list, in order
 *   candidates in descending (g, expert): pop a slot from the END of the free list and start a
 *            read (action ADMIT), or count no_slot
 *   evict: while spare - free - cooling > 0, the routed slot with the smallest (last_use, slot)
 *            whose expert is not wanted is unrouted (served_bias <- -1e30, slot_of <- absent,
 *            last_use <- +inf, appended to cooling with stamp `step`)
 * The host's part: set landed[e] when a read finishes, clear it once it sees the ROUTE action;
 * start a read for every ADMIT action.  Actions are appended to `actions` as (kind, expert, slot).
 * ------------------------------------------------------------------------------------------ */
typedef enum keepvq_residency_action {
  KEEPVQ_ACTION_ROUTE = 1,
  KEEPVQ_ACTION_UNROUTE = 2,
  KEEPVQ_ACTION_ADMIT = 3
} keepvq_residency_action;

typedef enum keepvq_residency_stat {
  KEEPVQ_STAT_CALLS = 0, KEEPVQ_STAT_TOKENS, KEEPVQ_STAT_DEMAND, KEEPVQ_STAT_RESIDENT, KEEPVQ_STAT_WANTED,
  KEEPVQ_STAT_ADMITTED, KEEPVQ_STAT_INSTALLED, KEEPVQ_STAT_EVICTED, KEEPVQ_STAT_BYTES, KEEPVQ_STAT_NO_SLOT,
  KEEPVQ_STAT_COUNT
} keepvq_residency_stat;

typedef struct keepvq_residency_args {
  /* state of the layer, owned by the caller, updated in place */
  int32_t* slot_expert;     /* [slots] expert in the slot, -1 = unrouted */
  uint32_t* slot_of;        /* [pool]  slot of the expert, KEEPVQ_NO_RESIDUAL = absent */
  float* served_bias;       /* [pool]  the router's served bias (see keepvq_routed_topk_args) */
  const float* pool_bias;   /* [pool]  or NULL (zero) */
  double* last_use;         /* [slots] */
  int32_t* free_list;       /* [slots] */
  int32_t* cooling;         /* [slots][2] (slot, stamp) */
  int32_t* reading;         /* [slots][2] (expert, slot) */
  int32_t* counts;          /* [3] entries in free_list, cooling, reading */
  int64_t* stats;           /* [KEEPVQ_STAT_COUNT] */
  int64_t pool;
  int64_t slots;
  /* the demand being harvested */
  const uint32_t* want;     /* [tokens, top_k] */
  const float* want_score;  /* [tokens, top_k] */
  int64_t tokens;
  int32_t top_k;
  uint8_t* landed;          /* [pool] flags the installer raises when an expert's bytes are in its slot; the
                               tick that routes the expert clears its flag */
  int64_t call;
  int64_t step;
  float tau;
  float route_scale;
  int32_t spare;
  int32_t first_layer;      /* non-zero: this layer counts calls and tokens */
  /* what happened, for the host to act on */
  int32_t* actions;         /* [max_actions][3] (kind, expert, slot) */
  int32_t* action_count;    /* [1] running count; the caller resets it */
  int32_t max_actions;
} keepvq_residency_args;

int keepvq_residency_tick(const keepvq_residency_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * keepvq_grouped_projection: out[r] = W[rhs[r]] @ x[r], one activation row per route, on the
 * int8 tensor-core kernels.  What gather_vqmm_sorted_routes reaches in the reference for prefill
 * (src/ramp/ops/vq_switch.py:620-913 -> src/ramp/kernels/gather_vqmm.py:597-928 and the native
 * nax_e8p_fp16_sorted_matmul_steel, src/ramp/kernels/nax.py:330-366).  Routes are grouped by
 * expert on the device, so they need not arrive sorted; rhs 0xFFFFFFFF gives a zero row.
 * Returns KEEPVQ_ERR_UNSUPPORTED when the shapes or the table do not fit these kernels (16-bit
 * codes, in_dim % 256 == 0, whole scale groups per 256 inputs, every table nibble odd): the
 * caller then uses keepvq_routed_matvec.  Activations are rounded to 16-bit fixed point per row:
 * an element's error is at most 2^-16 of the row's largest magnitude, whatever the input dtype
 * (fp32 rows are narrowed too; keepvq_routed_matvec keeps 24 bits of them).  On a row with one
 * channel far above the rest the small channels therefore lose relative precision: with an
 * outlier of 300 (3000) times the row's RMS the output error stays near 1e-3 of the output's
 * largest magnitude, while against the output the row would give WITHOUT the outlier channel it
 * is about 0.5 % (3 %).  Everything else is exact integer arithmetic.  Rows of routes without an
 * expert are written as zeros.
 * The scratch also holds, at keepvq_grouped_projection_status_offset, the int32 the tcgen05
 * kernel sets when a bounded wait expires (see keepvq_moe_layer_status_offset).
 * ------------------------------------------------------------------------------------------ */
typedef struct keepvq_grouped_projection_args {
  const void* x;             /* [x_rows, in_dim]; fp16 or bf16 (fp32 rows belong to keepvq_routed_matvec, which keeps 24 bits of them) */
  int32_t x_dtype;
  int64_t routes;
  const uint32_t* rhs;       /* [routes] expert (slot) of each route */
  const uint16_t* codes;     /* [slots, out_dim, in_dim/8] */
  const void* scales;        /* [slots, out_dim, groups] */
  int32_t scales_dtype;
  int64_t slots, out_dim, in_dim, groups;
  const uint32_t* codebook;  /* E8P packed abs grid */
  int32_t codebook_all_odd;  /* as in keepvq_moe_layer_args */
  void* out;                 /* [routes, out_dim] */
  int32_t out_dtype;
  void* workspace;           /* keepvq_grouped_projection_workspace_bytes(), 256-byte aligned */
  int64_t workspace_bytes;
  /* Route r reads activation row r / x_div: 1 (or 0) = a row per route, top_k = the token layout
     of e8p_m1_token_layout (src/ramp/kernels/e8p_m1.py:134-157).  x_rows = routes / x_div. */
  int32_t x_div;
  /* Optional nested residual, as in keepvq_matvec_args (e8p_nested_m1.py:90-112); res_codes == NULL
     turns it off.  Needs at least 48 routes and whole residual scale groups per 256 inputs,
     otherwise KEEPVQ_ERR_UNSUPPORTED. */
  const uint8_t* res_codes;    /* [res_rows, out_dim, in_dim/8] */
  const void* res_scales;      /* [res_rows, out_dim, res_groups], dtype scales_dtype */
  int64_t res_rows;
  int64_t res_groups;
  const uint32_t* res_table;   /* KEEPVQ_TABLE_HALF2_PAIRS */
  const uint32_t* hot_of_slot; /* [slots] */
} keepvq_grouped_projection_args;

int64_t keepvq_grouped_projection_workspace_bytes(int64_t routes, int64_t in_dim);
int64_t keepvq_grouped_projection_status_offset(int64_t routes, int64_t in_dim);
int keepvq_grouped_projection(const keepvq_grouped_projection_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Expert parallelism: packing routes for the dispatch all-to-all and summing them after the
 * combine all-to-all.
 *
 * The reference's only expert-parallel form replicates every token on every rank, runs the
 * rank's slice of the experts and all-reduces the outputs
 * (tests/fixtures/v41_reference/model.py:869-872,891-906).  Here a token's hidden state visits
 * only the ranks that own its experts; the sum over its k picks is the same.
 *
 * Every (source, destination) pair owns a fixed block of `capacity` rows in the exchange
 * buffers, so the all-to-all has constant split sizes and no routing fact reaches the host.
 * Rank w owns experts [w * experts_per_rank, (w + 1) * experts_per_rank).
 *
 * keepvq_ep_pack    for route r (token r / top_k, pick r % top_k) with a live expert e:
 *                   dest = e / experts_per_rank, pos = number of earlier live routes with the same
 *                   dest (stable); position[r] = dest * capacity + pos; x's row is copied to
 *                   send_x[position[r]] and send_meta[position[r]] = (e % experts_per_rank, bits of
 *                   the route's weight).  Dead routes (expert 0xFFFFFFFF), routes whose expert is
 *                   out of range and routes beyond a block's capacity get position = world *
 *                   capacity.  Unused rows of send_x are zero, of send_meta (-1, 0).
 * keepvq_ep_combine out[t] = sum over picks j, in pick order, of back[position[t, j]] in fp32,
 *                   rounded once to the row dtype; positions >= rows add nothing.
 * ------------------------------------------------------------------------------------------ */
typedef struct keepvq_ep_pack_args {
  const void* x;                  /* [tokens, row_bytes] this rank's token rows */
  int64_t row_bytes;              /* multiple of 16 */
  const uint32_t* served_expert;  /* [tokens, top_k] global expert ids, 0xFFFFFFFF = dead pick */
  const float* served_weight;     /* [tokens, top_k] */
  int64_t tokens;
  int32_t top_k;
  int32_t world;                  /* 1..64 ranks */
  int32_t experts_per_rank;
  int64_t capacity;               /* rows per (source, destination) block */
  void* send_x;                   /* [world * capacity, row_bytes] */
  int32_t* send_meta;             /* [world * capacity, 2] */
  int32_t* position;              /* [tokens, top_k] */
} keepvq_ep_pack_args;

int keepvq_ep_pack(const keepvq_ep_pack_args* args, void* stream);

typedef struct keepvq_ep_combine_args {
  const void* back;               /* [rows, hidden] expert outputs, returned to their send positions */
  int32_t dtype;                  /* keepvq_dtype of back and out */
  int64_t rows;
  int64_t hidden;                 /* multiple of 8 */
  const int32_t* position;        /* [tokens, top_k] */
  int64_t tokens;
  int32_t top_k;
  void* out;                      /* [tokens, hidden] */
} keepvq_ep_combine_args;

int keepvq_ep_combine(const keepvq_ep_combine_args* args, void* stream);

/* The same exchange without a collective library in the data path: ranks write rows straight into
 * each other's buffers over NVLink (peer-mapped memory the caller sets up once and describes
 * here), and a flag barrier with a bounded wait orders the phases.  One process per GPU; every
 * rank makes the same sequence of calls.
 *
 * keepvq_ep_dispatch_peer  the plan of keepvq_ep_pack, with rows, slots and weights stored
 *                          directly at row (rank * capacity + pos) of the destination rank's
 *                          recv_x / recv_meta (slot and weight planes), then a barrier: when the call's work is done on
 *                          this rank's stream, every rank's rows for it have landed.
 * keepvq_ep_return_peer    row r of y (a live route received from rank r / capacity) goes to row
 *                          (rank * capacity + r % capacity) of that rank's `back`, then a barrier;
 *                          keepvq_ep_combine then runs on the local `back` with the positions
 *                          keepvq_ep_dispatch_peer wrote.
 *
 * Each of the two calls is one kernel launch: its blocks count themselves off in `arrivals`
 * behind their stores, and the block that finishes last runs the barrier.
 *
 * One set of buffers is enough for back-to-back layers: a rank leaves the second barrier of a
 * layer only after every rank has finished reading what the first phase wrote.  A wait that
 * expires (a peer that never arrives) sets *status to 1 and the kernel returns; nothing traps. */
typedef struct keepvq_ep_peer_args {
  int32_t world, rank;
  int64_t capacity;             /* rows per (source, destination) block */
  int64_t row_bytes;            /* multiple of 16 */
  void* const* recv_x;          /* device array [world]: each rank's [world * capacity, row_bytes] */
  int32_t* const* recv_meta;    /* device array [world]: each rank's [2, world * capacity]: local slots (-1 = no
                                   route), then the bits of the routes' weights; the two planes can be handed to
                                   keepvq_moe_decode_stages as served_slot and served_weight as they are */
  void* const* back;            /* device array [world]: each rank's [world * capacity, row_bytes] */
  int32_t* const* flags;        /* device array [world]: each rank's [world] arrival words, zero at start */
  int32_t* epoch;               /* [1] this rank's barrier count, zero at start */
  int32_t* status;              /* [1] */
  uint32_t wait_spins;          /* polls (about a microsecond each) before a barrier gives up; 0 = 8,388,608 */
  int32_t* arrivals;            /* [1] this rank's count of finished blocks of the running exchange kernel, zero at start
                                   (the last block to finish runs the barrier and clears it) */
} keepvq_ep_peer_args;

int keepvq_ep_dispatch_peer(const keepvq_ep_pack_args* pack, const keepvq_ep_peer_args* peer, void* stream);
int keepvq_ep_return_peer(const void* y, const keepvq_ep_peer_args* peer, void* stream);

/* ------------------------------------------------------------------------------------------
 * keepvq_moe_decode_layer for callers that cannot hand over scratch memory.  It has no
 * counterpart in the reference.
 *
 * Who needs it: a host that gave all device memory to its own pool at start-up and has nothing
 * left to allocate from, or one that must never stall (cudaMalloc / cudaFree synchronise the
 * device).  This entry point allocates nothing, on the host or on the device, and neither does
 * anything it calls.  `workspace` and `workspace_bytes` of the arguments are ignored; the scratch
 * is a fixed KEEPVQ_STATIC_SCRATCH_BYTES array inside the library that every GPU loading the
 * library holds until the process exits.  Inputs and outputs are still the caller's.
 *
 *  - A request whose scratch need (keepvq_moe_layer_workspace_bytes) exceeds the array returns
 *    KEEPVQ_ERR_CAPACITY and launches nothing.  8 MiB covers, for example, 16 decode tokens of a
 *    top-6 layer with hidden 4096 and inter 2048.
 *  - The first call on a device looks up the array's device address (with that device current).
 *    Make that first call before any stream capture begins.
 *  - All calls on a device share the one array, and it keeps the last call's contents.  Calls
 *    that overlap on the GPU race on it: keep them on one stream or order them with events.
 *    Nothing in the array needs clearing between calls.
 * ------------------------------------------------------------------------------------------ */
#define KEEPVQ_STATIC_SCRATCH_BYTES (8u << 20)
int keepvq_moe_decode_layer_static(const keepvq_moe_layer_args* args, void* stream);

/* ------------------------------------------------------------------------------------------
 * Self-test of the bounded waits of the tcgen05 kernels.  Runs one thread block of the prefill
 * projection kernel on a tiny problem laid out inside `workspace`, with the producers of its
 * activation tiles told never to publish.  The consumer's wait must run into its deadline
 * (`wait_ns` nanoseconds on the GPU's global timer, at most one second), after which the block
 * writes 1 into the first int32 of `workspace`, releases its tensor memory and returns; the
 * device stays usable.  A host checks that word after synchronising.  No counterpart in the
 * reference.
 * ------------------------------------------------------------------------------------------ */
int64_t keepvq_wait_selftest_workspace_bytes(void);
int keepvq_wait_selftest(void* workspace, int64_t workspace_bytes, int64_t wait_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KEEPVQ_H */
