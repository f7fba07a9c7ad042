// keepvq_moe_decode_layer: one routed MoE layer at decode as a single launch sequence.
//
// Sequence on the caller's stream (no host read anywhere):
//   1 router logits            router.cu
//   2 dual top-k + admission   router.cu
//   3 gate and up projections  routed matvec, token layout, rounded to the activation dtype
//   4 h = silu(G) * U * g      this file
//   5 down projection          routed matvec, one row per route
//   6 fp32 sum over the k picks, one rounding       this file
// The rounding points are the served path's (scripts/v41_build/omlx_lattice.py:356-371,583-589).
//
// Two sets of kernels serve steps 3-5.  The tensor-core set (moe_fast.cu, projection_slab.cu,
// prefill_umma.cu) groups routes by slot, quantises activations to 16-bit fixed point and runs the
// projections on the int8 tensor cores, SwiGLU fused into the gate/up epilogue; it needs a table
// whose entries are all odd half-units (true of the E8P table; the caller vouches with
// `codebook_all_odd`) and input dims and scale groups that are multiples of 256.  Everything else
// takes the general kernel (rowdot.cu).
//
// Scratch layout (all regions 256-byte aligned):
//   logits [tokens, pool] f32 | gate [routes, inter] | up [routes, inter] | h [routes, inter]
//   | down [routes, hidden]     (activation dtype)
//   | quantised x, quantised h, their scales and group sums, the route groups   (tensor-core set)
#include <algorithm>
#include <type_traits>

#include "common.cuh"
#include "moe_fast.cuh"

namespace keepvq {

template <typename T>
struct dtype_tag_of {
  static constexpr int value = sizeof(T) == 4 ? KEEPVQ_F32 : (std::is_same<T, __half>::value ? KEEPVQ_F16 : KEEPVQ_BF16);
};

static inline int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

// The tcgen05 kernels decode a code once per 96 routes of an expert but cost the same for one
// route as for 96; the mma.sync kernels stream an expert's codes once per 8 routes.  Which one
// pays depends on routes per expert, and the host only knows its upper bound routes / slots
// (reading the routing back would stall the stream): from 24 on, three passes of the decode
// kernels cost more than the one pass of the tcgen05 kernels.
constexpr int64_t PREFILL_MIN_ROUTES = 1024;
constexpr int64_t PREFILL_MIN_ROUTES_PER_SLOT = 24;

struct LayerScratch {
  int64_t logits, gate, up, h, down;
  int64_t xq, xscale, xsums, hq, hscale, hsums, gcount, gslot, gstart, gsize, groutes, status;
  int64_t total;
};

static LayerScratch plan_scratch(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k) {
  const int64_t routes = tokens * top_k;
  LayerScratch s;
  int64_t at = 0;
  s.logits = at; at += align256(tokens * pool * 4);
  s.gate = at;   at += align256(routes * inter * 4);  // sized for fp32 activations
  s.up = at;     at += align256(routes * inter * 4);
  s.h = at;      at += align256(routes * inter * 4);
  s.down = at;   at += align256(routes * hidden * 4);
  // calls large enough for the tcgen05 kernels quantise the token rows once per route, in grouped order
  const int64_t x_rows = routes >= PREFILL_MIN_ROUTES ? routes : tokens;
  s.xq = at;     at += align256((x_rows + 1) * hidden * 2);  // + the zero row
  s.xscale = at; at += align256((x_rows + 1) * 4);
  s.xsums = at;  at += align256(std::max((tokens + 1) * (hidden / 8) * 4, (x_rows + 1) * 4));  // room for one scale group per codeword (one per row in grouped order)
  s.hq = at;     at += align256((routes + 1) * inter * 2);
  s.hscale = at; at += align256((routes + 1) * 4);
  s.hsums = at;  at += align256((routes + 1) * (inter / 8) * 4);
  s.gcount = at; at += 256;
  s.gslot = at;  at += align256(routes * 4);
  s.gstart = at; at += align256(routes * 4);
  s.gsize = at;  at += align256(routes * 4);
  s.groutes = at; at += align256(routes * 4);
  s.status = at; at += 256;
  s.total = at;
  return s;
}

// h[r, n] = round(silu(G) * U * g_r); a switched-off route (weight 0 / no slot) gives zeros.
template <typename T>
__global__ void __launch_bounds__(256) swiglu_weight_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                            const float* __restrict__ weight, T* __restrict__ h,
                                                            int64_t routes, int64_t inter, float limit) {
  constexpr int tag = dtype_tag_of<T>::value;
  const int64_t total = routes * inter;
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int64_t r = i / inter;
    float g = load_as_float(gate, tag, i);
    float u = load_as_float(up, tag, i);
    if (limit > 0.0f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    const float v = g / (1.0f + expf(-g)) * u * weight[r];
    store_from_float(h, tag, i, v);
  }
}

// out[t, d] = round(sum_j float(down[t*k + j, d]) + shared[t, d]), summed in pick order.  A pick
// without a slot adds nothing (the grouped kernels never touch its row of `down`).  `shared` (may
// be null) is the shared expert's fp32 output: it joins the routed sum before the one rounding, as
// the reference's shared down kernel adds the routed sum and rounds once
// (scripts/v41_build/omlx_lattice.py:372-389).
template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ down, const uint32_t* __restrict__ served_slot, int64_t slots,
                                                      const float* __restrict__ shared, T* __restrict__ out, int64_t tokens, int64_t hidden, int top_k) {
  grid_launch_dependents();
  grid_wait();
  const int64_t vectors = hidden / 8, total = tokens * vectors;  // eight values (16 or 32 bytes) per thread and step
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int64_t t = i / vectors, d = (i - t * vectors) * 8;
    float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      if (served_slot[t * top_k + j] >= static_cast<uint64_t>(slots)) continue;
      float v[8];
      load8_as_float<T>(down + (t * top_k + j) * hidden + d, v);
#pragma unroll
      for (int q = 0; q < 8; ++q) y[q] += v[q];
    }
    if (shared) {
      const float4 lo = *reinterpret_cast<const float4*>(shared + t * hidden + d), hi = *reinterpret_cast<const float4*>(shared + t * hidden + d + 4);
      y[0] += lo.x; y[1] += lo.y; y[2] += lo.z; y[3] += lo.w; y[4] += hi.x; y[5] += hi.y; y[6] += hi.z; y[7] += hi.w;
    }
    store8_from_float<T>(out + t * hidden + d, y);
  }
}

template <typename T>
static void launch_elementwise(const keepvq_moe_layer_args& a, const LayerScratch& sc, cudaStream_t s, bool combine) {
  char* ws = reinterpret_cast<char*>(a.workspace);
  const int64_t routes = a.tokens * a.top_k;
  if (!combine) {
    const int64_t total = routes * a.inter;
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 16));
    swiglu_weight_kernel<T><<<blocks, 256, 0, s>>>(reinterpret_cast<const T*>(ws + sc.gate), reinterpret_cast<const T*>(ws + sc.up),
                                                   a.served_weight, reinterpret_cast<T*>(ws + sc.h), routes, a.inter, a.swiglu_limit);
  } else {
    const int64_t total = a.tokens * (a.hidden / 8);
    const unsigned blocks = static_cast<unsigned>(std::min<int64_t>((total + 255) / 256, 148 * 16));
    launch_after(a.tokens <= 256, combine_kernel<T>, blocks, 256, 0, s, reinterpret_cast<const T*>(ws + sc.down), static_cast<const uint32_t*>(a.served_slot), a.slots,
                 a.shared, reinterpret_cast<T*>(a.out), a.tokens, a.hidden, static_cast<int>(a.top_k));
  }
}

static int projection(const keepvq_moe_layer_args& a, const keepvq_expert_weights& w, const void* x, int64_t x_rows,
                      int64_t in_dim, int64_t out_dim, int32_t x_div, void* out, void* stream) {
  keepvq_matvec_args m = {};
  m.x = x; m.x_dtype = a.x_dtype; m.x_rows = x_rows;
  m.codes = w.codes; m.code_bits = 16; m.scales = w.scales; m.scales_dtype = a.scales_dtype;
  m.experts = a.slots; m.out_dim = out_dim; m.in_dim = in_dim; m.groups = w.groups;
  m.codebook = a.codebook; m.codebook_layout = KEEPVQ_TABLE_PACKED;
  m.rhs = a.served_slot; m.lhs = nullptr; m.x_div = x_div; m.routes = a.tokens * a.top_k;
  if (w.res_codes && a.res_rows > 0) {
    m.res_codes = w.res_codes; m.res_scales = w.res_scales; m.res_scales_dtype = a.scales_dtype;
    m.res_rows = a.res_rows; m.res_groups = w.res_groups; m.res_table = a.res_table; m.hot_of_slot = a.hot_of_slot;
  }
  m.out = out; m.out_dtype = a.x_dtype;
  return keepvq_routed_matvec(&m, stream);
}

}  // namespace keepvq

extern "C" int64_t keepvq_moe_layer_workspace_bytes(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k) {
  if (tokens < 0 || hidden <= 0 || inter <= 0 || pool <= 0 || top_k <= 0) return KEEPVQ_ERR_SHAPE;
  return keepvq::plan_scratch(tokens, hidden, inter, pool, top_k).total + 256;
}

extern "C" int64_t keepvq_moe_layer_status_offset(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k) {
  if (tokens < 0 || hidden <= 0 || inter <= 0 || pool <= 0 || top_k <= 0) return KEEPVQ_ERR_SHAPE;
  return keepvq::plan_scratch(tokens, hidden, inter, pool, top_k).status;
}

extern "C" int64_t keepvq_moe_layer_route_output_offset(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k) {
  if (tokens < 0 || hidden <= 0 || inter <= 0 || pool <= 0 || top_k <= 0) return KEEPVQ_ERR_SHAPE;
  return keepvq::plan_scratch(tokens, hidden, inter, pool, top_k).down;
}

extern "C" int64_t keepvq_moe_layer_route_hidden_offset(int64_t tokens, int64_t hidden, int64_t inter, int64_t pool, int32_t top_k) {
  if (tokens < 0 || hidden <= 0 || inter <= 0 || pool <= 0 || top_k <= 0) return KEEPVQ_ERR_SHAPE;
  return keepvq::plan_scratch(tokens, hidden, inter, pool, top_k).h;
}

extern "C" int keepvq_moe_decode_stages(const keepvq_moe_layer_args* args, int32_t stages, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_moe_layer_args& a = *args;
  if (!valid_dtype(a.x_dtype) || !valid_dtype(a.router_dtype) || !valid_dtype(a.scales_dtype)) return KEEPVQ_ERR_DTYPE;
  if (a.tokens < 0 || a.hidden <= 0 || a.inter <= 0 || a.pool <= 0 || a.slots <= 0 || a.top_k <= 0) return KEEPVQ_ERR_SHAPE;
  if (a.hidden % 8 || a.inter % 8) return KEEPVQ_ERR_SHAPE;
  if (a.tokens == 0) return KEEPVQ_OK;
  if (!a.x || !a.router_w || !a.out || !a.workspace || !a.codebook) return KEEPVQ_ERR_NULL;
  if (!a.w1.codes || !a.w3.codes || !a.w2.codes || !a.w1.scales || !a.w3.scales || !a.w2.scales) return KEEPVQ_ERR_NULL;
  if (!a.served_expert || !a.served_slot || !a.served_weight || !a.want || !a.want_score) return KEEPVQ_ERR_NULL;
  if (a.w1.groups <= 0 || a.w3.groups != a.w1.groups || a.w2.groups <= 0) return KEEPVQ_ERR_SHAPE;
  const LayerScratch sc = plan_scratch(a.tokens, a.hidden, a.inter, a.pool, a.top_k);
  if (!aligned_to(a.workspace, 256) || (a.shared && !aligned_to(a.shared, 16))) return KEEPVQ_ERR_ALIGN;
  if (a.workspace_bytes < sc.total) return KEEPVQ_ERR_CAPACITY;
  char* ws = reinterpret_cast<char*>(a.workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t routes = a.tokens * a.top_k;
  const bool residual = a.res_rows > 0 && (a.w1.res_codes || a.w3.res_codes || a.w2.res_codes);
  // a residual tier stays on the tensor-core kernels when all three projections carry it and the
  // call has enough routes for the kernel that holds the residual pass
  const bool residual_fits = !residual || (a.w1.res_codes && a.w3.res_codes && a.w2.res_codes && a.res_table && a.hot_of_slot &&
                                           a.w3.res_groups == a.w1.res_groups && fast::residual_supported(routes, a.hidden, a.w1.res_groups) &&
                                           fast::residual_supported(routes, a.inter, a.w2.res_groups));
  // (fp32 activations take the general kernel, which keeps 24 bits of a row instead of 16)
  const bool tensor_path = a.x_dtype != KEEPVQ_F32 && a.codebook_all_odd && residual_fits && fast::shapes_supported(a.inter, a.hidden, a.w1.groups) &&
                           fast::shapes_supported(a.hidden, a.inter, a.w2.groups);
  int rc = KEEPVQ_OK;
  // many routes per expert: the tcgen05 kernels, which decode a code once per 96 routes
  const int64_t live = a.expected_routes > 0 && a.expected_routes < routes ? a.expected_routes : routes;
  const bool prefill = tensor_path && !residual && live >= PREFILL_MIN_ROUTES && live >= PREFILL_MIN_ROUTES_PER_SLOT * a.slots &&
                       fast::prefill_supported(a.inter, a.hidden, a.w1.groups) && fast::prefill_supported(a.hidden, a.inter, a.w2.groups);
  // (the sums regions have room for a scale group per codeword; the tensor-core kernels' rows have at
  // most one per 256 inputs, and their sums per 256 inputs go behind those)
  fast::QuantRows xq = {reinterpret_cast<uint8_t*>(ws + sc.xq), reinterpret_cast<float*>(ws + sc.xscale), reinterpret_cast<int32_t*>(ws + sc.xsums),
                        tensor_path && !prefill ? reinterpret_cast<int32_t*>(ws + sc.xsums) + (a.tokens + 1) * a.w1.groups : nullptr};
  bool x_quantized = false;  // the router's launch took the quantisation of the token rows along
  // a caller that expects few of the routes to be live (an expert-parallel rank's padded receive
  // buffer) has the quantisation skip the rows no live route reads; otherwise the look at the
  // slots would only put a dependent load in front of every row
  const uint32_t* padded = live < routes ? a.served_slot : nullptr;

  if (stages & KEEPVQ_STAGE_ROUTER) {
    keepvq_router_logits_args rl = {};
    rl.x = a.x; rl.x_dtype = a.x_dtype; rl.router_w = a.router_w; rl.router_dtype = a.router_dtype;
    rl.tokens = a.tokens; rl.pool = a.pool; rl.hidden = a.hidden; rl.gate_temp = a.gate_temp;
    rl.logits = reinterpret_cast<float*>(ws + sc.logits);
    // few tokens: the logits and the quantised token rows of the projections in one launch
    const bool front = (stages & KEEPVQ_STAGE_PREPARE) && tensor_path && !prefill && valid_dtype(a.router_dtype) && a.router_w && a.gate_temp > 0.0f &&
                       aligned_to(a.x, 16) && aligned_to(a.router_w, 16) && fast::logits_and_quantize_supported(rl, a.w1.groups);
    if (front) {
      if ((rc = fast::logits_and_quantize(rl, a.w1.groups, xq, s))) return rc;
      x_quantized = true;
    } else if ((rc = keepvq_router_logits(&rl, stream))) return rc;
    keepvq_routed_topk_args tk = {};
    tk.logits = rl.logits; tk.tokens = a.tokens; tk.pool = a.pool; tk.top_k = a.top_k; tk.score_func = a.score_func;
    tk.norm_topk_prob = a.norm_topk_prob; tk.route_scale = a.route_scale; tk.tau = a.tau;
    tk.served_bias = a.served_bias; tk.pool_bias = a.pool_bias; tk.slot_of = a.slot_of;
    tk.served_expert = a.served_expert; tk.served_slot = a.served_slot; tk.served_weight = a.served_weight;
    tk.want = a.want; tk.want_score = a.want_score; tk.admit = a.admit;
    if ((rc = keepvq_routed_topk(&tk, stream))) return rc;
  }

  if (tensor_path) {
    fast::RouteGroups groups = {reinterpret_cast<int32_t*>(ws + sc.gcount), reinterpret_cast<int32_t*>(ws + sc.gslot),
                                reinterpret_cast<int32_t*>(ws + sc.gstart), reinterpret_cast<int32_t*>(ws + sc.gsize),
                                reinterpret_cast<int32_t*>(ws + sc.groutes)};
    fast::QuantRows hq = {reinterpret_cast<uint8_t*>(ws + sc.hq), reinterpret_cast<float*>(ws + sc.hscale), reinterpret_cast<int32_t*>(ws + sc.hsums),
                          prefill ? nullptr : reinterpret_cast<int32_t*>(ws + sc.hsums) + (routes + 1) * a.w2.groups};
    int32_t* wait_status = reinterpret_cast<int32_t*>(ws + sc.status);
    const int group_cols = prefill ? fast::PREFILL_GROUP_ROUTES : fast::decode_group_routes(live, a.slots, std::max(a.hidden, a.inter));
    if (stages & KEEPVQ_STAGE_PREPARE) {
      if (!x_quantized && !prefill && fast::group_with_quantize_supported(routes, a.slots)) {  // one launch for both
        if ((rc = fast::quantize_rows_and_group(a.x, a.x_dtype, a.tokens, a.hidden, a.w1.groups, xq, false, s, padded, a.top_k, a.slots,
                                                a.served_slot, routes, group_cols, groups, wait_status))) return rc;
      } else {
        if ((rc = fast::group_routes(a.served_slot, routes, a.slots, group_cols, groups, wait_status, s))) return rc;
        if (prefill) {
          if ((rc = fast::quantize_rows_sorted(a.x, a.x_dtype, routes, a.hidden, a.w1.groups, xq, {groups.routes, groups.count, a.top_k}, s))) return rc;
        } else if (!x_quantized && (rc = fast::quantize_rows(a.x, a.x_dtype, a.tokens, a.hidden, a.w1.groups, xq, false, s, padded, a.top_k, a.slots))) return rc;
      }
    }
    fast::FastProjectionArgs p = {};
    p.scales_dtype = a.scales_dtype; p.codebook = a.codebook; p.groups_of_routes = groups; p.max_routes = routes; p.group_cols = group_cols; p.status = wait_status;
    p.few_groups = prefill ? 0 : fast::few_route_groups(live, a.slots);
    p.out_dtype = a.x_dtype; p.swiglu_limit = a.swiglu_limit; p.route_weight = a.served_weight;
    if (stages & KEEPVQ_STAGE_GATE_UP) {
      p.a = {a.w1.codes, a.w1.scales, a.w1.res_codes, a.w1.res_scales}; p.b = {a.w3.codes, a.w3.scales, a.w3.res_codes, a.w3.res_scales};
      if (residual) { p.res_groups = a.w1.res_groups; p.hot_of_slot = a.hot_of_slot; p.res_table = a.res_table; }
      p.out_dim = a.inter; p.in_dim = a.hidden; p.groups = a.w1.groups; p.x = xq; p.x_zero_row = prefill ? routes : a.tokens; p.x_div = a.top_k; p.out = ws + sc.h;
      if ((rc = prefill ? fast::prefill_gate_up(p, wait_status, s) : fast::gate_up(p, s))) return rc;
    }
    if (stages & KEEPVQ_STAGE_DOWN) {
      if (prefill) {
        if ((rc = fast::quantize_rows_sorted(ws + sc.h, a.x_dtype, routes, a.inter, a.w2.groups, hq, {groups.routes, groups.count, 1}, s))) return rc;
      } else if ((rc = fast::quantize_rows(ws + sc.h, a.x_dtype, routes, a.inter, a.w2.groups, hq, false, s, padded, 1, a.slots))) return rc;
      p.a = {a.w2.codes, a.w2.scales, a.w2.res_codes, a.w2.res_scales}; p.b = {nullptr, nullptr, nullptr, nullptr};
      if (residual) { p.res_groups = a.w2.res_groups; p.hot_of_slot = a.hot_of_slot; p.res_table = a.res_table; }
      p.out_dim = a.hidden; p.in_dim = a.inter; p.groups = a.w2.groups; p.x = hq; p.x_zero_row = routes; p.x_div = 1; p.out = ws + sc.down;
      if ((rc = prefill ? fast::prefill_down(p, wait_status, s) : fast::down(p, s))) return rc;
    }
  } else {
    if (stages & KEEPVQ_STAGE_GATE_UP) {
      if ((rc = projection(a, a.w1, a.x, a.tokens, a.hidden, a.inter, a.top_k, ws + sc.gate, stream))) return rc;
      if ((rc = projection(a, a.w3, a.x, a.tokens, a.hidden, a.inter, a.top_k, ws + sc.up, stream))) return rc;
      if (a.x_dtype == KEEPVQ_F32) launch_elementwise<float>(a, sc, s, false);
      else if (a.x_dtype == KEEPVQ_F16) launch_elementwise<__half>(a, sc, s, false);
      else launch_elementwise<__nv_bfloat16>(a, sc, s, false);
      KEEPVQ_CHECK_LAUNCH();
    }
    if (stages & KEEPVQ_STAGE_DOWN) {
      if ((rc = projection(a, a.w2, ws + sc.h, routes, a.inter, a.hidden, 1, ws + sc.down, stream))) return rc;
    }
  }

  if (stages & KEEPVQ_STAGE_COMBINE) {
    if (a.x_dtype == KEEPVQ_F32) launch_elementwise<float>(a, sc, s, true);
    else if (a.x_dtype == KEEPVQ_F16) launch_elementwise<__half>(a, sc, s, true);
    else launch_elementwise<__nv_bfloat16>(a, sc, s, true);
    KEEPVQ_CHECK_LAUNCH();
  }
  return KEEPVQ_OK;
}

extern "C" int keepvq_moe_decode_layer(const keepvq_moe_layer_args* args, void* stream) {
  return keepvq_moe_decode_stages(args, KEEPVQ_STAGE_ALL, stream);
}

// ------------------------------------------------------------------------------------------
// The decode layer for callers that have no scratch buffer to give.
//
// Some hosts cannot allocate device memory at call time: a serving process that handed every
// byte of the GPU to its own pool at start-up, or a loop that may not stall (cudaMalloc and
// cudaFree synchronise the device).  For them the scratch lives in this library's image: a
// fixed array in device memory that every GPU loading the library holds until the process
// exits.  All calls on a device share it, so two calls that overlap on the GPU (different
// streams, or a graph replay racing a direct call) corrupt each other; serialise them.  The
// array keeps whatever the last call left there.  Nothing in it has to start at zero: every
// region is written by an earlier stage of the same call before a later stage reads it.
// ------------------------------------------------------------------------------------------
namespace keepvq {

static __device__ __align__(256) unsigned char g_layer_scratch[KEEPVQ_STATIC_SCRATCH_BYTES];

// Device address of g_layer_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel can use; the runtime translates it,
// per device.  Looked up once per device, on the first call made with that device current.
static int layer_scratch_address(void** out) {
  constexpr int MAX_DEVICES = 64;
  static void* cached[MAX_DEVICES] = {};
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return note_cuda_error(e);
  if (device < 0 || device >= MAX_DEVICES) return KEEPVQ_ERR_CAPACITY;
  if (!cached[device]) {
    void* address = nullptr;
    e = cudaGetSymbolAddress(&address, g_layer_scratch);
    if (e != cudaSuccess) return note_cuda_error(e);
    cached[device] = address;
  }
  *out = cached[device];
  return KEEPVQ_OK;
}

}  // namespace keepvq

extern "C" int keepvq_moe_decode_layer_static(const keepvq_moe_layer_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  if (args->tokens < 0 || args->hidden <= 0 || args->inter <= 0 || args->pool <= 0 || args->top_k <= 0) return KEEPVQ_ERR_SHAPE;
  const int64_t need = plan_scratch(args->tokens, args->hidden, args->inter, args->pool, args->top_k).total;
  if (need > static_cast<int64_t>(KEEPVQ_STATIC_SCRATCH_BYTES)) return KEEPVQ_ERR_CAPACITY;  // too many tokens for the built-in scratch
  void* scratch = nullptr;
  const int rc = layer_scratch_address(&scratch);
  if (rc) return rc;
  keepvq_moe_layer_args with_scratch = *args;
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = static_cast<int64_t>(KEEPVQ_STATIC_SCRATCH_BYTES);
  return keepvq_moe_decode_stages(&with_scratch, KEEPVQ_STAGE_ALL, stream);
}
