// Tensor-core decode path for the routed E8P experts: activation quantisation, route grouping
// and the choice of projection kernel.  See moe_fast.cuh for the arithmetic identity it rests on.
//
// The projection kernels themselves (HBM-bound by design: every code byte is read once per group
// of routes) live in their own files: projection_slab.cu (calls with many route groups, and their
// split form for a residual tier with few), projection_sweep.cu (few route groups) and
// prefill_umma.cu (many routes per expert, tcgen05).  They share:
//   - a codeword becomes the A fragment of an m16n8k32 int8 MMA through two 4-byte table reads
//     (abs byte, sign byte; 32 replicas each so lanes never share a bank) XORed and spread from
//     nibbles to bytes: the nibble decoder of moe_fast.cuh;
//   - the K order inside an MMA is permuted (byte j of the low word is table nibble 3-j, of the
//     high word nibble 7-j); the activations are stored in that same order by quantize_rows;
//   - accumulation is exact in int32; one conversion to fp32 per scale group.
#include <stdlib.h>

#include <algorithm>

#include "moe_fast.cuh"
#include "router_logits.cuh"

namespace keepvq {
namespace fast {

// ------------------------------------------------------------------------------------------
// Activation quantisation: x -> 16-bit fixed point with a power-of-two scale per row.
// ------------------------------------------------------------------------------------------
// One row per block of 256 threads; row == rows is the extra all-zero row.
template <typename XT>
__device__ __forceinline__ void quantize_row(const XT* __restrict__ x, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, int planes, int64_t row, int64_t source_row) {
  __shared__ float warp_max[8];
  __shared__ float row_scale;
  extern __shared__ int32_t group_sum[];
  const int64_t cw = in_dim / 8, per_group = cw / groups;
  if (row == rows) {  // one extra all-zero row: the B operand of MMA columns that carry no route
    // (both layouts: the buffer is (rows + 1) * cw * 16 bytes either way)
    for (int64_t c = threadIdx.x; c < cw; c += 256) {
      if (planes) {
        reinterpret_cast<uint2*>(out.q)[row * cw + c] = make_uint2(0, 0);
        reinterpret_cast<uint2*>(out.q + (rows + 1) * cw * 8)[row * cw + c] = make_uint2(0, 0);
      } else {
        reinterpret_cast<uint4*>(out.q)[row * cw + c] = make_uint4(0, 0, 0, 0);
      }
    }
    for (int64_t g = threadIdx.x; g < groups; g += 256) out.sums[row * groups + g] = 0;
    if (out.chunk_sums)
      for (int64_t c = threadIdx.x; c < cw / 32; c += 256) out.chunk_sums[row * (cw / 32) + c] = 0;
    if (threadIdx.x == 0) out.scale[row] = 1.0f;
    return;
  }
  const XT* xr = x + source_row * in_dim;
  for (int64_t g = threadIdx.x; g < groups; g += 256) group_sum[g] = 0;

  float amax = 0.0f;
  for (int64_t c = threadIdx.x; c < cw; c += 256) {
    float v[8];
    load8_as_float<XT>(xr + c * 8, v);
#pragma unroll
    for (int d = 0; d < 8; ++d) amax = fmaxf(amax, fabsf(v[d]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.0f;
    for (int w = 0; w < 8; ++w) m = fmaxf(m, warp_max[w]);
    float s = 1.0f;
    if (m > 0.0f && isfinite(m)) {
      int ex;
      frexpf(m, &ex);            // m < 2^ex
      s = ldexpf(1.0f, ex - 15);  // |x| / s < 2^15
      if (m / s > 32639.0f) s *= 2.0f;  // 127 * 256 + 127: the largest value two signed bytes hold
    }
    row_scale = s;
    out.scale[row] = s;
  }
  __syncthreads();
  const float inv = 1.0f / row_scale;  // exact: a power of two

  for (int64_t c = threadIdx.x; c < cw; c += 256) {
    float v[8];
    load8_as_float<XT>(xr + c * 8, v);
    int q[8], total = 0;
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      q[d] = max(-32639, min(32639, __float2int_rn(v[d] * inv)));
      total += q[d];
    }
    atomicAdd(&group_sum[c / per_group], total);
    if (out.chunk_sums) {  // a warp's 32 codewords are one chunk of 256 inputs (the row is a multiple of that when these are asked for)
      const int chunk_total = __reduce_add_sync(0xFFFFFFFFu, total);
      if ((threadIdx.x & 31) == 0) out.chunk_sums[row * (cw / 32) + c / 32] = chunk_total;
    }
    // byte j of word 0 pairs with table nibble 3-j = dim 6-2j; of word 1 with nibble 7-j = dim 7-2j
    uint32_t hi0 = 0, hi1 = 0, lo0 = 0, lo1 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // x' = 256 * hi + lo with both bytes signed, so the two MMAs are the same s8 x s8 kind
      const int e = q[6 - 2 * j], o = q[7 - 2 * j];
      const int eh = (e + 128) >> 8, oh = (o + 128) >> 8;
      hi0 |= static_cast<uint32_t>(eh & 0xFF) << (8 * j);
      lo0 |= static_cast<uint32_t>((e - 256 * eh) & 0xFF) << (8 * j);
      hi1 |= static_cast<uint32_t>(oh & 0xFF) << (8 * j);
      lo1 |= static_cast<uint32_t>((o - 256 * oh) & 0xFF) << (8 * j);
    }
    if (planes) {  // high bytes of every row first, then the low bytes: what the tcgen05 B tiles copy from
      reinterpret_cast<uint2*>(out.q)[row * cw + c] = make_uint2(hi0, hi1);
      reinterpret_cast<uint2*>(out.q + (rows + 1) * cw * 8)[row * cw + c] = make_uint2(lo0, lo1);
    } else {
      reinterpret_cast<uint4*>(out.q)[row * cw + c] = make_uint4(hi0, hi1, lo0, lo1);
    }
  }
  __syncthreads();
  for (int64_t g = threadIdx.x; g < groups; g += 256) out.sums[row * groups + g] = group_sum[g];
}

// `live` (may be null): the slots of the routes that read the rows, `per_row` of them per row; a row
// none of whose routes has a slot below `slots` is skipped (no kernel reads it: projections only
// follow live routes).  An expert-parallel rank quantises 8 x capacity rows of which an eighth is live.
struct LiveRows { const uint32_t* slot; int32_t per_row; int64_t slots; };

// One more block (the last) may group the routes of the call, which needs nothing of the rows:
// one launch less in front of the projections.
struct GroupJob { const uint32_t* served_slot; int32_t routes, slots, max_group; RouteGroups out; int32_t* clear; };

template <typename XT>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const XT* __restrict__ x, int64_t rows, int64_t in_dim, int64_t groups, QuantRows out, int planes, LiveRows live, GroupJob job) {
  grid_launch_dependents();
  grid_wait();
  const int64_t row = blockIdx.x;
  if (row > rows) {  // only launched when there is a job
    extern __shared__ int32_t group_scratch[];
    group_routes_block<256>(job.served_slot, job.routes, job.slots, job.max_group, job.out, job.clear, group_scratch);
    return;
  }
  if (live.slot && row < rows) {
    bool any = false;
    for (int j = 0; j < live.per_row; ++j) any = any || live.slot[row * live.per_row + j] < static_cast<uint64_t>(live.slots);
    if (!any) return;  // uniform over the block
  }
  quantize_row<XT>(x, rows, in_dim, groups, out, planes, row, row);
}

// Byte planes with the rows in grouped order (what the tcgen05 kernels' TMA boxes copy).
template <typename XT>
__global__ void __launch_bounds__(256) quantize_rows_sorted_kernel(const XT* __restrict__ x, int64_t rows, int64_t in_dim, int64_t groups, QuantRows out, SortedRows sorted) {
  grid_launch_dependents();
  grid_wait();
  const int64_t row = blockIdx.x;
  if (row < rows && row >= sorted.count[1]) return;  // not a grouped route: nothing reads the row (uniform over the block)
  quantize_row<XT>(x, rows, in_dim, groups, out, 1, row, row < rows ? sorted.routes[row] / sorted.x_div : 0);
}

// The front of a decode layer call in one launch: the router's logits (the few-token kernel's
// blocks, router_logits.cuh) and the quantisation of the same token rows for the projections
// (rows + 1 further blocks).  Neither needs the other's result, and at a handful of tokens a launch
// costs more than either does.
template <typename XT, typename WT>
__global__ void __launch_bounds__(256) logits_and_quantize_kernel(keepvq_router_logits_args a, int logit_blocks_x, int logit_blocks, int64_t groups, QuantRows out) {
  static_assert(RL_WARPS * 32 == 256, "both halves run on blocks of 256 threads");
  grid_launch_dependents();
  grid_wait();
  const int b = static_cast<int>(blockIdx.x);
  if (b < logit_blocks) router_logits_block<XT, WT>(a, b % logit_blocks_x, b / logit_blocks_x);
  else quantize_row<XT>(reinterpret_cast<const XT*>(a.x), a.tokens, a.hidden, groups, out, 0, b - logit_blocks, b - logit_blocks);
}

template <typename XT>
static cudaError_t launch_front(const keepvq_router_logits_args& a, int bx, int blocks, int64_t groups, const QuantRows& out, size_t smem, cudaStream_t s) {
  const unsigned grid = static_cast<unsigned>(blocks + a.tokens + 1);
  if (a.router_dtype == KEEPVQ_F32) return launch_after(true, logits_and_quantize_kernel<XT, float>, grid, 256, smem, s, a, bx, blocks, groups, out);
  if (a.router_dtype == KEEPVQ_F16) return launch_after(true, logits_and_quantize_kernel<XT, __half>, grid, 256, smem, s, a, bx, blocks, groups, out);
  return launch_after(true, logits_and_quantize_kernel<XT, __nv_bfloat16>, grid, 256, smem, s, a, bx, blocks, groups, out);
}

bool logits_and_quantize_supported(const keepvq_router_logits_args& a, int64_t groups) {
  return a.tokens > 0 && a.tokens <= FRONT_MAX_TOKENS && a.x_dtype != KEEPVQ_F32 && a.hidden % 8 == 0 && groups * sizeof(int32_t) <= 40 * 1024 &&
         (a.pool + RL_ROWS - 1) / RL_ROWS * ((a.tokens + RL_TOKENS - 1) / RL_TOKENS) <= EARLY_LAUNCH_MAX_BLOCKS;
}

int logits_and_quantize(const keepvq_router_logits_args& a, int64_t groups, const QuantRows& out, cudaStream_t s) {
  const int bx = static_cast<int>((a.pool + RL_ROWS - 1) / RL_ROWS), by = static_cast<int>((a.tokens + RL_TOKENS - 1) / RL_TOKENS);
  const size_t smem = static_cast<size_t>(groups) * sizeof(int32_t);
  const cudaError_t err = a.x_dtype == KEEPVQ_F16 ? launch_front<__half>(a, bx, bx * by, groups, out, smem, s) : launch_front<__nv_bfloat16>(a, bx, bx * by, groups, out, smem, s);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

int quantize_rows(const void* x, int32_t x_dtype, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, bool planes, cudaStream_t s,
                  const uint32_t* live_slot, int32_t per_row, int64_t slots) {
  return quantize_rows_and_group(x, x_dtype, rows, in_dim, groups, out, planes, s, live_slot, per_row, slots, nullptr, 0, 0, RouteGroups{}, nullptr);
}

int quantize_rows_sorted(const void* x, int32_t x_dtype, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, const SortedRows& sorted, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(groups) * sizeof(int32_t);
  if (smem > 40 * 1024) return KEEPVQ_ERR_CAPACITY;
  const unsigned grid = static_cast<unsigned>(rows + 1);  // + the zero row
  cudaError_t err;
  if (x_dtype == KEEPVQ_F32) err = launch_after(false, quantize_rows_sorted_kernel<float>, grid, 256, smem, s, reinterpret_cast<const float*>(x), rows, in_dim, groups, out, sorted);
  else if (x_dtype == KEEPVQ_F16) err = launch_after(false, quantize_rows_sorted_kernel<__half>, grid, 256, smem, s, reinterpret_cast<const __half*>(x), rows, in_dim, groups, out, sorted);
  else err = launch_after(false, quantize_rows_sorted_kernel<__nv_bfloat16>, grid, 256, smem, s, reinterpret_cast<const __nv_bfloat16*>(x), rows, in_dim, groups, out, sorted);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

bool group_with_quantize_supported(int64_t routes, int64_t slots) { return routes <= 4096 && slots * 3 * sizeof(int32_t) <= 40 * 1024; }

int quantize_rows_and_group(const void* x, int32_t x_dtype, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, bool planes, cudaStream_t s,
                            const uint32_t* live_slot, int32_t per_row, int64_t slots,
                            const uint32_t* served_slot, int64_t routes, int max_group, const RouteGroups& route_groups, int32_t* clear) {
  const LiveRows live = {live_slot, per_row, slots};
  const GroupJob job = {served_slot, static_cast<int32_t>(routes), static_cast<int32_t>(slots), max_group, route_groups, clear};
  size_t smem = static_cast<size_t>(groups) * sizeof(int32_t);
  if (smem > 40 * 1024) return KEEPVQ_ERR_CAPACITY;
  if (served_slot) {
    if (!group_with_quantize_supported(routes, slots)) return KEEPVQ_ERR_UNSUPPORTED;
    smem = std::max(smem, static_cast<size_t>(slots) * 3 * sizeof(int32_t));
  }
  const unsigned grid = static_cast<unsigned>(rows + 1 + (served_slot ? 1 : 0));  // + the zero row (+ the grouping block)
  const bool early = rows < EARLY_LAUNCH_MAX_BLOCKS;
  cudaError_t err;
  if (x_dtype == KEEPVQ_F32) err = launch_after(early, quantize_rows_kernel<float>, grid, 256, smem, s, reinterpret_cast<const float*>(x), rows, in_dim, groups, out, planes ? 1 : 0, live, job);
  else if (x_dtype == KEEPVQ_F16) err = launch_after(early, quantize_rows_kernel<__half>, grid, 256, smem, s, reinterpret_cast<const __half*>(x), rows, in_dim, groups, out, planes ? 1 : 0, live, job);
  else err = launch_after(early, quantize_rows_kernel<__nv_bfloat16>, grid, 256, smem, s, reinterpret_cast<const __nv_bfloat16*>(x), rows, in_dim, groups, out, planes ? 1 : 0, live, job);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

// ------------------------------------------------------------------------------------------
// Route grouping: routes that are served from the same slot share the code stream.  One block;
// counting sort by slot, then each slot's routes are cut into groups of at most 8.
// ------------------------------------------------------------------------------------------
constexpr int GR_THREADS = 1024;

__global__ void __launch_bounds__(GR_THREADS) group_routes_kernel(const uint32_t* __restrict__ served_slot, int routes, int slots, int max_group, RouteGroups out, int32_t* clear) {
  grid_launch_dependents();
  grid_wait();
  extern __shared__ int32_t group_scratch[];
  group_routes_block<GR_THREADS>(served_slot, routes, slots, max_group, out, clear, group_scratch);
}

int group_routes(const uint32_t* served_slot, int64_t routes, int64_t slots, int max_group, const RouteGroups& out, int32_t* clear, cudaStream_t s) {
  if (routes > (1 << 20) || slots > 16384) return KEEPVQ_ERR_CAPACITY;
  const size_t smem = static_cast<size_t>(slots) * 3 * sizeof(int32_t);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(group_routes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
  }
  cudaError_t err = launch_after(routes <= 4 * EARLY_LAUNCH_MAX_BLOCKS, group_routes_kernel, 1, GR_THREADS, smem, s, served_slot, static_cast<int>(routes), static_cast<int>(slots), max_group, out, clear);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

// ------------------------------------------------------------------------------------------
// Which kernel runs a grouped projection.
// ------------------------------------------------------------------------------------------
constexpr int CHUNK_CODES = 32;               // codewords of a row a warp consumes per step: inputs come in multiples of 256

bool shapes_supported(int64_t out_dim, int64_t in_dim, int64_t groups) {
  if (in_dim % (8 * CHUNK_CODES) != 0 || groups <= 0) return false;
  const int64_t chunks = in_dim / (8 * CHUNK_CODES);
  return chunks % groups == 0 && out_dim > 0;
}

// Enough routes to give every CTA of the machine its own (group, slab) items, and activations
// that fit the shared-memory stage?
static bool many_items(const FastProjectionArgs& p) {
  return p.max_routes >= SMALL_CALL_ROUTES && p.in_dim <= slab_max_in_dim(p.group_cols > PAIRED_GROUP_ROUTES ? MAX_GROUP_ROUTES : PAIRED_GROUP_ROUTES);
}
// Few route groups of at most four routes.  Small calls run the sweep kernel (measured on a B200 at
// 4096 inputs: ahead of the split slab kernel up to four tokens of top-6, behind it at eight); the
// rest, and every layer with a residual tier (the slab kernels hold the residual pass), the split
// form of the slab kernel when the activations leave it room.  0 = neither, 1 = split slab, 2 = sweep.
static int few_items(const FastProjectionArgs& p) {
  if (!p.few_groups || p.group_cols > PAIRED_GROUP_ROUTES) return 0;
  const bool split_fits = p.in_dim <= slab_split_max_in_dim(), sweep_fits = !p.res_table && sweep_supported(p.in_dim);
  if (p.few_groups == 2 && sweep_fits) return 2;
  return split_fits ? 1 : sweep_fits ? 2 : 0;
}

#ifdef KEEPVQ_DIAG
static int g_force_cols = 0;
extern "C" void keepvq_diag_set_group_cols(int cols) { g_force_cols = cols; }
#endif

int decode_group_routes(int64_t live, int64_t slots, int64_t widest_in_dim) {
#ifdef KEEPVQ_DIAG
  if (g_force_cols) return g_force_cols;
#endif
  if (live < SMALL_CALL_ROUTES) return PAIRED_GROUP_ROUTES;  // the sweep kernel (the split slab kernel with a residual tier)
  if (widest_in_dim > slab_max_in_dim(MAX_GROUP_ROUTES)) return PAIRED_GROUP_ROUTES;
  return live <= 2 * slots ? PAIRED_GROUP_ROUTES : MAX_GROUP_ROUTES;
}

// The residual pass lives in the slab kernels only: a layer with a residual tier needs activations
// that fit their stage (three quarters of it for calls with few routes) and residual scale groups
// that close on chunk boundaries.
bool residual_supported(int64_t routes, int64_t in_dim, int64_t res_groups) {
  const int64_t widest = routes < SMALL_CALL_ROUTES ? slab_split_max_in_dim() : slab_max_in_dim(PAIRED_GROUP_ROUTES);
  if (in_dim > widest || in_dim % (8 * CHUNK_CODES) != 0 || res_groups <= 0) return false;
  return (in_dim / (8 * CHUNK_CODES)) % res_groups == 0;
}

int gate_up(const FastProjectionArgs& p, cudaStream_t s) {
  if (const int few = few_items(p)) return few == 2 ? sweep_gate_up(p, s) : slab_split_gate_up(p, s);
  if (!many_items(p)) return KEEPVQ_ERR_UNSUPPORTED;
  return slab_gate_up(p, p.group_cols > PAIRED_GROUP_ROUTES ? MAX_GROUP_ROUTES : PAIRED_GROUP_ROUTES, s);
}
int down(const FastProjectionArgs& p, cudaStream_t s) {
  if (const int few = few_items(p)) return few == 2 ? sweep_down(p, s) : slab_split_down(p, s);
  if (!many_items(p)) return KEEPVQ_ERR_UNSUPPORTED;
  return slab_down(p, p.group_cols > PAIRED_GROUP_ROUTES ? MAX_GROUP_ROUTES : PAIRED_GROUP_ROUTES, s);
}

}  // namespace fast
}  // namespace keepvq
