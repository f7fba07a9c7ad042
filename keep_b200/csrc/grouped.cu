// One expert-grouped projection over routes, on the int8 tensor-core kernels: the operator-level
// counterpart of the reference's sorted-route prefill kernels
// (src/ramp/kernels/gather_vqmm.py:597-928, native/vq_nax_ext/kernels/nax_fp16_matmul.metal:904-1062).
//
// out[r] = W[rhs[r]] @ x[r] for r < routes; x holds one activation row per route (the caller
// gathers them, as the reference does before its kernels, src/ramp/ops/vq_switch.py:758-761).
// The sequence is the down projection of the layer call: quantise the rows, group the routes by
// expert on the device, then the tcgen05 kernel (24 or more routes per expert on average) or the
// mma.sync one.  Routes need not be sorted; a route with expert 0xFFFFFFFF gives a zero row.
#include "moe_fast.cuh"

namespace keepvq {

struct GroupedScratch {
  int64_t xq, xscale, xsums, gcount, gslot, gstart, gsize, groutes, status, total;
};

static inline int64_t up256(int64_t v) { return (v + 255) / 256 * 256; }

// The grouped kernels never touch the output row of a route that names no expert: this does.
__global__ void __launch_bounds__(128) zero_dead_rows_kernel(const uint32_t* __restrict__ rhs, int64_t slots, void* out, int64_t row_bytes) {
  if (rhs[blockIdx.x] < static_cast<uint64_t>(slots)) return;
  uint8_t* row = reinterpret_cast<uint8_t*>(out) + static_cast<int64_t>(blockIdx.x) * row_bytes;
  for (int64_t i = threadIdx.x * 2; i < row_bytes; i += 256) *reinterpret_cast<uint16_t*>(row + i) = 0;
}

static GroupedScratch plan_grouped(int64_t routes, int64_t in_dim) {
  GroupedScratch s;
  int64_t at = 0;
  s.xq = at;      at += up256((routes + 1) * in_dim * 2);
  s.xscale = at;  at += up256((routes + 1) * 4);
  s.xsums = at;   at += up256((routes + 1) * (in_dim / 8) * 4);
  s.gcount = at;  at += 256;
  s.gslot = at;   at += up256(routes * 4);
  s.gstart = at;  at += up256(routes * 4);
  s.gsize = at;   at += up256(routes * 4);
  s.groutes = at; at += up256(routes * 4);
  s.status = at;  at += 256;
  s.total = at;
  return s;
}

}  // namespace keepvq

extern "C" int64_t keepvq_grouped_projection_workspace_bytes(int64_t routes, int64_t in_dim) {
  if (routes < 0 || in_dim <= 0 || in_dim % 8) return KEEPVQ_ERR_SHAPE;
  return keepvq::plan_grouped(routes, in_dim).total;
}

extern "C" int64_t keepvq_grouped_projection_status_offset(int64_t routes, int64_t in_dim) {
  if (routes < 0 || in_dim <= 0 || in_dim % 8) return KEEPVQ_ERR_SHAPE;
  return keepvq::plan_grouped(routes, in_dim).status;
}

extern "C" int keepvq_grouped_projection(const keepvq_grouped_projection_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_grouped_projection_args& a = *args;
  if (!valid_dtype(a.x_dtype) || !valid_dtype(a.scales_dtype)) return KEEPVQ_ERR_DTYPE;
  if (a.routes < 0 || a.slots <= 0 || a.out_dim <= 0 || a.in_dim <= 0 || a.in_dim % 8 || a.groups <= 0) return KEEPVQ_ERR_SHAPE;
  if (a.routes == 0) return KEEPVQ_OK;
  if (!a.x || !a.rhs || !a.codes || !a.scales || !a.codebook || !a.out || !a.workspace) return KEEPVQ_ERR_NULL;
  if (a.x_dtype == KEEPVQ_F32) return KEEPVQ_ERR_UNSUPPORTED;  // these kernels keep 16 bits of a row: not what an fp32 caller asked for
  if (!a.codebook_all_odd || !fast::shapes_supported(a.out_dim, a.in_dim, a.groups)) return KEEPVQ_ERR_UNSUPPORTED;
  const int32_t x_div = a.x_div > 0 ? a.x_div : 1;
  if (a.routes % x_div) return KEEPVQ_ERR_SHAPE;
  const int64_t x_rows = a.routes / x_div;
  const bool residual = a.res_codes != nullptr;
  if (residual) {
    if (!a.res_scales || !a.res_table || !a.hot_of_slot) return KEEPVQ_ERR_NULL;
    if (a.res_rows <= 0 || a.res_groups <= 0) return KEEPVQ_ERR_SHAPE;
    if (!fast::residual_supported(a.routes, a.in_dim, a.res_groups)) return KEEPVQ_ERR_UNSUPPORTED;
    if (!aligned_to(a.res_codes, 8)) return KEEPVQ_ERR_ALIGN;
  }
  if (!aligned_to(a.x, 16) || !aligned_to(a.codes, 16) || !aligned_to(a.workspace, 256)) return KEEPVQ_ERR_ALIGN;
  const GroupedScratch sc = plan_grouped(a.routes, a.in_dim);
  if (a.workspace_bytes < sc.total) return KEEPVQ_ERR_CAPACITY;
  char* ws = reinterpret_cast<char*>(a.workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  fast::RouteGroups groups = {reinterpret_cast<int32_t*>(ws + sc.gcount), reinterpret_cast<int32_t*>(ws + sc.gslot),
                              reinterpret_cast<int32_t*>(ws + sc.gstart), reinterpret_cast<int32_t*>(ws + sc.gsize),
                              reinterpret_cast<int32_t*>(ws + sc.groutes)};
  const bool many = !residual && a.routes >= 1024 && a.routes >= 24 * a.slots && fast::prefill_supported(a.out_dim, a.in_dim, a.groups);
  // (the sums region has room for a scale group per codeword; these kernels' rows have at most one
  // per 256 inputs, and their sums per 256 inputs go behind those)
  fast::QuantRows xq = {reinterpret_cast<uint8_t*>(ws + sc.xq), reinterpret_cast<float*>(ws + sc.xscale), reinterpret_cast<int32_t*>(ws + sc.xsums),
                        many ? nullptr : reinterpret_cast<int32_t*>(ws + sc.xsums) + (x_rows + 1) * a.groups};
  int32_t* wait_status = reinterpret_cast<int32_t*>(ws + sc.status);
  int rc;
  const int group_cols = many ? fast::PREFILL_GROUP_ROUTES : fast::decode_group_routes(a.routes, a.slots, a.in_dim);
  if ((rc = fast::group_routes(a.rhs, a.routes, a.slots, group_cols, groups, wait_status, s))) return rc;
  if (many) {  // the tcgen05 kernels copy rows in grouped order
    if ((rc = fast::quantize_rows_sorted(a.x, a.x_dtype, a.routes, a.in_dim, a.groups, xq, {groups.routes, groups.count, static_cast<int32_t>(x_div)}, s))) return rc;
  } else if ((rc = fast::quantize_rows(a.x, a.x_dtype, x_rows, a.in_dim, a.groups, xq, false, s))) return rc;
  fast::FastProjectionArgs p = {};
  p.a = {a.codes, a.scales, a.res_codes, a.res_scales}; p.b = {nullptr, nullptr, nullptr, nullptr};
  if (residual) { p.res_groups = a.res_groups; p.hot_of_slot = a.hot_of_slot; p.res_table = a.res_table; }
  p.scales_dtype = a.scales_dtype; p.codebook = a.codebook; p.groups_of_routes = groups; p.max_routes = a.routes; p.group_cols = group_cols; p.status = wait_status;
  p.few_groups = many ? 0 : fast::few_route_groups(a.routes, a.slots);
  p.out_dim = a.out_dim; p.in_dim = a.in_dim; p.groups = a.groups; p.x = xq; p.x_zero_row = many ? a.routes : x_rows; p.x_div = x_div;
  p.out = a.out; p.out_dtype = a.out_dtype; p.swiglu_limit = 0.0f; p.route_weight = nullptr;
  if (a.routes > 0x7FFFFFFFll) return KEEPVQ_ERR_CAPACITY;
  zero_dead_rows_kernel<<<static_cast<unsigned>(a.routes), 128, 0, s>>>(a.rhs, a.slots, a.out, a.out_dim * dtype_size(a.out_dtype));
  KEEPVQ_CHECK_LAUNCH();
  return many ? fast::prefill_down(p, wait_status, s) : fast::down(p, s);
}

// ------------------------------------------------------------------------------------------
// Self-test of the bounded waits of the tcgen05 kernel: one CTA on a tiny problem laid out in the
// caller's scratch, whose activation loaders never publish their tiles.  The MMA issuer's first
// wait then runs into its deadline (wait_ns on the global timer); the CTA must set the status
// word to 1, free its tensor memory and return, and the context must stay usable.  Nothing
// faults and nothing spins without a limit.  No counterpart in the reference.
// ------------------------------------------------------------------------------------------
namespace keepvq {
constexpr int64_t SELFTEST_BYTES = 32 * 1024;
__global__ void selftest_init_kernel(int32_t* count, int32_t* size, int32_t* routes, float* x_scale) {
  if (threadIdx.x == 0) { count[0] = 1; size[0] = 16; }
  if (threadIdx.x < 16) routes[threadIdx.x] = threadIdx.x;
  if (threadIdx.x < 17) x_scale[threadIdx.x] = 1.0f;
}
}  // namespace keepvq

extern "C" int64_t keepvq_wait_selftest_workspace_bytes(void) { return keepvq::SELFTEST_BYTES; }

extern "C" int keepvq_wait_selftest(void* workspace, int64_t workspace_bytes, int64_t wait_ns, void* stream) {
  using namespace keepvq;
  if (!workspace) return KEEPVQ_ERR_NULL;
  if (workspace_bytes < SELFTEST_BYTES) return KEEPVQ_ERR_CAPACITY;
  if (!aligned_to(workspace, 256)) return KEEPVQ_ERR_ALIGN;
  if (wait_ns <= 0 || wait_ns > 1000000000ll) return KEEPVQ_ERR_SHAPE;  // a self-test may hold the GPU for a second at most
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* ws = reinterpret_cast<char*>(workspace);
  cudaError_t e = cudaMemsetAsync(ws, 0, SELFTEST_BYTES, s);
  if (e != cudaSuccess) return note_cuda_error(e);
  // status 0 | groups 256.. | routes 1280 | table 2048 | scales 3072 | codes 4096 | planes 8192 | x scale 16384 | x sums 16640 | out 20480
  fast::RouteGroups groups = {reinterpret_cast<int32_t*>(ws + 256), reinterpret_cast<int32_t*>(ws + 512), reinterpret_cast<int32_t*>(ws + 768),
                              reinterpret_cast<int32_t*>(ws + 1024), reinterpret_cast<int32_t*>(ws + 1280)};
  fast::QuantRows xq = {reinterpret_cast<uint8_t*>(ws + 8192), reinterpret_cast<float*>(ws + 16384), reinterpret_cast<int32_t*>(ws + 16640), nullptr};
  selftest_init_kernel<<<1, 32, 0, s>>>(groups.count, groups.size, groups.routes, xq.scale);
  KEEPVQ_CHECK_LAUNCH();
  fast::FastProjectionArgs p = {};
  p.a = {reinterpret_cast<const uint16_t*>(ws + 4096), ws + 3072, nullptr, nullptr};
  p.scales_dtype = KEEPVQ_F16; p.out_dim = 128; p.in_dim = 128; p.groups = 1;
  p.codebook = reinterpret_cast<const uint32_t*>(ws + 2048);
  p.x = xq; p.x_zero_row = 16; p.x_div = 1; p.groups_of_routes = groups; p.max_routes = 16; p.group_cols = fast::PREFILL_GROUP_ROUTES;
  p.out = ws + 20480; p.out_dtype = KEEPVQ_BF16;
  return fast::prefill_wait_selftest(p, reinterpret_cast<int32_t*>(ws), static_cast<uint64_t>(wait_ns), s);
}
