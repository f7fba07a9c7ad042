// Internal interface of the tensor-core decode path (moe_fast.cu), used by moe_layer.cu.
//
// The idea.  A 16-bit E8P codeword decodes to eight weights w = s*h/2 + p/4, with h an odd
// integer from the abs table (|h| in {1,3,5}), s the sign bit and p = +-1 by the parity of the
// sign byte.  Then 4w = 2q + 1 for the integer q = h ^ (neg ? 0xFE : 0) ^ parity, which is pure
// bit arithmetic on a byte.  So a row's dot product with integer activations x' is
//     4 * sum_k w_k x'_k = 2 * sum_k q_k x'_k + sum_k x'_k,
// an exact int8 tensor-core product plus one per-token constant.  Activations are quantised per
// row to 16-bit fixed point (power-of-two scale) and fed as two signed bytes (x' = 256 hi + lo).
// The only rounding in a projection is that fixed-point step.  The kernels hand the tensor cores
// u = q + 8 (a 4-bit unsigned value, two table words XORed) and take 8 * sum(x') off afterwards.
#pragma once

#include "common.cuh"

namespace keepvq {
namespace fast {

constexpr int MAX_GROUP_ROUTES = 8;     // routes of one expert that share an mma.sync tile (its 8 columns)
constexpr int SMALL_CALL_ROUTES = 48;   // calls with fewer routes never run the plain slab kernel
constexpr int FEW_ROUTE_GROUPS = 96;    // below this many route groups a CTA's warps share rows AND inputs (sweep kernel, split slab kernel)
constexpr int PAIRED_GROUP_ROUTES = 4;  // ... when a route's two byte planes take a column each (one MMA per step)
constexpr int PREFILL_GROUP_ROUTES = 96;   // routes of one expert per tcgen05 item (its accumulators and two operand stages fill tensor memory)


// ------------------------------------------------------------------------------------------
// The codeword decoder shared by the decode kernels (projection_slab.cu, projection_sweep.cu) and
// the tcgen05 kernel (prefill_umma.cu), and the entries its tables are built from.
// Entry bytes: byte j of the low word is table nibble 3 - j, of the high word nibble 7 - j.
// ------------------------------------------------------------------------------------------
// The eight bytes q (4w = 2q + 1 for positive signs) of abs row `word` under one parity.
__device__ __forceinline__ uint2 abs_table_entry(uint32_t word, uint32_t par) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int nl = 3 - j, nh = 7 - j;
    uint32_t hl = ((word >> (4 * nl)) & 0xFu) - 8u, hh = ((word >> (4 * nh)) & 0xFu) - 8u;
    if (par) { hl = nl == 0 ? ~hl : hl ^ 1u; hh ^= 1u; }
    lo |= (hl & 0xFFu) << (8 * j);
    hi |= (hh & 0xFFu) << (8 * j);
  }
  return make_uint2(lo, hi);
}
// The XOR masks of sign byte `sb`: 0xFE where the sign bit is set; ^1 everywhere (^0xFF on nibble 0) on odd parity.
__device__ __forceinline__ uint2 sign_table_entry(uint32_t sb) {
  const uint32_t par = __popc(sb) & 1u;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int nl = 3 - j, nh = 7 - j;
    uint32_t ml = ((sb >> nl) & 1u) ? 0xFEu : 0u, mh = ((sb >> nh) & 1u) ? 0xFEu : 0u;
    if (par) { ml ^= nl == 0 ? 0xFFu : 0x01u; mh ^= 0x01u; }
    lo |= ml << (8 * j);
    hi |= mh << (8 * j);
  }
  return make_uint2(lo, hi);
}

__device__ __forceinline__ uint2 table_entry(uint32_t addr) {  // tables never change after the set-up barrier: free to schedule
  uint2 v;
  asm("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// The nibble decoder.  Both tables hold an entry as eight 4-bit values in ONE word, u = q + 8 for the
// abs table (even parity) and the XOR masks of the sign byte for the other (4-bit XOR on q + 8 is
// the same as on q), 32 replicas each, interleaved in one 64 KB region on a 64 KB boundary:
//   abs entry  at region + abs byte * 256 + lane * 4,   sign entry at region + 128 + sign byte * 256 + lane * 4,
// so each address is one byte permute and each read one shared-memory wavefront (an 8-byte entry
// costs two).  The operand bytes are u (0..15, an UNSIGNED A operand); the caller
// takes 8 * sum(x') off the integer dot product to get back to sum(q x').
template <bool ODD>
__device__ __forceinline__ void decode_codeword_nibble(uint32_t word, uint32_t abs_lane, uint32_t sign_lane, uint32_t& lo, uint32_t& hi) {
  uint32_t e, m;
  asm("ld.shared.u32 %0, [%1];" : "=r"(e) : "r"(__byte_perm(word, abs_lane, ODD ? 0x7634 : 0x7614)));
  asm("ld.shared.u32 %0, [%1];" : "=r"(m) : "r"(__byte_perm(word, sign_lane, ODD ? 0x7624 : 0x7604)));
  // (e ^ m) & mask as ONE three-input logic operation each (written out: the compiler otherwise
  // turns the second into a shift and two operations), and one shift
  uint32_t top;
  asm("lop3.b32 %0, %1, %2, 0x0F0F0F0F, 0x28;" : "=r"(lo) : "r"(e), "r"(m));
  asm("lop3.b32 %0, %1, %2, 0xF0F0F0F0, 0x28;" : "=r"(top) : "r"(e), "r"(m));
  hi = top >> 4;
}
__device__ __forceinline__ uint32_t pack_nibbles(uint2 v) { return (v.x & 0x0F0F0F0Fu) | ((v.y & 0x0F0F0F0Fu) << 4); }
// All `threads` threads of the CTA (whole warps) fill the 64 KB region at `region` (shared address on
// a 64 KB boundary): a thread works out one entry (one load of the codebook, all in flight together),
// then its warp writes its 32 entries one after the other, the 32 replicas of an entry side by side.
__device__ __forceinline__ void build_nibble_tables(uint32_t region, const uint32_t* __restrict__ codebook, int tid, int threads) {
  const int lane = tid & 31;
  for (int base = 0; base < 512; base += threads) {
    const int e = base + tid;
    uint32_t v = 0;
    if (e < 256) v = pack_nibbles(abs_table_entry(codebook[e], 0)) ^ 0x88888888u;
    else if (e < 512) v = pack_nibbles(sign_table_entry(e - 256));
    const int first = e - lane;  // the warp's first entry
#pragma unroll 8
    for (int i = 0; i < 32; ++i) {
      const uint32_t vi = __shfl_sync(0xFFFFFFFFu, v, i);
      const int ee = first + i;
      if (ee < 512) asm volatile("st.shared.u32 [%0], %1;" ::"r"(region + (ee & 255) * 256 + (ee >> 8) * 128 + lane * 4), "r"(vi) : "memory");
    }
  }
}
// Quantised activation rows: the B operand of the projections.
struct QuantRows {
  uint8_t* q;       // [rows + 1, in_dim/8, 16] (last row all zero): per codeword 4 words: hi(dims 6,4,2,0) hi(7,5,3,1) lo(...) lo(...)
  float* scale;     // [rows + 1] power of two: x ~= scale * x'
  int32_t* sums;    // [rows + 1, groups] sum of x' over each scale group
  int32_t* chunk_sums;  // [rows + 1, in_dim / 256] sum of x' over every 256 inputs, or null: for kernels whose warps split a scale group
};

// Routes grouped by the slot they are served from.
struct RouteGroups {
  int32_t* count;        // [2] number of groups, number of routes in them (the live ones)
  int32_t* slot;         // [max_groups]
  int32_t* start;        // [max_groups] first entry in `routes`
  int32_t* size;         // [max_groups] 1..max_group
  int32_t* routes;       // [routes] route ids ordered by group
};

// ------------------------------------------------------------------------------------------
// Route grouping: routes that are served from the same slot share the code stream.  One block;
// counting sort by slot, then each slot's routes are cut into groups of at most max_group.
// ------------------------------------------------------------------------------------------
// One block of THREADS threads (a multiple of 32, at most 1024); `sm`: 3 * slots ints of shared memory.
template <int THREADS>
__device__ __forceinline__ void group_routes_block(const uint32_t* __restrict__ served_slot, int routes, int slots, int max_group, const RouteGroups& out, int32_t* clear, int32_t* sm) {
  constexpr int GR_THREADS = THREADS;
  if (clear && threadIdx.x == 0) *clear = 0;
  int32_t* count = sm;               // [slots] routes per slot, then running cursor
  int32_t* first = sm + slots;       // [slots] first position of the slot in `routes`
  int32_t* gfirst = sm + 2 * slots;  // [slots] first group index of the slot
  __shared__ int32_t warp_a[32], warp_b[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int s = tid; s < slots; s += GR_THREADS) count[s] = 0;
  __syncthreads();
  for (int r = tid; r < routes; r += GR_THREADS) {
    const uint32_t s = served_slot[r];
    if (s < static_cast<uint32_t>(slots)) atomicAdd(&count[s], 1);
  }
  __syncthreads();
  // exclusive scans of (routes, groups) per slot: each thread owns a contiguous run of slots
  const int per = (slots + GR_THREADS - 1) / GR_THREADS;
  const int lo = min(tid * per, slots), hi = min(lo + per, slots);
  int a = 0, b = 0;
  for (int s = lo; s < hi; ++s) { a += count[s]; b += (count[s] + max_group - 1) / max_group; }
  int ia = a, ib = b;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int ta = __shfl_up_sync(0xFFFFFFFFu, ia, o), tb = __shfl_up_sync(0xFFFFFFFFu, ib, o);
    if (lane >= o) { ia += ta; ib += tb; }
  }
  if (lane == 31) { warp_a[warp] = ia; warp_b[warp] = ib; }
  __syncthreads();
  if (warp == 0) {
    int wa = lane < THREADS / 32 ? warp_a[lane] : 0, wb = lane < THREADS / 32 ? warp_b[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int ta = __shfl_up_sync(0xFFFFFFFFu, wa, o), tb = __shfl_up_sync(0xFFFFFFFFu, wb, o);
      if (lane >= o) { wa += ta; wb += tb; }
    }
    warp_a[lane] = wa; warp_b[lane] = wb;
  }
  __syncthreads();
  int base_a = ia - a + (warp ? warp_a[warp - 1] : 0), base_b = ib - b + (warp ? warp_b[warp - 1] : 0);
  for (int s = lo; s < hi; ++s) {
    first[s] = base_a; gfirst[s] = base_b;
    const int c = count[s], g = (c + max_group - 1) / max_group;
    for (int i = 0; i < g; ++i) {
      out.slot[base_b + i] = s;
      out.start[base_b + i] = base_a + i * max_group;
      out.size[base_b + i] = min(max_group, c - i * max_group);
    }
    base_a += c; base_b += g;
  }
  if (tid == GR_THREADS - 1) { out.count[0] = warp_b[31]; out.count[1] = warp_a[31]; }  // groups, grouped (live) routes
  __syncthreads();
  for (int s = tid; s < slots; s += GR_THREADS) count[s] = 0;  // reuse as cursors
  __syncthreads();
  for (int r = tid; r < routes; r += GR_THREADS) {
    const uint32_t s = served_slot[r];
    if (s < static_cast<uint32_t>(slots)) out.routes[first[s] + atomicAdd(&count[s], 1)] = r;
  }
}

struct Projection {
  const uint16_t* codes;  // [slots, out_dim, in_dim/8]
  const void* scales;     // [slots, out_dim, groups]
  const uint8_t* res_codes;  // [hot rows, out_dim, in_dim/8] 8-bit residual codes, or nullptr
  const void* res_scales;    // [hot rows, out_dim, res_groups]
};

struct FastProjectionArgs {
  Projection a;           // gate (or down)
  Projection b;           // up, or {nullptr, nullptr} for a single projection
  int32_t scales_dtype;
  int64_t out_dim, in_dim, groups;
  const uint32_t* codebook;
  QuantRows x;            // activations
  int64_t x_zero_row;     // index of the all-zero row quantize_rows appends
  int32_t x_div;          // activation row of route r is r / x_div
  RouteGroups groups_of_routes;
  const float* route_weight;  // [routes] gate weight (gate/up only)
  float swiglu_limit;
  void* out;              // [routes, out_dim]
  int32_t out_dtype;
  int64_t max_routes;
  int32_t* status;        // device word a kernel sets when it gives up (bounded wait expired: 1; unexpected shared window: 2), or null
  int32_t group_cols;     // most routes a group holds: PAIRED_GROUP_ROUTES or MAX_GROUP_ROUTES (what group_routes was given)
  int32_t few_groups;     // what few_route_groups said of the call: 0 many route groups, 1 few, 2 a small call
  // nested residual tier (all null / 0 when the layer has none): slot s adds the 8-bit residual of
  // row hot_of_slot[s] unless that is 0xFFFFFFFF.  res_table is [256][4] fp16 pairs (dims 2k, 2k+1).
  int64_t res_groups;
  const uint32_t* hot_of_slot;
  const uint32_t* res_table;
};

// True when the shapes fit the tensor-core path (in_dim % 256 == 0, group size % 256 == 0, ...).
bool shapes_supported(int64_t out_dim, int64_t in_dim, int64_t groups);
// True when gate_up / down can also add a nested residual with these scale groups to `routes` routes.
bool residual_supported(int64_t routes, int64_t in_dim, int64_t res_groups);

// planes = false: 16 bytes per codeword (hi 8, lo 8), what the mma.sync kernels read;
// planes = true: all high bytes [rows + 1, in_dim] then all low bytes (quantize_rows_sorted writes that form).
// live_slot (may be null): [rows, per_row] slots of the routes that read the rows; rows whose routes are all dead (slot >= slots) are skipped.
int quantize_rows(const void* x, int32_t x_dtype, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, bool planes, cudaStream_t s,
                  const uint32_t* live_slot = nullptr, int32_t per_row = 1, int64_t slots = 0);
// What the tcgen05 kernels' TMA boxes copy: byte planes (all high bytes [rows + 1, in_dim], then all
// low bytes) with the rows IN GROUPED ORDER: output row r is input row sorted.routes[r] / x_div for
// r below sorted.count[1] (group_routes must have run), rows beyond that are left alone; scale and
// sums are per output row.
struct SortedRows { const int32_t* routes; const int32_t* count; int32_t x_div; };
int quantize_rows_sorted(const void* x, int32_t x_dtype, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, const SortedRows& sorted, cudaStream_t s);
// `clear` (may be null): a status word the kernel zeroes for the projection kernels that follow it.
// The router's logits and quantize_rows (planes = false) of the same token rows in one launch, for
// calls of at most FRONT_MAX_TOKENS tokens with fp16 / bf16 activations.
constexpr int64_t FRONT_MAX_TOKENS = 23;  // from 24 tokens on the logits have a faster kernel of their own (router.cu)
bool logits_and_quantize_supported(const keepvq_router_logits_args& logits, int64_t groups);
int logits_and_quantize(const keepvq_router_logits_args& logits, int64_t groups, const QuantRows& out, cudaStream_t s);
// quantize_rows with one more block that groups the routes (group_routes): calls of at most 4096 routes.
bool group_with_quantize_supported(int64_t routes, int64_t slots);
int quantize_rows_and_group(const void* x, int32_t x_dtype, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, bool planes, cudaStream_t s,
                            const uint32_t* live_slot, int32_t per_row, int64_t slots,
                            const uint32_t* served_slot, int64_t routes, int max_group, const RouteGroups& route_groups, int32_t* clear);
int group_routes(const uint32_t* served_slot, int64_t routes, int64_t slots, int max_group, const RouteGroups& out, int32_t* clear, cudaStream_t s);
// Routes per group for a decode call: four while experts rarely get more (the kernels then run one
// MMA per step for both byte planes), eight beyond.  `live` = routes expected to carry a slot.
int decode_group_routes(int64_t live, int64_t slots, int64_t widest_in_dim);
// Whether a decode call with `live` routes over `slots` experts forms few route groups: 0 no, 1 yes, 2 a small call.
inline int few_route_groups(int64_t live, int64_t slots) { return live < SMALL_CALL_ROUTES ? 2 : (live < slots ? live : slots) < FEW_ROUTE_GROUPS ? 1 : 0; }
int gate_up(const FastProjectionArgs& args, cudaStream_t s);   // h = round(silu(G) * U * weight)
int down(const FastProjectionArgs& args, cudaStream_t s);      // out = round(W2 h)

// The persistent slab kernels behind gate_up / down for calls with many route groups (projection_slab.cu).
int slab_max_in_dim(int cols);
int slab_gate_up(const FastProjectionArgs& args, int cols, cudaStream_t s);
int slab_down(const FastProjectionArgs& args, int cols, cudaStream_t s);
// ... and their split form for calls with few route groups (groups of at most four routes).
int slab_split_max_in_dim();
int slab_split_gate_up(const FastProjectionArgs& args, cudaStream_t s);
int slab_split_down(const FastProjectionArgs& args, cudaStream_t s);
// The sweep kernels for calls with few route groups and no residual tier (projection_sweep.cu):
// inputs of any width in multiples of 256.
bool sweep_supported(int64_t in_dim);
int sweep_gate_up(const FastProjectionArgs& args, cudaStream_t s);
int sweep_down(const FastProjectionArgs& args, cudaStream_t s);

// tcgen05 kernels for many routes per expert (prefill_umma.cu).  `status` is a device word that
// a CTA sets to 1 if one of its bounded waits expires.
bool prefill_supported(int64_t out_dim, int64_t in_dim, int64_t groups);
int prefill_gate_up(const FastProjectionArgs& args, int32_t* status, cudaStream_t s);
int prefill_down(const FastProjectionArgs& args, int32_t* status, cudaStream_t s);
// One CTA whose activation loaders never publish, with a deadline of wait_ns: the wait runs out, the CTA sets *status = 1 and returns.
int prefill_wait_selftest(const FastProjectionArgs& args, int32_t* status, uint64_t wait_ns, cudaStream_t s);

}  // namespace fast
}  // namespace keepvq
