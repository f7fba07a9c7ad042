// Tensor-core decode path for the routed E8P experts: activation quantisation, route grouping
// and the grouped projection kernels.  See moe_fast.cuh for the arithmetic identity it rests on.
//
// Projection kernel layout (HBM-bound: every code byte is read once per group of routes):
//   - persistent CTAs, one per SM, 16 warps = 2 teams of 8.  A team takes a work item = (route
//     group, block of 32 or 64 output rows) and splits the input dimension across its 8 warps in
//     chunks of 32 codewords; partial sums meet in shared memory in a fixed order.
//   - a lane loads 16 bytes (8 codewords) per row per chunk, straight to registers
//     (ld.global.nc, no L1 allocation): 4 lanes cover 64 contiguous bytes of a row.
//   - a codeword becomes the A fragment of one m16n8k32 int8 MMA with: one popc, one 8-byte
//     shared-memory read from a table indexed by (abs row, parity), two integer multiplies that
//     spread the eight sign bits to byte tops, two byte-permutes that widen them to byte masks,
//     two XORs.  The table is replicated 16x so lanes never share a bank.
//   - the K order inside an MMA is permuted (byte j of the low word is table nibble 3-j, of the
//     high word nibble 7-j); the activations are stored in that same order by quantize_rows.
//   - accumulation is exact in int32; one conversion to fp32 per scale group.
#include <stdlib.h>

#include <algorithm>

#include "moe_fast.cuh"

namespace keepvq {
namespace fast {

// ------------------------------------------------------------------------------------------
// Activation quantisation: x -> 16-bit fixed point with a power-of-two scale per row.
// ------------------------------------------------------------------------------------------
template <typename XT>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const XT* __restrict__ x, int64_t rows, int64_t in_dim, int64_t groups, QuantRows out, int planes) {
  grid_launch_dependents();
  grid_wait();
  __shared__ float warp_max[8];
  __shared__ float row_scale;
  extern __shared__ int32_t group_sum[];
  const int64_t row = blockIdx.x, cw = in_dim / 8, per_group = cw / groups;
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
    if (threadIdx.x == 0) out.scale[row] = 1.0f;
    return;
  }
  const XT* xr = x + row * in_dim;
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

int quantize_rows(const void* x, int32_t x_dtype, int64_t rows, int64_t in_dim, int64_t groups, const QuantRows& out, bool planes, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(groups) * sizeof(int32_t);
  if (smem > 40 * 1024) return KEEPVQ_ERR_CAPACITY;
  const unsigned grid = static_cast<unsigned>(rows + 1);  // + the zero row
  const bool early = rows < EARLY_LAUNCH_MAX_BLOCKS;
  cudaError_t err;
  if (x_dtype == KEEPVQ_F32) err = launch_after(early, quantize_rows_kernel<float>, grid, 256, smem, s, reinterpret_cast<const float*>(x), rows, in_dim, groups, out, planes ? 1 : 0);
  else if (x_dtype == KEEPVQ_F16) err = launch_after(early, quantize_rows_kernel<__half>, grid, 256, smem, s, reinterpret_cast<const __half*>(x), rows, in_dim, groups, out, planes ? 1 : 0);
  else err = launch_after(early, quantize_rows_kernel<__nv_bfloat16>, grid, 256, smem, s, reinterpret_cast<const __nv_bfloat16*>(x), rows, in_dim, groups, out, planes ? 1 : 0);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

// ------------------------------------------------------------------------------------------
// Route grouping: routes that are served from the same slot share the code stream.  One block;
// counting sort by slot, then each slot's routes are cut into groups of at most 8.
// ------------------------------------------------------------------------------------------
constexpr int GR_THREADS = 1024;

__global__ void __launch_bounds__(GR_THREADS) group_routes_kernel(const uint32_t* __restrict__ served_slot, int routes, int slots, int max_group, RouteGroups out) {
  grid_launch_dependents();
  grid_wait();
  extern __shared__ int32_t sm[];
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
    int wa = warp_a[lane], wb = warp_b[lane];
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
  if (tid == GR_THREADS - 1) out.count[0] = warp_b[31];
  __syncthreads();
  for (int s = tid; s < slots; s += GR_THREADS) count[s] = 0;  // reuse as cursors
  __syncthreads();
  for (int r = tid; r < routes; r += GR_THREADS) {
    const uint32_t s = served_slot[r];
    if (s < static_cast<uint32_t>(slots)) out.routes[first[s] + atomicAdd(&count[s], 1)] = r;
  }
}

int group_routes(const uint32_t* served_slot, int64_t routes, int64_t slots, int max_group, const RouteGroups& out, cudaStream_t s) {
  if (routes > (1 << 20) || slots > 16384) return KEEPVQ_ERR_CAPACITY;
  const size_t smem = static_cast<size_t>(slots) * 3 * sizeof(int32_t);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(group_routes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
  }
  cudaError_t err = launch_after(routes <= 4 * EARLY_LAUNCH_MAX_BLOCKS, group_routes_kernel, 1, GR_THREADS, smem, s, served_slot, static_cast<int>(routes), static_cast<int>(slots), max_group, out);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

// ------------------------------------------------------------------------------------------
// Grouped projections on the int8 tensor cores.
// ------------------------------------------------------------------------------------------
constexpr int TEAM_WARPS = 8;
constexpr int TEAMS = 2;
constexpr int CTA_THREADS = TEAMS * TEAM_WARPS * 32;
constexpr int CHUNK_CODES = 32;               // codewords of a row one warp consumes per step
constexpr int LUT_REPLICAS = 16;
constexpr int LUT_BYTES = 2 * 256 * LUT_REPLICAS * 8;  // [abs row][parity][replica] 8-byte entries
// Spreads of the sign byte: S * SPREAD_LO puts sign bits 3,2,1,0 on bits 7,15,23,31 and
// S * SPREAD_HI puts bits 7,6,5,4 there; the shifted copies of S never overlap, so no carries.
constexpr uint32_t SPREAD_LO = (1u << 4) | (1u << 13) | (1u << 22) | (1u << 31);
constexpr uint32_t SPREAD_HI = 1u | (1u << 9) | (1u << 18) | (1u << 27);

__device__ __forceinline__ uint32_t top_bits_to_byte_masks(uint32_t v) {
  uint32_t m;  // selector nibble 8+j: replicate the top bit of byte j over the output byte
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(v), "r"(0u), "r"(0xBA98u));
  return m;
}

__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// One codeword -> two A-fragment words.  `sign` is its low byte, `abs_off` its high byte * 256,
// `lut_lane` the 32-bit shared-memory address of this lane's replica.
// q = table[abs][parity] ^ (neg ? 0xFE : 0).
__device__ __forceinline__ void decode_to_fragment(uint32_t lut_lane, uint32_t sign, uint32_t abs_off, uint32_t& lo, uint32_t& hi) {
  const uint32_t parity_off = (__popc(sign) & 1u) << 7;
  uint32_t ex, ey;
  // volatile: keeps the table reads after the code prefetch that precedes them in program order,
  // so the compiler cannot sink that prefetch to the end of the step to save registers
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(ex), "=r"(ey) : "r"(lut_lane + abs_off + parity_off));
  lo = ex ^ (top_bits_to_byte_masks(sign * SPREAD_LO) & 0xFEFEFEFEu);
  hi = ey ^ (top_bits_to_byte_masks(sign * SPREAD_HI) & 0xFEFEFEFEu);
}

__device__ __forceinline__ void team_barrier(int team) {
  asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(TEAM_WARPS * 32) : "memory");
}

template <int M, int TILES>
__global__ void __launch_bounds__(CTA_THREADS, 1) projection_kernel(FastProjectionArgs p) {
  extern __shared__ __align__(16) uint8_t smem[];
  grid_launch_dependents();
  uint8_t* lut = smem;
  constexpr int ACCS = M * TILES * 4;  // fp32 partials per lane
  float* red = reinterpret_cast<float*>(smem + LUT_BYTES);  // [team][warp][ACCS][32]

  // ---- table: entry (abs, parity) = eight bytes q for a positive sign pattern -----------------
  for (int e = threadIdx.x; e < 512; e += CTA_THREADS) {
    const uint32_t word = p.codebook[e >> 1], par = e & 1;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int nl = 3 - j, nh = 7 - j;
      uint32_t hl = ((word >> (4 * nl)) & 0xFu) - 8u, hh = ((word >> (4 * nh)) & 0xFu) - 8u;
      if (par) { hl = nl == 0 ? ~hl : hl ^ 1u; hh ^= 1u; }
      lo |= (hl & 0xFFu) << (8 * j);
      hi |= (hh & 0xFFu) << (8 * j);
    }
    uint2* dst = reinterpret_cast<uint2*>(lut) + e * LUT_REPLICAS;
#pragma unroll
    for (int r = 0; r < LUT_REPLICAS; ++r) dst[r] = make_uint2(lo, hi);
  }
  grid_wait();  // the tables came from constants; everything below reads what earlier kernels of the stream wrote
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = (threadIdx.x >> 5) % TEAM_WARPS, team = threadIdx.x / (TEAM_WARPS * 32);
  const int g = lane >> 2, t = lane & 3;
  const uint32_t lut_lane = static_cast<uint32_t>(__cvta_generic_to_shared(lut)) + (lane & (LUT_REPLICAS - 1)) * 8;
  float* team_red = red + static_cast<size_t>(team) * TEAM_WARPS * ACCS * 32;
  const int64_t N = p.out_dim, cw = p.in_dim / 8;
  const int n_chunks = static_cast<int>(cw / CHUNK_CODES);
  const int chunks_per_group = n_chunks / static_cast<int>(p.groups);
  const int rows_per_item = 16 * TILES;
  const int row_blocks = static_cast<int>((N + rows_per_item - 1) / rows_per_item);
  const int items = p.groups_of_routes.count[0] * row_blocks;
  const Projection mats[2] = {p.a, p.b};

  for (int item = blockIdx.x * TEAMS + team; item < items; item += gridDim.x * TEAMS) {
    const int gi = item / row_blocks, rb = item - gi * row_blocks;
    const int64_t slot = p.groups_of_routes.slot[gi];
    const int gsize = p.groups_of_routes.size[gi], gstart = p.groups_of_routes.start[gi];
    const int64_t row0 = static_cast<int64_t>(rb) * rows_per_item;
    const int my_route = g < gsize ? p.groups_of_routes.routes[gstart + g] : -1;
    const uint4* bsrc = reinterpret_cast<const uint4*>(p.x.q) + (my_route < 0 ? p.x_zero_row : static_cast<int64_t>(my_route / p.x_div)) * cw;

    float part[M][TILES][4];
    int acc_h[M][TILES][4], acc_l[M][TILES][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int r = 0; r < 4; ++r) { part[m][tl][r] = 0.0f; acc_h[m][tl][r] = 0; acc_l[m][tl][r] = 0; }

    for (int c = warp; c < n_chunks; c += TEAM_WARPS) {
      const int64_t cb = static_cast<int64_t>(c) * CHUNK_CODES + t * 8;
      uint4 codes[M][2 * TILES];
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 2 * TILES; ++j) {
          const int64_t row = min(row0 + 8 * j + g, N - 1);
          codes[m][j] = ld_stream_u4(mats[m].codes + (slot * N + row) * cw + cb);
        }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 b = bsrc[cb + i];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int tl = 0; tl < TILES; ++tl) {
            uint32_t a[4];
#pragma unroll
            for (int half = 0; half < 2; ++half) {  // rows g and g + 8 of the tile
              const uint4 v = codes[m][2 * tl + half];
              const uint32_t word = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
              uint32_t sign, abs_off;
              if (i & 1) {
                asm("prmt.b32 %0, %1, %2, %3;" : "=r"(sign) : "r"(word), "r"(0u), "r"(0x4442u));
                asm("prmt.b32 %0, %1, %2, %3;" : "=r"(abs_off) : "r"(word), "r"(0u), "r"(0x4434u));
              } else {
                sign = word & 0xFFu;
                abs_off = word & 0xFF00u;
              }
              decode_to_fragment(lut_lane, sign, abs_off, a[half], a[2 + half]);
            }
            mma_s8s8(acc_h[m][tl], a[0], a[1], a[2], a[3], b.x, b.y);
            mma_s8s8(acc_l[m][tl], a[0], a[1], a[2], a[3], b.z, b.w);
          }
      }
      // close the scale group when this warp's next chunk belongs to another one
      const int group = c / chunks_per_group;
      if (c + TEAM_WARPS >= n_chunks || (c + TEAM_WARPS) / chunks_per_group != group) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int64_t row = min(row0 + 16 * tl + g + (r >= 2 ? 8 : 0), N - 1);
              const float sc = load_as_float(mats[m].scales, p.scales_dtype, (slot * N + row) * p.groups + group);
              part[m][tl][r] = fmaf(sc, 256.0f * static_cast<float>(acc_h[m][tl][r]) + static_cast<float>(acc_l[m][tl][r]), part[m][tl][r]);
              acc_h[m][tl][r] = 0;
              acc_l[m][tl][r] = 0;
            }
      }
    }

    // ---- meet the other warps of the team ---------------------------------------------------
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int r = 0; r < 4; ++r) team_red[(warp * ACCS + (m * TILES + tl) * 4 + r) * 32 + lane] = part[m][tl][r];
    team_barrier(team);

    const int tid = threadIdx.x % (TEAM_WARPS * 32);
    for (int o = tid; o < TILES * 4 * 32; o += TEAM_WARPS * 32) {
      const int tl = o / 128, r = (o >> 5) & 3, ln = o & 31;
      const int col = 2 * (ln & 3) + (r & 1);
      const int64_t row = row0 + 16 * tl + (ln >> 2) + (r >= 2 ? 8 : 0);
      if (col >= gsize || row >= N) continue;
      const int route = p.groups_of_routes.routes[gstart + col];
      const int64_t xrow = route / p.x_div;
      float y[M];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        float dot = 0.0f;
#pragma unroll
        for (int w = 0; w < TEAM_WARPS; ++w) dot += team_red[(w * ACCS + (m * TILES + tl) * 4 + r) * 32 + ln];
        float shift = 0.0f;  // the +-1/4 of every weight, folded into sum(x') per scale group
        for (int64_t q = 0; q < p.groups; ++q)
          shift = fmaf(load_as_float(mats[m].scales, p.scales_dtype, (slot * N + row) * p.groups + q),
                       static_cast<float>(p.x.sums[xrow * p.groups + q]), shift);
        y[m] = p.x.scale[xrow] * (0.5f * dot + 0.25f * shift);
      }
      float result;
      if (M == 2) {
        // round G and U to the activation dtype first, as the separate kernels of the reference do
        float gt = y[0], up = y[1];
        if (p.out_dtype == KEEPVQ_BF16) { gt = __bfloat162float(__float2bfloat16_rn(gt)); up = __bfloat162float(__float2bfloat16_rn(up)); }
        else if (p.out_dtype == KEEPVQ_F16) { gt = __half2float(__float2half_rn(gt)); up = __half2float(__float2half_rn(up)); }
        if (p.swiglu_limit > 0.0f) { gt = fminf(gt, p.swiglu_limit); up = fminf(fmaxf(up, -p.swiglu_limit), p.swiglu_limit); }
        result = gt / (1.0f + expf(-gt)) * up * p.route_weight[route];
      } else {
        result = y[0];
      }
      store_from_float(p.out, p.out_dtype, static_cast<int64_t>(route) * N + row, result);
    }
    team_barrier(team);  // the reduction buffer is reused by the next item
  }
}

// ------------------------------------------------------------------------------------------
// The same projection for batches with many route groups.  A CTA takes (route group, slab of
// output rows); its 16 warps each own 16*TILES rows of the slab over the whole input dimension,
// so there is no split-K reduction.
//   - Codes stream through a private two-stage cp.async ring per warp (a lane copies and later
//     reads back its own 16-byte pieces), so the next chunk is always in flight behind the one
//     being decoded, whatever order the compiler gives the instructions.
//   - The group's quantised activations (the B operand, up to 64 KB) are staged once per item
//     into shared memory in MMA-fragment order.
//   - Two decoders share the work so that neither the integer pipe nor shared-memory bandwidth
//     is the only limit: the arithmetic one of the team kernel (one table read), and one that
//     reads a second table indexed by the sign byte, whose entry is the XOR mask the arithmetic
//     computes (sign flips, the parity bit of every byte, the extra flip of table nibble 0 on
//     odd parity).  TABLE_STEPS says which steps of a chunk use the second.
// ------------------------------------------------------------------------------------------
constexpr int CK_WARPS = 16;
constexpr int CK_THREADS = CK_WARPS * 32;
constexpr int CK_MAX_CHUNKS = 16;                                   // in_dim <= 4096
constexpr int CK_B_BYTES = CK_MAX_CHUNKS * 8 * 32 * 16;             // 64 KB
constexpr int CK_MAX_CHUNKS_WIDE = 24;                              // in_dim <= 6144: the activations take the sign table's room too
constexpr int CK_ABS_BYTES = LUT_BYTES;                             // 64 KB: [abs row][parity][replica]
constexpr int CK_SIGN_BYTES = 256 * LUT_REPLICAS * 8;               // 32 KB: [sign byte][replica]
constexpr int CK_STAGES = 2;
constexpr unsigned TABLE_STEPS = 0xEEu;  // bit i set: step i of a chunk decodes through the sign table

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// The int8 MMA has a long dependent-accumulate latency (about 290 cycles measured), so each
// (matrix, tile, byte) keeps two accumulators, used by alternate steps, to double the number of
// independent MMA chains in flight.
// MODE 0 is the product.  The others are measurement aids selected by KEEPVQ_PROJECTION_MODE and
// their outputs are meaningless: 1 = loads only, 3 = no decode (raw words into the MMA),
// 4 = no MMA.
template <int M, int TILES, int MODE, bool USE_SIGN_TABLE>
__device__ __forceinline__ void decode_chunk(uint32_t abs_lane, uint32_t sign_lane, const uint4 (&codes)[M][2 * TILES], uint32_t b_addr,
                                             int (&acc_h)[2][M][TILES][4], int (&acc_l)[2][M][TILES][4]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint4 b = lds128(b_addr + i * 512);  // (hi k0-3, hi k16-19, lo k0-3, lo k16-19) of step i
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
        uint32_t a[4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {  // rows g and g + 8 of the tile
          const uint4 v = codes[m][2 * tl + half];
          const uint32_t word = (i >> 1) == 0 ? v.x : (i >> 1) == 1 ? v.y : (i >> 1) == 2 ? v.z : v.w;
          uint32_t sign, abs_off;  // sign byte; abs row * 256 (its even-parity entry, 16 replicas of 8 bytes)
          if (i & 1) {
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(sign) : "r"(word), "r"(0u), "r"(0x4442u));
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(abs_off) : "r"(word), "r"(0u), "r"(0x4434u));
          } else {
            sign = word & 0xFFu;
            abs_off = word & 0xFF00u;
          }
          if (MODE == 3) {
            a[half] = sign;
            a[2 + half] = abs_off;
          } else if (USE_SIGN_TABLE && ((TABLE_STEPS >> i) & 1u)) {
            const uint2 e = lds64(abs_lane + abs_off), x = lds64(sign_lane + (sign << 7));
            a[half] = e.x ^ x.x;
            a[2 + half] = e.y ^ x.y;
          } else {
            decode_to_fragment(abs_lane, sign, abs_off, a[half], a[2 + half]);
          }
        }
        if (MODE == 4) {
#pragma unroll
          for (int r = 0; r < 4; ++r) acc_h[i & 1][m][tl][r] += a[r] ^ b.x;
        } else {
          mma_s8s8(acc_h[i & 1][m][tl], a[0], a[1], a[2], a[3], b.x, b.y);
          mma_s8s8(acc_l[i & 1][m][tl], a[0], a[1], a[2], a[3], b.z, b.w);
        }
      }
  }
}

// NESTED: the layer has a residual tier.  The second table then holds the residual codebook
// instead of the sign masks (the base decode does its signs on the integer pipe in every step),
// and an item whose slot is hot runs a second pass over the residual's 8-bit codes: one table
// read per codeword gives the int8 operand 2v directly (no signs, no parity, no offset term).
// WIDE: input dimensions of 4097..6144 (the shipped artifacts' 5120).  Their staged activations
// need 96 KB, so the sign table goes and every step decodes its signs on the integer pipe.
template <int M, int TILES, int MODE, bool NESTED, bool WIDE = false>
__global__ void __launch_bounds__(CK_THREADS, 1) projection_cta_kernel(FastProjectionArgs p) {
  static_assert(!(NESTED && WIDE), "the residual table and the wide activation stage want the same shared memory");
  extern __shared__ __align__(16) uint8_t smem[];
  grid_launch_dependents();
  // ---- tables -----------------------------------------------------------------------------
  for (int e = threadIdx.x; e < (WIDE ? 512 : 768); e += CK_THREADS) {
    uint32_t lo = 0, hi = 0;
    if (e >= 512 && NESTED) {  // residual entry: byte j of the low word is 2 * v[6 - 2j], of the high word 2 * v[7 - 2j]
      const uint32_t* row = p.res_table + (e - 512) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 pair = *reinterpret_cast<const __half2*>(&row[3 - j]);  // dims 6 - 2j, 7 - 2j
        lo |= (static_cast<uint32_t>(__float2int_rn(2.0f * __low2float(pair))) & 0xFFu) << (8 * j);
        hi |= (static_cast<uint32_t>(__float2int_rn(2.0f * __high2float(pair))) & 0xFFu) << (8 * j);
      }
    } else if (e < 512) {  // abs entry (row e/2, parity e&1): byte j of the low word is table nibble 3-j, of the high word 7-j
      const uint32_t word = p.codebook[e >> 1], par = e & 1;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int nl = 3 - j, nh = 7 - j;
        uint32_t hl = ((word >> (4 * nl)) & 0xFu) - 8u, hh = ((word >> (4 * nh)) & 0xFu) - 8u;
        if (par) { hl = nl == 0 ? ~hl : hl ^ 1u; hh ^= 1u; }
        lo |= (hl & 0xFFu) << (8 * j);
        hi |= (hh & 0xFFu) << (8 * j);
      }
    } else {        // sign entry: 0xFE where the sign bit is set, ^1 everywhere (^0xFF on nibble 0) on odd parity
      const uint32_t sb = e - 512, par = __popc(sb) & 1u;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int nl = 3 - j, nh = 7 - j;
        uint32_t ml = ((sb >> nl) & 1u) ? 0xFEu : 0u, mh = ((sb >> nh) & 1u) ? 0xFEu : 0u;
        if (par) { ml ^= nl == 0 ? 0xFFu : 0x01u; mh ^= 0x01u; }
        lo |= ml << (8 * j);
        hi |= mh << (8 * j);
      }
    }
    uint2* dst = reinterpret_cast<uint2*>(smem) + e * LUT_REPLICAS;  // abs table, then sign table
#pragma unroll
    for (int r = 0; r < LUT_REPLICAS; ++r) dst[r] = make_uint2(lo, hi);
  }

  grid_wait();  // the tables came from constants; everything below reads what earlier kernels of the stream wrote
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t abs_lane = smem_base + (lane & (LUT_REPLICAS - 1)) * 8;
  const uint32_t sign_lane = abs_lane + CK_ABS_BYTES;
  const uint32_t b_base = smem_base + CK_ABS_BYTES + (WIDE ? 0 : CK_SIGN_BYTES);
  constexpr int B_BYTES = CK_B_BYTES + (WIDE ? CK_SIGN_BYTES : 0);
  constexpr int STREAMS = M * 2 * TILES;                 // 16-byte pieces a lane owns per chunk
  constexpr int STAGE_BYTES = STREAMS * 512;             // per warp
  const uint32_t ring = b_base + B_BYTES + warp * (CK_STAGES * STAGE_BYTES) + lane * 16;
  const int64_t N = p.out_dim, cw = p.in_dim / 8;
  const int n_chunks = static_cast<int>(cw / CHUNK_CODES);
  const int chunks_per_group = n_chunks / static_cast<int>(p.groups);
  constexpr int ROWS = 16 * TILES;              // per warp
  constexpr int SLAB = ROWS * CK_WARPS;         // per CTA item
  const int slabs = static_cast<int>((N + SLAB - 1) / SLAB);
  const int items = p.groups_of_routes.count[0] * slabs;
  const Projection mats[2] = {p.a, p.b};

  // A CTA takes a contiguous run of items, so consecutive items mostly belong to one route group
  // and its activations are staged once for all of them.
  // (With a residual tier the items of a hot slot cost half as much again, and a run of them on
  // one CTA would unbalance the grid: those layers deal the items out round-robin instead.)
  const int per_cta = (items + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int first_item = NESTED ? static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x) * per_cta;
  const int last_item = NESTED ? items : min(items, first_item + per_cta);
  const int item_step = NESTED ? static_cast<int>(gridDim.x) : 1;
  int staged_group = -1;
  for (int item = first_item; item < last_item; item += item_step) {
    const int gi = item / slabs, slab = item - gi * slabs;
    const int64_t slot = p.groups_of_routes.slot[gi];
    const int gsize = p.groups_of_routes.size[gi], gstart = p.groups_of_routes.start[gi];
    const int64_t row0 = static_cast<int64_t>(slab) * SLAB + warp * ROWS;
    const bool active = row0 < N;
    const uint16_t* row_ptr[M][2 * TILES];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int j = 0; j < 2 * TILES; ++j)
        row_ptr[m][j] = mats[m].codes + (slot * N + min(row0 + 8 * j + g, N - 1)) * cw + t * 8;
    auto fetch = [&](int c) {  // chunk c of this lane's row streams -> ring stage c % CK_STAGES
      if (active && c < n_chunks) {
        const uint32_t dst = ring + (c % CK_STAGES) * STAGE_BYTES;
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int j = 0; j < 2 * TILES; ++j) cp_async16(dst + (m * 2 * TILES + j) * 512, row_ptr[m][j] + c * CHUNK_CODES);
      }
      cp_async_commit();
    };

    if (gi != staged_group) {
      __syncthreads();  // every warp is done with the previous group's activations (and the tables are built)
      {                 // stage this group's activations in fragment order: [chunk * 8 + step][lane]
        const int route = g < gsize ? p.groups_of_routes.routes[gstart + g] : -1;
        const uint4* src = reinterpret_cast<const uint4*>(p.x.q) + (route < 0 ? p.x_zero_row : static_cast<int64_t>(route / p.x_div)) * cw + t * 8;
        for (int step = warp; step < n_chunks * 8; step += CK_WARPS)
          cp_async16(b_base + lane * 16 + step * 512, src + (step >> 3) * CHUNK_CODES + (step & 7));
        cp_async_commit();
      }
      fetch(0);
      cp_async_wait<1>();  // the activations (the older group) have landed
      __syncthreads();
      staged_group = gi;
    } else {
      fetch(0);
    }
    if (!active) { cp_async_wait<0>(); continue; }

    float part[M][TILES][4];
    int acc_h[2][M][TILES][4], acc_l[2][M][TILES][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          part[m][tl][r] = 0.0f;
          acc_h[0][m][tl][r] = acc_h[1][m][tl][r] = 0;
          acc_l[0][m][tl][r] = acc_l[1][m][tl][r] = 0;
        }
    // what the epilogue needs of this lane's two routes (columns 2t, 2t + 1), asked for now so
    // that the loads fly behind the main loop instead of in front of the stores
    int ep_route[2];
    float ep_xs[2], ep_weight[2], ep_sum[2];
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int col = 2 * t + cc;
      ep_route[cc] = col < gsize ? p.groups_of_routes.routes[gstart + col] : -1;
      const int64_t xrow = ep_route[cc] < 0 ? p.x_zero_row : static_cast<int64_t>(ep_route[cc] / p.x_div);
      ep_xs[cc] = p.x.scale[xrow];
      ep_weight[cc] = (M == 2 && ep_route[cc] >= 0) ? p.route_weight[ep_route[cc]] : 1.0f;
      ep_sum[cc] = static_cast<float>(p.x.sums[xrow * p.groups]);  // the only group when the rows have one scale
    }
    float row_scale[M][TILES][4];  // the last scale group's scale of each accumulator row

    for (int c = 0; c < n_chunks; ++c) {
      fetch(c + 1);
      cp_async_wait<1>();  // chunk c has landed (the younger group may still fly)
      uint4 cur[M][2 * TILES];
      const uint32_t src = ring + (c % CK_STAGES) * STAGE_BYTES;
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 2 * TILES; ++j) cur[m][j] = lds128(src + (m * 2 * TILES + j) * 512);
      if (MODE == 1) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int j = 0; j < 2 * TILES; ++j) acc_h[0][m][j / 2][j & 1] += cur[m][j].x ^ cur[m][j].y ^ cur[m][j].z ^ cur[m][j].w;
      } else {
        decode_chunk<M, TILES, MODE, !NESTED && !WIDE>(abs_lane, sign_lane, cur, b_base + lane * 16 + c * 8 * 512, acc_h, acc_l);
      }
      const int group = c / chunks_per_group;
      if (c + 1 == n_chunks || (c + 1) / chunks_per_group != group) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              const int64_t row = min(row0 + 16 * tl + g + (r >= 2 ? 8 : 0), N - 1);
              const float sc = load_as_float(mats[m].scales, p.scales_dtype, (slot * N + row) * p.groups + group);
              const int hi = acc_h[0][m][tl][r] + acc_h[1][m][tl][r], lo = acc_l[0][m][tl][r] + acc_l[1][m][tl][r];
              part[m][tl][r] = fmaf(sc, 256.0f * static_cast<float>(hi) + static_cast<float>(lo), part[m][tl][r]);
              row_scale[m][tl][r] = sc;
              acc_h[0][m][tl][r] = acc_h[1][m][tl][r] = 0;
              acc_l[0][m][tl][r] = acc_l[1][m][tl][r] = 0;
            }
      }
    }
    cp_async_wait<0>();

    // ---- the residual of a hot slot: a second pass over its 8-bit codes ---------------------
    float rpart[M][TILES][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int r = 0; r < 4; ++r) rpart[m][tl][r] = 0.0f;
    if (NESTED) {
      const uint32_t hot = p.hot_of_slot[slot];
      if (hot != 0xFFFFFFFFu) {
        const int chunks_per_res_group = n_chunks / static_cast<int>(p.res_groups);
        const uint8_t* res_ptr[M][2 * TILES];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int j = 0; j < 2 * TILES; ++j)
            res_ptr[m][j] = mats[m].res_codes + (static_cast<int64_t>(hot) * N + min(row0 + 8 * j + g, N - 1)) * cw + t * 8;
        auto fetch_res = [&](int c) {  // 8 codes of 8 bits per row stream
          if (c < n_chunks) {
            const uint32_t dst = ring + (c % CK_STAGES) * STAGE_BYTES;
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
              for (int j = 0; j < 2 * TILES; ++j)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst + (m * 2 * TILES + j) * 512), "l"(res_ptr[m][j] + c * CHUNK_CODES) : "memory");
          }
          cp_async_commit();
        };
        fetch_res(0);
        for (int c = 0; c < n_chunks; ++c) {
          fetch_res(c + 1);
          cp_async_wait<1>();
          uint2 cur[M][2 * TILES];
          const uint32_t src = ring + (c % CK_STAGES) * STAGE_BYTES;
#pragma unroll
          for (int m = 0; m < M; ++m)
#pragma unroll
            for (int j = 0; j < 2 * TILES; ++j) cur[m][j] = lds64(src + (m * 2 * TILES + j) * 512);
          const uint32_t b_addr = b_base + lane * 16 + c * 8 * 512;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint4 b = lds128(b_addr + i * 512);
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
              for (int tl = 0; tl < TILES; ++tl) {
                uint32_t a[4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                  const uint2 v = cur[m][2 * tl + half];
                  const uint32_t code = ((i < 4 ? v.x : v.y) >> (8 * (i & 3))) & 0xFFu;
                  const uint2 e = lds64(sign_lane + (code << 7));  // the second table is the residual codebook here
                  a[half] = e.x;
                  a[2 + half] = e.y;
                }
                mma_s8s8(acc_h[i & 1][m][tl], a[0], a[1], a[2], a[3], b.x, b.y);
                mma_s8s8(acc_l[i & 1][m][tl], a[0], a[1], a[2], a[3], b.z, b.w);
              }
          }
          const int group = c / chunks_per_res_group;
          if (c + 1 == n_chunks || (c + 1) / chunks_per_res_group != group) {
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
              for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                  const int64_t row = min(row0 + 16 * tl + g + (r >= 2 ? 8 : 0), N - 1);
                  const float sc = load_as_float(mats[m].res_scales, p.scales_dtype, (static_cast<int64_t>(hot) * N + row) * p.res_groups + group);
                  const int hi = acc_h[0][m][tl][r] + acc_h[1][m][tl][r], lo = acc_l[0][m][tl][r] + acc_l[1][m][tl][r];
                  rpart[m][tl][r] = fmaf(sc, 256.0f * static_cast<float>(hi) + static_cast<float>(lo), rpart[m][tl][r]);
                  acc_h[0][m][tl][r] = acc_h[1][m][tl][r] = 0;
                  acc_l[0][m][tl][r] = acc_l[1][m][tl][r] = 0;
                }
          }
        }
        cp_async_wait<0>();
      }
    }

    // ---- epilogue in registers: lane (g, t) holds rows {g, g+8} of each tile, columns {2t, 2t+1}
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int route = ep_route[cc];
      if (route < 0) continue;
      const int64_t xrow = route / p.x_div;
      const float xs = ep_xs[cc];
      const float weight = ep_weight[cc];
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int r = 2 * rr + cc;
          const int64_t row = row0 + 16 * tl + g + 8 * rr;
          if (row >= N) continue;
          float y[M];
#pragma unroll
          for (int m = 0; m < M; ++m) {
            float shift = 0.0f;  // the +-1/4 of every weight, folded into sum(x') per scale group
            if (p.groups == 1) {
              shift = row_scale[m][tl][r] * ep_sum[cc];
            } else {
              for (int64_t q = 0; q < p.groups; ++q)
                shift = fmaf(load_as_float(mats[m].scales, p.scales_dtype, (slot * N + row) * p.groups + q),
                             static_cast<float>(p.x.sums[xrow * p.groups + q]), shift);
            }
            y[m] = xs * (0.5f * (part[m][tl][r] + rpart[m][tl][r]) + 0.25f * shift);  // a residual weight is q / 2 with no offset
          }
          float result;
          if (M == 2) {
            float gt = y[0], up = y[M - 1];
            if (p.out_dtype == KEEPVQ_BF16) { gt = __bfloat162float(__float2bfloat16_rn(gt)); up = __bfloat162float(__float2bfloat16_rn(up)); }
            else if (p.out_dtype == KEEPVQ_F16) { gt = __half2float(__float2half_rn(gt)); up = __half2float(__float2half_rn(up)); }
            if (p.swiglu_limit > 0.0f) { gt = fminf(gt, p.swiglu_limit); up = fminf(fmaxf(up, -p.swiglu_limit), p.swiglu_limit); }
            result = gt / (1.0f + expf(-gt)) * up * weight;
          } else {
            result = y[0];
          }
          store_from_float(p.out, p.out_dtype, static_cast<int64_t>(route) * N + row, result);
        }
    }
  }
  cp_async_wait<0>();
}

bool shapes_supported(int64_t out_dim, int64_t in_dim, int64_t groups) {
  if (in_dim % (8 * CHUNK_CODES) != 0 || groups <= 0) return false;
  const int64_t chunks = in_dim / (8 * CHUNK_CODES);
  return chunks % groups == 0 && out_dim > 0;
}

static int sm_count() {
  static int cached = 0;
  if (!cached) {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached = n > 0 ? n : 148;
  }
  return cached;
}

template <int M, int TILES>
static int launch_projection(const FastProjectionArgs& p, cudaStream_t s) {
  constexpr size_t smem = LUT_BYTES + static_cast<size_t>(TEAMS) * TEAM_WARPS * (M * TILES * 4) * 32 * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(projection_kernel<M, TILES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
    configured = true;
  }
  cudaError_t err = launch_after(true, projection_kernel<M, TILES>, sm_count(), CTA_THREADS, smem, s, p);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

template <int M, int TILES, int MODE, bool NESTED = false, bool WIDE = false>
static int launch_projection_cta_mode(const FastProjectionArgs& p, cudaStream_t s) {
  constexpr size_t smem = CK_ABS_BYTES + CK_SIGN_BYTES + CK_B_BYTES + CK_WARPS * CK_STAGES * (M * 2 * TILES * 512);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(projection_cta_kernel<M, TILES, MODE, NESTED, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
    configured = true;
  }
  cudaError_t err = launch_after(true, projection_cta_kernel<M, TILES, MODE, NESTED, WIDE>, sm_count(), CK_THREADS, smem, s, p);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

static int diagnostic_mode() {
  static int mode = -1;
  if (mode < 0) {
    const char* v = getenv("KEEPVQ_PROJECTION_MODE");
    mode = v ? atoi(v) : 0;
    if (mode < 0 || mode > 4) mode = 0;
  }
  return mode;
}

template <int M, int TILES>
static int launch_projection_cta(const FastProjectionArgs& p, cudaStream_t s) {
  if (p.res_table) return launch_projection_cta_mode<M, TILES, 0, true>(p, s);
  if (p.in_dim > 8 * CHUNK_CODES * CK_MAX_CHUNKS) return launch_projection_cta_mode<M, TILES, 0, false, true>(p, s);
  switch (diagnostic_mode()) {
    case 1: return launch_projection_cta_mode<M, TILES, 1>(p, s);
    case 3: return launch_projection_cta_mode<M, TILES, 3>(p, s);
    case 4: return launch_projection_cta_mode<M, TILES, 4>(p, s);
    default: return launch_projection_cta_mode<M, TILES, 0>(p, s);
  }
}

// Enough routes to give every CTA of the machine its own (group, slab) items, and activations
// that fit the shared-memory stage?
static bool many_items(const FastProjectionArgs& p) {
  const int64_t widest = 8 * CHUNK_CODES * (p.res_table ? CK_MAX_CHUNKS : CK_MAX_CHUNKS_WIDE);
  return p.max_routes >= 48 && p.in_dim <= widest;
}

// The residual pass lives in the CTA kernel only: a layer with a residual tier needs enough routes
// for that kernel and residual scale groups that close on chunk boundaries.
bool residual_supported(int64_t routes, int64_t in_dim, int64_t res_groups) {
  if (routes < 48 || in_dim > 8 * CHUNK_CODES * CK_MAX_CHUNKS || in_dim % (8 * CHUNK_CODES) != 0 || res_groups <= 0) return false;
  return (in_dim / (8 * CHUNK_CODES)) % res_groups == 0;
}

int gate_up(const FastProjectionArgs& p, cudaStream_t s) {
  if (p.res_table && !many_items(p)) return KEEPVQ_ERR_UNSUPPORTED;
  return many_items(p) ? launch_projection_cta<2, 1>(p, s) : launch_projection<2, 2>(p, s);
}
int down(const FastProjectionArgs& p, cudaStream_t s) {
  if (p.res_table && !many_items(p)) return KEEPVQ_ERR_UNSUPPORTED;
  return many_items(p) ? launch_projection_cta<1, 2>(p, s) : launch_projection<1, 4>(p, s);
}

}  // namespace fast
}  // namespace keepvq
