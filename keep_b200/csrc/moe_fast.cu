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

__global__ void __launch_bounds__(GR_THREADS) group_routes_kernel(const uint32_t* __restrict__ served_slot, int routes, int slots, int max_group, RouteGroups out, int32_t* clear) {
  grid_launch_dependents();
  grid_wait();
  if (clear && threadIdx.x == 0) *clear = 0;
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

bool shapes_supported(int64_t out_dim, int64_t in_dim, int64_t groups) {
  if (in_dim % (8 * CHUNK_CODES) != 0 || groups <= 0) return false;
  const int64_t chunks = in_dim / (8 * CHUNK_CODES);
  return chunks % groups == 0 && out_dim > 0;
}

// SM count of the current device (cached per device ordinal).
static int sm_count(int* device_out) {
  constexpr int MAX_DEVICES = 64;
  static int cached[MAX_DEVICES] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (device_out) *device_out = dev;
  if (dev < 0 || dev >= MAX_DEVICES) return 148;
  if (!cached[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

template <int M, int TILES>
static int launch_projection(const FastProjectionArgs& p, cudaStream_t s) {
  constexpr size_t smem = LUT_BYTES + static_cast<size_t>(TEAMS) * TEAM_WARPS * (M * TILES * 4) * 32 * sizeof(float);
  static uint64_t configured = 0;  // one bit per device: the shared-memory opt-in is a per-device attribute of the function
  int dev = 0;
  const int sms = sm_count(&dev);
  if (dev < 0 || dev >= 64 || !((configured >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(projection_kernel<M, TILES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
    if (dev >= 0 && dev < 64) configured |= 1ull << dev;
  }
  cudaError_t err = launch_after(true, projection_kernel<M, TILES>, sms, CTA_THREADS, smem, s, p);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

// Enough routes to give every CTA of the machine its own (group, slab) items, and activations
// that fit the shared-memory stage?
static bool many_items(const FastProjectionArgs& p) {
  return p.max_routes >= SMALL_CALL_ROUTES && p.in_dim <= slab_max_in_dim(p.group_cols > PAIRED_GROUP_ROUTES ? MAX_GROUP_ROUTES : PAIRED_GROUP_ROUTES);
}
// Few route groups of at most four routes, activations that leave room in the stage: the split slab kernel.
static bool few_items(const FastProjectionArgs& p) {
  return p.few_groups && p.group_cols <= PAIRED_GROUP_ROUTES && p.in_dim <= slab_split_max_in_dim();
}

#ifdef KEEPVQ_DIAG
static int g_force_cols = 0;
extern "C" void keepvq_diag_set_group_cols(int cols) { g_force_cols = cols; }
#endif

int decode_group_routes(int64_t live, int64_t slots, int64_t widest_in_dim) {
#ifdef KEEPVQ_DIAG
  if (g_force_cols) return g_force_cols;
#endif
  if (live < SMALL_CALL_ROUTES) return widest_in_dim <= slab_split_max_in_dim() ? PAIRED_GROUP_ROUTES : MAX_GROUP_ROUTES;  // split slab kernel | team kernel
  if (widest_in_dim > slab_max_in_dim(MAX_GROUP_ROUTES)) return PAIRED_GROUP_ROUTES;
  return live <= 2 * slots ? PAIRED_GROUP_ROUTES : MAX_GROUP_ROUTES;
}

// The residual pass lives in the slab kernels only: a layer with a residual tier needs activations
// that fit their stage (half of it for calls with few routes) and residual scale groups that close
// on chunk boundaries.
bool residual_supported(int64_t routes, int64_t in_dim, int64_t res_groups) {
  const int64_t widest = routes < SMALL_CALL_ROUTES ? slab_split_max_in_dim() : slab_max_in_dim(PAIRED_GROUP_ROUTES);
  if (in_dim > widest || in_dim % (8 * CHUNK_CODES) != 0 || res_groups <= 0) return false;
  return (in_dim / (8 * CHUNK_CODES)) % res_groups == 0;
}

int gate_up(const FastProjectionArgs& p, cudaStream_t s) {
  if (few_items(p)) return slab_split_gate_up(p, s);
  if (p.res_table && !many_items(p)) return KEEPVQ_ERR_UNSUPPORTED;
  return many_items(p) ? slab_gate_up(p, p.group_cols > PAIRED_GROUP_ROUTES ? MAX_GROUP_ROUTES : PAIRED_GROUP_ROUTES, s) : launch_projection<2, 2>(p, s);
}
int down(const FastProjectionArgs& p, cudaStream_t s) {
  if (few_items(p)) return slab_split_down(p, s);
  if (p.res_table && !many_items(p)) return KEEPVQ_ERR_UNSUPPORTED;
  return many_items(p) ? slab_down(p, p.group_cols > PAIRED_GROUP_ROUTES ? MAX_GROUP_ROUTES : PAIRED_GROUP_ROUTES, s) : launch_projection<1, 4>(p, s);
}

}  // namespace fast
}  // namespace keepvq
