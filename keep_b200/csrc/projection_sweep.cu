// Decode projections for calls with few route groups (a handful of tokens): the sweep kernel.
//
// With six experts touched, a call is twelve matrices of codes and nothing else; what decides its
// time is that every SM gets an equal share, that every warp has loads in flight, and that no
// instruction is spent on anything but codewords.  So the work is cut into units of two MMA row
// tiles of one route group (16 rows of both matrices of a gate/up pair, or 32 rows of a single
// matrix), the units are dealt to the CTAs as
// contiguous runs of equal length, and inside a CTA the 16 warps split the INPUT dimension: warp
// (row set, k part) walks down its row set's units and takes only its own chunk(s) of 32 codewords
// per row from each.  Its slice of the group's quantised activations is 16 registers, kept across
// the units of a group; its codes arrive through a private cp.async ring that runs ahead across
// units.  A warp leaves the partial sums of up to eight units in shared memory; then the CTA meets
// once and the warps share the units' epilogues (sum over the k parts, scales, SwiGLU, store).
// Units are walked by increments: no division, no per-unit barrier.
//
// Same arithmetic as the slab kernel (projection_slab.cu): int8 mma.sync m16n8k32 with a route's
// two byte planes as neighbouring columns, codes decoded through the permute-addressed tables.
#include <type_traits>
#include <utility>

#include "moe_fast.cuh"

namespace keepvq {
namespace fast {

constexpr int SW_WARPS = 16;
constexpr int SW_THREADS = SW_WARPS * 32;
constexpr int SW_CHUNK = 32;                     // codewords of a row per step of a warp
constexpr int SW_PASS_UNITS = 8;                 // units a warp carries in registers between two meetings of the CTA
constexpr int SW_SMEM_BYTES = 227 * 1024;
constexpr uint32_t SW_TABLE_BYTES = 64 * 1024;   // the nibble decoder's two tables, on a 64 KB boundary of the shared window
constexpr uint32_t SW_RED_BYTES = SW_PASS_UNITS * SW_WARPS * 4 * 128;  // 64 KB: [unit of the pass][k part][value][lane] fp32

template <int N, typename F, int... I>
__device__ __forceinline__ void sw_static_for_impl(F&& f, std::integer_sequence<int, I...>) { (f(std::integral_constant<int, I>{}), ...); }
template <int N, typename F>
__device__ __forceinline__ void sw_static_for(F&& f) { sw_static_for_impl<N>(static_cast<F&&>(f), std::make_integer_sequence<int, N>{}); }

template <int OFF>
__device__ __forceinline__ void sw_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0+%2], [%1], 16;" ::"r"(dst), "l"(src), "n"(OFF) : "memory");
}
template <int OFF>
__device__ __forceinline__ uint4 sw_lds128(uint32_t addr) {  // data a cp.async wrote: ordered by the volatile wait before it
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ void sw_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// The first MMA of a chain: accumulates onto zero, so the accumulators need no clearing.
__device__ __forceinline__ void sw_mma_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
template <int I>
__device__ __forceinline__ uint32_t sw_word(const uint4& v) {
  return (I >> 1) == 0 ? v.x : (I >> 1) == 1 ? v.y : (I >> 1) == 2 ? v.z : v.w;
}

// M = 2: gate and up over the same rows, fused by SwiGLU; M = 1: one matrix.
// The decode is the nibble decoder (moe_fast.cuh): unsigned operand bytes q + 8, whose offset
// 8 * sum(x') comes off each chunk's integer dot product (the quantised rows carry sum(x') per 256 inputs).
// DEPTH: stages of one chunk per warp in the code ring.
// `status` (may be null) is set to 2 if the shared window does not have the expected shape.
// RAGGED: the output rows are not a multiple of a unit's rows, so the last unit of a group clamps its row indices.
template <int M, int DEPTH, bool RAGGED>
__global__ void __launch_bounds__(SW_THREADS, 1) projection_sweep_kernel(FastProjectionArgs p, int32_t* status, int ks) {
  extern __shared__ __align__(16) uint8_t smem[];
  grid_launch_dependents();
  // A unit is two MMA row tiles: the same 16 rows of the gate and of the up matrix (M = 2), or 32
  // consecutive rows of the one matrix (M = 1).
  constexpr int ROWS = M == 2 ? 16 : 32;               // output rows per unit
  constexpr int STREAMS = 4;                           // row g and row g + 8 of each sub-tile
  constexpr int VALUES = 4;                            // per lane and unit: (sub-tile, row g | g + 8) for the lane's route
  constexpr uint32_t STAGE_BYTES = STREAMS * 512;      // per warp: 16 bytes per lane and stream
  constexpr uint32_t RING_BYTES = DEPTH * STAGE_BYTES;

  // ---- the shared window: rings below the first 64 KB boundary as far as they fit, then the two
  // tables (one 64 KB region) on the boundary, the partial sums, the remaining rings
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t a0 = (base + 0xFFFFu) & ~0xFFFFu;
  const int low_warps = min(SW_WARPS, static_cast<int>((a0 - base) / RING_BYTES));
  const uint32_t red_base = a0 + SW_TABLE_BYTES;
  const uint32_t high_rings = red_base + SW_RED_BYTES;
  if (high_rings + (SW_WARPS - low_warps) * RING_BYTES > base + SW_SMEM_BYTES) {  // uniform over the grid
    if (status && threadIdx.x == 0) atomicExch(status, 2);
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  // ---- tables (from constants: before the wait on the previous kernel) -------------------------
  build_nibble_tables(a0, p.codebook, threadIdx.x, SW_THREADS);
  grid_wait();  // everything below reads what earlier kernels of the stream wrote
  __syncthreads();

  const uint32_t abs_lane = a0 + lane * 4u, sign_lane = a0 + 128u + lane * 4u;
  const uint32_t ring = (warp < low_warps ? base + warp * RING_BYTES : high_rings + (warp - low_warps) * RING_BYTES) + lane * 16;
  const int64_t N = p.out_dim, cw = p.in_dim / 8;
  const int n_chunks = static_cast<int>(cw / SW_CHUNK);
  const int chunks_per_group = n_chunks / static_cast<int>(p.groups);
  // `ks` warps per row set (the host picks it from the number of chunks, sweep_k_parts below);
  // warps beyond row_sets * ks have no units and only help with the epilogues
  const int row_sets = SW_WARPS / ks;
  const int row_set = warp / ks, k_part = warp - row_set * ks;
  const bool spare = row_set >= row_sets;
  const int c_first = k_part * n_chunks / ks, c_end = (k_part + 1) * n_chunks / ks;
  const int my_chunks = c_end - c_first;
  const int units_per_group = static_cast<int>((N + ROWS - 1) / ROWS);
  const int64_t units = static_cast<int64_t>(p.groups_of_routes.count[0]) * units_per_group;
  const int grid = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const int u_begin = static_cast<int>(units * cta / grid), u_end = static_cast<int>(units * (cta + 1) / grid);
  const Projection mats[2] = {p.a, M == 2 ? p.b : p.a};

  // A warp's walk over its units (u_begin + row_set, + row_sets, ...), kept twice: once for the
  // code fetches, which run ahead, once for the arithmetic.
  const int last_row = static_cast<int>(N - 1);
  const uint64_t codes0 = reinterpret_cast<uint64_t>(mats[0].codes), row_bytes = static_cast<uint64_t>(cw) * 2u;
  const uint64_t matrix_delta = reinterpret_cast<uint64_t>(mats[1].codes) - codes0;  // wraps for a lower address: the sum is taken modulo 2^64 again
  const uint64_t lane_offset = static_cast<uint64_t>(g) * row_bytes + static_cast<uint64_t>(c_first * SW_CHUNK + t * 8) * 2u;
  const uint64_t unit_stride = static_cast<uint64_t>(row_sets) * ROWS * row_bytes;
  const uint64_t sub_delta = M == 2 ? matrix_delta : 16u * row_bytes;  // from the first sub-tile's codes to the second's
  struct Walk {
    int u, gi, tile;     // unit, its group and its place among the group's units
    int c;               // next chunk of the unit
    int64_t slot_rows;   // slot * N
    uint64_t codes;      // address of this lane's first codes of the unit: matrix 0, row tile * ROWS + g, chunk c_first
  };
  auto enter_group = [&](Walk& w) {
    w.slot_rows = static_cast<int64_t>(p.groups_of_routes.slot[w.gi]) * N;
    w.codes = codes0 + static_cast<uint64_t>(w.slot_rows + w.tile * ROWS) * row_bytes + lane_offset;
  };
  auto start_walk = [&](Walk& w) {
    w.u = spare ? u_end : u_begin + row_set;
    w.gi = w.u / units_per_group;
    w.tile = w.u - w.gi * units_per_group;
    w.c = c_first;
    w.slot_rows = 0;
    w.codes = 0;
    if (w.u < u_end) enter_group(w);
  };
  auto next_unit = [&](Walk& w) {
    w.u += row_sets;
    w.tile += row_sets;
    w.c = c_first;
    w.codes += unit_stride;
    if (w.tile >= units_per_group) {  // (a loop: tiny outputs have fewer units per group than a CTA has row sets)
      while (w.tile >= units_per_group) { w.tile -= units_per_group; ++w.gi; }
      if (w.u < u_end) enter_group(w);
    }
  };
  uint32_t fetch_turn = 0, use_turn = 0;
  Walk ahead;
  start_walk(ahead);
  auto fetch = [&]() {  // the next chunk of the walk `ahead` -> ring stage fetch_turn % DEPTH; always commits a group
    if (ahead.u < u_end && my_chunks > 0) {
      const uint32_t dst = ring + (fetch_turn % DEPTH) * STAGE_BYTES;
      // stream 0 = row g of the first sub-tile; the others are fixed byte distances away
      const uint64_t first = ahead.codes + static_cast<uint32_t>(ahead.c - c_first) * (SW_CHUNK * 2u);
      sw_static_for<STREAMS>([&](auto s) {
        constexpr int S = decltype(s)::value;
        uint64_t from = first + ((S & 1) ? 8u * row_bytes : 0u) + ((S >> 1) ? sub_delta : 0u);
        if (RAGGED) {
          const int row = min(ahead.tile * ROWS + (M == 1 ? 16 * (S >> 1) : 0) + g + 8 * (S & 1), last_row);
          from = codes0 + ((M == 2 && (S >> 1)) ? matrix_delta : 0u) + static_cast<uint64_t>((ahead.slot_rows + row) * cw + ahead.c * SW_CHUNK + t * 8) * 2u;
        }
        sw_cp_async16<S * 512>(dst, reinterpret_cast<const void*>(from));
      });
      if (++ahead.c == c_end) next_unit(ahead);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    ++fetch_turn;
  };
#pragma unroll
  for (int i = 0; i < DEPTH - 1; ++i) fetch();

  Walk at;
  start_walk(at);
  const uint8_t* x_lane = nullptr;
  const int32_t* chunk_sums = nullptr;
  int held_sum = 0;  // a warp with one chunk per unit keeps its chunk's sum as it keeps the slice
  int x_group = -1;  // whose activations x_lane points at
  uint2 b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = make_uint2(0u, 0u);
  auto load_slice = [&](int c) {
#pragma unroll
    for (int i = 0; i < 8; ++i)  // (volatile: held in registers, not re-issued at every use)
      asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(b[i].x), "=r"(b[i].y) : "l"(x_lane + (static_cast<int64_t>(c) * SW_CHUNK + i) * 16));
  };
  const int local_units = u_end - u_begin;
  const int per_pass = SW_PASS_UNITS * row_sets;  // units of the CTA per pass
  const uint32_t red_mine = red_base + ((row_set * ks + k_part) * 128u + lane) * 4u;  // + j * pass_stride + v * 128 bytes
  const uint32_t pass_stride = static_cast<uint32_t>(row_sets * ks) * 512u;         // one partial tile per (unit, k part)
  for (int pass_first = 0; pass_first < local_units; pass_first += per_pass) {
    // ---- this warp's units of the pass: the partial sums of unit j go straight to their place in
    // shared memory, so the loop stays rolled (unrolled eight times it did not fit the instruction cache)
    const int pass_end = u_begin + pass_first + per_pass;
#pragma unroll 1
    for (int j = 0; j < SW_PASS_UNITS && at.u < u_end && at.u < pass_end; ++j) {
      float part[VALUES];
#pragma unroll
      for (int v = 0; v < VALUES; ++v) part[v] = 0.0f;
      // The lane's slice of the group's activations: 8 bytes of one plane per step of a chunk.  The
      // reads are scattered (sixteen cache lines per warp-wide load), so a warp with one chunk per
      // unit keeps them across the units of a group.
      if (at.gi != x_group) {
        const int gsize = p.groups_of_routes.size[at.gi], gstart = p.groups_of_routes.start[at.gi];
        // column g of the MMA is (route g / 2, byte plane g % 2); a lane whose column carries no route
        // reads route 0's bytes (always there), and nothing ever looks at its column
        const int col_route = (g >> 1) < gsize ? (g >> 1) : 0;
        const int route = p.groups_of_routes.routes[gstart + col_route];
        x_lane = p.x.q + (static_cast<int64_t>(route / p.x_div) * cw + t * 8) * 16 + (g & 1) * 8;
        x_group = at.gi;
        // columns 2t, 2t + 1 of the accumulators are route t's: its sums of x' per chunk
        const int64_t sums_row = t < gsize ? p.groups_of_routes.routes[gstart + t] / p.x_div : p.x_zero_row;
        chunk_sums = p.x.chunk_sums + sums_row * n_chunks;
        if (my_chunks == 1) { load_slice(c_first); held_sum = chunk_sums[c_first]; }
      }
      for (int c = c_first; c < c_end; ++c) {
        if (my_chunks != 1) { load_slice(c); held_sum = chunk_sums[c]; }
        fetch();
        asm volatile("cp.async.wait_group %0;" ::"n"(DEPTH - 1) : "memory");  // this chunk has landed
        const uint32_t src = ring + (use_turn % DEPTH) * STAGE_BYTES;
        ++use_turn;
        uint4 cur[STREAMS];
        sw_static_for<STREAMS>([&](auto s) { cur[decltype(s)::value] = sw_lds128<decltype(s)::value * 512>(src); });
        float sc[2][2];  // with one scale per row the epilogue applies it; otherwise asked for now, used behind the MMAs
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            sc[sub][rr] = 1.0f;
            if (p.groups > 1) {
              const int64_t row = min(static_cast<int64_t>(at.tile) * ROWS + (M == 1 ? 16 * sub : 0) + g + 8 * rr, N - 1);
              sc[sub][rr] = load_as_float(mats[M == 2 ? sub : 0].scales, p.scales_dtype, (at.slot_rows + row) * p.groups + c / chunks_per_group);
            }
          }
        int acc[2][2][4];  // two chains per sub-tile, used by alternate steps: the MMA's dependent latency is long
        sw_static_for<8>([&](auto index) {
          constexpr int I = decltype(index)::value;
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            uint32_t a[4];
            decode_codeword_nibble<(I & 1) != 0>(sw_word<I>(cur[2 * sub]), abs_lane, sign_lane, a[0], a[2]);      // row g
            decode_codeword_nibble<(I & 1) != 0>(sw_word<I>(cur[2 * sub + 1]), abs_lane, sign_lane, a[1], a[3]);  // row g + 8
            if (I < 2) sw_mma_first(acc[I][sub], a[0], a[1], a[2], a[3], b[I].x, b[I].y);
            else sw_mma(acc[I & 1][sub], a[0], a[1], a[2], a[3], b[I].x, b[I].y);
          }
        });
        // columns 2t, 2t + 1 of the MMA are this lane's route: high plane, low plane
#pragma unroll
        for (int sub = 0; sub < 2; ++sub)
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            // 256 * high + low of one chunk fits 32 bits (256 products of at most 2^15 each, times 256);
            // less 8 * sum(x') it is sum(q x') over the chunk
            const int dot = ((acc[0][sub][2 * rr] + acc[1][sub][2 * rr]) << 8) + acc[0][sub][2 * rr + 1] + acc[1][sub][2 * rr + 1] - 8 * held_sum;
            part[2 * sub + rr] = fmaf(sc[sub][rr], static_cast<float>(dot), part[2 * sub + rr]);
          }
      }
#pragma unroll
      for (int v = 0; v < VALUES; ++v)
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(red_mine + j * pass_stride + v * 128u), "f"(part[v]) : "memory");
      next_unit(at);
    }

    // ---- the CTA meets: epilogues shared out -----------------------------------------------------
    __syncthreads();
    const int in_pass = min(per_pass, local_units - pass_first);
    for (int e = warp; e < in_pass; e += SW_WARPS) {  // unit e of the pass: j = e / row_sets of row set e % row_sets
      const int u = u_begin + pass_first + e;
      const int gi = u / units_per_group, tile = u - gi * units_per_group;
      const int gsize = p.groups_of_routes.size[gi], gstart = p.groups_of_routes.start[gi];
      const int64_t slot_rows = static_cast<int64_t>(p.groups_of_routes.slot[gi]) * N;
      if (t >= gsize) continue;  // lane (g, t) holds rows g and g + 8 of each sub-tile for route t
      const int route = p.groups_of_routes.routes[gstart + t];
      const int64_t xrow = route / p.x_div;
      const float xs = p.x.scale[xrow];
      float sum[VALUES];
#pragma unroll
      for (int v = 0; v < VALUES; ++v) sum[v] = 0.0f;
      for (int k = 0; k < ks; ++k)
#pragma unroll
        for (int v = 0; v < VALUES; ++v) {
          float got;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(got) : "r"(red_base + (((e * ks + k) * 4 + v) * 32 + lane) * 4u));
          sum[v] += got;
        }
      // y of (sub-tile, row g | g + 8): scale and the +-1/4 of every weight, folded into sum(x') per scale group
      auto finish = [&](int sub, float dot, int64_t row) {
        const void* scales = mats[M == 2 ? sub : 0].scales;
        float shift = 0.0f;
        if (p.groups == 1) {
          const float sc = load_as_float(scales, p.scales_dtype, slot_rows + row);
          dot *= sc;
          shift = sc * static_cast<float>(p.x.sums[xrow]);
        } else {
          for (int64_t q = 0; q < p.groups; ++q)
            shift = fmaf(load_as_float(scales, p.scales_dtype, (slot_rows + row) * p.groups + q), static_cast<float>(p.x.sums[xrow * p.groups + q]), shift);
        }
        return xs * (0.5f * dot + 0.25f * shift);
      };
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        if (M == 2) {  // gate and up of one row: round G and U to the activation dtype first, as the separate kernels of the reference do
          const int64_t row = static_cast<int64_t>(tile) * ROWS + g + 8 * rr;
          if (row >= N) continue;
          float gt = finish(0, sum[rr], row), up = finish(1, sum[2 + rr], row);
          if (p.out_dtype == KEEPVQ_BF16) { gt = __bfloat162float(__float2bfloat16_rn(gt)); up = __bfloat162float(__float2bfloat16_rn(up)); }
          else if (p.out_dtype == KEEPVQ_F16) { gt = __half2float(__float2half_rn(gt)); up = __half2float(__float2half_rn(up)); }
          if (p.swiglu_limit > 0.0f) { gt = fminf(gt, p.swiglu_limit); up = fminf(fmaxf(up, -p.swiglu_limit), p.swiglu_limit); }
          store_from_float(p.out, p.out_dtype, static_cast<int64_t>(route) * N + row, gt / (1.0f + expf(-gt)) * up * p.route_weight[route]);
        } else {
#pragma unroll
          for (int sub = 0; sub < 2; ++sub) {
            const int64_t row = static_cast<int64_t>(tile) * ROWS + 16 * sub + g + 8 * rr;
            if (row < N) store_from_float(p.out, p.out_dtype, static_cast<int64_t>(route) * N + row, finish(sub, sum[2 * sub + rr], row));
          }
        }
      }
    }
    __syncthreads();  // the partial sums are read; the next pass may overwrite them
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- launch -----------------------------------------------------------------------------------

bool sweep_supported(int64_t in_dim) { return in_dim % (8 * SW_CHUNK) == 0; }

// Warps per row set for `n_chunks` chunks of inputs: the split that keeps most of the 16 warps busy.
// A warp with one chunk per unit keeps its slice of the activations in registers; with more it
// re-reads a slice per chunk (scattered reads: about a fifth slower, measured), so e.g. 16 chunks
// are 16 parts of one, 20 chunks four parts of five (not sixteen of one or two), 9 chunks three of three.
static int sweep_k_parts(int n_chunks) {
  int best = 1;
  double best_score = 0.0;
  for (int ks = 1; ks <= SW_WARPS && ks <= n_chunks; ++ks) {
    const int most = (n_chunks + ks - 1) / ks, row_sets = SW_WARPS / ks;
    const double score = static_cast<double>(n_chunks) / (ks * most) * (ks * row_sets) / SW_WARPS * (most == 1 ? 1.0 : 0.8);
    if (score >= best_score) { best_score = score; best = ks; }
  }
  return best;
}

template <int M, int DEPTH, bool RAGGED>
static int launch_sweep_kernel(const FastProjectionArgs& p, cudaStream_t s) {
  auto kernel = projection_sweep_kernel<M, DEPTH, RAGGED>;
  static uint64_t configured = 0;  // one bit per device: the shared-memory opt-in is a per-device attribute of the function
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !((configured >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SW_SMEM_BYTES);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (dev >= 0 && dev < 64) configured |= 1ull << dev;
  }
  static int cached_sms[64] = {};
  if (dev >= 0 && dev < 64) {
    if (!cached_sms[dev]) {
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cached_sms[dev] = sms > 0 ? sms : 148;
    }
    sms = cached_sms[dev];
  }
  cudaError_t err = launch_after(true, kernel, sms, SW_THREADS, SW_SMEM_BYTES, s, p, p.status, sweep_k_parts(static_cast<int>(p.in_dim / (8 * SW_CHUNK))));
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

template <int M, int DEPTH>
static int launch_sweep(const FastProjectionArgs& p, cudaStream_t s) {
  if (!p.x.chunk_sums) return KEEPVQ_ERR_NULL;
  if (p.out_dim % (M == 2 ? 16 : 32) == 0) return launch_sweep_kernel<M, DEPTH, false>(p, s);
  // a gate/up pair's outputs are the down projection's inputs, which come in multiples of 256
  if (M == 2) return KEEPVQ_ERR_UNSUPPORTED;
  return launch_sweep_kernel<1, DEPTH, true>(p, s);
}

#ifdef KEEPVQ_DIAG
static int g_sweep_variant = 0;  // measurement build only: 0 = code ring of 2 stages, 1 = of 3
extern "C" void keepvq_diag_set_sweep(int variant) { g_sweep_variant = variant; }
int sweep_gate_up(const FastProjectionArgs& p, cudaStream_t s) { return g_sweep_variant ? launch_sweep<2, 3>(p, s) : launch_sweep<2, 2>(p, s); }
int sweep_down(const FastProjectionArgs& p, cudaStream_t s) { return g_sweep_variant ? launch_sweep<1, 3>(p, s) : launch_sweep<1, 2>(p, s); }
#else
int sweep_gate_up(const FastProjectionArgs& p, cudaStream_t s) { return launch_sweep<2, 2>(p, s); }
int sweep_down(const FastProjectionArgs& p, cudaStream_t s) { return launch_sweep<1, 2>(p, s); }
#endif

}  // namespace fast
}  // namespace keepvq
