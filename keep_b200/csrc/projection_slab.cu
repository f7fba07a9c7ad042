// Decode projections for batches with many route groups: the kernel the HBM roofline of a decode
// layer is measured on.
//
// A persistent CTA per SM takes (route group, slab of output rows) items; each of its 16 warps owns
// 16 * TILES rows of the slab over the whole input dimension, so there is no split-K reduction.
// The kernel is bound by turning codes into int8 operands, not by memory, so every instruction a
// codeword costs was counted (ncu's executed-instruction counters per opcode):
//   - a group holds at most four routes, and their high-byte and low-byte planes sit side by side
//     as the eight columns of ONE m16n8k32 MMA (a lane ends up with both planes of its route);
//     groups of up to eight routes (two MMAs per tile and step) serve calls with more routes per
//     expert;
//   - the nibble decoder (moe_fast.cuh): the abs entry and the sign byte's XOR masks are one
//     32-bit word of eight 4-bit values each, 32 replicas, interleaved in one 64 KB region on a
//     64 KB boundary of the shared window, so the abs (sign) byte of the code word dropped into
//     byte 1 of (region + lane offset) IS the entry's address: two byte permutes, two 4-byte
//     table reads, two masked XORs and a shift per codeword.  The operand bytes are q + 8
//     (unsigned A), and 8 * sum(x') comes off the integer dot product when a scale group closes;
//   - codes stream through a private cp.async ring per warp; a group's quantised activations are
//     staged once per run of items in MMA-fragment order, and a lane whose column carries no
//     route re-reads a live column's bytes (its own MMA column is never looked at), so the
//     activation reads cost one wavefront for the typical one-route group.
// Calls with few route groups (a handful of tokens) run the SPLIT form: the warps of a CTA share a
// slab's rows AND the input dimension (`ks` warps per row set, each over 1/ks of the codewords),
// their partial sums meet in shared memory, and `ks` is picked on the device from the number of
// groups so that every SM gets several items however few experts the call touches.
#include <type_traits>
#include <utility>

#include "moe_fast.cuh"

namespace keepvq {
namespace fast {

constexpr int SK_WARPS = 16;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_CHUNK = 32;                              // codewords of a row per ring stage and lane quartet
constexpr int SK_STAGES = 2;
constexpr int SK_SMEM_BYTES = 227 * 1024;                 // the whole opt-in window: the tables want a fixed 64 KB boundary inside it
constexpr int SK_WARP_RING = SK_STAGES * 4 * 512;         // four 16-byte streams per lane and stage
constexpr uint32_t SK_TABLE_BYTES = 64 * 1024;            // the nibble decoder's two tables
constexpr uint32_t SK_RES_REPLICAS = 16;
constexpr uint32_t SK_RES_BYTES = 256 * SK_RES_REPLICAS * 8;   // 32 KB: the residual codebook, signed bytes, [code][replica] x 8 bytes

// Shared window, in absolute shared addresses.  A0 = the first 64 KB boundary at or above the
// dynamic base (the runtime keeps 1 KB below it, so A0 = 64 KB):
//   [base, A0)            cp.async rings of as many warps as fit (15)
//   [A0, +64 KB)          the two tables
//   no residual tier      [+64 KB, +128 KB) activations: 8 columns x 8192 inputs or 16 x 4096
//   residual tier         [+64 KB, +96 KB) residual codebook | [+96 KB, +160 KB) activations
//   [+160 KB, ...)        the remaining rings
constexpr uint32_t SK_RING_HIGH_OFF = 160 * 1024;

template <int N, typename F, int... I>
__device__ __forceinline__ void sk_static_for_impl(F&& f, std::integer_sequence<int, I...>) { (f(std::integral_constant<int, I>{}), ...); }
template <int N, typename F>
__device__ __forceinline__ void sk_static_for(F&& f) { sk_static_for_impl<N>(static_cast<F&&>(f), std::make_integer_sequence<int, N>{}); }

template <int OFF>
__device__ __forceinline__ void sk_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0+%2], [%1], 16;" ::"r"(dst), "l"(src), "n"(OFF) : "memory");
}
template <int OFF>
__device__ __forceinline__ void sk_cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0+%2], [%1], 8;" ::"r"(dst), "l"(src), "n"(OFF) : "memory");
}
__device__ __forceinline__ void sk_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void sk_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int OFF>
__device__ __forceinline__ uint4 sk_lds128(uint32_t addr) {  // data a cp.async wrote: ordered by the volatile wait before it
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint2 sk_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
__device__ __forceinline__ void sk_sts64(uint32_t addr, uint32_t lo, uint32_t hi) {
  asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
}

__device__ __forceinline__ void sk_mma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void sk_mma_u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {  // A unsigned
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int I>
__device__ __forceinline__ uint32_t sk_word(const uint4& v) {
  return (I >> 1) == 0 ? v.x : (I >> 1) == 1 ? v.y : (I >> 1) == 2 ? v.z : v.w;
}

// COLS = routes per group: 4 (both byte planes of a route in one MMA) or 8 (one MMA per plane).
// NESTED: the layer has a residual tier; the residual codebook (signed bytes) sits behind the
// tables, and an item whose slot is hot runs a second pass over the residual's 8-bit codes.
// `status` (may be null) is set to 2 if the shared window does not have the expected shape.
// SPLIT: see the head of the file; the partial sums (16 KB) live at the end of the 64 KB activation
// stage, which leaves 48 KB for the activations (eight columns of 6144 inputs).  A warp's share of
// a scale group needs sum(x') over just that share: the quantised rows carry it per 256 inputs.
constexpr uint32_t SK_SPLIT_RED_OFF = 48 * 1024;          // from the start of the activation stage
constexpr int SK_SPLIT_ITEMS_PER_CTA = 4;                 // items per CTA the split factor aims for

template <int M, int TILES, int COLS, bool NESTED, bool SPLIT>
__global__ void __launch_bounds__(SK_THREADS, 1) projection_slab_kernel(FastProjectionArgs p, int32_t* status) {
  static_assert(COLS == 4 || COLS == 8, "a group is four or eight routes");
  static_assert(!SPLIT || COLS == 4, "the split form keeps its partial sums at the end of the 64 KB activation stage");
  static_assert(M * 2 * TILES == 4, "four code streams per lane");
  extern __shared__ __align__(16) uint8_t smem[];
  grid_launch_dependents();
  constexpr int PLANES = COLS == 4 ? 1 : 2;     // MMAs per tile and step
  constexpr int RPL = COLS == 4 ? 1 : 2;        // routes a lane holds in the epilogue
  constexpr int PARTS = 2 * RPL;                // (row g | g + 8) x routes of the lane
  constexpr int B_LANE = COLS == 4 ? 8 : 16;    // bytes of the B operand a lane reads per step
  constexpr int B_STEP = 32 * B_LANE;

  const uint32_t smem_base = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const uint32_t a0 = (smem_base + 0xFFFFu) & ~0xFFFFu;
  const int low_warps = min(SK_WARPS, static_cast<int>((a0 - smem_base) / SK_WARP_RING));
  if (a0 + SK_RING_HIGH_OFF + (SK_WARPS - low_warps) * SK_WARP_RING > smem_base + SK_SMEM_BYTES) {  // uniform over the grid
    if (status && threadIdx.x == 0) atomicExch(status, 2);
    return;
  }

  // ---- tables -----------------------------------------------------------------------------
  build_nibble_tables(a0, p.codebook, threadIdx.x, SK_THREADS);
  if (NESTED) {
    // the residual codebook: byte j of an entry's low word is 2 * v[6 - 2j], of its high word
    // 2 * v[7 - 2j].  A thread works out one entry; its warp then writes its 32 entries two at a
    // time, sixteen lanes storing the sixteen replicas of one entry side by side (no bank conflicts)
    for (int e = threadIdx.x; e < 256; e += SK_THREADS) {
      uint32_t lo = 0, hi = 0;
      const uint32_t* row = p.res_table + e * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 pair = *reinterpret_cast<const __half2*>(&row[3 - j]);  // dims 6 - 2j, 7 - 2j
        lo |= (static_cast<uint32_t>(__float2int_rn(2.0f * __low2float(pair))) & 0xFFu) << (8 * j);
        hi |= (static_cast<uint32_t>(__float2int_rn(2.0f * __high2float(pair))) & 0xFFu) << (8 * j);
      }
      const int e_warp = e & ~31, ln = threadIdx.x & 31;
      const uint32_t dst_warp = a0 + SK_TABLE_BYTES + e_warp * (SK_RES_REPLICAS * 8);
#pragma unroll 4
      for (int i = 0; i < 32; i += 2) {
        const int from = i + (ln >> 4);
        const uint32_t vlo = __shfl_sync(0xFFFFFFFFu, lo, from), vhi = __shfl_sync(0xFFFFFFFFu, hi, from);
        sk_sts64(dst_warp + from * (SK_RES_REPLICAS * 8) + (ln & (SK_RES_REPLICAS - 1)) * 8, vlo, vhi);
      }
    }
  }

  grid_wait();  // the tables came from constants; everything below reads what earlier kernels of the stream wrote
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const uint32_t abs_lane = a0 + lane * 4u, sign_lane = a0 + 128u + lane * 4u;
  const uint32_t res_lane = a0 + SK_TABLE_BYTES + static_cast<uint32_t>(lane & (SK_RES_REPLICAS - 1)) * 8u;
  const uint32_t b_base = a0 + SK_TABLE_BYTES + (NESTED ? SK_RES_BYTES : 0u);
  constexpr int STAGE_BYTES = 4 * 512;                   // per warp
  const uint32_t ring = (warp < low_warps ? smem_base + warp * SK_WARP_RING : a0 + SK_RING_HIGH_OFF + (warp - low_warps) * SK_WARP_RING) + lane * 16;
  const int64_t N = p.out_dim, cw = p.in_dim / 8;
  const int n_chunks = static_cast<int>(cw / SK_CHUNK);
  const int chunks_per_group = n_chunks / static_cast<int>(p.groups);
  const int chunks_per_res_group = NESTED ? n_chunks / static_cast<int>(p.res_groups) : n_chunks;
  constexpr int ROWS = 16 * TILES;              // per warp
  const int grid = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  // `ks` warps share a row set, each over n_chunks / ks chunks of the input dimension.  It grows
  // (in powers of two, as far as the chunks allow) until every CTA has several items.
  int ks = 1;
  if (SPLIT) {
    const int64_t want = static_cast<int64_t>(SK_SPLIT_ITEMS_PER_CTA) * grid, found = p.groups_of_routes.count[0];
    while (2 * ks <= SK_WARPS && n_chunks % (2 * ks) == 0 && found * ((N * ks + ROWS * SK_WARPS - 1) / (ROWS * SK_WARPS)) < want) ks *= 2;
  }
  const int row_sets = SK_WARPS / ks;           // row sets of a CTA item
  const int row_set = SPLIT ? warp / ks : warp, k_part = SPLIT ? warp % ks : 0;
  const int c_first = k_part * (n_chunks / ks), c_end = c_first + n_chunks / ks;  // this warp's chunks
  const int slab_rows = ROWS * row_sets;        // per CTA item
  const int slabs = static_cast<int>((N + slab_rows - 1) / slab_rows);
  const int items = p.groups_of_routes.count[0] * slabs;
  const Projection mats[2] = {p.a, p.b};
  const uint32_t red_base = b_base + SK_SPLIT_RED_OFF;  // [turn & 1][warp][value][lane] fp32
  uint32_t red_turn = 0;                                // items this row set has reduced

  // A CTA takes a contiguous run of items, so consecutive items mostly belong to one route group
  // and its activations are staged once for all of them.  (With a residual tier the items of a
  // hot slot cost half as much again, and a run of them on one CTA would unbalance the grid:
  // those layers deal the items out round-robin instead.)
  const int first_item = NESTED ? cta : static_cast<int>(static_cast<int64_t>(items) * cta / grid);
  const int last_item = NESTED ? items : static_cast<int>(static_cast<int64_t>(items) * (cta + 1) / grid);
  const int item_step = NESTED ? grid : 1;
  // What a lane needs to know of an item.  The next item's first chunk is requested while the
  // current item's last chunk is being decoded, so an item does not start with an exposed wait.
  struct Item {
    int gi, gsize, gstart;
    int64_t slot, row0;
    bool active;
    const uint16_t* row_ptr[4];  // stream s = matrix s / (2 * TILES), rows g + 8 * (s % (2 * TILES))
  };
  auto describe = [&](int item) {
    Item it;
    it.gi = item / slabs;
    const int slab = item - it.gi * slabs;
    it.slot = p.groups_of_routes.slot[it.gi];
    it.gsize = p.groups_of_routes.size[it.gi];
    it.gstart = p.groups_of_routes.start[it.gi];
    it.row0 = static_cast<int64_t>(slab) * slab_rows + row_set * ROWS;
    it.active = it.row0 < N;
#pragma unroll
    for (int s = 0; s < 4; ++s)
      it.row_ptr[s] = mats[s / (2 * TILES)].codes + (it.slot * N + min(it.row0 + 8 * (s % (2 * TILES)) + g, N - 1)) * cw + t * 8;
    return it;
  };
  uint32_t ring_turn = 0;  // chunks this warp has consumed: picks the ring stage
  auto fetch = [&](const Item& it, int c, uint32_t turn) {  // chunk c of the lane's row streams -> ring stage turn % SK_STAGES
    if (it.active && c < c_end) {
      const uint32_t dst = ring + (turn % SK_STAGES) * STAGE_BYTES;
      sk_static_for<4>([&](auto s) { sk_cp_async16<decltype(s)::value * 512>(dst, it.row_ptr[decltype(s)::value] + c * SK_CHUNK); });
    }
    sk_commit();
  };
  constexpr bool CARRY = !NESTED;  // the residual pass borrows the ring, so those layers start every item cold
  Item next_item = {};
  if (first_item < last_item) {
    next_item = describe(first_item);
    if (CARRY) fetch(next_item, c_first, ring_turn);
  }
  int staged_group = -1;
  for (int item = first_item; item < last_item; item += item_step) {
    const Item it = next_item;
    const bool has_next = item + item_step < last_item;
    if (has_next) next_item = describe(item + item_step);
    const int gi = it.gi, gsize = it.gsize, gstart = it.gstart;
    const int64_t slot = it.slot, row0 = it.row0;
    const bool active = it.active;

    // column g of the MMA is (route g / 2, byte plane g % 2) with four routes, route g (both planes) with eight
    const int col_route = COLS == 4 ? (g >> 1) : g;
    const bool column_live = col_route < gsize;
    if (gi != staged_group) {
      __syncthreads();  // every warp is done with the previous group's activations (and the tables are built)
      if (column_live) {  // stage this group's activations in fragment order: [chunk * 8 + step][lane]
        const int route = p.groups_of_routes.routes[gstart + col_route];
        const uint8_t* src = p.x.q + (static_cast<int64_t>(route / p.x_div) * cw + t * 8) * 16 + (COLS == 4 ? (g & 1) * 8 : 0);
        const uint32_t dst = b_base + lane * B_LANE;
        for (int step = warp; step < n_chunks * 8; step += SK_WARPS) {
          const uint8_t* from = src + ((step >> 3) * SK_CHUNK + (step & 7)) * 16;
          if (COLS == 4) sk_cp_async8<0>(dst + step * B_STEP, from);
          else sk_cp_async16<0>(dst + step * B_STEP, from);
        }
      }
      sk_commit();
      if (CARRY) {
        sk_wait<0>();  // the activations, and the first chunk asked for earlier
      } else {
        fetch(it, c_first, ring_turn);
        sk_wait<1>();  // the activations (the older group) have landed
      }
      __syncthreads();
      staged_group = gi;
    } else if (!CARRY) {
      fetch(it, c_first, ring_turn);
    }
    if (!active) {
      if (CARRY && has_next) fetch(next_item, c_first, ring_turn);
      else sk_wait<0>();
      continue;
    }
    // a lane whose column carries no route reads the bytes of route 0's column instead (always
    // live): same addresses as live lanes, so no extra shared-memory traffic, and nothing ever
    // looks at its column of the accumulators
    const uint32_t b_lane = b_base + (column_live ? lane : (COLS == 4 ? (g & 1) * 4 + t : t)) * B_LANE;

    float part[M][TILES][PARTS];
    int acc[PLANES][2][M][TILES][4];  // two chains per (plane, matrix, tile), used by alternate steps: the MMA's dependent latency is long
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
#pragma unroll
        for (int r = 0; r < PARTS; ++r) part[m][tl][r] = 0.0f;
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int pl = 0; pl < PLANES; ++pl) acc[pl][0][m][tl][r] = acc[pl][1][m][tl][r] = 0;
      }
    // what the epilogue needs of this lane's routes, asked for now so that the loads fly behind
    // the main loop instead of in front of the stores
    int ep_route[RPL];
    const int32_t* ep_sums[RPL];  // the lane's routes' sums of x' per scale group
    uint32_t share_sum[RPL];      // split form: sum of x' over this warp's chunks since the last close
    float ep_xs[RPL], ep_weight[RPL], ep_sum[RPL];
#pragma unroll
    for (int cc = 0; cc < RPL; ++cc) {
      const int col = RPL * t + cc;
      ep_route[cc] = col < gsize ? p.groups_of_routes.routes[gstart + col] : -1;
      const int64_t xrow = ep_route[cc] < 0 ? p.x_zero_row : static_cast<int64_t>(ep_route[cc] / p.x_div);
      ep_xs[cc] = p.x.scale[xrow];
      ep_weight[cc] = (M == 2 && ep_route[cc] >= 0) ? p.route_weight[ep_route[cc]] : 1.0f;
      ep_sums[cc] = SPLIT ? p.x.chunk_sums + xrow * n_chunks : p.x.sums + xrow * p.groups;  // split form: per 256 inputs, added up over the warp's share
      ep_sum[cc] = static_cast<float>(p.x.sums[xrow * p.groups]);  // the only group when the rows have one scale
      share_sum[cc] = 0u;
    }
    float row_scale[M][TILES][2];  // the last scale group's scale of rows g and g + 8

    // accumulators -> fp32 partials at the end of a scale group
    auto close_group = [&](const void* const (&scales)[2], int64_t row_base, int64_t groups, int group, float (&into)[M][TILES][PARTS], bool keep_scale) {
      // keep_scale marks the base pass: its operand was u = q + 8, which added 8 * sum(x') of the
      // group (of the warp's share of it) to the integer dot product
      uint32_t offset[RPL];
#pragma unroll
      for (int cc = 0; cc < RPL; ++cc) {
        offset[cc] = keep_scale ? 8u * (SPLIT ? share_sum[cc] : static_cast<uint32_t>(ep_sums[cc][group])) : 0u;
        if (keep_scale) share_sum[cc] = 0u;
      }
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const int64_t row = min(row0 + 16 * tl + g + 8 * rr, N - 1);
            const float sc = load_as_float(scales[m], p.scales_dtype, (row_base + row) * groups + group);
            if (keep_scale) row_scale[m][tl][rr] = sc;
#pragma unroll
            for (int cc = 0; cc < RPL; ++cc) {
              int hi, lo;
              if (COLS == 4) {  // columns 2t, 2t+1 of the one MMA are this lane's route: high plane, low plane
                hi = acc[0][0][m][tl][2 * rr] + acc[0][1][m][tl][2 * rr];
                lo = acc[0][0][m][tl][2 * rr + 1] + acc[0][1][m][tl][2 * rr + 1];
              } else {
                hi = acc[0][0][m][tl][2 * rr + cc] + acc[0][1][m][tl][2 * rr + cc];
                lo = acc[PLANES - 1][0][m][tl][2 * rr + cc] + acc[PLANES - 1][1][m][tl][2 * rr + cc];
              }
              // 256 hi + lo - 8 sum(x') in wrapping 32-bit arithmetic: the true value, sum(q x'), fits
              const int dot = static_cast<int>(static_cast<uint32_t>(hi) * 256u + static_cast<uint32_t>(lo) - offset[cc]);
              into[m][tl][rr * RPL + cc] = fmaf(sc, static_cast<float>(dot), into[m][tl][rr * RPL + cc]);
            }
#pragma unroll
            for (int pl = 0; pl < PLANES; ++pl)
#pragma unroll
              for (int r = 2 * rr; r < 2 * rr + 2; ++r) acc[pl][0][m][tl][r] = acc[pl][1][m][tl][r] = 0;
          }
    };

    int group = c_first / chunks_per_group, left_in_group = chunks_per_group - c_first % chunks_per_group;
    for (int c = c_first; c < c_end; ++c, ++ring_turn) {
      if (CARRY && c + 1 == c_end && has_next) fetch(next_item, c_first, ring_turn + 1);
      else fetch(it, c + 1, ring_turn + 1);
      sk_wait<1>();  // chunk c has landed (the younger group may still fly)
      uint4 cur[4];
      const uint32_t src = ring + (ring_turn % SK_STAGES) * STAGE_BYTES;
      sk_static_for<4>([&](auto s) { cur[decltype(s)::value] = sk_lds128<decltype(s)::value * 512>(src); });
      if (SPLIT) {
#pragma unroll
        for (int cc = 0; cc < RPL; ++cc) share_sum[cc] += static_cast<uint32_t>(ep_sums[cc][c]);
      }
      const uint32_t b_addr = b_lane + c * 8 * B_STEP;
      sk_static_for<8>([&](auto index) {
        constexpr int I = decltype(index)::value;
        uint32_t b[4];
        if (COLS == 4) { const uint2 v = sk_lds64<I * B_STEP>(b_addr); b[0] = v.x; b[1] = v.y; }
        else { const uint4 v = sk_lds128<I * B_STEP>(b_addr); b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w; }
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int tl = 0; tl < TILES; ++tl) {
            uint32_t a[4];
            decode_codeword_nibble<(I & 1) != 0>(sk_word<I>(cur[(m * TILES + tl) * 2]), abs_lane, sign_lane, a[0], a[2]);      // row g
            decode_codeword_nibble<(I & 1) != 0>(sk_word<I>(cur[(m * TILES + tl) * 2 + 1]), abs_lane, sign_lane, a[1], a[3]);  // row g + 8
            sk_mma_u8(acc[0][I & 1][m][tl], a[0], a[1], a[2], a[3], b[0], b[1]);
            if (PLANES == 2) sk_mma_u8(acc[PLANES - 1][I & 1][m][tl], a[0], a[1], a[2], a[3], b[2], b[3]);
          }
      });
      if (--left_in_group == 0) {
        const void* const scales[2] = {mats[0].scales, mats[1].scales};
        close_group(scales, slot * N, p.groups, group, part, true);
        ++group;
        left_in_group = chunks_per_group;
      }
    }
    if (SPLIT && left_in_group != chunks_per_group) {  // this warp's share ends inside a scale group
      const void* const scales[2] = {mats[0].scales, mats[1].scales};
      close_group(scales, slot * N, p.groups, group, part, true);
    }
    if (!CARRY) sk_wait<0>();

    // ---- the residual of a hot slot: a second pass over its 8-bit codes ---------------------
    float rpart[M][TILES][PARTS];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int r = 0; r < PARTS; ++r) rpart[m][tl][r] = 0.0f;
    if (NESTED) {
      const uint32_t hot = p.hot_of_slot[slot];
      if (hot != 0xFFFFFFFFu) {
        const uint8_t* res_ptr[4];
#pragma unroll
        for (int s = 0; s < 4; ++s)
          res_ptr[s] = mats[s / (2 * TILES)].res_codes + (static_cast<int64_t>(hot) * N + min(row0 + 8 * (s % (2 * TILES)) + g, N - 1)) * cw + t * 8;
        auto fetch_res = [&](int c) {  // 8 codes of 8 bits per row stream
          if (c < c_end) {
            const uint32_t dst = ring + (c % SK_STAGES) * STAGE_BYTES;  // the ring is idle here: the base pass has drained it
            sk_static_for<4>([&](auto s) { sk_cp_async8<decltype(s)::value * 512>(dst, res_ptr[decltype(s)::value] + c * SK_CHUNK); });
          }
          sk_commit();
        };
        fetch_res(c_first);
        int res_group = c_first / chunks_per_res_group, left_in_res_group = chunks_per_res_group - c_first % chunks_per_res_group;
        for (int c = c_first; c < c_end; ++c) {
          fetch_res(c + 1);
          sk_wait<1>();
          uint2 cur[4];
          const uint32_t src = ring + (c % SK_STAGES) * STAGE_BYTES;
          sk_static_for<4>([&](auto s) { cur[decltype(s)::value] = sk_lds64<decltype(s)::value * 512>(src); });
          const uint32_t b_addr = b_lane + c * 8 * B_STEP;
          sk_static_for<8>([&](auto index) {
            constexpr int I = decltype(index)::value;
            uint32_t b[4];
            if (COLS == 4) { const uint2 v = sk_lds64<I * B_STEP>(b_addr); b[0] = v.x; b[1] = v.y; }
            else { const uint4 v = sk_lds128<I * B_STEP>(b_addr); b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w; }
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
              for (int tl = 0; tl < TILES; ++tl) {
                uint32_t a[4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                  const uint2 v = cur[(m * TILES + tl) * 2 + half];
                  const uint32_t code = ((I < 4 ? v.x : v.y) >> (8 * (I & 3))) & 0xFFu;
                  const uint2 e = table_entry(code * 128u + res_lane);
                  a[half] = e.x;
                  a[2 + half] = e.y;
                }
                sk_mma(acc[0][I & 1][m][tl], a[0], a[1], a[2], a[3], b[0], b[1]);
                if (PLANES == 2) sk_mma(acc[PLANES - 1][I & 1][m][tl], a[0], a[1], a[2], a[3], b[2], b[3]);
              }
          });
          if (--left_in_res_group == 0) {
            const void* const scales[2] = {mats[0].res_scales, mats[1].res_scales};
            close_group(scales, static_cast<int64_t>(hot) * N, p.res_groups, res_group, rpart, false);
            ++res_group;
            left_in_res_group = chunks_per_res_group;
          }
        }
        if (SPLIT && left_in_res_group != chunks_per_res_group) {
          const void* const scales[2] = {mats[0].res_scales, mats[1].res_scales};
          close_group(scales, static_cast<int64_t>(hot) * N, p.res_groups, res_group, rpart, false);
        }
        sk_wait<0>();
      }
    }

    // ---- split form: the row set's warps add up their shares; its first warp carries on --------
    if (SPLIT && ks > 1) {
      constexpr int VALUES = M * TILES * PARTS;
      const uint32_t mine = red_base + (((red_turn & 1u) * SK_WARPS + warp) * VALUES) * 128u + lane * 4u;
      ++red_turn;
      if (k_part != 0) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
            for (int r = 0; r < PARTS; ++r)
              asm volatile("st.shared.f32 [%0], %1;" ::"r"(mine + ((m * TILES + tl) * PARTS + r) * 128u), "f"(part[m][tl][r] + rpart[m][tl][r]) : "memory");
      }
      // a barrier of the row set's warps only (ids 1..8; id 0 is __syncthreads).  Two buffers by
      // turn: a warp writes buffer (n & 1) again only after the barrier of turn n + 1, which the
      // reading warp joins after it has finished with turn n.
      asm volatile("bar.sync %0, %1;" ::"r"(row_set + 1), "r"(ks * 32) : "memory");
      if (k_part != 0) continue;
      for (int w = 1; w < ks; ++w) {
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
          for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
            for (int r = 0; r < PARTS; ++r) {
              float v;
              asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(mine + (w * VALUES + (m * TILES + tl) * PARTS + r) * 128u));
              part[m][tl][r] += v;
            }
      }
    }

    // ---- epilogue in registers: lane (g, t) holds rows {g, g+8} of each tile for its route(s)
#pragma unroll
    for (int cc = 0; cc < RPL; ++cc) {
      const int route = ep_route[cc];
      if (route < 0) continue;
      const int64_t xrow = route / p.x_div;
      const float xs = ep_xs[cc];
      const float weight = ep_weight[cc];
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int r = rr * RPL + cc;
          const int64_t row = row0 + 16 * tl + g + 8 * rr;
          if (row >= N) continue;
          float y[M];
#pragma unroll
          for (int m = 0; m < M; ++m) {
            float shift = 0.0f;  // the +-1/4 of every weight, folded into sum(x') per scale group
            if (p.groups == 1) {
              shift = row_scale[m][tl][rr] * ep_sum[cc];
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
  sk_wait<0>();
}

// ---- launch -----------------------------------------------------------------------------------

int slab_max_in_dim(int cols) { return cols == 4 ? 8192 : 4096; }  // what the 64 KB activation stage holds

static int device_sm_count(int* device_out) {
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

template <int M, int TILES, int COLS, bool NESTED, bool SPLIT = false>
static int launch_slab(const FastProjectionArgs& p, cudaStream_t s) {
  auto kernel = projection_slab_kernel<M, TILES, COLS, NESTED, SPLIT>;
  static uint64_t configured = 0;  // one bit per device: the shared-memory opt-in is a per-device attribute of the function
  int dev = 0;
  const int sms = device_sm_count(&dev);
  if (dev < 0 || dev >= 64 || !((configured >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_BYTES);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (dev >= 0 && dev < 64) configured |= 1ull << dev;
  }
  cudaError_t err = launch_after(true, kernel, sms, SK_THREADS, SK_SMEM_BYTES, s, p, p.status);
  if (err != cudaSuccess) return note_cuda_error(err);
  return KEEPVQ_OK;
}

// Groups of four routes (inputs up to 8192) or eight (up to 4096).
template <int M, int TILES>
static int launch_slab_projection(const FastProjectionArgs& p, int cols, cudaStream_t s) {
  if (p.in_dim > slab_max_in_dim(cols)) return KEEPVQ_ERR_UNSUPPORTED;
  if (p.res_table) return cols == 4 ? launch_slab<M, TILES, 4, true>(p, s) : launch_slab<M, TILES, 8, true>(p, s);
  return cols == 4 ? launch_slab<M, TILES, 4, false>(p, s) : launch_slab<M, TILES, 8, false>(p, s);
}

int slab_gate_up(const FastProjectionArgs& p, int cols, cudaStream_t s) { return launch_slab_projection<2, 1>(p, cols, s); }
int slab_down(const FastProjectionArgs& p, int cols, cudaStream_t s) { return launch_slab_projection<1, 2>(p, cols, s); }

// The split form, for calls with few route groups (groups of at most four routes).
int slab_split_max_in_dim() { return static_cast<int>(SK_SPLIT_RED_OFF / 8); }  // eight activation columns in front of the partial sums
template <int M, int TILES>
static int launch_split(const FastProjectionArgs& p, cudaStream_t s) {
  if (p.in_dim > slab_split_max_in_dim()) return KEEPVQ_ERR_UNSUPPORTED;
  if (!p.x.chunk_sums) return KEEPVQ_ERR_NULL;  // the warps' shares of a scale group need sum(x') per 256 inputs
  if (p.res_table) return launch_slab<M, TILES, 4, true, true>(p, s);
  return launch_slab<M, TILES, 4, false, true>(p, s);
}
int slab_split_gate_up(const FastProjectionArgs& p, cudaStream_t s) { return launch_split<2, 1>(p, s); }
int slab_split_down(const FastProjectionArgs& p, cudaStream_t s) { return launch_split<1, 2>(p, s); }

}  // namespace fast
}  // namespace keepvq
