// keepvq_routed_matvec: the general routed kernel behind the operator surface (vq_qmv, vq_qmm,
// gather_vqmm direct, e8p_m1_*, e8_1bit_m1_*, e8p_nested_m1_*): any activation dtype, any scale
// group size, any row count, 16-bit E8P or 8-bit E8 codes, optional nested residual, any table.
// The layer kernels (projection_slab.cu, prefill_umma.cu) are the ones tuned for the rooflines;
// this one is built for generality, with the same exact integer arithmetic:
//
//   - every weight is a multiple of 1/4, so a codeword becomes eight int8 values 4w, and a dot
//     product with fixed-point activations is a chain of dp4a instructions, exact in int32;
//   - activations are quantised per row inside the kernel to fixed point with a power-of-two
//     step: 16 bits (two byte planes) for fp16/bf16 rows, 24 bits (three planes) for fp32 rows,
//     so an fp32 caller keeps fp32-grade inputs (relative 2^-23 of the row maximum);
//   - a thread owns one output row: no cross-lane reduction, and the activation bytes it needs
//     are the same address for the whole warp (a shared-memory broadcast).  The four warps of a
//     block split the input dimension by stages of 64 codewords; their partial sums meet in
//     shared memory in a fixed order;
//   - code rows are not contiguous across threads, so each warp copies its [32 rows x 128 bytes]
//     tile with coalesced cp.async pieces into a padded shared-memory tile, two stages deep;
//   - routes that name the same expert are served by one block (the first of them leads, the
//     others leave), four routes per pass, so an expert's codes are streamed once per four routes.
//
// Base and residual of a nested call accumulate apart and meet in one fp32 addition, and each
// part runs the same code as the stand-alone 16-bit / 8-bit call, so an fp32 nested output is
// bit for bit the fp32 sum of the two separate calls.
#include <type_traits>

#include "common.cuh"

namespace keepvq {

constexpr int RD_WARPS = 4;
constexpr int RD_THREADS = RD_WARPS * 32;
constexpr int RD_ROWS = 32;             // output rows per block: one per lane
constexpr int RD_STAGE_CW = 64;         // codewords of a row per stage
constexpr int RD_PASS = 4;              // routes of one expert per pass over its codes
constexpr int RD_REPLICAS = 16;
constexpr int RD_LIST = 1024;           // routes a leader can gather; larger calls run one block per route
constexpr int RD_PITCH16 = RD_STAGE_CW * 2 + 16;  // bytes between rows of a 16-bit code tile (bank-conflict-free 16-byte reads)
constexpr int RD_PITCH8 = RD_STAGE_CW + 16;
constexpr uint32_t RD_SPREAD_LO = (1u << 4) | (1u << 13) | (1u << 22) | (1u << 31);  // sign bits 3,2,1,0 -> bits 7,15,23,31
constexpr uint32_t RD_SPREAD_HI = 1u | (1u << 9) | (1u << 18) | (1u << 27);          // sign bits 7,6,5,4 -> the same places

enum RowdotMode { RD_E8P = 0, RD_E8 = 1, RD_NESTED = 2 };

// Byte order inside a codeword, shared by the tables and the activation planes: byte j of the low
// word is table nibble 3 - j (output dim 6 - 2j), of the high word nibble 7 - j (dim 7 - 2j).
__device__ __forceinline__ int rd_dim_of(int word, int j) { return (word ? 7 : 6) - 2 * j; }

// Table entry of an abs row for one parity: the eight bytes q with 4w = 2q + 1 for positive signs.
__device__ __forceinline__ uint2 rd_abs_entry(uint32_t word, uint32_t par) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int nl = 3 - j, nh = 7 - j;
    uint32_t hl = ((word >> (4 * nl)) & 0xFu) - 8u, hh = ((word >> (4 * nh)) & 0xFu) - 8u;
    if (par) { hl = nl == 0 ? ~hl : hl ^ 1u; hh ^= 1u; }  // odd parity: every weight drops by 1/2, nibble 0 flips sign
    lo |= (hl & 0xFFu) << (8 * j);
    hi |= (hh & 0xFFu) << (8 * j);
  }
  return make_uint2(lo, hi);
}

// The eight values 4w of an 8-bit codeword, from whichever table layout the caller holds.
__device__ __forceinline__ uint2 rd_residual_entry(const uint32_t* table, int layout, int code) {
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int word = 0; word < 2; ++word)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int d = rd_dim_of(word, j);
      int v4;  // 4 * weight of dim d
      if (layout == KEEPVQ_TABLE_HALF2_PAIRS) {
        const __half2 pair = *reinterpret_cast<const __half2*>(&table[code * 4 + (d >> 1)]);
        v4 = __float2int_rn(4.0f * ((d & 1) ? __high2float(pair) : __low2float(pair)));
      } else {
        const int nibble = layout == KEEPVQ_TABLE_PAIR_PACKED ? ((d >> 1) + 4 * (d & 1)) : d;
        v4 = 2 * (static_cast<int>((table[code] >> (4 * nibble)) & 0xFu) - 8);
      }
      (word ? hi : lo) |= (static_cast<uint32_t>(v4) & 0xFFu) << (8 * j);
    }
  return make_uint2(lo, hi);
}

__device__ __forceinline__ uint32_t rd_byte_masks(uint32_t v) {  // the top bit of every byte, spread over the byte
  uint32_t m;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(v), "r"(0u), "r"(0xBA98u));
  return m;
}

// 16-bit E8P codeword -> eight int8 values 4w.  Fast form for tables whose nibbles are all odd
// (negation is then an XOR); any other table goes value by value.
__device__ __forceinline__ uint2 rd_decode_e8p(const uint8_t* abs_table, const uint32_t* raw_table, bool all_odd, uint32_t code, uint32_t lane8) {
  const uint32_t sign = code & 0xFFu, abs_row = code >> 8, parity = __popc(sign) & 1u;
  if (all_odd) {
    const uint2 e = *reinterpret_cast<const uint2*>(abs_table + abs_row * 256u + parity * 128u + lane8);
    const uint32_t ql = e.x ^ (rd_byte_masks(sign * RD_SPREAD_LO) & 0xFEFEFEFEu);
    const uint32_t qh = e.y ^ (rd_byte_masks(sign * RD_SPREAD_HI) & 0xFEFEFEFEu);
    return make_uint2(((ql << 1) & 0xFEFEFEFEu) | 0x01010101u, ((qh << 1) & 0xFEFEFEFEu) | 0x01010101u);  // 2q + 1 per byte
  }
  const uint32_t word = raw_table[abs_row], eff = sign ^ parity;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int w = 0; w < 2; ++w)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int nibble = (w ? 7 : 3) - j;
      int h = static_cast<int>((word >> (4 * nibble)) & 0xFu) - 8;
      if ((eff >> nibble) & 1u) h = -h;
      const int v4 = 2 * h + (parity ? -1 : 1);
      (w ? hi : lo) |= (static_cast<uint32_t>(v4) & 0xFFu) << (8 * j);
    }
  return make_uint2(lo, hi);
}

template <typename XT>
__device__ __forceinline__ float rd_load_x(const XT* p, int64_t i);
template <> __device__ __forceinline__ float rd_load_x<float>(const float* p, int64_t i) { return p[i]; }
template <> __device__ __forceinline__ float rd_load_x<__half>(const __half* p, int64_t i) { return __half2float(p[i]); }
template <> __device__ __forceinline__ float rd_load_x<__nv_bfloat16>(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }

struct RowdotShared {  // fixed-size part of the block's shared memory
  int32_t list[RD_LIST];
  int32_t count;
  int32_t flag;
  float x_scale[RD_PASS];
  float warp_max[RD_WARPS];
  uint32_t raw_table[256];
};

template <typename XT, int MODE>
__global__ void __launch_bounds__(RD_THREADS) routed_rowdot_kernel(keepvq_matvec_args a, int vector_copies) {
  constexpr int PLANES = sizeof(XT) == 4 ? 3 : 2;
  constexpr int QMAX = PLANES == 3 ? 8355711 : 32639;   // 127 in every signed byte plane
  constexpr int QBITS = PLANES == 3 ? 23 : 15;
  constexpr bool BASE16 = MODE != RD_E8;                // the routed codes are 16-bit E8P
  constexpr bool HAS8 = MODE != RD_E8P;                 // an 8-bit stream exists (the codes themselves, or the residual)
  extern __shared__ __align__(16) uint8_t dyn[];
  // layout: fixed part | abs table (E8P) | 8-bit table | reduction | per warp: code tiles, 8-bit tiles, activation planes
  RowdotShared& sh = *reinterpret_cast<RowdotShared*>(dyn);
  constexpr int FIXED = (sizeof(RowdotShared) + 15) / 16 * 16;
  constexpr int ABS_BYTES = BASE16 ? 256 * 2 * RD_REPLICAS * 8 : 0;
  constexpr int T8_BYTES = HAS8 ? 256 * RD_REPLICAS * 8 : 0;
  constexpr int RED_BYTES = 2 * RD_WARPS * RD_PASS * RD_ROWS * 4;
  constexpr int TILE16 = BASE16 ? 2 * RD_ROWS * RD_PITCH16 : 0;
  constexpr int TILE8 = HAS8 ? 2 * RD_ROWS * RD_PITCH8 : 0;
  constexpr int XPLANES = RD_PASS * PLANES * RD_STAGE_CW * 8;
  constexpr int PER_WARP = TILE16 + TILE8 + XPLANES;
  uint8_t* abs_table = dyn + FIXED;
  uint8_t* table8 = abs_table + ABS_BYTES;
  float* red = reinterpret_cast<float*>(table8 + T8_BYTES);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* mine = reinterpret_cast<uint8_t*>(red) + RED_BYTES + warp * PER_WARP;
  uint8_t* tile16 = mine;
  uint8_t* tile8 = mine + TILE16;
  uint8_t* xplanes = mine + TILE16 + TILE8;   // [route][plane][codeword][8]
  const uint32_t lane8 = static_cast<uint32_t>(lane & (RD_REPLICAS - 1)) * 8u;

  const int64_t N = a.out_dim, cw = a.in_dim / 8;
  const int64_t route0 = blockIdx.x;
  const int64_t row = static_cast<int64_t>(blockIdx.y) * RD_ROWS + lane;
  const int64_t row_c = min(row, N - 1);
  const uint32_t slot = a.rhs[route0];

  // ---- a route that is switched off (or names no expert) writes zeros ---------------------------
  if (slot >= static_cast<uint64_t>(a.experts)) {
    if (warp == 0 && row < N) store_from_float(a.out, a.out_dtype, route0 * N + row, 0.0f);
    return;
  }

  // ---- which routes this block serves: all that name `slot`, if none of them comes earlier -------
  const bool gather = a.routes <= RD_LIST;
  if (threadIdx.x == 0) { sh.count = 0; sh.flag = 0; }
  __syncthreads();
  if (gather) {
    for (int64_t r = threadIdx.x; r < route0; r += RD_THREADS)
      if (a.rhs[r] == slot) sh.flag = 1;
    __syncthreads();
    if (sh.flag) return;  // an earlier route of this expert leads
    for (int64_t r = route0 + threadIdx.x; r < a.routes; r += RD_THREADS)
      if (a.rhs[r] == slot) sh.list[atomicAdd(&sh.count, 1)] = static_cast<int32_t>(r);
  } else if (threadIdx.x == 0) {
    sh.list[0] = static_cast<int32_t>(route0);
    sh.count = 1;
  }

  // ---- tables --------------------------------------------------------------------------------------
  bool odd_here = true;
  if (BASE16) {
    for (int e = threadIdx.x; e < 512; e += RD_THREADS) {
      const uint32_t word = a.codebook[e >> 1];
      if (e & 1) sh.raw_table[e >> 1] = word;
      odd_here = odd_here && ((word & 0x11111111u) == 0x11111111u);
      const uint2 entry = rd_abs_entry(word, e & 1);
      uint2* dst = reinterpret_cast<uint2*>(abs_table) + e * RD_REPLICAS;
#pragma unroll
      for (int r = 0; r < RD_REPLICAS; ++r) dst[r] = entry;
    }
  }
  if (HAS8) {
    const uint32_t* table = MODE == RD_E8 ? a.codebook : a.res_table;
    const int layout = MODE == RD_E8 ? a.codebook_layout : KEEPVQ_TABLE_HALF2_PAIRS;
    for (int e = threadIdx.x; e < 256; e += RD_THREADS) {
      const uint2 entry = rd_residual_entry(table, layout, e);
      uint2* dst = reinterpret_cast<uint2*>(table8) + e * RD_REPLICAS;
#pragma unroll
      for (int r = 0; r < RD_REPLICAS; ++r) dst[r] = entry;
    }
  }
  const bool all_odd = __syncthreads_and(odd_here) != 0;  // also orders the tables and the route list
  const int count = sh.count;

  uint32_t hot = KEEPVQ_NO_RESIDUAL;
  if (MODE == RD_NESTED) {
    hot = a.hot_of_slot[slot];
    if (hot >= static_cast<uint64_t>(a.res_rows)) hot = KEEPVQ_NO_RESIDUAL;
  }
  const bool with_res = MODE == RD_NESTED && hot != KEEPVQ_NO_RESIDUAL;

  const int n_stages = static_cast<int>((cw + RD_STAGE_CW - 1) / RD_STAGE_CW);
  const int64_t per_group = cw / a.groups;
  const int64_t res_per_group = MODE == RD_NESTED ? cw / a.res_groups : per_group;
  const uint8_t* codes_base = reinterpret_cast<const uint8_t*>(a.codes) + static_cast<int64_t>(slot) * N * cw * (BASE16 ? 2 : 1);
  const uint8_t* res_base = with_res ? a.res_codes + static_cast<int64_t>(hot) * N * cw : nullptr;
  const int64_t tile_row0 = static_cast<int64_t>(blockIdx.y) * RD_ROWS;

  // copy stage `st` of the block's 32 code rows into this warp's tile buffer `buf`
  auto stage_codes = [&](const uint8_t* base, int code_bytes, uint8_t* tile, int pitch, int st, int buf) {
    const int64_t first = static_cast<int64_t>(st) * RD_STAGE_CW;
    const int n = static_cast<int>(min(static_cast<int64_t>(RD_STAGE_CW), cw - first));  // codewords of this stage
    uint8_t* dst = tile + buf * RD_ROWS * pitch;
    if (vector_copies) {  // 16-byte pieces: eight (four) lanes cover a row's 128 (64) bytes
      const int pieces_per_row = RD_STAGE_CW * code_bytes / 16, live = (n * code_bytes + 15) / 16;
      for (int p = lane; p < RD_ROWS * pieces_per_row; p += 32) {
        const int r = p / pieces_per_row, c = p - r * pieces_per_row;
        if (c >= live) continue;
        const int64_t src_row = min(tile_row0 + r, N - 1);
        const uint32_t to = static_cast<uint32_t>(__cvta_generic_to_shared(dst + r * pitch + c * 16));
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(base + (src_row * cw + first) * code_bytes + c * 16) : "memory");
      }
    } else {  // rows that do not start on 16-byte boundaries: plain loads
      for (int p = lane; p < RD_ROWS * n * code_bytes; p += 32) {
        const int r = p / (n * code_bytes), c = p - r * (n * code_bytes);
        const int64_t src_row = min(tile_row0 + r, N - 1);
        dst[r * pitch + c] = base[(src_row * cw + first) * code_bytes + c];
      }
    }
  };

  for (int pass = 0; pass < count; pass += RD_PASS) {
    const int nr = min(RD_PASS, count - pass);
    __syncthreads();  // the previous pass is done with x_scale and the reduction buffer
    // ---- row scales of this pass's activation rows: a power of two that puts the row maximum below QMAX ----
    const XT* x_rows[RD_PASS];
#pragma unroll
    for (int r = 0; r < RD_PASS; ++r) {
      const int64_t route = sh.list[pass + min(r, nr - 1)];
      x_rows[r] = reinterpret_cast<const XT*>(a.x) + (a.lhs ? static_cast<int64_t>(a.lhs[route]) : route / a.x_div) * a.in_dim;
    }
    for (int r = 0; r < nr; ++r) {
      float amax = 0.0f;
      for (int64_t i = threadIdx.x; i < a.in_dim; i += RD_THREADS) amax = fmaxf(amax, fabsf(rd_load_x<XT>(x_rows[r], i)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      if (lane == 0) sh.warp_max[warp] = amax;
      __syncthreads();
      if (threadIdx.x == 0) {
        float m = 0.0f;
        for (int w = 0; w < RD_WARPS; ++w) m = fmaxf(m, sh.warp_max[w]);
        float s = 1.0f;
        if (m > 0.0f && isfinite(m)) {
          int ex;
          frexpf(m, &ex);                 // m < 2^ex
          s = ldexpf(1.0f, ex - QBITS);   // |x| / s < 2^QBITS
          if (m / s > static_cast<float>(QMAX)) s *= 2.0f;
        }
        sh.x_scale[r] = s;
      }
      __syncthreads();
    }
    float inv_scale[RD_PASS];
#pragma unroll
    for (int r = 0; r < RD_PASS; ++r) inv_scale[r] = 1.0f / sh.x_scale[min(r, nr - 1)];  // exact: powers of two

    float part[RD_PASS], rpart[RD_PASS];
#pragma unroll
    for (int r = 0; r < RD_PASS; ++r) part[r] = rpart[r] = 0.0f;

    // ---- this warp's stages: warp w takes stages w, w + 4, ... ---------------------------------
    int buf = 0;
    if (warp < n_stages) {
      if (BASE16) stage_codes(codes_base, 2, tile16, RD_PITCH16, warp, 0);
      else stage_codes(codes_base, 1, tile8, RD_PITCH8, warp, 0);
      if (with_res) stage_codes(res_base, 1, tile8, RD_PITCH8, warp, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int st = warp; st < n_stages; st += RD_WARPS, buf ^= 1) {
      if (st + RD_WARPS < n_stages) {
        if (BASE16) stage_codes(codes_base, 2, tile16, RD_PITCH16, st + RD_WARPS, buf ^ 1);
        else stage_codes(codes_base, 1, tile8, RD_PITCH8, st + RD_WARPS, buf ^ 1);
        if (with_res) stage_codes(res_base, 1, tile8, RD_PITCH8, st + RD_WARPS, buf ^ 1);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      const int64_t first = static_cast<int64_t>(st) * RD_STAGE_CW;
      const int n = static_cast<int>(min(static_cast<int64_t>(RD_STAGE_CW), cw - first));
      // activation planes of the stage: lane l converts codewords l and l + 32 of every route
      for (int r = 0; r < nr; ++r)
        for (int c = lane; c < n; c += 32) {
          uint32_t words[PLANES][2];
#pragma unroll
          for (int pl = 0; pl < PLANES; ++pl) words[pl][0] = words[pl][1] = 0;
#pragma unroll
          for (int w = 0; w < 2; ++w)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float v = rd_load_x<XT>(x_rows[r], (first + c) * 8 + rd_dim_of(w, j));
              int q = max(-QMAX, min(QMAX, __float2int_rn(v * inv_scale[r])));
#pragma unroll
              for (int pl = 0; pl < PLANES; ++pl) {  // signed bytes, least significant plane first
                const int up = (q + 128) >> 8;
                words[pl][w] |= static_cast<uint32_t>((q - 256 * up) & 0xFF) << (8 * j);
                q = up;
              }
            }
#pragma unroll
          for (int pl = 0; pl < PLANES; ++pl)
            *reinterpret_cast<uint2*>(xplanes + ((r * PLANES + pl) * RD_STAGE_CW + c) * 8) = make_uint2(words[pl][0], words[pl][1]);
        }
      asm volatile("cp.async.wait_group 1;" ::: "memory");  // this stage's codes have landed (the next may still fly)
      __syncwarp();

      // ---- the thread's row against every route of the pass ------------------------------------
      auto run = [&](auto is_residual) {
        constexpr bool RES = decltype(is_residual)::value;
        constexpr bool WIDE = BASE16 && !RES;  // 16-bit codes in this stream
        const uint8_t* my = (WIDE ? tile16 + buf * RD_ROWS * RD_PITCH16 + lane * RD_PITCH16 : tile8 + buf * RD_ROWS * RD_PITCH8 + lane * RD_PITCH8);
        const int64_t group_cw = RES ? res_per_group : per_group;
        const void* scales = RES ? a.res_scales : a.scales;
        const int scales_dtype = RES ? a.res_scales_dtype : a.scales_dtype;
        const int64_t scale_row = RES ? (static_cast<int64_t>(hot) * N + row_c) * a.res_groups : (static_cast<int64_t>(slot) * N + row_c) * a.groups;
        float (&into)[RD_PASS] = RES ? rpart : part;
        int acc[RD_PASS][PLANES];
#pragma unroll
        for (int r = 0; r < RD_PASS; ++r)
#pragma unroll
          for (int pl = 0; pl < PLANES; ++pl) acc[r][pl] = 0;
        // one codeword of the row against every route of the pass
        auto consume = [&](uint32_t code, int c) {
          uint2 w4;
          if (WIDE) w4 = rd_decode_e8p(abs_table, sh.raw_table, all_odd, code, lane8);
          else w4 = *reinterpret_cast<const uint2*>(table8 + code * 128u + lane8);
#pragma unroll
          for (int r = 0; r < RD_PASS; ++r) {
            if (r >= nr) break;
#pragma unroll
            for (int pl = 0; pl < PLANES; ++pl) {
              const uint2 xv = *reinterpret_cast<const uint2*>(xplanes + ((r * PLANES + pl) * RD_STAGE_CW + c) * 8);  // one address for the whole warp
              acc[r][pl] = __dp4a(static_cast<int>(w4.x), static_cast<int>(xv.x), __dp4a(static_cast<int>(w4.y), static_cast<int>(xv.y), acc[r][pl]));
            }
          }
        };
        // exact int32 sums -> fp32, times the scale of the group they belong to
        auto close = [&](int64_t group) {
          const float sc = load_as_float(scales, scales_dtype, scale_row + group);
#pragma unroll
          for (int r = 0; r < RD_PASS; ++r) {
            float v = static_cast<float>(acc[r][PLANES - 1]);
#pragma unroll
            for (int pl = PLANES - 2; pl >= 0; --pl) v = fmaf(v, 256.0f, static_cast<float>(acc[r][pl]));
            into[r] = fmaf(sc, v, into[r]);
#pragma unroll
            for (int pl = 0; pl < PLANES; ++pl) acc[r][pl] = 0;
          }
        };
        int64_t group = first / group_cw;
        int64_t left = group_cw - (first - group * group_cw);  // codewords until the scale group ends
        int c = 0;
        bool open = false;
        while (c < n) {
          if (left >= 8 && c + 8 <= n && (c & 7) == 0) {  // eight codewords from one conflict-free 16-byte (8-byte) read
            uint32_t words[4];
            if (WIDE) {
              const uint4 v = *reinterpret_cast<const uint4*>(my + c * 2);
              words[0] = v.x; words[1] = v.y; words[2] = v.z; words[3] = v.w;
            } else {
              const uint2 v = *reinterpret_cast<const uint2*>(my + c);
              words[0] = v.x; words[1] = v.y; words[2] = words[3] = 0;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
              consume(WIDE ? (words[i >> 1] >> (16 * (i & 1))) & 0xFFFFu : (words[i >> 2] >> (8 * (i & 3))) & 0xFFu, c + i);
            c += 8;
            left -= 8;
          } else {
            consume(WIDE ? reinterpret_cast<const uint16_t*>(my)[c] : my[c], c);
            ++c;
            --left;
          }
          open = true;
          if (left == 0) {
            close(group);
            ++group;
            left = group_cw;
            open = false;
          }
        }
        if (open) close(group);  // the group goes on in a later stage
      };
      run(std::false_type{});
      if (with_res) run(std::true_type{});
      __syncwarp();  // the planes are rewritten by the next stage
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- the four warps' partial sums meet in a fixed order --------------------------------------
#pragma unroll
    for (int r = 0; r < RD_PASS; ++r) {
      red[((0 * RD_WARPS + warp) * RD_PASS + r) * RD_ROWS + lane] = part[r];
      red[((1 * RD_WARPS + warp) * RD_PASS + r) * RD_ROWS + lane] = rpart[r];
    }
    __syncthreads();
    if (warp == 0 && row < N) {
      for (int r = 0; r < nr; ++r) {
        float base = 0.0f, res = 0.0f;
#pragma unroll
        for (int w = 0; w < RD_WARPS; ++w) {
          base += red[((0 * RD_WARPS + w) * RD_PASS + r) * RD_ROWS + lane];
          res += red[((1 * RD_WARPS + w) * RD_PASS + r) * RD_ROWS + lane];
        }
        const float xs = 0.25f * sh.x_scale[r];  // the tables hold 4w
        float total = xs * base;
        if (with_res) total += xs * res;
        store_from_float(a.out, a.out_dtype, static_cast<int64_t>(sh.list[pass + r]) * N + row, total);
      }
    }
  }
}

template <typename XT, int MODE>
static int launch_rowdot(const keepvq_matvec_args& a, int vector_copies, cudaStream_t s) {
  constexpr int PLANES = sizeof(XT) == 4 ? 3 : 2;
  constexpr bool BASE16 = MODE != RD_E8, HAS8 = MODE != RD_E8P;
  constexpr size_t smem = (sizeof(RowdotShared) + 15) / 16 * 16 + (BASE16 ? 256 * 2 * RD_REPLICAS * 8 : 0) + (HAS8 ? 256 * RD_REPLICAS * 8 : 0) +
                          2 * RD_WARPS * RD_PASS * RD_ROWS * 4 +
                          RD_WARPS * ((BASE16 ? 2 * RD_ROWS * RD_PITCH16 : 0) + (HAS8 ? 2 * RD_ROWS * RD_PITCH8 : 0) + RD_PASS * PLANES * RD_STAGE_CW * 8);
  static uint64_t configured = 0;  // one bit per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !((configured >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(routed_rowdot_kernel<XT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
    if (dev >= 0 && dev < 64) configured |= 1ull << dev;
  }
  const int64_t row_tiles = (a.out_dim + RD_ROWS - 1) / RD_ROWS;
  if (row_tiles > 65535 || a.routes > 0x7FFFFFFFll) return KEEPVQ_ERR_CAPACITY;
  const dim3 grid(static_cast<unsigned>(a.routes), static_cast<unsigned>(row_tiles));
  routed_rowdot_kernel<XT, MODE><<<grid, RD_THREADS, smem, s>>>(a, vector_copies);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}

template <typename XT>
static int launch_rowdot_mode(const keepvq_matvec_args& a, int vector_copies, cudaStream_t s) {
  if (a.res_codes) return launch_rowdot<XT, RD_NESTED>(a, vector_copies, s);
  if (a.code_bits == 16) return launch_rowdot<XT, RD_E8P>(a, vector_copies, s);
  return launch_rowdot<XT, RD_E8>(a, vector_copies, s);
}

}  // namespace keepvq

extern "C" int keepvq_routed_matvec(const keepvq_matvec_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_matvec_args& a = *args;
  if (!a.x || !a.codes || !a.scales || !a.codebook || !a.rhs || !a.out) return KEEPVQ_ERR_NULL;
  if (a.code_bits != 8 && a.code_bits != 16) return KEEPVQ_ERR_DTYPE;
  if (!valid_dtype(a.x_dtype) || !valid_dtype(a.scales_dtype) || !valid_dtype(a.out_dtype)) return KEEPVQ_ERR_DTYPE;
  if (a.in_dim <= 0 || a.out_dim <= 0 || a.experts <= 0 || a.groups <= 0 || a.routes < 0) return KEEPVQ_ERR_SHAPE;
  if (a.in_dim % 8 != 0) return KEEPVQ_ERR_SHAPE;
  const int64_t cw = a.in_dim / 8;
  if (cw % a.groups != 0) return KEEPVQ_ERR_SHAPE;
  if (!a.lhs && a.x_div <= 0) return KEEPVQ_ERR_SHAPE;
  if (a.code_bits == 16 && a.codebook_layout != KEEPVQ_TABLE_PACKED) return KEEPVQ_ERR_UNSUPPORTED;
  if (a.codebook_layout < KEEPVQ_TABLE_PACKED || a.codebook_layout > KEEPVQ_TABLE_HALF2_PAIRS) return KEEPVQ_ERR_DTYPE;
  if (a.res_codes) {
    if (a.code_bits != 16) return KEEPVQ_ERR_UNSUPPORTED;
    if (!a.res_scales || !a.res_table || !a.hot_of_slot) return KEEPVQ_ERR_NULL;
    if (!valid_dtype(a.res_scales_dtype)) return KEEPVQ_ERR_DTYPE;
    if (a.res_groups <= 0 || cw % a.res_groups != 0 || a.res_rows <= 0) return KEEPVQ_ERR_SHAPE;
  }
  if (a.routes == 0) return KEEPVQ_OK;
  if (!aligned_to(a.x, dtype_size(a.x_dtype)) || !aligned_to(a.codes, a.code_bits / 8)) return KEEPVQ_ERR_ALIGN;
  // 16-byte copies need every code row to start on a 16-byte boundary; anything else takes plain loads
  const int code_bytes = a.code_bits / 8;
  int vector_copies = aligned_to(a.codes, 16) && (cw * code_bytes) % 16 == 0;
  if (a.res_codes && !(aligned_to(a.res_codes, 16) && cw % 16 == 0)) vector_copies = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.x_dtype == KEEPVQ_F32) return launch_rowdot_mode<float>(a, vector_copies, s);
  if (a.x_dtype == KEEPVQ_F16) return launch_rowdot_mode<__half>(a, vector_copies, s);
  return launch_rowdot_mode<__nv_bfloat16>(a, vector_copies, s);
}
