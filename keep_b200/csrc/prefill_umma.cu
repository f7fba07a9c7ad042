// Expert-grouped projections for many tokens per expert (prefill) on the 5th-generation tensor
// cores: tcgen05.mma kind::i8 with accumulators in tensor memory.
//
// Stands in for the reference's expert-block prefill kernels
// (native/vq_nax_ext/kernels/nax_fp16_matmul.metal:904-1062,11562-11674 and
// src/ramp/kernels/gather_vqmm.py:690-928): routes sorted by expert, codes decoded inside the
// kernel into operand tiles, a dense contraction per (expert, row tile).
//
// Arithmetic: the same exact-integer form as the decode kernels (moe_fast.cuh).  A codeword
// becomes eight int8 values q with 4w = 2q + 1; activations are 16-bit fixed point split in a
// signed high and an unsigned low byte.  Per (expert, 128 output rows, up to 96 routes):
//   [D_hi | D_lo][128 x 2N] += Q[128 x K] * [Xhi ; Xlo][2N x K]^T   (int32, exact, in TMEM)
//   y = scale_row * scale_x * (0.5 * (256 D_hi + D_lo) + 0.25 * sum(x'))
// The weights are the M operand (128 rows per tile) and the routes the N operand (their high-byte
// rows stacked on their low-byte rows, so one MMA reads the decoded tile once for both), so a
// ragged expert group costs at most 15 padded columns, and a code is decoded once per 96 routes.
//
// Pipeline per CTA (persistent, one per SM, 20 warps).  An item is (expert, two A tiles, <= 96
// routes): the gate and the up matrix over the same 128 rows, or two consecutive 128-row tiles of
// a single matrix; either way one set of activation tiles serves both.
//   warps 0-7    decode: a thread owns half a row of the K block (8 codewords per tile); codes
//                arrive through a private cp.async ring; one abs-table read plus sign arithmetic
//                per codeword, 16-byte stores into a K-major SWIZZLE_128B tile (3 stages).
//   warp  8      issues the MMAs (one thread) into the accumulators in tensor memory (a second
//                buffer when the item's columns leave room for one), commits stages back.
//   warps 9-11   cp.async the routes' quantised activations into the B tiles (3 stages).
//   warps 12-19  epilogue, two warps per quarter of the rows taking alternate 16-column chunks:
//                tcgen05.ld of the finished buffer, dequantisation, SwiGLU, stores.
// mbarrier full/empty pairs carry every dependency.  Every wait is bounded: on expiry the CTA
// raises a flag in `status`, stops issuing work, frees its tensor memory and returns.
#include <stdlib.h>

#include "moe_fast.cuh"

namespace keepvq {
namespace fast {

constexpr int PF_DECODE_WARPS = 8;
constexpr int PF_B_WARPS = 3;
constexpr int PF_EPI_WARPS = 8;                 // two per quarter of the rows, alternating 16-column chunks
constexpr int PF_THREADS = (PF_DECODE_WARPS + 1 + PF_B_WARPS + PF_EPI_WARPS) * 32;  // 640
constexpr int PF_A_STAGES = 3;
constexpr int PF_B_STAGES = 3;
constexpr int PF_B_LAG = 1;                     // K blocks of activation copies in flight behind the one being published
static_assert(PF_B_LAG >= 1 && PF_B_LAG <= PF_B_STAGES - 2 && PF_B_LAG <= 2, "see the loader's publication rule");
constexpr int PF_N_MAX = PREFILL_GROUP_ROUTES;  // routes per item
constexpr int PF_ROWS = 128;                    // output rows per item
constexpr int PF_KBLOCK_CODES = 16;             // codewords of a row per K block = 128 bytes of int8
constexpr int PF_TILE_BYTES = PF_ROWS * 128;    // 16 KB: one A tile
constexpr int PF_B_STAGE_BYTES = 2 * PF_N_MAX * 128;  // high-byte rows of the routes, then their low-byte rows
constexpr int PF_TABLE_BYTES = 256 * 16 * 8;     // abs table, 16 replicas of 8 bytes
constexpr int PF_CODE_RING_BYTES = 16 * 1024;    // per-thread code prefetch ring of the decode warps
constexpr uint32_t PF_SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait.  Returns false when the limit expires or another thread of the CTA gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t spin = 0; spin < PF_SPIN_LIMIT; ++spin) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// sign * PF_SPREAD_LO puts sign bits 3,2,1,0 on bits 7,15,23,31; PF_SPREAD_HI does so for bits 7,6,5,4
// (the shifted copies of an 8-bit value never overlap).  sign_masks then fills each byte with its top bit.
constexpr uint32_t PF_SPREAD_LO = (1u << 4) | (1u << 13) | (1u << 22) | (1u << 31);
constexpr uint32_t PF_SPREAD_HI = 1u | (1u << 9) | (1u << 18) | (1u << 27);
__device__ __forceinline__ uint32_t sign_masks(uint32_t v) {
  uint32_t m;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(v), "r"(0u), "r"(0xBA98u));
  return m;
}

// K-major SWIZZLE_128B operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t tile_addr) {
  return static_cast<uint64_t>((tile_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint32_t swizzled(uint32_t row, uint32_t chunk) {  // byte offset of a 16-byte chunk
  return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                 "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr) : "memory");
}

__device__ __forceinline__ void cp_async16_pf(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// GLU: the M = 2 A tiles are the gate and the up matrix over the same 128 rows, fused by SwiGLU.
// !GLU: the M tiles are consecutive 128-row tiles of one matrix, so an item covers 128 * M rows
// and its activation (B) stages serve all of them (the copies are what bounds a single projection).
template <int M, bool GLU>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_projection_kernel(FastProjectionArgs p, int32_t* status, int diag) {
  constexpr int ITEM_ROWS = GLU ? PF_ROWS : PF_ROWS * M;
  extern __shared__ uint8_t smem_raw[];
  // SWIZZLE_128B tiles want 1024-byte alignment; the launch reserves the slack
  uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
  // layout: A stages [2][M x 16 KB] | B stages [4][hi rows | lo rows] | abs table 32 KB | code ring
  constexpr int A_STAGE_BYTES = M * PF_TILE_BYTES;
  constexpr int A_BYTES = PF_A_STAGES * A_STAGE_BYTES, B_BYTES = PF_B_STAGES * PF_B_STAGE_BYTES;
  uint8_t* tables = smem + A_BYTES + B_BYTES;
  enum { A_FULL = 0, A_EMPTY = A_FULL + PF_A_STAGES, B_FULL = A_EMPTY + PF_A_STAGES, B_EMPTY = B_FULL + PF_B_STAGES,
         ACC_FULL = B_EMPTY + PF_B_STAGES, ACC_EMPTY = ACC_FULL + 2, N_BARS = ACC_EMPTY + 2 };
  __shared__ __align__(8) uint64_t bars[N_BARS];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  // per-warp copies, so that a role needs no barrier of its own (every cross-warp wait is an mbarrier with a limit)
  __shared__ int4 epi_all[4][PF_N_MAX];  // per row quarter: route, x scale, x sum / 4, gate weight (each epilogue warp fills and reads its own chunks)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto bar = [&](int which, int index) { return bar0 + 8u * static_cast<uint32_t>(which + index); };
  constexpr uint32_t ACC_COLS = 2 * M * PF_N_MAX;   // one accumulator buffer: per matrix the high-byte then the low-byte columns
  constexpr int ACC_BUFS = (2 * ACC_COLS <= 512) ? 2 : 1;  // a second buffer lets the epilogue overlap the next item
  constexpr uint32_t TMEM_COLS = 512;

  // ---- set-up: tables, barriers, tensor memory ------------------------------------------------
  for (int e = tid; e < 256; e += PF_THREADS) {
    // abs entry: byte j of the low word is table nibble 3-j, of the high word 7-j, each as h = nibble - 8
    const uint32_t word = p.codebook[e];
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= ((((word >> (4 * (3 - j))) & 0xFu) - 8u) & 0xFFu) << (8 * j);
      hi |= ((((word >> (4 * (7 - j))) & 0xFu) - 8u) & 0xFFu) << (8 * j);
    }
    uint2* dst = reinterpret_cast<uint2*>(tables) + e * 16;
#pragma unroll
    for (int r = 0; r < 16; ++r) dst[r] = make_uint2(lo, hi);
  }
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < PF_A_STAGES; ++s) { mbar_init(bar(A_FULL, s), PF_DECODE_WARPS); mbar_init(bar(A_EMPTY, s), 1); }
    for (int s = 0; s < PF_B_STAGES; ++s) { mbar_init(bar(B_FULL, s), PF_B_WARPS); mbar_init(bar(B_EMPTY, s), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(bar(ACC_FULL, s), 1); mbar_init(bar(ACC_EMPTY, s), PF_EPI_WARPS); }  // ACC_BUFS of them in use
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == PF_DECODE_WARPS) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_slot;

  const int64_t N_out = p.out_dim, cw = p.in_dim / 8;
  const int k_blocks = static_cast<int>(cw / PF_KBLOCK_CODES);
  const int row_tiles = static_cast<int>((N_out + ITEM_ROWS - 1) / ITEM_ROWS);
  const int items = p.groups_of_routes.count[0] * row_tiles;
  const Projection mats[2] = {p.a, GLU ? p.b : p.a};
  constexpr int TILE_STEP = GLU ? 0 : PF_ROWS;  // rows between the A tiles of an item
  volatile int* aborted = &abort_flag;

  // Every role walks the same item list on its own clock; barriers carry the dependencies.
  uint32_t iter = 0;  // K blocks since the start: picks stages and phases
  int n_item = 0;
  for (int item = blockIdx.x; item < items && !*aborted; item += gridDim.x, ++n_item, iter += k_blocks) {
    const int gi = item / row_tiles, tile = item - gi * row_tiles;
    const int64_t slot = p.groups_of_routes.slot[gi];
    const int gsize = p.groups_of_routes.size[gi], gstart = p.groups_of_routes.start[gi];
    const int n_pad = (gsize + 15) & ~15;  // the N of the MMA
    const int64_t row0 = static_cast<int64_t>(tile) * ITEM_ROWS;
    const int acc_buf = n_item % ACC_BUFS;
    const uint32_t acc_phase = (n_item / ACC_BUFS) & 1u;

    if (warp < PF_DECODE_WARPS) {
      // ================= decode producers =====================================================
      const uint32_t abs_lane = smem_addr(tables) + (lane & 15) * 8;
      const int row = tid >> 1, half = tid & 1;  // half a row of the K block: 8 codewords
      const uint16_t* src[M];
#pragma unroll
      for (int m = 0; m < M; ++m) src[m] = mats[m].codes + (slot * N_out + min(row0 + m * TILE_STEP + row, N_out - 1)) * cw + half * 8;
      // codes arrive through a private cp.async ring, RING - 1 K blocks ahead of the decode
      constexpr int RING = PF_CODE_RING_BYTES / (M * 256 * 16);
      const uint32_t ring = smem_base + A_BYTES + B_BYTES + PF_TABLE_BYTES + tid * 16;
      auto fetch = [&](int kb) {
        if (kb < k_blocks && diag != 5) {
#pragma unroll
          for (int m = 0; m < M; ++m) cp_async16_pf(ring + ((kb % RING) * M + m) * (256 * 16), src[m] + kb * PF_KBLOCK_CODES);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      };
#pragma unroll
      for (int kb = 0; kb < RING - 1; ++kb) fetch(kb);
      uint32_t it = iter;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        fetch(kb + RING - 1);
        asm volatile("cp.async.wait_group %0;" ::"n"(RING - 1) : "memory");
        uint4 cur[M];
#pragma unroll
        for (int m = 0; m < M; ++m)
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(cur[m].x), "=r"(cur[m].y), "=r"(cur[m].z), "=r"(cur[m].w)
                       : "r"(ring + ((kb % RING) * M + m) * (256 * 16)));
        const uint32_t stage = it % PF_A_STAGES, phase = (it / PF_A_STAGES) & 1u;
        if (!mbar_wait(bar(A_EMPTY, stage), phase ^ 1u, aborted)) break;
        const uint32_t stage_base = smem_base + stage * A_STAGE_BYTES;
#pragma unroll
        for (int m = 0; m < M && diag != 2; ++m) {
          const uint32_t words[4] = {cur[m].x, cur[m].y, cur[m].z, cur[m].w};
#pragma unroll
          for (int pair = 0; pair < 4; ++pair) {  // two codewords = one 16-byte chunk of the row
            const uint32_t w = words[pair];
            uint32_t q[4];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              // q = h ^ (sign bit ? 0xFE : 0); on odd parity of the sign byte ^1 everywhere and ^0xFF on nibble 0
              const uint32_t sign = (w >> (16 * c)) & 0xFFu, odd = 0u - (__popc(sign) & 1u);
              uint32_t ex, ey;
              asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(ex), "=r"(ey) : "r"(abs_lane + ((c ? (w >> 17) : (w >> 1)) & 0x7F80u)));
              q[2 * c] = ex ^ (sign_masks(sign * PF_SPREAD_LO) & 0xFEFEFEFEu) ^ (odd & 0xFF010101u);
              q[2 * c + 1] = ey ^ (sign_masks(sign * PF_SPREAD_HI) & 0xFEFEFEFEu) ^ (odd & 0x01010101u);
            }
            const uint32_t dst = stage_base + m * PF_TILE_BYTES + swizzled(row, half * 4 + pair);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(q[0]), "r"(q[1]), "r"(q[2]), "r"(q[3]) : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(A_FULL, stage));
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp == PF_DECODE_WARPS) {
      // ================= MMA issuer ============================================================
      if (lane == 0) {
        // N = 2 * n_pad: the high-byte rows and the low-byte rows of the routes are one B operand
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n_pad >> 2) << 17) | ((PF_ROWS >> 4) << 24);
        bool ok = mbar_wait(bar(ACC_EMPTY, acc_buf), acc_phase ^ 1u, aborted);  // the epilogue has drained this buffer
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + acc_buf * ACC_COLS;
        uint32_t it = iter;
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const uint32_t sa = it % PF_A_STAGES, sb = it % PF_B_STAGES;
          ok = mbar_wait(bar(A_FULL, sa), (it / PF_A_STAGES) & 1u, aborted) && mbar_wait(bar(B_FULL, sb), (it / PF_B_STAGES) & 1u, aborted);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_base = smem_base + sa * A_STAGE_BYTES, b_base = smem_base + A_BYTES + sb * PF_B_STAGE_BYTES;
          const uint64_t b_desc = umma_desc(b_base);
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const uint64_t a_desc = umma_desc(a_base + m * PF_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < 4 && diag != 4; ++k)  // 32 bytes of K per instruction: advance both start addresses by 2 x 16 B
              umma_i8(acc + m * (2 * PF_N_MAX), a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(bar(A_EMPTY, sa));  // the stages may be refilled once these MMAs have read them
          umma_commit(bar(B_EMPTY, sb));
        }
        if (ok) umma_commit(bar(ACC_FULL, acc_buf));
      }
    } else if (warp < PF_DECODE_WARPS + 1 + PF_B_WARPS) {
      // ================= activation (B operand) loaders =======================================
      // cp.async straight into the swizzled tiles (16 bytes = two codewords of one route); a K
      // block is published when its copies have landed, PF_B_LAG later ones already in flight.
      // A thread keeps one (chunk, plane) and every sixth route: sources and destinations are
      // worked out once per item, a K block then costs an add and a copy per route.
      const int loader = tid - (PF_DECODE_WARPS + 1) * 32;  // 0..95
      constexpr int SLOTS = PF_N_MAX * 16 / (PF_B_WARPS * 32);  // routes per thread
      static_assert(SLOTS * PF_B_WARPS * 32 == PF_N_MAX * 16 && (PF_B_WARPS * 32) % 16 == 0, "loader split");
      const int c = (loader >> 1) & 7, pl = loader & 1, n0 = loader >> 4;
      const int64_t row_bytes = cw * 8;
      const uint8_t* plane = p.x.q + (pl ? (p.x_zero_row + 1) * row_bytes : 0) + c * 16;
      const uint8_t* src[SLOTS];
      uint32_t dst[SLOTS];
#pragma unroll
      for (int i = 0; i < SLOTS; ++i) {
        const int n = n0 + i * (PF_B_WARPS * 2);
        const int route = n < gsize ? p.groups_of_routes.routes[gstart + n] : -1;
        src[i] = plane + (route < 0 ? p.x_zero_row : static_cast<int64_t>(route / p.x_div)) * row_bytes;
        dst[i] = swizzled(pl * n_pad + n, c);
      }
      uint32_t it = iter;
      bool ok = true;
      auto publish = [&](uint32_t which) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_FULL, which % PF_B_STAGES));
      };
      for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
        const uint32_t stage = it % PF_B_STAGES, phase = (it / PF_B_STAGES) & 1u;
        ok = mbar_wait(bar(B_EMPTY, stage), phase ^ 1u, aborted);
        if (!ok) break;
        const uint32_t b_stage = smem_base + A_BYTES + stage * PF_B_STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < SLOTS; ++i)
          if (n0 + i * (PF_B_WARPS * 2) < n_pad && diag != 3) cp_async16_pf(b_stage + dst[i], src[i] + kb * 128);
        asm volatile("cp.async.commit_group;" ::: "memory");
        // Publish K block kb - LAG once its copies have landed, with LAG <= stages - 2: the copies
        // of kb reuse the stage of kb - stages, so publishing kb - LAG then waits on nothing newer
        // than MMAs two blocks before it.  With LAG = stages - 1 every publication waited for the
        // MMAs just before it and the whole pipeline ran in lock step.
        if (kb >= PF_B_LAG) {
          asm volatile("cp.async.wait_group %0;" ::"n"(PF_B_LAG) : "memory");
          publish(it - PF_B_LAG);
        }
      }
      if (ok) {  // drain: publish the last K blocks in order
        const int tail = k_blocks < PF_B_LAG ? k_blocks : PF_B_LAG;
        if (tail >= 2) { asm volatile("cp.async.wait_group 1;" ::: "memory"); publish(it - 2); }
        if (tail >= 1) { asm volatile("cp.async.wait_group 0;" ::: "memory"); publish(it - 1); }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
      // ================= epilogue: accumulators -> y -> (SwiGLU) -> out =======================
      const int epi = warp - (PF_DECODE_WARPS + 1 + PF_B_WARPS), quarter = epi & 3, half = epi >> 2;  // quarter = warp % 4: its TMEM lanes
      if (half == 0) {  // pull the code rows of this CTA's next item into L2 while the current one is being multiplied
        const int next = item + gridDim.x;
        if (next < items) {
          const int ngi = next / row_tiles, ntile = next - ngi * row_tiles;
          const int64_t nrow = static_cast<int64_t>(ntile) * ITEM_ROWS + quarter * 32 + lane;
          const int64_t nslot = p.groups_of_routes.slot[ngi];
#pragma unroll
          for (int m = 0; m < M; ++m)
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(mats[m].codes + (nslot * N_out + min(nrow + m * TILE_STEP, N_out - 1)) * cw), "r"(static_cast<uint32_t>(cw * 2)) : "memory");
        }
      }
      int4* per_route = epi_all[quarter];
      __syncwarp();
      for (int n = half * 16 + (lane & 15) + (lane >> 4) * 32; n < n_pad; n += 64) {  // the columns of this warp's chunks
        const int route = n < gsize ? p.groups_of_routes.routes[gstart + n] : -1;
        const int64_t xrow = route < 0 ? p.x_zero_row : static_cast<int64_t>(route / p.x_div);
        const float weight = (GLU && route >= 0) ? p.route_weight[route] : 1.0f;
        per_route[n] = make_int4(route, __float_as_int(p.x.scale[xrow]), __float_as_int(0.25f * static_cast<float>(p.x.sums[xrow])), __float_as_int(weight));
      }
      __syncwarp();
      const int64_t erow = row0 + quarter * 32 + lane;
      float scale[M];
#pragma unroll
      for (int m = 0; m < M; ++m) scale[m] = load_as_float(mats[m].scales, p.scales_dtype, slot * N_out + min(erow + m * TILE_STEP, N_out - 1));
      if (mbar_wait(bar(ACC_FULL, acc_buf), acc_phase, aborted)) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc_base = tmem + acc_buf * ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
        // One instantiation per output dtype, and no branch inside the column loop except the
        // predicated store: the sixteen columns of a chunk are independent chains the compiler
        // can interleave, which is what hides the latencies of a single warp.
        const float limit = p.swiglu_limit > 0.0f ? p.swiglu_limit : INFINITY;
        const bool row_ok = erow < N_out;
        auto drain = [&](auto round_out, auto store_out) {
          for (int c0 = half * 16; c0 < n_pad && diag != 1; c0 += 32) {
            uint32_t acc[M][2][16];
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
              for (int piece = 0; piece < 2; ++piece) tmem_ld16(acc_base + m * (2 * PF_N_MAX) + piece * n_pad + c0, acc[m][piece]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int4 pr = per_route[c0 + j];
              const float x_scale = __int_as_float(pr.y), x_sum4 = __int_as_float(pr.z);
              float y[M];
#pragma unroll
              for (int m = 0; m < M; ++m) {
                const float dot = 256.0f * static_cast<float>(static_cast<int>(acc[m][0][j])) + static_cast<float>(static_cast<int>(acc[m][1][j]));
                y[m] = scale[m] * x_scale * (0.5f * dot + x_sum4);
              }
              if (GLU) {  // round G and U to the activation dtype first, as the separate kernels of the reference do
                const float gt = fminf(round_out(y[0]), limit);
                const float up = fminf(fmaxf(round_out(y[M - 1]), -limit), limit);
                const float result = gt / (1.0f + expf(-gt)) * up * __int_as_float(pr.w);
                if (pr.x >= 0 && row_ok) store_out(static_cast<int64_t>(pr.x) * N_out + erow, result);
              } else {
#pragma unroll
                for (int m = 0; m < M; ++m)
                  if (pr.x >= 0 && erow + m * TILE_STEP < N_out) store_out(static_cast<int64_t>(pr.x) * N_out + erow + m * TILE_STEP, y[m]);
              }
            }
          }
        };
        if (p.out_dtype == KEEPVQ_BF16)
          drain([](float v) { return __bfloat162float(__float2bfloat16_rn(v)); },
                [&](int64_t i, float v) { static_cast<__nv_bfloat16*>(p.out)[i] = __float2bfloat16_rn(v); });
        else if (p.out_dtype == KEEPVQ_F16)
          drain([](float v) { return __half2float(__float2half_rn(v)); },
                [&](int64_t i, float v) { static_cast<__half*>(p.out)[i] = __float2half_rn(v); });
        else
          drain([](float v) { return v; }, [&](int64_t i, float v) { static_cast<float*>(p.out)[i] = v; });
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(ACC_EMPTY, acc_buf));
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------------
  if (*aborted && tid == 0 && status) atomicExch(status, 1);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == PF_DECODE_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

bool prefill_supported(int64_t out_dim, int64_t in_dim, int64_t groups) {
  return groups == 1 && in_dim % (8 * PF_KBLOCK_CODES) == 0 && out_dim > 0;
}

#ifdef KEEPVQ_DIAG
static int g_prefill_diag = 0;
extern "C" void keepvq_diag_set_prefill(int mode) { g_prefill_diag = mode; }
#endif

template <int M, bool GLU>
static int launch_prefill(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) {
  constexpr size_t smem = PF_A_STAGES * M * PF_TILE_BYTES + PF_B_STAGES * PF_B_STAGE_BYTES + PF_TABLE_BYTES + PF_CODE_RING_BYTES + 1024;
  static uint64_t configured = 0;  // one bit per device: the shared-memory opt-in is a per-device attribute of the function
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !((configured >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(prefill_projection_kernel<M, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
    if (dev >= 0 && dev < 64) configured |= 1ull << dev;
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int diag = 0;
#ifdef KEEPVQ_DIAG
  // measurement build only (outputs meaningless): 1 no epilogue, 2 no decode, 3 no activation copies, 4 no MMAs, 5 no code fetches
  diag = g_prefill_diag;
#endif
  prefill_projection_kernel<M, GLU><<<sms, PF_THREADS, smem, s>>>(p, status, diag);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}

int prefill_gate_up(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) { return launch_prefill<2, true>(p, status, s); }
// a single projection takes two row tiles per item when it has them (the activation copies serve both)
int prefill_down(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) {
  return p.out_dim > PF_ROWS ? launch_prefill<2, false>(p, status, s) : launch_prefill<1, false>(p, status, s);
}

}  // namespace fast
}  // namespace keepvq
