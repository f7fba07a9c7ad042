// Expert-grouped projections for many tokens per expert (prefill) on the 5th-generation tensor
// cores: tcgen05.mma kind::i8 with both the A operand and the accumulators in tensor memory.
//
// Stands in for the reference's expert-block prefill kernels
// (native/vq_nax_ext/kernels/nax_fp16_matmul.metal:904-1062,11562-11674 and
// src/ramp/kernels/gather_vqmm.py:690-928): routes sorted by expert, codes decoded inside the
// kernel into operand tiles, a dense contraction per (expert, row tile).
//
// Arithmetic: the same exact-integer form as the decode kernels (moe_fast.cuh).  A codeword
// becomes eight int8 values q with 4w = 2q + 1; activations are 16-bit fixed point split in a
// signed high and a signed low byte.  Per (expert, 128 output rows, up to 96 routes):
//   [D_hi | D_lo][128 x 2N] += Q[128 x K] * [Xhi ; Xlo][2N x K]^T   (int32, exact, in TMEM)
//   y = scale_row * scale_x * (0.5 * (256 D_hi + D_lo) + 0.25 * sum(x'))
// The weights are the M operand (128 rows per tile) and the routes the N operand (their high-byte
// rows stacked on their low-byte rows, so one MMA reads the decoded tile once for both), so a
// ragged expert group costs at most 15 padded columns, and a code is decoded once per 96 routes.
//
// What bounds this kernel is turning codes into int8 operands, so the roles are cut for that
// (measured with each part switched off in turn: without MMAs, without activation copies or
// without code fetches the kernel took the same time; only the decode mattered):
//   warps 0-15   decode, then drain.  A thread's row of the tile is its lane of tensor memory
//                (warp w reaches lanes 32 * (w % 4) ...); warps 0-7 decode the first tile of an
//                item, warps 8-15 the second, half a row of the K block each (8 codewords).  Codes
//                arrive through a private cp.async ring; the decode is the slab kernel's nibble
//                decoder (two 4-byte table reads at byte-permute addresses, unsigned bytes q + 8);
//                the bytes go straight into TENSOR MEMORY (tcgen05.st), two stages deep, so the
//                A operand never touches shared memory.  When an item's MMAs are done the same
//                warps read its accumulators (tcgen05.ld: same lanes), dequantise, apply SwiGLU
//                and the gate weight, round and store.
//   warp  16     issues the MMAs (one thread): A from tensor memory, B from shared memory.  Its
//                other lanes gather what the drain needs per route (route id, activation scale
//                and sum, gate weight) into shared memory.
//   warp  17     one thread brings the routes' quantised activations into the B tiles (3 stages)
//                with TMA: the rows were quantised in grouped order, so a group's high bytes and
//                its low bytes are two runs of rows of one [2 x rows, K] byte matrix, and a K block
//                of them is a handful of cp.async.bulk.tensor.2d boxes of 16 rows x 128 bytes that
//                land swizzled, ready for the MMA; the boxes report to the stage's mbarrier
//                (expect_tx / complete_tx).
// mbarrier full/empty pairs carry every dependency.  Every wait is bounded by a deadline on the
// global timer: on expiry the CTA raises a flag in `status`, stops issuing work, waits (bounded)
// for the MMAs in flight, frees its tensor memory and returns.
#include <cuda.h>  // CUtensorMap (types only: the one driver entry point is looked up through the runtime)

#include "moe_fast.cuh"

namespace keepvq {
namespace fast {

constexpr int PF_DECODE_WARPS = 16;
constexpr int PF_MMA_WARP = PF_DECODE_WARPS;
constexpr int PF_THREADS = (PF_DECODE_WARPS + 2) * 32;  // 576: decode warps, the MMA warp, the TMA warp
constexpr int PF_A_STAGES = 2;                  // in tensor memory: 32 columns per tile and stage
constexpr int PF_B_STAGES = 4;
constexpr int PF_N_MAX = PREFILL_GROUP_ROUTES;  // routes per item
static_assert(PF_N_MAX % 16 == 0, "an item's routes pad to a multiple of sixteen columns");
constexpr int PF_ROWS = 128;                    // output rows per tile
constexpr int PF_KBLOCK_CODES = 16;             // codewords of a row per K block = 128 bytes of int8
constexpr int PF_A_TILE_COLS = PF_KBLOCK_CODES * 2;   // a decoded K block of one tile: 128 bytes per row = 32 columns
constexpr int PF_B_STAGE_BYTES = 2 * PF_N_MAX * 128;  // high-byte rows of the routes, then their low-byte rows
constexpr int PF_RING = 4;                      // K blocks of codes in flight per decode thread
constexpr int PF_RING_BYTES = PF_RING * PF_DECODE_WARPS * 32 * 16;  // 32 KB
static_assert(PF_RING == 4, "the decode loop's wait counts are written out for a lookahead of up to three K blocks");
constexpr uint32_t PF_TABLE_BYTES = 64 * 1024;  // the nibble decoder's two tables, interleaved (moe_fast.cuh)
// Shared window, absolute addresses.  A0 = the 64 KB boundary the tables sit on:
//   [A0 - 56 KB, A0 - 24 KB) code rings | [A0 - 24 KB, A0) B stage 0 | [A0, +64 KB) tables |
//   [+64 KB, ...) the other B stages
constexpr uint32_t PF_LOW_BYTES = PF_RING_BYTES + PF_B_STAGE_BYTES;
constexpr uint32_t PF_HIGH_BYTES = PF_TABLE_BYTES + (PF_B_STAGES - 1) * PF_B_STAGE_BYTES;
constexpr int PF_SMEM_BYTES = 220 * 1024;       // dynamic request: covers A0 + 144 KB from any base below A0 - 56 KB
constexpr uint64_t PF_DEFAULT_WAIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Wait bounded by time.  Returns false when the deadline passes (the caller's CTA then gives up:
// the flag is raised for every role) or when another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t deadline, volatile int* abort_flag) {
  for (uint32_t spin = 0;; ++spin) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 31u) == 31u) {
      if (*abort_flag) return false;
      if (global_timer_ns() > deadline) { *abort_flag = 1; return false; }
    }
  }
}

// K-major SWIZZLE_128B operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t tile_addr) {
  return static_cast<uint64_t>((tile_addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// A operand in tensor memory: row m of the tile in lane m, K packed along the columns (four int8 per column).  B: shared-memory descriptor.
__device__ __forceinline__ void umma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
               ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Sixteen consecutive columns of this thread's lane of tensor memory.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                 "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
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

// One TMA box of the tensor map -> shared memory; completion is counted on `bar` in bytes.
// x (bytes along K) is a multiple of 128 here and y a row index: both inside the rules for x.
__device__ __forceinline__ void tma_box_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void cp_async16_pf(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

#ifdef KEEPVQ_DIAG
// Measurement build only: where block 0's roles spend their cycles.
// 0 issuer: wait A  1 issuer: wait B  2 issuer: issue + commit  3 issuer: wait accumulators drained  4 issuer: total
// 5 decode warp 0: ring wait + decode  6 decode: wait stage empty  7 decode: store + publish  8 decode: wait accumulators full  9 decode: drain  10 decode: total
__device__ unsigned long long g_pf_timers[16];
#define PF_TICK(var) const long long var = clock64()
#define PF_ADD(slot, from, to) timers[slot] += (to) - (from)
#else
#define PF_TICK(var)
#define PF_ADD(slot, from, to)
#endif

// GLU: the M = 2 A tiles are the gate and the up matrix over the same 128 rows, fused by SwiGLU.
// !GLU: the M tiles are consecutive 128-row tiles of one matrix, so an item covers 128 * M rows
// and its activation (B) stages serve all of them (the copies are what bounds a single projection).
// `stall` != 0 is the wait self-test: the activation loader never publishes, so the MMA issuer's
// first wait runs into the deadline.
template <int M, bool GLU>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_projection_kernel(FastProjectionArgs p, const __grid_constant__ CUtensorMap x_map, int32_t* status, int diag, int stall, uint64_t wait_ns) {
  constexpr int ITEM_ROWS = GLU ? PF_ROWS : PF_ROWS * M;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  enum { A_FULL = 0, A_EMPTY = A_FULL + PF_A_STAGES, B_FULL = A_EMPTY + PF_A_STAGES, B_EMPTY = B_FULL + PF_B_STAGES,
         ACC_FULL = B_EMPTY + PF_B_STAGES, ACC_EMPTY = ACC_FULL + 1, INFO_FULL = ACC_EMPTY + 1, DRAINED = INFO_FULL + 2, N_BARS = DRAINED + 1 };
  __shared__ __align__(8) uint64_t bars[N_BARS];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int4 route_info[2][PF_N_MAX];  // per item (two in flight): route, x scale, x sum / 4, gate weight
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar0 = smem_addr(&bars[0]);
  auto bar = [&](int which, int index) { return bar0 + 8u * static_cast<uint32_t>(which + index); };
  constexpr uint32_t ACC_COLS = 2 * M * PF_N_MAX;   // per matrix the high-byte then the low-byte columns
  constexpr uint32_t A_STAGE_COLS = M * PF_A_TILE_COLS;
  constexpr uint32_t A_COL0 = ACC_COLS;             // the decoded A stages sit behind the accumulators
  constexpr uint32_t TMEM_COLS = 512;
  static_assert(A_COL0 + PF_A_STAGES * A_STAGE_COLS <= TMEM_COLS, "tensor memory holds the accumulators and the A stages");
  const uint64_t deadline = global_timer_ns() + (wait_ns ? wait_ns : PF_DEFAULT_WAIT_NS);

  // ---- the shared window --------------------------------------------------------------------------
  const uint32_t dyn_base = smem_addr(smem_raw);
  const uint32_t a0 = (dyn_base + PF_LOW_BYTES + 0xFFFFu) & ~0xFFFFu;
  const bool window_ok = a0 + PF_HIGH_BYTES <= dyn_base + PF_SMEM_BYTES;  // uniform over the grid
  const uint32_t ring_base = a0 - PF_LOW_BYTES;
  auto b_stage_addr = [&](uint32_t stage) { return stage == 0 ? a0 - PF_B_STAGE_BYTES : a0 + PF_TABLE_BYTES + (stage - 1) * PF_B_STAGE_BYTES; };

  // ---- set-up: tables, barriers, tensor memory ------------------------------------------------
  if (window_ok) build_nibble_tables(a0, p.codebook, tid, PF_THREADS);
  if (tid == 0) {
    abort_flag = window_ok ? 0 : 1;
    for (int s = 0; s < PF_A_STAGES; ++s) { mbar_init(bar(A_FULL, s), M * 8); mbar_init(bar(A_EMPTY, s), 1); }
    for (int s = 0; s < PF_B_STAGES; ++s) { mbar_init(bar(B_FULL, s), 1); mbar_init(bar(B_EMPTY, s), 1); }
    mbar_init(bar(ACC_FULL, 0), 1);
    mbar_init(bar(ACC_EMPTY, 0), PF_DECODE_WARPS);
    mbar_init(bar(INFO_FULL, 0), 1);
    mbar_init(bar(INFO_FULL, 1), 1);
    mbar_init(bar(DRAINED, 0), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == PF_MMA_WARP) {
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
  bool mma_issued = false;
#ifdef KEEPVQ_DIAG
  long long timers[16] = {};
  const long long t_begin = clock64();
#endif

  // Every role walks the same item list on its own clock; barriers carry the dependencies.
  uint32_t issue_a = 0, issue_a_phase = 0, issue_b = 0, issue_b_phase = 0;  // the issuer's place in the two stage rings
  uint32_t iter = 0;  // K blocks since the start: picks stages and phases
  int n_item = 0;
  for (int item = blockIdx.x; item < items && !*aborted; item += gridDim.x, ++n_item, iter += k_blocks) {
    const int gi = item / row_tiles, tile = item - gi * row_tiles;
    const int64_t slot = p.groups_of_routes.slot[gi];
    const int gsize = p.groups_of_routes.size[gi], gstart = p.groups_of_routes.start[gi];
    const int n_pad = (gsize + 15) & ~15;  // the N of the MMA
    const int64_t row0 = static_cast<int64_t>(tile) * ITEM_ROWS;
    const uint32_t item_phase = n_item & 1u;

    if (warp < PF_DECODE_WARPS) {
      // ================= decode, then drain =====================================================
      const int quadrant = warp & 3, half = (warp >> 2) & 1, m = warp >> 3;  // m: which tile of the item this warp decodes
      const int row = quadrant * 32 + lane;
      const uint32_t abs_lane = a0 + lane * 4u, sign_lane = a0 + 128u + lane * 4u;
      bool ok = true;
      if (m < M) {
        auto code_row = [&](int which_item) {  // this thread's code row (its half) of an item
          const int wgi = which_item / row_tiles, wtile = which_item - wgi * row_tiles;
          const int64_t wrow = static_cast<int64_t>(wtile) * ITEM_ROWS + m * TILE_STEP + row;
          return mats[m].codes + (static_cast<int64_t>(p.groups_of_routes.slot[wgi]) * N_out + min(wrow, N_out - 1)) * cw + half * 8;
        };
        const uint16_t* src = code_row(item);
        const int next = item + gridDim.x;
        const uint16_t* next_src = next < items ? code_row(next) : nullptr;
        // codes arrive through a private cp.async ring, PF_RING - 1 K blocks ahead of the decode; the
        // ring runs on across items (slot = K blocks since the kernel began), so an item's first K
        // blocks are already on their way while the previous item is being drained
        const uint32_t ring = ring_base + tid * 16;
        auto fetch = [&](const uint16_t* from, int kb, uint32_t turn) {
          if (from && kb < k_blocks && diag != 5) cp_async16_pf(ring + (turn % PF_RING) * (PF_DECODE_WARPS * 32 * 16), from + kb * PF_KBLOCK_CODES);
          asm volatile("cp.async.commit_group;" ::: "memory");
        };
        const int look = min(PF_RING - 1, k_blocks);  // K blocks ahead: never past the next item
        if (n_item == 0)
          for (int kb = 0; kb < look; ++kb) fetch(src, kb, iter + kb);
        const uint32_t my_tmem = tmem + (static_cast<uint32_t>(quadrant * 32) << 16) + A_COL0 + m * PF_A_TILE_COLS + half * 16;
        uint32_t it = iter;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          PF_TICK(t0);
          const int ahead = kb + look;
          if (ahead < k_blocks) fetch(src, ahead, it + look);
          else fetch(next_src, ahead - k_blocks, it + look);  // the next item's first K blocks
          if (look == 3) asm volatile("cp.async.wait_group 3;" ::: "memory");
          else if (look == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
          else asm volatile("cp.async.wait_group 1;" ::: "memory");
          uint4 cur;
          asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(cur.x), "=r"(cur.y), "=r"(cur.z), "=r"(cur.w)
                       : "r"(ring + (it % PF_RING) * (PF_DECODE_WARPS * 32 * 16)));
          // decode into registers first, then wait for the stage: the MMAs that read it have had a K block's time to finish
          uint32_t q[16];
          decode_codeword_nibble<false>(cur.x, abs_lane, sign_lane, q[0], q[1]);
          decode_codeword_nibble<true>(cur.x, abs_lane, sign_lane, q[2], q[3]);
          decode_codeword_nibble<false>(cur.y, abs_lane, sign_lane, q[4], q[5]);
          decode_codeword_nibble<true>(cur.y, abs_lane, sign_lane, q[6], q[7]);
          decode_codeword_nibble<false>(cur.z, abs_lane, sign_lane, q[8], q[9]);
          decode_codeword_nibble<true>(cur.z, abs_lane, sign_lane, q[10], q[11]);
          decode_codeword_nibble<false>(cur.w, abs_lane, sign_lane, q[12], q[13]);
          decode_codeword_nibble<true>(cur.w, abs_lane, sign_lane, q[14], q[15]);
          const uint32_t stage = it % PF_A_STAGES, phase = (it / PF_A_STAGES) & 1u;
          PF_TICK(t1);
          ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar(A_EMPTY, stage), phase ^ 1u, deadline, aborted));
          if (!ok) break;
          PF_TICK(t2);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (diag != 2) tmem_st16(my_tmem + stage * A_STAGE_COLS, q);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(A_FULL, stage));
          PF_TICK(t3);
          PF_ADD(5, t0, t1); PF_ADD(6, t1, t2); PF_ADD(7, t2, t3);
        }
      }

      // ---- drain: accumulators -> y -> (SwiGLU) -> out.  Four warps share a quadrant's columns.
      const int part = warp >> 2;  // takes the 16-column chunks part, part + 4, ...
      const int64_t erow = row0 + quadrant * 32 + lane;
      float scale[M];
#pragma unroll
      for (int mm = 0; mm < M; ++mm) scale[mm] = load_as_float(mats[mm].scales, p.scales_dtype, slot * N_out + min(erow + mm * TILE_STEP, N_out - 1));
      PF_TICK(t4);
      ok = ok && __all_sync(0xFFFFFFFFu, mbar_wait(bar(INFO_FULL, item_phase), (n_item >> 1) & 1u, deadline, aborted));
      ok = ok && __all_sync(0xFFFFFFFFu, mbar_wait(bar(ACC_FULL, 0), n_item & 1u, deadline, aborted));
      PF_TICK(t5);
      PF_ADD(8, t4, t5);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int4* per_route = route_info[item_phase];
        const uint32_t acc_base = tmem + (static_cast<uint32_t>(quadrant * 32) << 16);
        // One instantiation per output dtype, and no branch inside the column loop except the
        // predicated store: the sixteen columns of a chunk are independent chains the compiler
        // can interleave, which is what hides the latencies of a single warp.
        const float limit = p.swiglu_limit > 0.0f ? p.swiglu_limit : INFINITY;
        const bool row_ok = erow < N_out;
        // The accumulators are free again as soon as they are in registers: a warp gives its
        // arrival when the LAST of its chunks has been read, before the arithmetic and the stores
        // of that chunk, so the next item's MMAs start under them.
        auto drain = [&](auto round_out, auto store_out) {
          bool arrived = false;
          for (int c0 = part * 16; c0 < n_pad && diag != 1; c0 += 64) {
            uint32_t acc[M][2][16];
#pragma unroll
            for (int mm = 0; mm < M; ++mm)
#pragma unroll
              for (int piece = 0; piece < 2; ++piece) tmem_ld16(acc_base + mm * (2 * PF_N_MAX) + piece * n_pad + c0, acc[mm][piece]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (c0 + 64 >= n_pad) {
              asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
              __syncwarp();
              if (lane == 0) mbar_arrive(bar(ACC_EMPTY, 0));
              arrived = true;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int4 pr = per_route[c0 + j];
              const float x_scale = __int_as_float(pr.y), x_sum4 = 0.25f * static_cast<float>(pr.z);
              const uint32_t offset = 8u * static_cast<uint32_t>(pr.z);  // the A operand was u = q + 8: 8 * sum(x') too much
              float y[M];
#pragma unroll
              for (int mm = 0; mm < M; ++mm) {
                // 256 high + low - 8 sum(x') in wrapping 32-bit arithmetic: the true value, sum(q x'), fits
                const int dot = static_cast<int>(acc[mm][0][j] * 256u + acc[mm][1][j] - offset);
                y[mm] = scale[mm] * x_scale * (0.5f * static_cast<float>(dot) + x_sum4);
              }
              if (GLU) {  // round G and U to the activation dtype first, as the separate kernels of the reference do
                const float gt = fminf(round_out(y[0]), limit);
                const float up = fminf(fmaxf(round_out(y[M - 1]), -limit), limit);
                const float result = gt / (1.0f + expf(-gt)) * up * __int_as_float(pr.w);
                if (pr.x >= 0 && row_ok) store_out(static_cast<int64_t>(pr.x) * N_out + erow, result);
              } else {
#pragma unroll
                for (int mm = 0; mm < M; ++mm)
                  if (pr.x >= 0 && erow + mm * TILE_STEP < N_out) store_out(static_cast<int64_t>(pr.x) * N_out + erow + mm * TILE_STEP, y[mm]);
              }
            }
          }
          if (!arrived) {  // a warp without a chunk of this item
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ACC_EMPTY, 0));
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
        PF_TICK(t6);
        PF_ADD(9, t5, t6);
      }
    } else if (warp == PF_MMA_WARP) {
      // ================= per-route facts for the drain, then the MMAs ============================
      // The facts go into the buffer item n - 2 used; every warp finished that item's drain before
      // it produced the stages of item n - 1, all of which have been consumed by now (see the
      // __syncwarp at the end of this branch), so the buffer is free; the gathering hides behind
      // the drain of item n - 1.
      bool ok = true;
      {
        for (int n = lane; n < n_pad; n += 32) {
          const int route = n < gsize ? p.groups_of_routes.routes[gstart + n] : -1;
          const int64_t xrow = route < 0 ? p.x_zero_row : static_cast<int64_t>(gstart + n);  // the activation rows were quantised in grouped order
          const float weight = (GLU && route >= 0) ? p.route_weight[route] : 1.0f;
          route_info[item_phase][n] = make_int4(route, __float_as_int(p.x.scale[xrow]), p.x.sums[xrow], __float_as_int(weight));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(INFO_FULL, item_phase));
      }
      PF_TICK(m0);
      if (n_item >= 1) ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar(ACC_EMPTY, 0), (n_item - 1) & 1u, deadline, aborted));  // the previous item's accumulators are in registers
      PF_TICK(m1);
      PF_ADD(3, m0, m1);
      if (lane == 0 && ok) {
        // N = 2 * n_pad: the high-byte rows and the low-byte rows of the routes are one B operand
        // accumulator s32, A unsigned bytes (the nibble decoder's u = q + 8), B signed bytes
        const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | (static_cast<uint32_t>(n_pad >> 2) << 17) | ((PF_ROWS >> 4) << 24);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int kb = 0; kb < k_blocks && ok; ++kb) {
          const uint32_t sa = issue_a, sb = issue_b;
          PF_TICK(m2);
          ok = mbar_wait(bar(A_FULL, sa), issue_a_phase, deadline, aborted);
          PF_TICK(m3);
          ok = ok && mbar_wait(bar(B_FULL, sb), issue_b_phase, deadline, aborted);
          PF_TICK(m4);
          PF_ADD(0, m2, m3); PF_ADD(1, m3, m4);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_cols = tmem + A_COL0 + sa * A_STAGE_COLS;
          const uint64_t b_desc = umma_desc(b_stage_addr(sb));
#pragma unroll
          for (int m = 0; m < M; ++m) {
#pragma unroll
            for (int k = 0; k < 4 && diag != 4; ++k)  // 32 bytes of K per instruction: 8 columns of A, 2 x 16 bytes of the B start address
              umma_i8_ts(tmem + m * (2 * PF_N_MAX), a_cols + m * PF_A_TILE_COLS + 8 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          }
          mma_issued = true;
          umma_commit(bar(A_EMPTY, sa));  // the stages may be refilled once these MMAs have read them
          umma_commit(bar(B_EMPTY, sb));
          if (++issue_a == PF_A_STAGES) { issue_a = 0; issue_a_phase ^= 1u; }
          if (++issue_b == PF_B_STAGES) { issue_b = 0; issue_b_phase ^= 1u; }
          PF_TICK(m5);
          PF_ADD(2, m4, m5);
        }
        if (ok) umma_commit(bar(ACC_FULL, 0));
      }
      // The other lanes wait here for the issuing lane.  Without this they would run one item ahead
      // and refill the per-route buffer of item n - 1 while that item's drain is still doing the
      // arithmetic of its last chunks (the drain gives the accumulators back BEFORE that arithmetic).
      // Behind this point every K block of item n has been issued, which took the decode warps'
      // stages of item n, and they produce those only after they are done with item n - 1.
      __syncwarp();
    } else {
      // ================= activation (B operand) loader: TMA ====================================
      // Rows gstart .. gstart + n_pad - 1 of the high-byte plane and of the low-byte plane, 16 rows
      // per box (a box lands swizzled at a 2 KB step of the tile); rows past the group's own belong
      // to the next group or to nobody, and nobody looks at their columns.  One thread issues.
      if (warp == PF_MMA_WARP + 1 && lane == 0) {
        uint32_t it = iter;
        const int32_t plane_rows = static_cast<int32_t>(p.x_zero_row + 1);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t stage = it % PF_B_STAGES, phase = (it / PF_B_STAGES) & 1u;
          if (!mbar_wait(bar(B_EMPTY, stage), phase ^ 1u, deadline, aborted)) break;
          if (stall) continue;  // the wait self-test: nothing is ever published
          const uint32_t b_stage = b_stage_addr(stage), full = bar(B_FULL, stage);
          mbar_expect_tx(full, static_cast<uint32_t>(2 * n_pad * 128));
          if (diag != 3) {
            for (int r = 0; r < n_pad; r += 16) {
              tma_box_2d(b_stage + r * 128, &x_map, kb * 128, gstart + r, full);
              tma_box_2d(b_stage + (n_pad + r) * 128, &x_map, kb * 128, plane_rows + gstart + r, full);
            }
          } else {
            // measurement build only: the bytes never come, so count them off by hand
            asm volatile("mbarrier.complete_tx.shared::cta.b64 [%0], %1;" ::"r"(full), "r"(static_cast<uint32_t>(2 * n_pad * 128)) : "memory");
          }
        }
      }
    }
  }

#ifdef KEEPVQ_DIAG
  if (blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == PF_MMA_WARP)) {
    timers[warp == 0 ? 10 : 4] = clock64() - t_begin;
    for (int i = 0; i < 16; ++i) if (timers[i]) atomicAdd(&g_pf_timers[i], static_cast<unsigned long long>(timers[i]));
  }
#endif
  // ---- teardown ------------------------------------------------------------------------------
  if (*aborted) {
    if (tid == 0 && status) atomicExch(status, window_ok ? 1 : 2);
    // MMAs may still be in flight: one more commit arrives when they are all done; wait for it, bounded as every wait
    if (warp == PF_MMA_WARP && lane == 0 && mma_issued) {
      umma_commit(bar(DRAINED, 0));
      const uint64_t grace = global_timer_ns() + 100000000ull;
      for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar(DRAINED, 0)), "r"(0u) : "memory");
        if (done || ((spin & 31u) == 31u && global_timer_ns() > grace)) break;
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == PF_MMA_WARP) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

bool prefill_supported(int64_t out_dim, int64_t in_dim, int64_t groups) {
  return groups == 1 && in_dim % (8 * PF_KBLOCK_CODES) == 0 && out_dim > 0;
}

#ifdef KEEPVQ_DIAG
static int g_prefill_diag = 0;
extern "C" void keepvq_diag_set_prefill(int mode) { g_prefill_diag = mode; }
extern "C" void keepvq_diag_read_timers(unsigned long long* out) {  // host array of 16; reads and clears
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, g_pf_timers, sizeof(unsigned long long) * 16);
  unsigned long long zero[16] = {};
  cudaMemcpyToSymbol(g_pf_timers, zero, sizeof(zero));
}
#endif

// The tensor map of a projection's quantised activations: a [2 * (rows + 1), in_dim] byte matrix
// (the high-byte plane over the low-byte plane), boxes of 16 rows x 128 bytes, 128-byte swizzle.
// The map covers this GPU's own scratch memory only.
static int activation_map(const FastProjectionArgs& p, CUtensorMap* map) {
  typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiled encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (found != cudaDriverEntryPointSuccess || !fn) return KEEPVQ_ERR_UNSUPPORTED;
    encode = reinterpret_cast<EncodeTiled>(fn);
  }
  if (p.in_dim % 128 != 0 || (reinterpret_cast<uintptr_t>(p.x.q) & 15u) != 0) return KEEPVQ_ERR_ALIGN;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.in_dim), static_cast<cuuint64_t>(2 * (p.x_zero_row + 1))};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.in_dim)};
  const cuuint32_t box[2] = {128, 16}, element_strides[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, p.x.q, dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? KEEPVQ_OK : KEEPVQ_ERR_LAUNCH;
}

template <int M, bool GLU>
static int launch_prefill(const FastProjectionArgs& p, int32_t* status, cudaStream_t s, int stall = 0, uint64_t wait_ns = 0, int ctas = 0) {
  CUtensorMap x_map;
  if (const int rc = activation_map(p, &x_map)) return rc;
  static uint64_t configured = 0;  // one bit per device: the shared-memory opt-in is a per-device attribute of the function
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !((configured >> dev) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(prefill_projection_kernel<M, GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM_BYTES);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (dev >= 0 && dev < 64) configured |= 1ull << dev;
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int diag = 0;
#ifdef KEEPVQ_DIAG
  // measurement build only (outputs meaningless): 1 no drain, 2 no tensor-memory stores, 3 no activation copies, 4 no MMAs, 5 no code fetches
  diag = g_prefill_diag;
#endif
  prefill_projection_kernel<M, GLU><<<ctas > 0 ? ctas : sms, PF_THREADS, PF_SMEM_BYTES, s>>>(p, x_map, status, diag, stall, wait_ns);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}

int prefill_gate_up(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) { return launch_prefill<2, true>(p, status, s); }
// a single projection takes two row tiles per item when it has them (the activation copies serve both)
int prefill_down(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) {
  return p.out_dim > PF_ROWS ? launch_prefill<2, false>(p, status, s) : launch_prefill<1, false>(p, status, s);
}
// One CTA of the single-projection kernel whose activation loader never publishes, with a short
// deadline: the wait runs out, the CTA reports and returns.  `p` must describe a valid problem.
int prefill_wait_selftest(const FastProjectionArgs& p, int32_t* status, uint64_t wait_ns, cudaStream_t s) {
  return launch_prefill<1, false>(p, status, s, 1, wait_ns, 1);
}

}  // namespace fast
}  // namespace keepvq
