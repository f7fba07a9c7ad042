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
// signed high and a signed low byte.  Per (expert, 128 output rows, up to 128 routes):
//   D_hi[128 x N] += Q[128 x K] * Xhi[N x K]^T,   D_lo likewise   (int32, exact, in TMEM)
//   y = scale_row * scale_x * (0.5 * (256 D_hi + D_lo) + 0.25 * sum(x'))
// The weights are the M operand (128 rows per tile) and the routes the N operand, so a ragged
// expert group costs at most 15 padded columns, and a code is decoded once per 128 routes.
//
// Pipeline per CTA (persistent, one per SM, 12 warps):
//   warps 0-7   decode: a thread owns half a row of the K block (8 codewords per matrix): one
//               16-byte global load, two table reads and two XORs per codeword, 16-byte stores
//               into a K-major SWIZZLE_128B tile.  After the last K block the same warps read
//               the accumulators back (tcgen05.ld) and run the epilogue.
//   warp  8     issues the MMAs (one thread), commits stages back to the producers.
//   warps 9-11  copy the routes' quantised activations into the B tiles (high and low bytes).
// Two shared-memory stages, mbarrier full/empty pairs.  Every wait is bounded: on expiry the CTA
// raises a flag in `status`, stops issuing work, frees its tensor memory and returns.
#include "moe_fast.cuh"

namespace keepvq {
namespace fast {

constexpr int PF_THREADS = 384;
constexpr int PF_DECODE_WARPS = 8;
constexpr int PF_B_WARPS = 3;
constexpr int PF_STAGES = 2;
constexpr int PF_N_MAX = 128;                   // routes per item
constexpr int PF_ROWS = 128;                    // output rows per item
constexpr int PF_KBLOCK_CODES = 16;             // codewords of a row per K block = 128 bytes of int8
constexpr int PF_TILE_BYTES = PF_ROWS * 128;    // 16 KB
constexpr int PF_TABLE_BYTES = 2 * 256 * 16 * 8;  // abs + sign tables, 16 replicas of 8 bytes
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

template <int M>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_projection_kernel(FastProjectionArgs p, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  // SWIZZLE_128B tiles want 1024-byte alignment; the launch reserves the slack
  uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
  // layout: [stage][A tiles M x 16 KB | B_hi 16 KB | B_lo 16 KB] ... tables
  constexpr int STAGE_BYTES = (M + 2) * PF_TILE_BYTES;
  uint8_t* tables = smem + PF_STAGES * STAGE_BYTES;
  __shared__ __align__(8) uint64_t bars[2 * PF_STAGES + 2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int xrow_of[PF_N_MAX];  // activation row of each route of the current item (loader warps)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t smem_base = smem_addr(smem);
  const uint32_t full0 = smem_addr(&bars[0]), empty0 = smem_addr(&bars[PF_STAGES]);
  const uint32_t accum_full = smem_addr(&bars[2 * PF_STAGES]), accum_empty = smem_addr(&bars[2 * PF_STAGES + 1]);
  constexpr uint32_t TMEM_COLS = M == 2 ? 512 : 256;

  // ---- set-up: tables, barriers, tensor memory ------------------------------------------------
  for (int e = tid; e < 512; e += PF_THREADS) {
    uint32_t lo = 0, hi = 0;
    if (e < 256) {  // abs entry: byte j of the low word is table nibble 3-j, of the high word 7-j
      const uint32_t word = p.codebook[e];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= ((((word >> (4 * (3 - j))) & 0xFu) - 8u) & 0xFFu) << (8 * j);
        hi |= ((((word >> (4 * (7 - j))) & 0xFu) - 8u) & 0xFFu) << (8 * j);
      }
    } else {        // sign entry: 0xFE where the sign bit is set; on odd parity ^1 everywhere, ^0xFF on nibble 0
      const uint32_t sb = e - 256, par = __popc(sb) & 1u;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int nl = 3 - j, nh = 7 - j;
        uint32_t ml = ((sb >> nl) & 1u) ? 0xFEu : 0u, mh = ((sb >> nh) & 1u) ? 0xFEu : 0u;
        if (par) { ml ^= nl == 0 ? 0xFFu : 0x01u; mh ^= 0x01u; }
        lo |= ml << (8 * j);
        hi |= mh << (8 * j);
      }
    }
    uint2* dst = reinterpret_cast<uint2*>(tables) + e * 16;
#pragma unroll
    for (int r = 0; r < 16; ++r) dst[r] = make_uint2(lo, hi);
  }
  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < PF_STAGES; ++s) { mbar_init(full0 + 8 * s, PF_DECODE_WARPS + PF_B_WARPS); mbar_init(empty0 + 8 * s, 1); }
    mbar_init(accum_full, 1);
    mbar_init(accum_empty, PF_DECODE_WARPS);
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
  const int row_tiles = static_cast<int>((N_out + PF_ROWS - 1) / PF_ROWS);
  const int items = p.groups_of_routes.count[0] * row_tiles;
  const Projection mats[2] = {p.a, p.b};
  const uint32_t abs_lane = smem_addr(tables) + (lane & 15) * 8, sign_lane = abs_lane + 256 * 16 * 8;
  volatile int* aborted = &abort_flag;

  uint32_t iter = 0;  // K blocks handled so far by this CTA: picks the stage and its phase
  int n_item = 0;
  for (int item = blockIdx.x; item < items && !*aborted; item += gridDim.x, ++n_item) {
    const int gi = item / row_tiles, tile = item - gi * row_tiles;
    const int64_t slot = p.groups_of_routes.slot[gi];
    const int gsize = p.groups_of_routes.size[gi], gstart = p.groups_of_routes.start[gi];
    const int n_pad = (gsize + 15) & ~15;  // the N of the MMA
    const int64_t row0 = static_cast<int64_t>(tile) * PF_ROWS;

    if (warp < PF_DECODE_WARPS) {
      // ================= decode producers, then epilogue ======================================
      const int row = tid >> 1, half = tid & 1;  // half a row of the K block: 8 codewords
      const int64_t grow = min(row0 + row, N_out - 1);
      const uint16_t* src[M];
#pragma unroll
      for (int m = 0; m < M; ++m) src[m] = mats[m].codes + (slot * N_out + grow) * cw + half * 8;
      uint4 next[M];
#pragma unroll
      for (int m = 0; m < M; ++m) next[m] = ld_stream_u4(src[m]);
      uint32_t it = iter;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        uint4 cur[M];
#pragma unroll
        for (int m = 0; m < M; ++m) cur[m] = next[m];
        if (kb + 1 < k_blocks) {
#pragma unroll
          for (int m = 0; m < M; ++m) next[m] = ld_stream_u4(src[m] + (kb + 1) * PF_KBLOCK_CODES);
        }
        const uint32_t stage = it % PF_STAGES, phase = (it / PF_STAGES) & 1u;
        if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, aborted)) break;
        const uint32_t stage_base = smem_base + stage * STAGE_BYTES;
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint32_t words[4] = {cur[m].x, cur[m].y, cur[m].z, cur[m].w};
#pragma unroll
          for (int pair = 0; pair < 4; ++pair) {  // two codewords = one 16-byte chunk of the row
            const uint32_t w = words[pair];
            uint32_t e0x, e0y, s0x, s0y, e1x, e1y, s1x, s1y;
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(e0x), "=r"(e0y) : "r"(abs_lane + ((w >> 1) & 0x7F80u)));
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(s0x), "=r"(s0y) : "r"(sign_lane + ((w << 7) & 0x7F80u)));
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(e1x), "=r"(e1y) : "r"(abs_lane + ((w >> 17) & 0x7F80u)));
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(s1x), "=r"(s1y) : "r"(sign_lane + ((w >> 9) & 0x7F80u)));
            const uint32_t dst = stage_base + m * PF_TILE_BYTES + swizzled(row, half * 4 + pair);
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(e0x ^ s0x), "r"(e0y ^ s0y), "r"(e1x ^ s1x), "r"(e1y ^ s1y) : "memory");
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * stage);
      }
      // ---- epilogue: accumulators -> y -> (SwiGLU) -> out -----------------------------------
      if (!*aborted && mbar_wait(accum_full, n_item & 1, aborted)) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quarter = warp & 3, col_half = warp >> 2;
        const int64_t erow = row0 + quarter * 32 + lane;
        float scale[M];
#pragma unroll
        for (int m = 0; m < M; ++m) scale[m] = load_as_float(mats[m].scales, p.scales_dtype, slot * N_out + min(erow, N_out - 1));
        for (int c0 = col_half * 16; c0 < n_pad; c0 += 32) {  // the two warpgroups interleave 16-column chunks
          uint32_t acc[M][2][16];
#pragma unroll
          for (int m = 0; m < M; ++m)
#pragma unroll
            for (int piece = 0; piece < 2; ++piece)
              tmem_ld16(tmem + (static_cast<uint32_t>(quarter * 32) << 16) + (m * 2 + piece) * PF_N_MAX + c0, acc[m][piece]);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int col = c0 + j;
            if (col >= gsize || erow >= N_out) continue;
            const int route = p.groups_of_routes.routes[gstart + col];
            const int64_t xrow = route / p.x_div;
            const float xs = p.x.scale[xrow], xsum = static_cast<float>(p.x.sums[xrow]);
            float y[M];
#pragma unroll
            for (int m = 0; m < M; ++m) {
              const float dot = 256.0f * static_cast<float>(static_cast<int>(acc[m][0][j])) + static_cast<float>(static_cast<int>(acc[m][1][j]));
              y[m] = scale[m] * xs * (0.5f * dot + 0.25f * xsum);
            }
            float result;
            if (M == 2) {
              float gt = y[0], up = y[M - 1];
              if (p.out_dtype == KEEPVQ_BF16) { gt = __bfloat162float(__float2bfloat16_rn(gt)); up = __bfloat162float(__float2bfloat16_rn(up)); }
              else if (p.out_dtype == KEEPVQ_F16) { gt = __half2float(__float2half_rn(gt)); up = __half2float(__float2half_rn(up)); }
              if (p.swiglu_limit > 0.0f) { gt = fminf(gt, p.swiglu_limit); up = fminf(fmaxf(up, -p.swiglu_limit), p.swiglu_limit); }
              result = gt / (1.0f + expf(-gt)) * up * p.route_weight[route];
            } else {
              result = y[0];
            }
            store_from_float(p.out, p.out_dtype, static_cast<int64_t>(route) * N_out + erow, result);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(accum_empty);
      }
    } else if (warp == PF_DECODE_WARPS) {
      // ================= MMA issuer ============================================================
      if (lane == 0) {
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n_pad >> 3) << 17) | ((PF_ROWS >> 4) << 24);
        bool ok = mbar_wait(accum_empty, (n_item & 1) ^ 1u, aborted);  // the epilogue has drained the accumulators
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        uint32_t it = iter;
        for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
          const uint32_t stage = it % PF_STAGES, phase = (it / PF_STAGES) & 1u;
          ok = mbar_wait(full0 + 8 * stage, phase, aborted);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t stage_base = smem_base + stage * STAGE_BYTES;
#pragma unroll
          for (int m = 0; m < M; ++m) {
            const uint64_t a_desc = umma_desc(stage_base + m * PF_TILE_BYTES);
#pragma unroll
            for (int piece = 0; piece < 2; ++piece) {
              const uint64_t b_desc = umma_desc(stage_base + (M + piece) * PF_TILE_BYTES);
#pragma unroll
              for (int k = 0; k < 4; ++k)  // 32 bytes of K per instruction: advance both start addresses by 2 x 16 B
                umma_i8(tmem + (m * 2 + piece) * PF_N_MAX, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
            }
          }
          umma_commit(empty0 + 8 * stage);  // the stage may be refilled once these MMAs have read it
        }
        if (ok) umma_commit(accum_full);
      }
    } else {
      // ================= activation (B operand) loaders =======================================
      // cp.async straight into the swizzled tiles (16 bytes = two codewords of one route), one
      // K block in flight behind the one being handed to the MMA warp.
      const int loader = tid - (PF_DECODE_WARPS + 1) * 32;  // 0..95
      for (int n = loader; n < n_pad; n += PF_B_WARPS * 32) {
        const int route = n < gsize ? p.groups_of_routes.routes[gstart + n] : -1;
        xrow_of[n] = route < 0 ? static_cast<int>(p.x_zero_row) : route / p.x_div;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(PF_B_WARPS * 32) : "memory");  // the loader warps only
      const uint8_t* plane[2] = {p.x.q, p.x.q + (p.x_zero_row + 1) * cw * 8};
      const int64_t row_bytes = cw * 8;
      uint32_t it = iter;
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
        const uint32_t stage = it % PF_STAGES, phase = (it / PF_STAGES) & 1u;
        ok = mbar_wait(empty0 + 8 * stage, phase ^ 1u, aborted);
        if (!ok) break;
        const uint32_t b_tiles = smem_base + stage * STAGE_BYTES + M * PF_TILE_BYTES;
        for (int e = loader; e < n_pad * 16; e += PF_B_WARPS * 32) {  // e = (route n, 16-byte chunk c, plane)
          const int n = e >> 4, c = (e >> 1) & 7, pl = e & 1;
          cp_async16_pf(b_tiles + pl * PF_TILE_BYTES + swizzled(n, c), plane[pl] + xrow_of[n] * row_bytes + static_cast<int64_t>(kb) * 128 + c * 16);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (kb > 0) {  // the previous K block's copies have landed: publish it
          asm volatile("cp.async.wait_group 1;" ::: "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(full0 + 8 * ((it - 1) % PF_STAGES));
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      if (ok) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full0 + 8 * ((it - 1) % PF_STAGES));
      }
      asm volatile("bar.sync 1, %0;" ::"n"(PF_B_WARPS * 32) : "memory");  // xrow_of is rewritten for the next item
    }
    iter += k_blocks;
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

template <int M>
static int launch_prefill(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) {
  constexpr size_t smem = PF_STAGES * (M + 2) * PF_TILE_BYTES + PF_TABLE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_projection_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  prefill_projection_kernel<M><<<sms, PF_THREADS, smem, s>>>(p, status);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}

int prefill_gate_up(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) { return launch_prefill<2>(p, status, s); }
int prefill_down(const FastProjectionArgs& p, int32_t* status, cudaStream_t s) { return launch_prefill<1>(p, status, s); }

}  // namespace fast
}  // namespace keepvq
