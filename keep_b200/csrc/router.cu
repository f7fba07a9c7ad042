// Router for routed residency: logits, score function, and the dual top-k in one launch pair.
//
// What it stands in for (reference, jackmaxwil/keep):
//   - Gate.forward                 tests/fixtures/v41_reference/model.py:811-829
//   - gate_masked                  scripts/runpod/v41_reap/local_eval.py:69-90
//   - the fused served/demand top-k  scripts/v41_build/omlx_lattice.py:77-104,333-338
//   - the admission test (gate >= tau on renormalised demand weights)
//                                   scripts/v41_build/omlx_routed.py:184-203
//
// keepvq_router_logits: logits[t, e] = (x[t] . W[e]) / gate_temp, fp32.  A block owns 4 router
//   rows and a tile of 8 tokens, its warps split the hidden dimension.  Products of bf16 values
//   are exact in fp32; the order of additions is fixed (lane-sequential, a butterfly over lanes,
//   then over warps), so results are reproducible.
//   From 256 tokens on a tiled kernel takes over: bf16 x bf16 on the tensor cores (exact products,
//   fp32 accumulation in a fixed order), other dtypes as one fp32 FMA chain per logit, k ascending.
// keepvq_routed_topk: one warp per token (pool in registers up to 1024 experts, in shared memory
//   beyond).  Scores = f(logits); served = top-k of
//   scores + served_bias (absent experts carry -inf or anything <= -1e29); demand = top-k of
//   scores + pool_bias; ties go to the lowest expert id; picks come out in descending biased
//   score, the order torch.topk gives.  The bias selects only; weights come from raw scores.
#include <math.h>

#include "common.cuh"
#include "router_logits.cuh"

namespace keepvq {

template <typename XT, typename WT>
__global__ void __launch_bounds__(RL_WARPS * 32) router_logits_kernel(keepvq_router_logits_args a) {
  grid_launch_dependents();
  grid_wait();
  router_logits_block<XT, WT>(a, blockIdx.x, blockIdx.y);
}

// Many tokens: a 64 x 64 tile of logits per block, K staged through shared memory 32 at a time,
// 4 x 4 outputs per thread.  Each output is one chain of fp32 FMAs over k ascending, so it is
// reproducible and independent of the tiling.
constexpr int RT_TILE = 64, RT_K = 32, RT_THREADS = 256, RT_LD = RT_TILE + 4;
constexpr int RT_MIN_TOKENS = 256;  // below this the tile grid is too small to fill the GPU

template <typename XT, typename WT>
__global__ void __launch_bounds__(RT_THREADS) router_logits_tiled_kernel(keepvq_router_logits_args a) {
  grid_launch_dependents();
  grid_wait();
  __shared__ __align__(16) float xs[RT_K][RT_LD], ws[RT_K][RT_LD];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int64_t t0 = static_cast<int64_t>(blockIdx.y) * RT_TILE, e0 = static_cast<int64_t>(blockIdx.x) * RT_TILE;
  const XT* x = reinterpret_cast<const XT*>(a.x);
  const WT* w = reinterpret_cast<const WT*>(a.router_w);
  const int lrow = tid >> 2, lk = (tid & 3) * 8;  // staging: 64 rows x 4 pieces of 8 values
  const int64_t xt = min(t0 + lrow, a.tokens - 1), we = min(e0 + lrow, a.pool - 1);
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
  for (int64_t k0 = 0; k0 < a.hidden; k0 += RT_K) {
    float xv[8], wv[8];
    if (k0 + lk < a.hidden) {
      load8_as_float<XT>(x + xt * a.hidden + k0 + lk, xv);
      load8_as_float<WT>(w + we * a.hidden + k0 + lk, wv);
    } else {
#pragma unroll
      for (int d = 0; d < 8; ++d) xv[d] = wv[d] = 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int d = 0; d < 8; ++d) { xs[lk + d][lrow] = xv[d]; ws[lk + d][lrow] = wv[d]; }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < RT_K; ++k) {
      const float4 xa = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 wb = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float xr[4] = {xa.x, xa.y, xa.z, xa.w}, wr[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xr[i], wr[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t t = t0 + ty * 4 + i, e = e0 + tx * 4 + j;
      if (t < a.tokens && e < a.pool) a.logits[t * a.pool + e] = acc[i][j] / a.gate_temp;
    }
}

// Many bf16 tokens against a bf16 router: the same tile on the tensor cores (mma.sync m16n8k16:
// bf16 products are exact, sixteen of them are summed per instruction, the partial sums are added
// in fp32 with k ascending).  64 tokens x 64 experts per block of four warps, K staged 32 at a time through a
// three-stage cp.async ring; rows padded to 80 bytes so that every fragment load is conflict-free.
constexpr int RM_TILE = 64, RM_K = 32, RM_LD = 40, RM_STAGES = 3, RM_THREADS = 128;

__global__ void __launch_bounds__(RM_THREADS) router_logits_mma_kernel(keepvq_router_logits_args a) {
  __shared__ __align__(16) __nv_bfloat16 xs[RM_STAGES][RM_TILE][RM_LD], ws[RM_STAGES][RM_TILE][RM_LD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int wm = (warp & 1) * 32, wn = (warp >> 1) * 32;  // this warp's 32 x 32 corner of the tile
  const int64_t t0 = static_cast<int64_t>(blockIdx.y) * RM_TILE, e0 = static_cast<int64_t>(blockIdx.x) * RM_TILE;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(a.router_w);
  // staging: 64 rows x 4 pieces of 16 bytes per operand, two pieces per thread
  const int row_a = tid >> 2, piece = tid & 3, row_b = row_a + 32;
  const __nv_bfloat16* xsrc[2] = {x + min(t0 + row_a, a.tokens - 1) * a.hidden + piece * 8, x + min(t0 + row_b, a.tokens - 1) * a.hidden + piece * 8};
  const __nv_bfloat16* wsrc[2] = {w + min(e0 + row_a, a.pool - 1) * a.hidden + piece * 8, w + min(e0 + row_b, a.pool - 1) * a.hidden + piece * 8};
  auto stage_in = [&](int kb) {
    const int st = kb % RM_STAGES;
    if (kb * RM_K < a.hidden) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = h ? row_b : row_a;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&xs[st][row][piece * 8]))), "l"(xsrc[h] + kb * RM_K) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&ws[st][row][piece * 8]))), "l"(wsrc[h] + kb * RM_K) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;
  const int k_blocks = static_cast<int>(a.hidden / RM_K);
  stage_in(0);
  stage_in(1);
  for (int kb = 0; kb < k_blocks; ++kb) {
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // block kb has landed
    __syncthreads();                                          // ... for everyone, and block kb - 1 is no longer being read
    stage_in(kb + 2);
    const int st = kb % RM_STAGES;
#pragma unroll
    for (int ks = 0; ks < RM_K; ks += 16) {
      uint32_t af[2][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + 16 * i + g;
        af[i][0] = *reinterpret_cast<const uint32_t*>(&xs[st][r][ks + 2 * t]);
        af[i][1] = *reinterpret_cast<const uint32_t*>(&xs[st][r + 8][ks + 2 * t]);
        af[i][2] = *reinterpret_cast<const uint32_t*>(&xs[st][r][ks + 2 * t + 8]);
        af[i][3] = *reinterpret_cast<const uint32_t*>(&xs[st][r + 8][ks + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn + 8 * j + g;
        bf[j][0] = *reinterpret_cast<const uint32_t*>(&ws[st][n][ks + 2 * t]);
        bf[j][1] = *reinterpret_cast<const uint32_t*>(&ws[st][n][ks + 2 * t + 8]);
      }
      // Each MMA sums its sixteen exact products from zero; the running sums are kept by ordinary
      // fp32 additions (round to nearest).  Accumulating inside the tensor core over the whole K
      // truncates at every step and measured 4e-5 relative on softmax scores, too close to the
      // gaps that decide a top-k cut.
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float d0, d1, d2, d3;
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                       : "=f"(d0), "=f"(d1), "=f"(d2), "=f"(d3)
                       : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(bf[j][0]), "r"(bf[j][1]), "f"(0.0f));
          acc[i][j][0] += d0; acc[i][j][1] += d1; acc[i][j][2] += d2; acc[i][j][3] += d3;
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int64_t tok = t0 + wm + 16 * i + g + (r >= 2 ? 8 : 0), e = e0 + wn + 8 * j + 2 * t + (r & 1);
        if (tok < a.tokens && e < a.pool) a.logits[tok * a.pool + e] = acc[i][j][r] / a.gate_temp;
      }
}

// 16 to 255 bf16 tokens against a bf16 router: the same 64 x 64 tile and the same arithmetic, with the
// hidden dimension split over a cluster of eight blocks so that a call of 64 tokens is 48 blocks
// instead of 6.  Each block sums its eighth of K as above; the eight partial tiles meet through
// distributed shared memory, every block adding up eight rows of the tile over the ranks in rank
// order, so a logit is a fixed sequence of additions whatever the batch around it.
constexpr int RC_SPLIT = 8;
constexpr int RC_MIN_TOKENS = 24;  // below this the K-split kernel of the fp32 pipes is as fast, and shares its launch with the quantisation of the rows

__global__ void __cluster_dims__(RC_SPLIT, 1, 1) __launch_bounds__(RM_THREADS) router_logits_cluster_kernel(keepvq_router_logits_args a) {
  grid_launch_dependents();
  grid_wait();
  __shared__ __align__(16) __nv_bfloat16 xs[RM_STAGES][RM_TILE][RM_LD], ws[RM_STAGES][RM_TILE][RM_LD];
  __shared__ __align__(16) float red[RM_TILE][RM_TILE];  // this block's partial tile [token][expert]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int wm = (warp & 1) * 32, wn = (warp >> 1) * 32;
  const int rank = static_cast<int>(blockIdx.x);  // the cluster spans x: the block's share of K
  const int64_t t0 = static_cast<int64_t>(blockIdx.z) * RM_TILE, e0 = static_cast<int64_t>(blockIdx.y) * RM_TILE;
  const int64_t k_share = a.hidden / RC_SPLIT, k_first = rank * k_share;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x) + k_first;
  const __nv_bfloat16* w = reinterpret_cast<const __nv_bfloat16*>(a.router_w) + k_first;
  const int row_a = tid >> 2, piece = tid & 3, row_b = row_a + 32;
  const __nv_bfloat16* xsrc[2] = {x + min(t0 + row_a, a.tokens - 1) * a.hidden + piece * 8, x + min(t0 + row_b, a.tokens - 1) * a.hidden + piece * 8};
  const __nv_bfloat16* wsrc[2] = {w + min(e0 + row_a, a.pool - 1) * a.hidden + piece * 8, w + min(e0 + row_b, a.pool - 1) * a.hidden + piece * 8};
  const int k_blocks = static_cast<int>(k_share / RM_K);
  auto stage_in = [&](int kb) {
    const int st = kb % RM_STAGES;
    if (kb < k_blocks) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = h ? row_b : row_a;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&xs[st][row][piece * 8]))), "l"(xsrc[h] + kb * RM_K) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(&ws[st][row][piece * 8]))), "l"(wsrc[h] + kb * RM_K) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;
  stage_in(0);
  stage_in(1);
  for (int kb = 0; kb < k_blocks; ++kb) {
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    stage_in(kb + 2);
    const int st = kb % RM_STAGES;
#pragma unroll
    for (int ks = 0; ks < RM_K; ks += 16) {
      uint32_t af[2][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + 16 * i + g;
        af[i][0] = *reinterpret_cast<const uint32_t*>(&xs[st][r][ks + 2 * t]);
        af[i][1] = *reinterpret_cast<const uint32_t*>(&xs[st][r + 8][ks + 2 * t]);
        af[i][2] = *reinterpret_cast<const uint32_t*>(&xs[st][r][ks + 2 * t + 8]);
        af[i][3] = *reinterpret_cast<const uint32_t*>(&xs[st][r + 8][ks + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn + 8 * j + g;
        bf[j][0] = *reinterpret_cast<const uint32_t*>(&ws[st][n][ks + 2 * t]);
        bf[j][1] = *reinterpret_cast<const uint32_t*>(&ws[st][n][ks + 2 * t + 8]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {  // sixteen exact products summed from zero per instruction; running sums in plain fp32 (see the kernel above)
          float d0, d1, d2, d3;
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                       : "=f"(d0), "=f"(d1), "=f"(d2), "=f"(d3)
                       : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(bf[j][0]), "r"(bf[j][1]), "f"(0.0f));
          acc[i][j][0] += d0; acc[i][j][1] += d1; acc[i][j][2] += d2; acc[i][j][3] += d3;
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) red[wm + 16 * i + g + (r >= 2 ? 8 : 0)][wn + 8 * j + 2 * t + (r & 1)] = acc[i][j][r];
  // every partial tile is in place (release / acquire at cluster scope)
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  // this block adds up tokens 8 * rank .. 8 * rank + 7 of the tile over the ranks in order: 512 logits, four per thread
  const uint32_t red_local = static_cast<uint32_t>(__cvta_generic_to_shared(&red[0][0]));
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const int idx = tid + v * RM_THREADS;               // 0..511
    const int row = rank * (RM_TILE / RC_SPLIT) + idx / RM_TILE, col = idx % RM_TILE;
    float sum = 0.0f;
#pragma unroll
    for (int q = 0; q < RC_SPLIT; ++q) {
      uint32_t remote;
      float part;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(red_local + static_cast<uint32_t>((row * RM_TILE + col) * 4)), "r"(q));
      asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part) : "r"(remote) : "memory");
      sum += part;
    }
    const int64_t tok = t0 + row, e = e0 + col;
    if (tok < a.tokens && e < a.pool) a.logits[tok * a.pool + e] = sum / a.gate_temp;
  }
  // nobody leaves while a peer may still be reading its tile
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// (value, index) max with ties to the lower index, across a warp.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    const int oi = __shfl_xor_sync(0xFFFFFFFFu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

constexpr int TK_WARPS = 4;
constexpr int TK_MAX_K = 16;

// Floats as unsigned keys of the same order (-inf lowest of the real values); 0 is below all of them.
__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One warp per token with the pool in registers (NPL experts per lane, expert e = lane + 32 i).
// A pick is a register scan, one warp max and one warp min (redux.sync); no shared memory and no
// loads inside the selection loops.  Same arithmetic and the same results as routed_topk_kernel.
template <int NPL>
__global__ void __launch_bounds__(TK_WARPS * 32) routed_topk_reg_kernel(keepvq_routed_topk_args a) {
  grid_launch_dependents();
  grid_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * TK_WARPS + warp;
  if (t >= a.tokens) return;
  const int P = static_cast<int>(a.pool), K = a.top_k;
  const float* lg = a.logits + t * P;
  float sc[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) { const int e = lane + 32 * i; sc[i] = e < P ? lg[e] : -INFINITY; }

  // ---- score function --------------------------------------------------------------------
  if (a.score_func == KEEPVQ_SCORE_SOFTMAX) {
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPL; ++i) m = fmaxf(m, sc[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < NPL; ++i)
      if (lane + 32 * i < P) { sc[i] = expf(sc[i] - m); s += sc[i]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
#pragma unroll
    for (int i = 0; i < NPL; ++i) sc[i] = sc[i] / s;
  } else if (a.score_func == KEEPVQ_SCORE_SIGMOID) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) sc[i] = 1.0f / (1.0f + expf(-sc[i]));
  } else {
#pragma unroll
    for (int i = 0; i < NPL; ++i) { const float v = sc[i]; sc[i] = sqrtf(v > 20.0f ? v : log1pf(expf(v))); }
  }
  if (a.scores) {
#pragma unroll
    for (int i = 0; i < NPL; ++i)
      if (lane + 32 * i < P) a.scores[t * P + lane + 32 * i] = sc[i];
  }

  // ---- two selections over the same scores -------------------------------------------------
  for (int pass = 0; pass < 2; ++pass) {
    const float* bias = pass == 0 ? a.served_bias : a.pool_bias;
    uint32_t key[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      key[i] = e < P ? max(ordered_key(sc[i] + (bias ? bias[e] : 0.0f)), 1u) : 0u;
    }
    int my_e = 0;       // lane j keeps pick j
    float my_raw = 0.0f;
    for (int j = 0; j < K; ++j) {
      uint32_t bu = 0u, bi = 0xFFFFFFFFu;
#pragma unroll
      for (int i = 0; i < NPL; ++i)
        if (key[i] > bu) { bu = key[i]; bi = lane + 32 * i; }
      const uint32_t top = __reduce_max_sync(0xFFFFFFFFu, bu);
      const uint32_t win = __reduce_min_sync(0xFFFFFFFFu, bu == top ? bi : 0xFFFFFFFFu);  // ties: the lowest expert id
      float raw = 0.0f;
#pragma unroll
      for (int i = 0; i < NPL; ++i)
        if (static_cast<uint32_t>(lane + 32 * i) == win) { raw = sc[i]; key[i] = 0u; }
      raw = __shfl_sync(0xFFFFFFFFu, raw, win & 31u);
      if (lane == j) { my_e = static_cast<int>(win); my_raw = raw; }
    }
    float raw = 0.0f;
    bool live = false;
    if (lane < K) {
      raw = my_raw;
      live = pass == 1 || !a.served_bias || a.served_bias[my_e] > ABSENT_BIAS;
      if (!live) raw = 0.0f;  // a masked pick carries no weight (local_eval.py:87)
    }
    float sum = raw;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane < K) {
      const int e = my_e;
      const int64_t o = t * K + lane;
      if (pass == 0) {
        float w = raw;
        if (a.norm_topk_prob && K > 1) w = w / (sum + 1e-20f);
        w *= a.route_scale;
        a.served_weight[o] = w;
        a.served_expert[o] = live ? static_cast<uint32_t>(e) : KEEPVQ_NO_RESIDUAL;
        a.served_slot[o] = live ? (a.slot_of ? a.slot_of[e] : static_cast<uint32_t>(e)) : KEEPVQ_NO_RESIDUAL;
      } else {
        a.want[o] = static_cast<uint32_t>(e);
        a.want_score[o] = raw;
        if (a.admit) {
          // the policy's own normalisation: always over the k demanded scores (omlx_routed.py:186)
          const float g = raw / (sum + 1e-20f) * a.route_scale;
          const bool absent = a.served_bias && a.served_bias[e] <= ABSENT_BIAS;
          a.admit[o] = (absent && g >= a.tau) ? e : -1;
        }
      }
    }
  }
}

__global__ void __launch_bounds__(TK_WARPS * 32) routed_topk_kernel(keepvq_routed_topk_args a) {
  grid_launch_dependents();
  grid_wait();
  extern __shared__ float smem[];  // per warp: scores[pool]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t t = static_cast<int64_t>(blockIdx.x) * TK_WARPS + warp;
  if (t >= a.tokens) return;
  const int P = static_cast<int>(a.pool), K = a.top_k;
  float* sc = smem + static_cast<size_t>(warp) * P;
  const float* lg = a.logits + t * P;

  // ---- score function --------------------------------------------------------------------
  if (a.score_func == KEEPVQ_SCORE_SOFTMAX) {
    float m = -INFINITY;
    for (int e = lane; e < P; e += 32) m = fmaxf(m, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    float s = 0.0f;
    for (int e = lane; e < P; e += 32) { const float v = expf(lg[e] - m); sc[e] = v; s += v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
    for (int e = lane; e < P; e += 32) sc[e] = sc[e] / s;
  } else if (a.score_func == KEEPVQ_SCORE_SIGMOID) {
    for (int e = lane; e < P; e += 32) sc[e] = 1.0f / (1.0f + expf(-lg[e]));
  } else {  // sqrt(softplus), softplus linear above 20 as torch computes it
    for (int e = lane; e < P; e += 32) { const float v = lg[e]; sc[e] = sqrtf(v > 20.0f ? v : log1pf(expf(v))); }
  }
  __syncwarp();
  if (a.scores)
    for (int e = lane; e < P; e += 32) a.scores[t * P + e] = sc[e];

  // ---- two selections over the same scores -------------------------------------------------
  int picked[TK_MAX_K];
  for (int pass = 0; pass < 2; ++pass) {
    const float* bias = pass == 0 ? a.served_bias : a.pool_bias;
    for (int j = 0; j < K; ++j) {
      float best = -INFINITY;
      int besti = 0x7FFFFFFF;
      for (int e = lane; e < P; e += 32) {
        bool used = false;
        for (int q = 0; q < j; ++q) used |= picked[q] == e;
        if (used) continue;
        const float key = sc[e] + (bias ? bias[e] : 0.0f);
        if (key > best || (key == best && e < besti) || besti == 0x7FFFFFFF) { best = key; besti = e; }
      }
      warp_argmax(best, besti);
      picked[j] = besti;
    }
    // every lane now holds the same picks; lane j finishes pick j
    float raw = 0.0f;
    bool live = false;
    if (lane < K) {
      const int e = picked[lane];
      raw = sc[e];
      live = pass == 1 || !a.served_bias || a.served_bias[e] > ABSENT_BIAS;
      if (!live) raw = 0.0f;  // a masked pick carries no weight (local_eval.py:87)
    }
    float sum = raw;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (lane < K) {
      const int e = picked[lane];
      const int64_t o = t * K + lane;
      if (pass == 0) {
        float w = raw;
        if (a.norm_topk_prob && K > 1) w = w / (sum + 1e-20f);
        w *= a.route_scale;
        a.served_weight[o] = w;
        a.served_expert[o] = live ? static_cast<uint32_t>(e) : KEEPVQ_NO_RESIDUAL;
        a.served_slot[o] = live ? (a.slot_of ? a.slot_of[e] : static_cast<uint32_t>(e)) : KEEPVQ_NO_RESIDUAL;
      } else {
        a.want[o] = static_cast<uint32_t>(e);
        a.want_score[o] = raw;
        if (a.admit) {
          // the policy's own normalisation: always over the k demanded scores (omlx_routed.py:186)
          const float g = raw / (sum + 1e-20f) * a.route_scale;
          const bool absent = a.served_bias && a.served_bias[e] <= ABSENT_BIAS;
          a.admit[o] = (absent && g >= a.tau) ? e : -1;
        }
      }
    }
  }
}

template <typename XT>
static void launch_logits_tiled(const keepvq_router_logits_args& a, dim3 grid, cudaStream_t s) {
  if (a.router_dtype == KEEPVQ_F32) launch_after(false, router_logits_tiled_kernel<XT, float>, grid, RT_THREADS, 0, s, a);
  else if (a.router_dtype == KEEPVQ_F16) launch_after(false, router_logits_tiled_kernel<XT, __half>, grid, RT_THREADS, 0, s, a);
  else launch_after(false, router_logits_tiled_kernel<XT, __nv_bfloat16>, grid, RT_THREADS, 0, s, a);
}

template <typename XT>
static void launch_logits(const keepvq_router_logits_args& a, dim3 grid, cudaStream_t s) {
  if (a.router_dtype == KEEPVQ_F32) launch_after(true, router_logits_kernel<XT, float>, grid, RL_WARPS * 32, 0, s, a);
  else if (a.router_dtype == KEEPVQ_F16) launch_after(true, router_logits_kernel<XT, __half>, grid, RL_WARPS * 32, 0, s, a);
  else launch_after(true, router_logits_kernel<XT, __nv_bfloat16>, grid, RL_WARPS * 32, 0, s, a);
}

}  // namespace keepvq

extern "C" int keepvq_router_logits(const keepvq_router_logits_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_router_logits_args& a = *args;
  if (!valid_dtype(a.x_dtype) || !valid_dtype(a.router_dtype)) return KEEPVQ_ERR_DTYPE;
  if (a.tokens < 0 || a.pool <= 0 || a.hidden <= 0 || a.hidden % 8 != 0) return KEEPVQ_ERR_SHAPE;
  if (!(a.gate_temp > 0.0f)) return KEEPVQ_ERR_SHAPE;
  if (a.tokens == 0) return KEEPVQ_OK;
  if (!a.x || !a.router_w || !a.logits) return KEEPVQ_ERR_NULL;
  if (!aligned_to(a.x, 16) || !aligned_to(a.router_w, 16)) return KEEPVQ_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.tokens >= RT_MIN_TOKENS) {  // many tokens: a tiled kernel, on the tensor cores when both operands are bf16
    const int64_t tiles = (a.tokens + RT_TILE - 1) / RT_TILE;
    if (tiles > 65535) return KEEPVQ_ERR_CAPACITY;
    if (a.x_dtype == KEEPVQ_BF16 && a.router_dtype == KEEPVQ_BF16 && a.hidden % RM_K == 0) {
      dim3 grid(static_cast<unsigned>((a.pool + RM_TILE - 1) / RM_TILE), static_cast<unsigned>(tiles));
      router_logits_mma_kernel<<<grid, RM_THREADS, 0, s>>>(a);
      KEEPVQ_CHECK_LAUNCH();
      return KEEPVQ_OK;
    }
    dim3 grid(static_cast<unsigned>((a.pool + RT_TILE - 1) / RT_TILE), static_cast<unsigned>(tiles));
    if (a.x_dtype == KEEPVQ_F32) launch_logits_tiled<float>(a, grid, s);
    else if (a.x_dtype == KEEPVQ_F16) launch_logits_tiled<__half>(a, grid, s);
    else launch_logits_tiled<__nv_bfloat16>(a, grid, s);
    KEEPVQ_CHECK_LAUNCH();
    return KEEPVQ_OK;
  }
  if (a.tokens >= RC_MIN_TOKENS && a.x_dtype == KEEPVQ_BF16 && a.router_dtype == KEEPVQ_BF16 && a.hidden % (RC_SPLIT * RM_K) == 0) {
    // a few dozen tokens: the tensor-core tile with the hidden dimension split over a cluster of eight blocks
    dim3 grid(RC_SPLIT, static_cast<unsigned>((a.pool + RM_TILE - 1) / RM_TILE), static_cast<unsigned>((a.tokens + RM_TILE - 1) / RM_TILE));
    if (grid.y > 65535) return KEEPVQ_ERR_CAPACITY;
    cudaError_t err = launch_after(true, router_logits_cluster_kernel, grid, RM_THREADS, 0, s, a);
    if (err != cudaSuccess) return note_cuda_error(err);
    return KEEPVQ_OK;
  }
  const int64_t token_tiles = (a.tokens + RL_TOKENS - 1) / RL_TOKENS;
  if (token_tiles > 65535) return KEEPVQ_ERR_CAPACITY;
  dim3 grid(static_cast<unsigned>((a.pool + RL_ROWS - 1) / RL_ROWS), static_cast<unsigned>(token_tiles));
  if (a.x_dtype == KEEPVQ_F32) launch_logits<float>(a, grid, s);
  else if (a.x_dtype == KEEPVQ_F16) launch_logits<__half>(a, grid, s);
  else launch_logits<__nv_bfloat16>(a, grid, s);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}

extern "C" int keepvq_routed_topk(const keepvq_routed_topk_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_routed_topk_args& a = *args;
  if (a.tokens < 0 || a.pool <= 0 || a.top_k <= 0 || a.top_k > TK_MAX_K || a.top_k > a.pool) return KEEPVQ_ERR_SHAPE;
  if (a.score_func < KEEPVQ_SCORE_SOFTMAX || a.score_func > KEEPVQ_SCORE_SQRT_SOFTPLUS) return KEEPVQ_ERR_DTYPE;
  if (a.tokens == 0) return KEEPVQ_OK;
  if (!a.logits || !a.served_slot || !a.served_expert || !a.served_weight || !a.want || !a.want_score) return KEEPVQ_ERR_NULL;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>((a.tokens + TK_WARPS - 1) / TK_WARPS);
  if (a.pool <= 1024) {  // the pool fits the registers of a warp
    if (a.pool <= 128) launch_after(blocks <= EARLY_LAUNCH_MAX_BLOCKS / 4, routed_topk_reg_kernel<4>, blocks, TK_WARPS * 32, 0, s, a);
    else if (a.pool <= 384) launch_after(blocks <= EARLY_LAUNCH_MAX_BLOCKS / 4, routed_topk_reg_kernel<12>, blocks, TK_WARPS * 32, 0, s, a);
    else launch_after(blocks <= EARLY_LAUNCH_MAX_BLOCKS / 4, routed_topk_reg_kernel<32>, blocks, TK_WARPS * 32, 0, s, a);
    KEEPVQ_CHECK_LAUNCH();
    return KEEPVQ_OK;
  }
  const size_t smem = static_cast<size_t>(TK_WARPS) * a.pool * sizeof(float);
  if (smem > 200 * 1024) return KEEPVQ_ERR_CAPACITY;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(routed_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
  }
  routed_topk_kernel<<<blocks, TK_WARPS * 32, smem, s>>>(a);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}
