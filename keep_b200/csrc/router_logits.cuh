// The few-token router logits block, shared by keepvq_router_logits (router.cu) and the layer
// call's front kernel, which runs it beside the activation quantisation (moe_fast.cu).
#pragma once

#include "common.cuh"

namespace keepvq {

constexpr int RL_WARPS = 8;    // warps per block; they split the hidden dimension
constexpr int RL_ROWS = 4;     // router rows per block
constexpr int RL_TOKENS = 8;   // tokens per block
constexpr float ABSENT_BIAS = -1e29f;  // served_bias at or below this marks an absent expert

// Few tokens: latency is what counts, so a block's 8 warps split the hidden dimension (every load
// of a lane is independent of the others) and a block covers 4 router rows x 8 tokens.  A logit is
// summed lane-sequentially, then by a butterfly over the lanes, then over the warps in order.
// Block (row_block, token_block) of the grid ceil(pool / RL_ROWS) x ceil(tokens / RL_TOKENS); RL_WARPS * 32 threads.
template <typename XT, typename WT>
__device__ __forceinline__ void router_logits_block(const keepvq_router_logits_args& a, int64_t row_block, int64_t token_block) {
  __shared__ float part[RL_WARPS][RL_ROWS * RL_TOKENS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t e0 = row_block * RL_ROWS, t0 = token_block * RL_TOKENS;
  const WT* w = reinterpret_cast<const WT*>(a.router_w);
  const XT* x = reinterpret_cast<const XT*>(a.x);
  float acc[RL_ROWS][RL_TOKENS];
#pragma unroll
  for (int r = 0; r < RL_ROWS; ++r)
#pragma unroll
    for (int i = 0; i < RL_TOKENS; ++i) acc[r][i] = 0.0f;
  const int64_t chunks = a.hidden / 8;
#pragma unroll 2
  for (int64_t c = warp * 32 + lane; c < chunks; c += RL_WARPS * 32) {
    float wv[RL_ROWS][8];
#pragma unroll
    for (int r = 0; r < RL_ROWS; ++r) load8_as_float<WT>(w + min(e0 + r, a.pool - 1) * a.hidden + c * 8, wv[r]);
#pragma unroll
    for (int i = 0; i < RL_TOKENS; ++i) {
      if (t0 + i < a.tokens) {
        float xv[8];
        load8_as_float<XT>(x + (t0 + i) * a.hidden + c * 8, xv);
#pragma unroll
        for (int r = 0; r < RL_ROWS; ++r)
#pragma unroll
          for (int d = 0; d < 8; ++d) acc[r][i] = fmaf(xv[d], wv[r][d], acc[r][i]);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < RL_ROWS; ++r)
#pragma unroll
    for (int i = 0; i < RL_TOKENS; ++i) {
      float v = acc[r][i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
      if (lane == 0) part[warp][r * RL_TOKENS + i] = v;
    }
  __syncthreads();
  if (threadIdx.x < RL_ROWS * RL_TOKENS) {
    float v = 0.0f;
#pragma unroll
    for (int q = 0; q < RL_WARPS; ++q) v += part[q][threadIdx.x];
    const int64_t e = e0 + threadIdx.x / RL_TOKENS, t = t0 + threadIdx.x % RL_TOKENS;
    if (e < a.pool && t < a.tokens) a.logits[t * a.pool + e] = v / a.gate_temp;
  }
}

}  // namespace keepvq
