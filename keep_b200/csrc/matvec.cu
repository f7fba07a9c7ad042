// keepvq_routed_matvec: the general few-row routed kernel (any dtype, any group size, 8- or
// 16-bit codes, optional nested residual).
//
// It serves the operator surface (vq_qmv, vq_qmm, gather_vqmm direct, e8p_m1_*, e8_1bit_m1_*,
// e8p_nested_m1_*).  The fused layer kernels in moe_decode.cu are the ones tuned for the HBM
// roofline; this one favours generality and mirrors the arithmetic of the reference's few-token
// kernels (src/ramp/kernels/e8p_m1.metal:48-103, e8_1bit_m1.metal, e8p_nested_m1.metal:60-127):
//   - a block column per route; a warp owns ROWS output rows; a lane takes CHUNK consecutive
//     codewords per step (one 16/8/4/2-byte load per row), its activations loaded once and
//     reused for every row;
//   - the table is expanded once per block into fp16 pairs in shared memory; a 16-bit codeword
//     costs one 16-byte shared read plus a sign XOR per pair, and its +-1/4 shift is applied as
//     +-1/4 * sum(x) outside the pair loop;
//   - fp32 accumulation per row, `part * scale` added per chunk, warp-shuffle reduction, one
//     rounding at the store.  Base and residual accumulate apart, so an fp32 nested output is
//     the fp32 sum of the two separate kernels bit for bit.
#include "common.cuh"

namespace keepvq {

constexpr int MV_WARPS = 4;
constexpr int MV_ROWS = 4;  // rows per warp

template <int CHUNK, int CODE_BITS>
__device__ __forceinline__ void load_code_chunk(const void* codes, int64_t first, uint32_t (&w)[4]) {
  // `first` = index of the chunk's first codeword within the whole codes array.
  if (CODE_BITS == 16) {
    const uint16_t* p = reinterpret_cast<const uint16_t*>(codes) + first;
    if (CHUNK == 8) { uint4 v = ld_stream_u4(p); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
    else if (CHUNK == 4) { uint2 v = ld_stream_u2(p); w[0] = v.x; w[1] = v.y; }
    else w[0] = *p;
  } else {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(codes) + first;
    if (CHUNK == 8) { uint2 v = ld_stream_u2(p); w[0] = v.x; w[1] = v.y; }
    else if (CHUNK == 4) w[0] = ld_stream_u1(p);
    else w[0] = *p;
  }
}

template <int CODE_BITS>
__device__ __forceinline__ uint32_t code_at(const uint32_t (&w)[4], int i) {
  if (CODE_BITS == 16) return (w[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu;
  return (w[i >> 2] >> ((i & 3) * 8)) & 0xFFu;
}

__device__ __forceinline__ float dot_pairs(const uint4& e, const float (&x)[8], float part) {
  const uint32_t pr[4] = {e.x, e.y, e.z, e.w};
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pr[k]));
    part = fmaf(f.x, x[2 * k], part);
    part = fmaf(f.y, x[2 * k + 1], part);
  }
  return part;
}

template <typename XT, int CHUNK, int CODE_BITS, bool NESTED>
__global__ void __launch_bounds__(MV_WARPS * 32) routed_matvec_kernel(keepvq_matvec_args a) {
  __shared__ uint4 lut[256];
  __shared__ uint4 res_lut[NESTED ? 256 : 1];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t route = blockIdx.x;
  const uint32_t slot = a.rhs[route];
  const int64_t N = a.out_dim, cw = a.in_dim / 8;
  const int64_t row0 = (static_cast<int64_t>(blockIdx.y) * MV_WARPS + warp) * MV_ROWS;

  if (slot == KEEPVQ_NO_RESIDUAL) {  // a route that is switched off writes zeros; uniform over the block
    if (lane == 0)
      for (int r = 0; r < MV_ROWS && row0 + r < N; ++r) store_from_float(a.out, a.out_dtype, route * N + row0 + r, 0.0f);
    return;
  }

  for (int idx = threadIdx.x; idx < 256; idx += MV_WARPS * 32) {
    if (CODE_BITS == 8 && a.codebook_layout == KEEPVQ_TABLE_HALF2_PAIRS) {
      lut[idx] = reinterpret_cast<const uint4*>(a.codebook)[idx];
    } else {
      uint32_t word = a.codebook[idx];
      if (CODE_BITS == 8 && a.codebook_layout == KEEPVQ_TABLE_PACKED) word = to_pair_packed(word);
      lut[idx] = expand_pair_packed(word);
    }
    if (NESTED) res_lut[idx] = reinterpret_cast<const uint4*>(a.res_table)[idx];
  }
  __syncthreads();

  uint32_t hot = KEEPVQ_NO_RESIDUAL;
  if (NESTED) hot = a.hot_of_slot[slot];
  const bool nested = NESTED && hot != KEEPVQ_NO_RESIDUAL;

  const int64_t xrow = a.lhs ? static_cast<int64_t>(a.lhs[route]) : route / a.x_div;
  const XT* x = reinterpret_cast<const XT*>(a.x) + xrow * a.in_dim;
  const int64_t per_group = cw / a.groups;
  const int64_t res_per_group = NESTED ? cw / a.res_groups : 1;

  float acc[MV_ROWS], res_acc[MV_ROWS];
#pragma unroll
  for (int r = 0; r < MV_ROWS; ++r) acc[r] = res_acc[r] = 0.0f;

  for (int64_t cw0 = static_cast<int64_t>(lane) * CHUNK; cw0 < cw; cw0 += 32 * CHUNK) {
    float xv[CHUNK][8], xs[CHUNK];
#pragma unroll
    for (int i = 0; i < CHUNK; ++i) {
      load8_as_float<XT>(x + (cw0 + i) * 8, xv[i]);
      float s = 0.0f;
#pragma unroll
      for (int d = 0; d < 8; ++d) s += xv[i][d];
      xs[i] = s;
    }
    const int64_t group = cw0 / per_group, res_group = cw0 / res_per_group;
#pragma unroll
    for (int r = 0; r < MV_ROWS; ++r) {
      const int64_t row = row0 + r;
      if (row >= N) break;
      const int64_t base = static_cast<int64_t>(slot) * N + row;
      uint32_t w[4];
      load_code_chunk<CHUNK, CODE_BITS>(a.codes, base * cw + cw0, w);
      float part = 0.0f;
#pragma unroll
      for (int i = 0; i < CHUNK; ++i) {
        const uint32_t code = code_at<CODE_BITS>(w, i);
        if (CODE_BITS == 16) {
          const uint32_t signs = code & 0xFFu;
          const uint32_t parity = __popc(signs) & 1u;
          const uint32_t eff = signs ^ parity;
          uint4 e = lut[code >> 8];
          // sign bits k and k+4 belong to pair k: move them to bits 15 and 31.
          const uint32_t spread = (eff & 0x0Fu) | ((eff & 0xF0u) << 12);
          e.x ^= (spread << 15) & 0x80008000u;
          e.y ^= (spread << 14) & 0x80008000u;
          e.z ^= (spread << 13) & 0x80008000u;
          e.w ^= (spread << 12) & 0x80008000u;
          part = dot_pairs(e, xv[i], part);
          part = fmaf(parity ? -0.25f : 0.25f, xs[i], part);
        } else {
          part = dot_pairs(lut[code], xv[i], part);
        }
      }
      acc[r] = fmaf(part, load_as_float(a.scales, a.scales_dtype, base * a.groups + group), acc[r]);
      if (nested) {
        const int64_t rbase = static_cast<int64_t>(hot) * N + row;
        uint32_t rw[4];
        load_code_chunk<CHUNK, 8>(a.res_codes, rbase * cw + cw0, rw);
        float rpart = 0.0f;
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) rpart = dot_pairs(res_lut[code_at<8>(rw, i)], xv[i], rpart);
        res_acc[r] = fmaf(rpart, load_as_float(a.res_scales, a.res_scales_dtype, rbase * a.res_groups + res_group), res_acc[r]);
      }
    }
  }

#pragma unroll
  for (int r = 0; r < MV_ROWS; ++r) {
    float total = acc[r], rtotal = res_acc[r];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      total += __shfl_xor_sync(0xFFFFFFFFu, total, o);
      if (NESTED) rtotal += __shfl_xor_sync(0xFFFFFFFFu, rtotal, o);
    }
    if (nested) total += rtotal;
    const int64_t row = row0 + r;
    if (lane == 0 && row < N) store_from_float(a.out, a.out_dtype, route * N + row, total);
  }
}

template <typename XT, int CHUNK>
static void launch_matvec(const keepvq_matvec_args& a, dim3 grid, cudaStream_t s) {
  const dim3 block(MV_WARPS * 32);
  if (a.res_codes) routed_matvec_kernel<XT, CHUNK, 16, true><<<grid, block, 0, s>>>(a);
  else if (a.code_bits == 16) routed_matvec_kernel<XT, CHUNK, 16, false><<<grid, block, 0, s>>>(a);
  else routed_matvec_kernel<XT, CHUNK, 8, false><<<grid, block, 0, s>>>(a);
}

template <typename XT>
static void launch_matvec_chunk(const keepvq_matvec_args& a, int chunk, dim3 grid, cudaStream_t s) {
  if (chunk == 8) launch_matvec<XT, 8>(a, grid, s);
  else if (chunk == 4) launch_matvec<XT, 4>(a, grid, s);
  else launch_matvec<XT, 1>(a, grid, s);
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
  int64_t per_group = cw / a.groups;
  if (a.res_codes) {
    if (a.code_bits != 16) return KEEPVQ_ERR_UNSUPPORTED;
    if (!a.res_scales || !a.res_table || !a.hot_of_slot) return KEEPVQ_ERR_NULL;
    if (!valid_dtype(a.res_scales_dtype)) return KEEPVQ_ERR_DTYPE;
    if (a.res_groups <= 0 || cw % a.res_groups != 0 || a.res_rows <= 0) return KEEPVQ_ERR_SHAPE;
    if (!aligned_to(a.res_table, 16)) return KEEPVQ_ERR_ALIGN;
  }
  if (a.routes == 0) return KEEPVQ_OK;
  if (!aligned_to(a.x, 16)) return KEEPVQ_ERR_ALIGN;
  if (a.x_dtype == KEEPVQ_F32 ? false : (a.in_dim * 2) % 16 != 0) return KEEPVQ_ERR_ALIGN;
  if (a.code_bits == 8 && a.codebook_layout == KEEPVQ_TABLE_HALF2_PAIRS && !aligned_to(a.codebook, 16)) return KEEPVQ_ERR_ALIGN;

  // Codewords per wide load: a chunk may not straddle a row or a scale group
  // (src/ramp/kernels/e8p_m1.py:98-104), and its address must be aligned to its width.
  int chunk = 1;
  const int64_t res_per_group = a.res_codes ? cw / a.res_groups : per_group;
  const int code_bytes = a.code_bits / 8;
  for (int c : {8, 4}) {
    if (per_group % c || res_per_group % c) continue;
    if (!aligned_to(a.codes, static_cast<size_t>(c) * code_bytes)) continue;
    if (a.res_codes && !aligned_to(a.res_codes, static_cast<size_t>(c))) continue;
    chunk = c;
    break;
  }

  const int64_t row_tiles = (a.out_dim + MV_WARPS * MV_ROWS - 1) / (MV_WARPS * MV_ROWS);
  if (row_tiles > 65535 || a.routes > 0x7FFFFFFFll) return KEEPVQ_ERR_CAPACITY;
  dim3 grid(static_cast<unsigned>(a.routes), static_cast<unsigned>(row_tiles));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.x_dtype == KEEPVQ_F32) launch_matvec_chunk<float>(a, chunk, grid, s);
  else if (a.x_dtype == KEEPVQ_F16) launch_matvec_chunk<__half>(a, chunk, grid, s);
  else launch_matvec_chunk<__nv_bfloat16>(a, chunk, grid, s);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}
