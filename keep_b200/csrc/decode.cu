// keepvq_decode_weights: codes (+ scales) -> dense weights, one thread per codeword.
//
// This is the code-to-weight map on its own, the part of the path that has to agree with the
// reference bit for bit (src/keep/vq/e8.py:542-571).  A grid value has 4 significant bits and an
// fp16 scale 11, so the fp32 product is exact and an fp32 output equals the reference's.
// HBM-bound: 2 (or 1) bytes in, 32 bytes out per thread at fp32; stores are two 16-byte
// writes per thread, coalesced across a warp.
#include "common.cuh"

namespace keepvq {

template <int CODE_BITS>
__global__ void __launch_bounds__(256) decode_weights_kernel(keepvq_decode_args a) {
  __shared__ uint32_t table[256];
  table[threadIdx.x] = a.codebook[threadIdx.x];
  __syncthreads();

  const int64_t total = a.rows * a.codewords;
  const int64_t per_group = a.codewords / a.groups;
  for (int64_t i = blockIdx.x * 256ll + threadIdx.x; i < total; i += 256ll * gridDim.x) {
    const int64_t row = i / a.codewords, cw = i - row * a.codewords;
    float scale = 1.0f;
    if (a.scales) scale = load_as_float(a.scales, a.scales_dtype, row * a.groups + cw / per_group);
    float v[8];
    if (CODE_BITS == 16) {
      const uint32_t code = reinterpret_cast<const uint16_t*>(a.codes)[i];
      const uint32_t word = table[code >> 8];
#pragma unroll
      for (int d = 0; d < 8; ++d) v[d] = e8p_value(code, word, d) * scale;
    } else {
      const uint32_t word = table[reinterpret_cast<const uint8_t*>(a.codes)[i]];
#pragma unroll
      for (int d = 0; d < 8; ++d) v[d] = e8_1bit_value(word, d) * scale;
    }
    if (a.out_dtype == KEEPVQ_F32) {
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + i * 8);
      o[0] = make_float4(v[0], v[1], v[2], v[3]);
      o[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int d = 0; d < 8; ++d) store_from_float(a.out, a.out_dtype, i * 8 + d, v[d]);
    }
  }
}

}  // namespace keepvq

extern "C" int keepvq_decode_weights(const keepvq_decode_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_decode_args& a = *args;
  if (a.code_bits != 8 && a.code_bits != 16) return KEEPVQ_ERR_DTYPE;
  if (!valid_dtype(a.out_dtype) || (a.scales && !valid_dtype(a.scales_dtype))) return KEEPVQ_ERR_DTYPE;
  if (a.rows < 0 || a.codewords < 0 || a.groups <= 0) return KEEPVQ_ERR_SHAPE;
  if (a.codewords % a.groups != 0) return KEEPVQ_ERR_SHAPE;
  if (a.rows == 0 || a.codewords == 0) return KEEPVQ_OK;  // nothing to do; empty tensors carry no pointer
  if (!a.codes || !a.codebook || !a.out) return KEEPVQ_ERR_NULL;
  if (!aligned_to(a.out, 16)) return KEEPVQ_ERR_ALIGN;
  const int64_t total = a.rows * a.codewords;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;  // grid-stride beyond that: 32 blocks per SM
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.code_bits == 16) decode_weights_kernel<16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(a);
  else decode_weights_kernel<8><<<static_cast<unsigned>(blocks), 256, 0, s>>>(a);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}
