/* TEST INFRASTRUCTURE: a plain C restatement of the reference's code-to-weight decode and of its
 * dense matvec, used only by tests, the smoke check and the benchmark's CPU baseline.  Never
 * shipped and never called by the product path.
 *
 * Follows, in the reference checkout:
 *   e8p_decode      keep.vq.e8.decode_e8p                     src/keep/vq/e8.py:210-234
 *   e8_1bit_decode  keep.vq.e8.decode_e8_1bit                 src/keep/vq/e8.py:165-200
 *   vq_qmv          ramp.kernels.vq_qmv.vq_qmv_reference_np   src/ramp/kernels/vq_qmv.py:126-160
 *                   (= decode_weight_matrix(codes, scales) @ x, src/keep/vq/e8.py:542-571)
 */
#include <stdint.h>

/* output dimension d of an E8P codeword reads nibble SHUFFLE[d] of its abs-table word */
static const int SHUFFLE[8] = {0, 4, 1, 5, 2, 6, 3, 7};

static inline void e8p_decode_one(uint16_t code, const uint32_t* abs_table, float* out) {
  const uint32_t signs = code & 0xFFu, word = abs_table[code >> 8];
  const uint32_t parity = (uint32_t)__builtin_popcount(signs) & 1u;
  const uint32_t eff = signs ^ parity;
  const float shift = parity ? -0.25f : 0.25f;
  for (int d = 0; d < 8; ++d) {
    const int p = SHUFFLE[d];
    float v = ((float)((word >> (4 * p)) & 0xFu) - 8.0f) * 0.5f;
    if ((eff >> p) & 1u) v = -v;
    out[d] = v + shift;
  }
}

void e8p_decode(const uint16_t* codes, int64_t n, const uint32_t* abs_table, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) e8p_decode_one(codes[i], abs_table, out + 8 * i);
}

/* 8-bit residual code: eight nibbles (2v + 8) in natural order, no shuffle, no parity */
void e8_1bit_decode(const uint8_t* codes, int64_t n, const uint32_t* table, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    const uint32_t word = table[codes[i]];
    for (int d = 0; d < 8; ++d) out[8 * i + d] = ((float)((word >> (4 * d)) & 0xFu) - 8.0f) * 0.5f;
  }
}

/* y[r] = sum_k float(decode(codes[r, k]) * scale[r, group of k]) * x[k], products in fp32 as the
 * reference forms its dense matrix, accumulation in double */
void vq_qmv(const uint16_t* codes, const float* scales, int64_t out_dim, int64_t codewords, int64_t groups,
            const float* x, const uint32_t* abs_table, double* y) {
  const int64_t per_group = codewords / groups;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < out_dim; ++r) {
    double acc = 0.0;
    for (int64_t k = 0; k < codewords; ++k) {
      float w[8];
      e8p_decode_one(codes[r * codewords + k], abs_table, w);
      const float s = scales[r * groups + k / per_group];
      for (int d = 0; d < 8; ++d) acc += (double)(w[d] * s) * (double)x[8 * k + d];
    }
    y[r] = acc;
  }
}
