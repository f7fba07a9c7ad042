// Shared device helpers: dtype tags, scalar loads/stores, and the E8 codeword arithmetic.
//
// E8P 16-bit codeword (reference: src/keep/vq/e8.py:210-234, src/ramp/kernels/common_e8.metal:27-58)
//   low byte  = sign bits, high byte = row of the 256-word abs table
//   parity    = popcount(low byte) & 1;  effective signs = low byte ^ parity
//   output dim d reads nibble p = {0,4,1,5,2,6,3,7}[d]:  v = (nibble_p - 8) / 2, negated when
//   bit p of the effective signs is set, then shifted by +1/4 (even parity) or -1/4 (odd).
//   Hence nibbles k and k+4 of a table word are output dims 2k and 2k+1.
// E8 8-bit residual codeword (e8.py:186-200): dim d = (nibble_d - 8) / 2 of table word [code].
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/keepvq.h"

namespace keepvq {

// Records the runtime's complaint for keepvq_last_cuda_error(); returns a keepvq_status.
int note_cuda_error(cudaError_t err);

#define KEEPVQ_CHECK_LAUNCH()                                   \
  do {                                                          \
    cudaError_t e__ = cudaGetLastError();                       \
    if (e__ != cudaSuccess) return ::keepvq::note_cuda_error(e__); \
  } while (0)

__host__ __device__ inline bool valid_dtype(int t) { return t >= KEEPVQ_F32 && t <= KEEPVQ_BF16; }
__host__ __device__ inline int dtype_size(int t) { return t == KEEPVQ_F32 ? 4 : 2; }

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

__device__ __forceinline__ float load_as_float(const void* base, int dtype, int64_t idx) {
  if (dtype == KEEPVQ_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  if (dtype == KEEPVQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return reinterpret_cast<const float*>(base)[idx];
}

__device__ __forceinline__ void store_from_float(void* base, int dtype, int64_t idx, float v) {
  if (dtype == KEEPVQ_F16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else if (dtype == KEEPVQ_BF16) reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(base)[idx] = v;
}

// ---- programmatic dependent launch ------------------------------------------------------------
// The kernels of a layer call run back to back on one stream.  Launched with launch_after(), a
// kernel may start while its predecessor is still running: it announces itself at once
// (grid_launch_dependents), does whatever needs none of the predecessor's results (building its
// shared-memory tables), then waits for the predecessor to finish and flush (grid_wait) before it
// reads or writes any global memory.  Both instructions are no-ops in a kernel launched the usual
// way, and a successor launched the usual way still waits for full completion.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Early start pays at decode sizes, where launch latency is a visible share of a call; grids of
// thousands of blocks gain nothing from it and measured slower (their early blocks crowd the SMs
// while they wait), so the callers pass `early = false` there and get an ordinary launch.
template <typename... Params, typename... Args>
inline cudaError_t launch_after(bool early, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute = {};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = early ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
constexpr int64_t EARLY_LAUNCH_MAX_BLOCKS = 1024;

// Streaming 128/64/32-bit loads that bypass L1 allocation: code bytes are read once.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream_u1(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// Eight consecutive activations widened to fp32.  `p` is 16-byte aligned.
template <typename T>
__device__ __forceinline__ void load8_as_float(const T* p, float (&v)[8]);

template <>
__device__ __forceinline__ void load8_as_float<float>(const float* p, float (&v)[8]) {
  float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8_as_float<__half>(const __half* p, float (&v)[8]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) { float2 f = __half22float2(h[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
}
template <>
__device__ __forceinline__ void load8_as_float<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) {  // a bf16 is the top half of an fp32
    v[2 * k] = __uint_as_float(w[k] << 16);
    v[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
  }
}

// Eight consecutive values rounded to T and stored at once.  `p` is aligned to 8 * sizeof(T).
template <typename T>
__device__ __forceinline__ void store8_from_float(T* p, const float (&v)[8]);

template <>
__device__ __forceinline__ void store8_from_float<float>(float* p, const float (&v)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8_from_float<__half>(__half* p, const float (&v)[8]) {
  uint4 raw;
  __half2* h = reinterpret_cast<__half2*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}
template <>
__device__ __forceinline__ void store8_from_float<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// ---- table expansion ----------------------------------------------------------------------

// Nibbles k and k+4 of `word` as an fp16 pair of (nibble - 8) / 2.
// 0x6400 | n is the fp16 1024 + n; (1024 + n) * 0.5 - 516 = (n - 8) / 2 exactly.
__device__ __forceinline__ uint32_t nibble_pair_to_half2(uint32_t word, int k) {
  uint32_t raw = ((word >> (4 * k)) & 0x000F000Fu) | 0x64006400u;
  __half2 h = __hfma2(*reinterpret_cast<__half2*>(&raw), __float2half2_rn(0.5f), __float2half2_rn(-516.0f));
  return *reinterpret_cast<uint32_t*>(&h);
}

// A table word whose nibbles k, k+4 hold dims 2k, 2k+1 -> four fp16 pairs in dim order.
__device__ __forceinline__ uint4 expand_pair_packed(uint32_t word) {
  return make_uint4(nibble_pair_to_half2(word, 0), nibble_pair_to_half2(word, 1),
                    nibble_pair_to_half2(word, 2), nibble_pair_to_half2(word, 3));
}

// A table word whose nibble d holds dim d -> the pair-packed arrangement.
__device__ __forceinline__ uint32_t to_pair_packed(uint32_t word) {
  uint32_t out = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    out |= ((word >> (8 * k)) & 0xFu) << (4 * k);
    out |= ((word >> (8 * k + 4)) & 0xFu) << (16 + 4 * k);
  }
  return out;
}

// Scalar decode of one output dim of an E8P codeword, for the reference-shaped paths.
__device__ __forceinline__ float e8p_value(uint32_t code, uint32_t table_word, int d) {
  uint32_t signs = code & 0xFFu;
  uint32_t parity = __popc(signs) & 1u;
  uint32_t eff = signs ^ parity;
  int p = (d >> 1) | ((d & 1) << 2);  // {0,4,1,5,2,6,3,7}[d]
  float v = (static_cast<float>((table_word >> (4 * p)) & 0xFu) - 8.0f) * 0.5f;
  if ((eff >> p) & 1u) v = -v;
  return v + (parity ? -0.25f : 0.25f);
}

__device__ __forceinline__ float e8_1bit_value(uint32_t table_word, int d) {
  return (static_cast<float>((table_word >> (4 * d)) & 0xFu) - 8.0f) * 0.5f;
}

}  // namespace keepvq
