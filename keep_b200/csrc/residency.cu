// keepvq_residency_tick: the routed cache's admission / eviction policy for one layer, as one
// small kernel (one block).  The demand statistics are gathered in parallel; the list surgery
// that follows is order-sensitive and tiny, so one thread does it, exactly in the order of the
// reference's host code (scripts/v41_build/omlx_routed.py:184-247).
#include <math.h>

#include "common.cuh"

namespace keepvq {

constexpr int RT_THREADS = 256;
constexpr float ROUTER_OFF = -1e30f;

__device__ __forceinline__ void log_action(const keepvq_residency_args& a, int kind, int expert, int slot) {
  const int at = atomicAdd(a.action_count, 1);
  if (at < a.max_actions) { a.actions[3 * at] = kind; a.actions[3 * at + 1] = expert; a.actions[3 * at + 2] = slot; }
}

__global__ void __launch_bounds__(RT_THREADS) residency_tick_kernel(keepvq_residency_args a) {
  extern __shared__ __align__(8) unsigned char raw[];
  unsigned long long* wanted = reinterpret_cast<unsigned long long*>(raw);  // [pool] bits of the max strong g (0 = not wanted)
  double* miss_g = reinterpret_cast<double*>(wanted + a.pool);                // [pool] candidates
  int* miss_e = reinterpret_cast<int*>(miss_g + a.pool);
  __shared__ int resident_hits;
  const int P = static_cast<int>(a.pool), S = static_cast<int>(a.slots), K = a.top_k;
  for (int e = threadIdx.x; e < P; e += RT_THREADS) wanted[e] = 0ull;
  if (threadIdx.x == 0) resident_hits = 0;
  __syncthreads();

  int hits = 0;
  for (int64_t t = threadIdx.x; t < a.tokens; t += RT_THREADS) {
    double sum = 0.0;
    for (int j = 0; j < K; ++j) sum += static_cast<double>(a.want_score[t * K + j]);
    for (int j = 0; j < K; ++j) {
      const uint32_t e = a.want[t * K + j];
      if (e >= static_cast<uint32_t>(P)) continue;
      hits += a.slot_of[e] != KEEPVQ_NO_RESIDUAL;
      const double g = static_cast<double>(a.want_score[t * K + j]) / (sum + 1e-20) * static_cast<double>(a.route_scale);
      if (g >= static_cast<double>(a.tau)) atomicMax(&wanted[e], static_cast<unsigned long long>(__double_as_longlong(g)));  // g > 0: bit order = value order
    }
  }
  atomicAdd(&resident_hits, hits);
  __syncthreads();
  if (threadIdx.x != 0) return;

  int n_free = a.counts[0], n_cool = a.counts[1], n_read = a.counts[2];
  if (a.first_layer) { a.stats[KEEPVQ_STAT_CALLS] += 1; a.stats[KEEPVQ_STAT_TOKENS] += a.tokens; }
  a.stats[KEEPVQ_STAT_DEMAND] += a.tokens * K;
  a.stats[KEEPVQ_STAT_RESIDENT] += resident_hits;

  // install: route the reads that have landed, keep the others in order
  int kept = 0;
  for (int i = 0; i < n_read; ++i) {
    const int e = a.reading[2 * i], slot = a.reading[2 * i + 1];
    if (a.landed && a.landed[e]) {
      a.served_bias[e] = a.pool_bias ? a.pool_bias[e] : 0.0f;
      a.slot_of[e] = static_cast<uint32_t>(slot);
      a.slot_expert[slot] = e;
      a.last_use[slot] = static_cast<double>(a.step);
      a.stats[KEEPVQ_STAT_INSTALLED] += 1;
      a.landed[e] = 0;  // consumed: a later read of the same expert raises it again
      log_action(a, KEEPVQ_ACTION_ROUTE, e, slot);
    } else {
      a.reading[2 * kept] = e; a.reading[2 * kept + 1] = slot; ++kept;
    }
  }
  n_read = kept;

  // refresh residents, collect candidates
  int n_miss = 0;
  for (int e = 0; e < P; ++e) {
    if (!wanted[e]) continue;
    const uint32_t slot = a.slot_of[e];
    if (slot != KEEPVQ_NO_RESIDUAL) { a.last_use[slot] = static_cast<double>(a.call); continue; }
    bool reading = false;
    for (int i = 0; i < n_read; ++i) reading |= a.reading[2 * i] == e;
    if (reading) continue;
    // insertion into descending (g, expert) order
    const double g = __longlong_as_double(static_cast<long long>(wanted[e]));
    int at = n_miss++;
    while (at > 0 && (miss_g[at - 1] < g || (miss_g[at - 1] == g && miss_e[at - 1] < e))) { miss_g[at] = miss_g[at - 1]; miss_e[at] = miss_e[at - 1]; --at; }
    miss_g[at] = g; miss_e[at] = e;
  }
  a.stats[KEEPVQ_STAT_WANTED] += n_miss;

  // cooled slots become free, in order
  kept = 0;
  for (int i = 0; i < n_cool; ++i) {
    const int slot = a.cooling[2 * i], since = a.cooling[2 * i + 1];
    if (since <= a.call) a.free_list[n_free++] = slot;
    else { a.cooling[2 * kept] = slot; a.cooling[2 * kept + 1] = since; ++kept; }
  }
  n_cool = kept;

  // admissions
  for (int i = 0; i < n_miss; ++i) {
    if (n_free == 0) { a.stats[KEEPVQ_STAT_NO_SLOT] += 1; continue; }
    const int slot = a.free_list[--n_free];
    a.reading[2 * n_read] = miss_e[i]; a.reading[2 * n_read + 1] = slot; ++n_read;
    a.stats[KEEPVQ_STAT_ADMITTED] += 1;
    log_action(a, KEEPVQ_ACTION_ADMIT, miss_e[i], slot);
  }

  // eviction: stable order of last_use, wanted experts spared
  for (int shortfall = a.spare - n_free - n_cool; shortfall > 0; --shortfall) {
    int victim = -1;
    double oldest = 0.0;
    for (int s = 0; s < S; ++s) {
      const int e = a.slot_expert[s];
      if (e < 0 || wanted[e]) continue;
      if (victim < 0 || a.last_use[s] < oldest) { victim = s; oldest = a.last_use[s]; }
    }
    if (victim < 0) break;
    const int e = a.slot_expert[victim];
    a.slot_of[e] = KEEPVQ_NO_RESIDUAL;
    a.slot_expert[victim] = -1;
    a.last_use[victim] = INFINITY;
    a.served_bias[e] = ROUTER_OFF;  // unrouted first; its bytes change only after earlier calls finished
    a.cooling[2 * n_cool] = victim; a.cooling[2 * n_cool + 1] = static_cast<int>(a.step); ++n_cool;
    a.stats[KEEPVQ_STAT_EVICTED] += 1;
    log_action(a, KEEPVQ_ACTION_UNROUTE, e, victim);
  }
  a.counts[0] = n_free; a.counts[1] = n_cool; a.counts[2] = n_read;
}

}  // namespace keepvq

extern "C" int keepvq_residency_tick(const keepvq_residency_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_residency_args& a = *args;
  if (!a.slot_expert || !a.slot_of || !a.served_bias || !a.last_use || !a.free_list || !a.cooling || !a.reading || !a.counts || !a.stats)
    return KEEPVQ_ERR_NULL;
  if (!a.actions || !a.action_count) return KEEPVQ_ERR_NULL;
  if (a.pool <= 0 || a.slots <= 0 || a.tokens < 0 || a.top_k <= 0 || a.max_actions < 0) return KEEPVQ_ERR_SHAPE;
  if (a.tokens > 0 && (!a.want || !a.want_score)) return KEEPVQ_ERR_NULL;
  const size_t smem = static_cast<size_t>(a.pool) * (8 + 8 + 4);
  if (smem > 160 * 1024) return KEEPVQ_ERR_CAPACITY;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(residency_tick_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
  }
  residency_tick_kernel<<<1, RT_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(a);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}
