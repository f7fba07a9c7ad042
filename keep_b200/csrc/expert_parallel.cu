// Expert parallelism: route packing before the dispatch all-to-all, pick summation after the
// combine all-to-all.  See include/keepvq.h for the contract; the transfers themselves are the
// caller's (NCCL all-to-all with constant split sizes).
//
// keepvq_ep_pack is a memset and two launches:
//   plan   one block.  A stable counting sort of the routes by destination rank: per 1024-route
//          chunk every warp ballots each destination, the block adds the warp counts up, and a
//          route's slot in its destination's block is the running base plus the routes before it.
//   copy   one block per route: its token row, 16 bytes per thread per step, to its position.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace keepvq {

constexpr int EP_PLAN_THREADS = 1024;
constexpr int EP_MAX_WORLD = 64;
constexpr uint32_t EP_DEAD = 0xFFFFFFFFu;

__global__ void __launch_bounds__(EP_PLAN_THREADS) ep_plan_kernel(keepvq_ep_pack_args a) {
  __shared__ int warp_count[32][EP_MAX_WORLD];  // routes of each warp per destination, this chunk
  __shared__ int base[EP_MAX_WORLD];            // routes per destination in earlier chunks
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t rows = static_cast<int64_t>(a.world) * a.capacity, routes = a.tokens * a.top_k;
  for (int64_t i = tid; i < rows; i += EP_PLAN_THREADS) { a.send_meta[2 * i] = -1; a.send_meta[2 * i + 1] = 0; }
  if (tid < a.world) base[tid] = 0;
  __syncthreads();
  for (int64_t chunk = 0; chunk < routes; chunk += EP_PLAN_THREADS) {
    const int64_t r = chunk + tid;
    const uint32_t e = r < routes ? a.served_expert[r] : EP_DEAD;
    int dest = -1;
    if (e != EP_DEAD && e / static_cast<uint32_t>(a.experts_per_rank) < static_cast<uint32_t>(a.world)) dest = static_cast<int>(e / a.experts_per_rank);
    int before = 0;  // routes of this warp with my destination and a lower lane
    for (int w = 0; w < a.world; ++w) {
      const unsigned votes = __ballot_sync(0xFFFFFFFFu, dest == w);
      if (lane == 0) warp_count[warp][w] = __popc(votes);
      if (dest == w) before = __popc(votes & ((1u << lane) - 1u));
    }
    __syncthreads();
    if (r < routes) {
      int64_t pos = rows;
      if (dest >= 0) {
        int slot = base[dest] + before;
        for (int i = 0; i < warp; ++i) slot += warp_count[i][dest];
        if (slot < a.capacity) {
          pos = static_cast<int64_t>(dest) * a.capacity + slot;
          a.send_meta[2 * pos] = static_cast<int32_t>(e % a.experts_per_rank);
          a.send_meta[2 * pos + 1] = __float_as_int(a.served_weight[r]);
        }
      }
      a.position[r] = static_cast<int32_t>(pos);
    }
    __syncthreads();
    if (tid < a.world) {
      int total = 0;
      for (int i = 0; i < 32; ++i) total += warp_count[i][tid];
      base[tid] += total;
    }
    __syncthreads();
  }
}

// ---- the exchange over peer-mapped memory --------------------------------------------------
// Flag barrier over the ranks, run by the LAST block of a kernel to finish (every block gives a
// ticket after a system-scope fence behind its stores; the block that draws the last ticket has
// all of this GPU's stores behind it).  Thread w tells rank w "I have arrived at barrier number e"
// and waits for rank w's word in this rank's flags; the system-scope fences order this GPU's
// stores before the flag stores and the peers' stores before whatever follows the kernel here.
// The wait is bounded (a few seconds by default): on expiry *status becomes 1 and the block returns.
constexpr uint32_t EP_WAIT_LIMIT = 1u << 23;

__device__ __forceinline__ void barrier_by_last_block(const keepvq_ep_peer_args& peer) {
  __shared__ int last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(peer.arrivals, 1);
    last = ticket == static_cast<int>(gridDim.x) - 1;
    if (last) *peer.arrivals = 0;  // every block has drawn: ready for the next kernel
  }
  __syncthreads();
  if (!last) return;
  const int w = threadIdx.x;
  const int32_t e = *peer.epoch + 1;
  __threadfence_system();
  if (w < peer.world) {
    volatile int32_t* theirs = peer.flags[w] + peer.rank;
    *theirs = e;
    volatile int32_t* mine = peer.flags[peer.rank] + w;
    const uint32_t limit = peer.wait_spins ? peer.wait_spins : EP_WAIT_LIMIT;
    uint32_t spin = 0;
    while (static_cast<int32_t>(*mine - e) < 0) {
      if (++spin >= limit) { atomicExch(peer.status, 1); break; }
      __nanosleep(100);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (w == 0) *peer.epoch = e;
}

// Dispatch in one launch.  Block r < routes takes route r: its place in the destination's block of
// rows is the number of earlier routes with the same destination (the stable counting sort of the
// NCCL form's plan, each block counting for itself: a decode call has a few hundred routes), its
// slot and weight go into the destination rank's tables and its token row into that rank's
// receive buffer, 16 bytes per thread and step.  Block routes + w marks the rows of this rank's
// block at rank w that no route took.  The last block to finish runs the barrier.
constexpr int EP_DISPATCH_THREADS = 256;

__global__ void __launch_bounds__(EP_DISPATCH_THREADS) ep_dispatch_peer_kernel(keepvq_ep_pack_args a, keepvq_ep_peer_args peer) {
  grid_launch_dependents();
  grid_wait();
  __shared__ int warp_sum[EP_DISPATCH_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t rows = static_cast<int64_t>(a.world) * a.capacity, routes = a.tokens * a.top_k;
  const int64_t b = blockIdx.x;
  auto dest_of = [&](int64_t r) {
    const uint32_t e = a.served_expert[r];
    return (e != EP_DEAD && e / static_cast<uint32_t>(a.experts_per_rank) < static_cast<uint32_t>(a.world)) ? static_cast<int>(e / a.experts_per_rank) : -1;
  };
  const int dest = b < routes ? dest_of(b) : static_cast<int>(b - routes);
  // routes bound for `dest`: the earlier ones (a route's block) or all of them (a marking block)
  const int64_t upto = b < routes ? b : routes;
  int count = 0;
  if (dest >= 0)
    for (int64_t r = tid; r < upto; r += EP_DISPATCH_THREADS) count += dest_of(r) == dest;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xFFFFFFFFu, count, o);
  if (lane == 0) warp_sum[warp] = count;
  __syncthreads();
  count = 0;
#pragma unroll
  for (int i = 0; i < EP_DISPATCH_THREADS / 32; ++i) count += warp_sum[i];
  if (b < routes) {
    int64_t pos = rows;
    if (dest >= 0 && count < a.capacity) {
      pos = static_cast<int64_t>(dest) * a.capacity + count;
      if (tid == 0) {
        int32_t* meta = peer.recv_meta[dest] + static_cast<int64_t>(peer.rank) * a.capacity + count;
        meta[0] = static_cast<int32_t>(a.served_expert[b] % a.experts_per_rank);  // slot plane
        meta[rows] = __float_as_int(a.served_weight[b]);                          // weight plane
      }
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.x) + (b / a.top_k) * a.row_bytes);
      uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(peer.recv_x[dest]) + (static_cast<int64_t>(peer.rank) * a.capacity + count) * a.row_bytes);
      for (int64_t i = tid; i < a.row_bytes / 16; i += EP_DISPATCH_THREADS) dst[i] = src[i];
    }
    if (tid == 0) a.position[b] = static_cast<int32_t>(pos);
  } else {
    for (int64_t slot = min(static_cast<int64_t>(count), a.capacity) + tid; slot < a.capacity; slot += EP_DISPATCH_THREADS) {
      int32_t* meta = peer.recv_meta[dest] + static_cast<int64_t>(peer.rank) * a.capacity + slot;
      meta[0] = -1;
      meta[rows] = 0;
    }
  }
  barrier_by_last_block(peer);
}

// Row r of y, if it is a live route, back to the rank it came from; the last block runs the barrier.
__global__ void __launch_bounds__(256) ep_return_peer_kernel(const uint8_t* __restrict__ y, keepvq_ep_peer_args peer) {
  grid_launch_dependents();
  grid_wait();
  const int64_t r = blockIdx.x;
  if (peer.recv_meta[peer.rank][r] >= 0) {
    const int64_t src_rank = r / peer.capacity, slot = r % peer.capacity;
    const uint4* src = reinterpret_cast<const uint4*>(y + r * peer.row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(peer.back[src_rank]) + (static_cast<int64_t>(peer.rank) * peer.capacity + slot) * peer.row_bytes);
    for (int64_t i = threadIdx.x; i < peer.row_bytes / 16; i += blockDim.x) dst[i] = src[i];
  }
  barrier_by_last_block(peer);
}

__global__ void __launch_bounds__(256) ep_copy_kernel(keepvq_ep_pack_args a) {
  const int64_t r = blockIdx.x, rows = static_cast<int64_t>(a.world) * a.capacity;
  const int64_t pos = a.position[r];
  if (pos >= rows) return;
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(a.x) + (r / a.top_k) * a.row_bytes);
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(a.send_x) + pos * a.row_bytes);
  for (int64_t i = threadIdx.x; i < a.row_bytes / 16; i += blockDim.x) dst[i] = src[i];
}

template <typename T>
__global__ void __launch_bounds__(256) ep_combine_kernel(keepvq_ep_combine_args a) {
  grid_launch_dependents();
  grid_wait();
  const int64_t t = blockIdx.x;
  const T* back = static_cast<const T*>(a.back);
  for (int64_t c = threadIdx.x * 8; c < a.hidden; c += blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < a.top_k; ++j) {  // pick order, as the single-GPU combine
      const int64_t pos = a.position[t * a.top_k + j];
      if (pos < 0 || pos >= a.rows) continue;
      float v[8];
      load8_as_float<T>(back + pos * a.hidden + c, v);
#pragma unroll
      for (int d = 0; d < 8; ++d) acc[d] += v[d];
    }
#pragma unroll
    for (int d = 0; d < 8; ++d) store_from_float(a.out, a.dtype, t * a.hidden + c + d, acc[d]);
  }
}

}  // namespace keepvq

extern "C" int keepvq_ep_pack(const keepvq_ep_pack_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_ep_pack_args& a = *args;
  if (a.tokens < 0 || a.top_k <= 0 || a.world <= 0 || a.world > EP_MAX_WORLD || a.experts_per_rank <= 0 || a.capacity <= 0) return KEEPVQ_ERR_SHAPE;
  if (a.row_bytes <= 0 || a.row_bytes % 16 != 0) return KEEPVQ_ERR_SHAPE;
  const int64_t rows = static_cast<int64_t>(a.world) * a.capacity, routes = a.tokens * a.top_k;
  if (rows >= (1ll << 31) || routes >= (1ll << 31)) return KEEPVQ_ERR_CAPACITY;
  if (!a.send_x || !a.send_meta) return KEEPVQ_ERR_NULL;
  if (routes > 0 && (!a.x || !a.served_expert || !a.served_weight || !a.position)) return KEEPVQ_ERR_NULL;
  if (!aligned_to(a.x, 16) || !aligned_to(a.send_x, 16)) return KEEPVQ_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(a.send_x, 0, static_cast<size_t>(rows) * a.row_bytes, s);
  if (e != cudaSuccess) return note_cuda_error(e);
  ep_plan_kernel<<<1, EP_PLAN_THREADS, 0, s>>>(a);
  KEEPVQ_CHECK_LAUNCH();
  if (routes > 0) {
    ep_copy_kernel<<<static_cast<unsigned>(routes), 256, 0, s>>>(a);
    KEEPVQ_CHECK_LAUNCH();
  }
  return KEEPVQ_OK;
}

extern "C" int keepvq_ep_combine(const keepvq_ep_combine_args* args, void* stream) {
  using namespace keepvq;
  if (!args) return KEEPVQ_ERR_NULL;
  const keepvq_ep_combine_args& a = *args;
  if (!valid_dtype(a.dtype)) return KEEPVQ_ERR_DTYPE;
  if (a.tokens < 0 || a.top_k <= 0 || a.rows < 0 || a.hidden <= 0 || a.hidden % 8 != 0) return KEEPVQ_ERR_SHAPE;
  if (a.tokens == 0) return KEEPVQ_OK;
  if (!a.position || !a.out || (a.rows > 0 && !a.back)) return KEEPVQ_ERR_NULL;
  if (!aligned_to(a.back, 16) || !aligned_to(a.out, 16)) return KEEPVQ_ERR_ALIGN;
  if (a.tokens >= (1ll << 31)) return KEEPVQ_ERR_CAPACITY;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(a.tokens);
  const bool early = a.tokens <= EARLY_LAUNCH_MAX_BLOCKS;
  if (a.dtype == KEEPVQ_F32) launch_after(early, ep_combine_kernel<float>, grid, 256, 0, s, a);
  else if (a.dtype == KEEPVQ_F16) launch_after(early, ep_combine_kernel<__half>, grid, 256, 0, s, a);
  else launch_after(early, ep_combine_kernel<__nv_bfloat16>, grid, 256, 0, s, a);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}

static int check_peer(const keepvq_ep_peer_args& p) {
  if (p.world <= 0 || p.world > keepvq::EP_MAX_WORLD || p.rank < 0 || p.rank >= p.world || p.capacity <= 0) return KEEPVQ_ERR_SHAPE;
  if (p.row_bytes <= 0 || p.row_bytes % 16 != 0) return KEEPVQ_ERR_SHAPE;
  if (!p.recv_x || !p.recv_meta || !p.back || !p.flags || !p.epoch || !p.status || !p.arrivals) return KEEPVQ_ERR_NULL;
  if (static_cast<int64_t>(p.world) * p.capacity >= (1ll << 31)) return KEEPVQ_ERR_CAPACITY;
  return KEEPVQ_OK;
}

extern "C" int keepvq_ep_dispatch_peer(const keepvq_ep_pack_args* pack, const keepvq_ep_peer_args* peer, void* stream) {
  using namespace keepvq;
  if (!pack || !peer) return KEEPVQ_ERR_NULL;
  const keepvq_ep_pack_args& a = *pack;
  const keepvq_ep_peer_args& p = *peer;
  if (int rc = check_peer(p)) return rc;
  if (a.tokens < 0 || a.top_k <= 0 || a.experts_per_rank <= 0) return KEEPVQ_ERR_SHAPE;
  if (a.world != p.world || a.capacity != p.capacity || a.row_bytes != p.row_bytes) return KEEPVQ_ERR_SHAPE;
  const int64_t routes = a.tokens * a.top_k;
  if (routes >= (1ll << 31)) return KEEPVQ_ERR_CAPACITY;
  if (routes > 0 && (!a.x || !a.served_expert || !a.served_weight || !a.position)) return KEEPVQ_ERR_NULL;
  if (!aligned_to(a.x, 16)) return KEEPVQ_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t blocks = routes + p.world;  // one per route, one per destination for the rows no route took
  launch_after(blocks <= EARLY_LAUNCH_MAX_BLOCKS, ep_dispatch_peer_kernel, static_cast<unsigned>(blocks), EP_DISPATCH_THREADS, 0, s, a, p);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}

extern "C" int keepvq_ep_return_peer(const void* y, const keepvq_ep_peer_args* peer, void* stream) {
  using namespace keepvq;
  if (!y || !peer) return KEEPVQ_ERR_NULL;
  const keepvq_ep_peer_args& p = *peer;
  if (int rc = check_peer(p)) return rc;
  if (!aligned_to(y, 16)) return KEEPVQ_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  launch_after(static_cast<int64_t>(p.world) * p.capacity <= EARLY_LAUNCH_MAX_BLOCKS, ep_return_peer_kernel, static_cast<unsigned>(p.world * p.capacity), 256, 0, s, static_cast<const uint8_t*>(y), p);
  KEEPVQ_CHECK_LAUNCH();
  return KEEPVQ_OK;
}
