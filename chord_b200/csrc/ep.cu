// Expert-parallel exchange around the local expert GEMMs, as kernels over peer memory.
//
// The reference has no communication code ("EP routing may carry only this rank's
// routes", docs/getting_started.md:21); a deployment shards the experts over the GPUs
// of one NVSwitch domain and has to move every routed row to the GPU that owns its
// expert and the result back.  Here that exchange is done by this library's own
// kernels through peer pointers (one process per GPU, buffers mapped into every
// process by the host side), not by a collective library:
//
//   plan      one CTA: how many of this rank's routes go to each expert (of any rank) and each
//             route's position among those of its expert; the counts row is stored into
//             every peer's count matrix, followed by a flag.
//   dispatch  a one-CTA kernel waits (bounded) for every rank's counts row and derives, per
//             expert, the first slot of this rank's rows in the owner's receive buffer:
//             the owner's rows are laid out in routing order - expert after expert, each
//             padded to whole routing blocks, inside an expert source rank after source
//             rank - so that the GEMMs load them as consecutive rows, with no copy into
//             slot order.  The copy kernel then stores each route's activation row and
//             its (source rank, route) tag straight into the owner's buffers with 16-byte
//             peer stores and flags every peer.
//   align     one CTA on the owner: waits (bounded) for every rank's rows and writes the
//             routing arrays of that layout (slot ids with sentinels for the padding,
//             expert of each block, padded count) and, per slot, the address of the row of
//             the source rank's result tensor that the down projection's epilogue will
//             store to (the combine step is that store).
//   signal / wait   after the down projection: flag every peer; wait (bounded) until
//             every owner has flagged this rank, after which its result tensor is complete.
//
// Flags carry the call's epoch (a counter every rank advances once per layer call), so
// nothing is reset between calls.  Every wait has a time limit after which the kernel
// records a status bit and goes on (with incomplete data) instead of hanging the GPU.
// No TMA is used here, and nothing is multicast: plain loads from local memory and
// plain stores to peer memory.
#include <cuda_bf16.h>

#include "../../include/chord_b200.h"
#include "common.h"

namespace chord {
namespace {

constexpr int kEpMaxRanks = 64;
constexpr int kEpMaxExperts = 1024;  // experts of all ranks together
constexpr long long kEpWaitCycles = 10000000000ll;  // about five seconds of SM clock
constexpr int32_t kEpStatusCountsTimeout = 1 << 8;
constexpr int32_t kEpStatusDispatchTimeout = 1 << 9;
constexpr int32_t kEpStatusCombineTimeout = 1 << 10;
constexpr int32_t kEpStatusOverflow = 1 << 11;

// Per-rank exchange state, in memory every peer can write.
struct EpState {
  int32_t counts[kEpMaxRanks][kEpMaxExperts];  // counts[src][expert], row src written by rank src
  int32_t flag_counts[kEpMaxRanks];            // epoch of the last counts row that landed from src
  int32_t flag_dispatch[kEpMaxRanks];          // epoch of the last complete set of rows from src
  int32_t flag_combine[kEpMaxRanks];           // epoch of the last complete set of results from owner
  int32_t slot_base[kEpMaxExperts];            // local: first slot of this rank's rows of each expert in its owner's buffers
  int32_t dispatch_ctas_done;                  // local: CTAs of the running dispatch kernel that finished
  int32_t status;                              // local: bits of waits that ran out
};

__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *flag >= epoch; false after kEpWaitCycles.
__device__ bool ep_wait_flag(const int32_t* flag, int32_t epoch) {
  if (ld_acquire_sys(flag) - epoch >= 0) return true;
  const long long start = clock64();
  while (ld_acquire_sys(flag) - epoch < 0) {
    if (clock64() - start > kEpWaitCycles) return false;
    __nanosleep(200);
  }
  return true;
}

constexpr int kPlanThreads = 1024;

// grid 1 x kPlanThreads.  send_pos[i] = position of route i among this rank's routes to
// the same expert, or -1 for an expert id outside [0, num_experts).  (Positions are handed
// out by a shared-memory counter: which route of an expert gets which slot does not change
// any result, a row's product depends on neither its slot nor its neighbours.)
__global__ void __launch_bounds__(kPlanThreads)
ep_plan_kernel(const int32_t* __restrict__ topk_ids, int32_t routes, int32_t num_experts, int32_t world,
               int32_t rank, int32_t* __restrict__ send_pos, EpState* const* __restrict__ peer_state,
               int32_t epoch) {
  __shared__ int32_t hist[kEpMaxExperts];
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  for (int32_t i = threadIdx.x; i < routes; i += blockDim.x) {
    const int32_t e = __ldg(topk_ids + i);
    send_pos[i] = (e >= 0 && e < num_experts) ? atomicAdd(&hist[e], 1) : -1;
  }
  __syncthreads();
  // This rank's counts row goes to every peer, then the flag that says so.
  for (int p = 0; p < world; ++p) {
    int32_t* row = peer_state[p]->counts[rank];
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) row[e] = hist[e];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(&peer_state[threadIdx.x]->flag_counts[rank], epoch);
}

// Rows of expert e on its owner, all source ranks together, rounded up to whole blocks.
__device__ __forceinline__ int32_t padded_rows(int32_t rows, int32_t block_m) {
  return (rows + block_m - 1) / block_m * block_m;
}

// grid 1 x kPlanThreads, after every rank's plan: slot_base[e] = first slot of this rank's
// rows of expert e in the receive buffer of e's owner.
__global__ void __launch_bounds__(kPlanThreads)
ep_offsets_kernel(EpState* state, int32_t num_experts, int32_t experts_per_rank, int32_t world, int32_t rank,
                  int32_t block_m, int32_t epoch) {
  __shared__ int32_t total[kEpMaxExperts];
  if (threadIdx.x < world && !ep_wait_flag(&state->flag_counts[threadIdx.x], epoch)) {
    atomicOr(&state->status, kEpStatusCountsTimeout);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int32_t acc = 0;
    for (int s = 0; s < world; ++s) acc += __ldcg(&state->counts[s][e]);
    total[e] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    const int32_t first = e / experts_per_rank * experts_per_rank;  // the owner's first expert
    int32_t base = 0;
    for (int j = first; j < e; ++j) base += padded_rows(total[j], block_m);
    for (int s = 0; s < rank; ++s) base += __ldcg(&state->counts[s][e]);
    state->slot_base[e] = base;
  }
}

// One warp per route.  x bf16 [tokens, hidden]; the owner's receive buffers hold
// `capacity` slots: recv_x bf16 [capacity, hidden], recv_tag int32 [capacity]
// (source rank << 24 | route).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_ids,
                   const int32_t* __restrict__ send_pos, int32_t routes, int32_t top_k, int32_t hidden,
                   int32_t experts_per_rank, int32_t world, int32_t rank, EpState* state,
                   EpState* const* __restrict__ peer_state, __nv_bfloat16* const* __restrict__ peer_recv_x,
                   int32_t* const* __restrict__ peer_recv_tag, int32_t capacity, int32_t epoch) {
  __shared__ int32_t ok;
  const int lane = threadIdx.x & 31;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  const int32_t vecs = hidden / 8;  // 16-byte pieces per row
  for (int32_t i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < routes; i += warps) {
    const int32_t pos = __ldg(send_pos + i);
    if (pos < 0) continue;
    const int32_t e = __ldg(topk_ids + i);
    const int32_t d = e / experts_per_rank;
    const int32_t slot = __ldcg(&state->slot_base[e]) + pos;
    if (d >= world || slot < 0 || slot >= capacity) {
      if (lane == 0) atomicOr(&state->status, kEpStatusOverflow);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(i / top_k) * hidden);
    uint4* dst = reinterpret_cast<uint4*>(peer_recv_x[d] + static_cast<size_t>(slot) * hidden);
    int32_t v = lane;
    for (; v + 96 < vecs; v += 128) {  // four loads in flight per lane
      const uint4 a = __ldg(src + v), b = __ldg(src + v + 32), c = __ldg(src + v + 64), q = __ldg(src + v + 96);
      dst[v] = a;
      dst[v + 32] = b;
      dst[v + 64] = c;
      dst[v + 96] = q;
    }
    for (; v < vecs; v += 32) dst[v] = __ldg(src + v);
    if (lane == 0) peer_recv_tag[d][slot] = (rank << 24) | i;
  }
  // Last CTA to finish tells every peer that this rank's rows have landed.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int32_t done = atomicAdd(&state->dispatch_ctas_done, 1);
    ok = done == static_cast<int32_t>(gridDim.x) - 1 ? 2 : 0;
  }
  __syncthreads();
  if (ok == 2) {
    __threadfence_system();
    if (threadIdx.x == 0) state->dispatch_ctas_done = 0;
    if (threadIdx.x < world) st_release_sys(&peer_state[threadIdx.x]->flag_dispatch[rank], epoch);
  }
}

constexpr int kAlignThreads = 1024;

// grid 1 x kAlignThreads: routing arrays of the received layout + result addresses.
__global__ void __launch_bounds__(kAlignThreads)
ep_align_kernel(EpState* state, const int32_t* recv_tag, int32_t capacity, int32_t world, int32_t rank,
                int32_t num_local_experts, int32_t block_m, int32_t* __restrict__ sorted_ids,
                int32_t sorted_cap, int32_t* __restrict__ expert_ids, int32_t expert_cap,
                int32_t* __restrict__ num_tokens_padded, int32_t* __restrict__ recv_count,
                __nv_bfloat16* const* __restrict__ peer_routed, int64_t routed_rows_per_rank, int32_t hidden,
                void** __restrict__ row_ptr, int32_t epoch) {
  __shared__ int32_t total[kEpMaxExperts];
  __shared__ int32_t first_slot[kEpMaxExperts + 1];
  if (threadIdx.x < world && !ep_wait_flag(&state->flag_dispatch[threadIdx.x], epoch)) {
    atomicOr(&state->status, kEpStatusDispatchTimeout);
  }
  __syncthreads();
  for (int le = threadIdx.x; le < num_local_experts; le += blockDim.x) {
    int32_t acc = 0;
    for (int s = 0; s < world; ++s) acc += __ldcg(&state->counts[s][rank * num_local_experts + le]);
    total[le] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t acc = 0;
    for (int le = 0; le < num_local_experts; ++le) {
      first_slot[le] = acc;
      acc += padded_rows(total[le], block_m);
    }
    const int32_t room = min(capacity, min(sorted_cap, expert_cap * block_m)) / block_m * block_m;
    if (acc > room) {
      atomicOr(&state->status, kEpStatusOverflow);
      acc = room;
    }
    first_slot[num_local_experts] = acc;
    *num_tokens_padded = acc;
    *recv_count = acc;
  }
  __syncthreads();
  const int32_t padded = first_slot[num_local_experts];
  for (int le = threadIdx.x; le < num_local_experts; le += blockDim.x) {
    const int32_t end = min(first_slot[le] + padded_rows(total[le], block_m), padded);
    for (int32_t s = first_slot[le]; s < end; s += block_m) expert_ids[s / block_m] = le;
  }
  __syncthreads();
  for (int32_t s = threadIdx.x; s < padded; s += blockDim.x) {
    const int32_t le = expert_ids[s / block_m];
    const bool used = s - first_slot[le] < total[le];
    const int32_t tag = used ? __ldcg(recv_tag + s) : 0;
    const int32_t src = (tag >> 24) & 0xFF, route = tag & 0xFFFFFF;
    const bool valid = used && src < world && route < routed_rows_per_rank;
    sorted_ids[s] = valid ? s : capacity;  // a slot's id is the slot itself; `capacity` = no row
    row_ptr[s] = valid ? peer_routed[src] + static_cast<size_t>(route) * hidden : nullptr;
  }
}

__global__ void ep_signal_kernel(EpState* const* __restrict__ peer_state, int32_t world, int32_t rank,
                                 int32_t epoch) {
  __threadfence_system();
  if (threadIdx.x < world) st_release_sys(&peer_state[threadIdx.x]->flag_combine[rank], epoch);
}

__global__ void ep_wait_kernel(EpState* state, int32_t world, int32_t epoch) {
  if (threadIdx.x < world && !ep_wait_flag(&state->flag_combine[threadIdx.x], epoch)) {
    atomicOr(&state->status, kEpStatusCombineTimeout);
  }
}

}  // namespace
}  // namespace chord

extern "C" {

int64_t chord_b200_ep_state_bytes(void) { return static_cast<int64_t>(sizeof(chord::EpState)); }

int chord_b200_ep_plan(const int32_t* topk_ids, int64_t routes, int64_t experts_per_rank, int64_t world,
                       int64_t rank, int32_t* send_pos, void* const* peer_state, int64_t epoch,
                       void* stream) {
  CHORD_REQUIRE(topk_ids != nullptr && send_pos != nullptr && peer_state != nullptr, "null pointer");
  CHORD_REQUIRE(routes > 0 && routes < (1ll << 24), "routes=%lld must be in [1, 2^24)",
                static_cast<long long>(routes));
  CHORD_REQUIRE(world >= 1 && world <= chord::kEpMaxRanks && rank >= 0 && rank < world,
                "rank %lld of %lld: at most %d ranks", static_cast<long long>(rank),
                static_cast<long long>(world), chord::kEpMaxRanks);
  CHORD_REQUIRE(experts_per_rank > 0 && world * experts_per_rank <= chord::kEpMaxExperts,
                "experts_per_rank=%lld: at most %d experts over all ranks",
                static_cast<long long>(experts_per_rank), chord::kEpMaxExperts);
  chord::ep_plan_kernel<<<1, chord::kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, static_cast<int32_t>(routes), static_cast<int32_t>(world * experts_per_rank),
      static_cast<int32_t>(world), static_cast<int32_t>(rank), send_pos,
      reinterpret_cast<chord::EpState* const*>(peer_state), static_cast<int32_t>(epoch));
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

int chord_b200_ep_dispatch(const void* x, const int32_t* topk_ids, const int32_t* send_pos, int64_t routes,
                           int64_t top_k, int64_t hidden, int64_t experts_per_rank, int64_t world,
                           int64_t rank, void* state, void* const* peer_state, void* const* peer_recv_x,
                           void* const* peer_recv_tag, int64_t capacity, int64_t block_m, int64_t epoch,
                           void* stream) {
  CHORD_REQUIRE(x != nullptr && topk_ids != nullptr && send_pos != nullptr && state != nullptr &&
                    peer_state != nullptr && peer_recv_x != nullptr && peer_recv_tag != nullptr,
                "null pointer");
  CHORD_REQUIRE(routes > 0 && routes < (1ll << 24) && top_k > 0 && routes % top_k == 0,
                "routes=%lld must be a positive multiple of top_k below 2^24", static_cast<long long>(routes));
  CHORD_REQUIRE(hidden > 0 && hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0,
                "rows must be 16-byte aligned multiples of 8 BF16");
  CHORD_REQUIRE(world >= 1 && world <= chord::kEpMaxRanks && rank >= 0 && rank < world, "bad rank");
  CHORD_REQUIRE(capacity > 0 && capacity < (1ll << 31), "bad capacity");
  CHORD_REQUIRE(experts_per_rank > 0 && world * experts_per_rank <= chord::kEpMaxExperts,
                "experts_per_rank=%lld: at most %d experts over all ranks",
                static_cast<long long>(experts_per_rank), chord::kEpMaxExperts);
  CHORD_REQUIRE(block_m > 0 && block_m % 8 == 0, "block_m must be a positive multiple of 8");
  chord::DeviceInfo dev;
  if (int rc = chord::current_device_info(&dev)) return rc;
  chord::ep_offsets_kernel<<<1, chord::kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<chord::EpState*>(state), static_cast<int32_t>(world * experts_per_rank),
      static_cast<int32_t>(experts_per_rank), static_cast<int32_t>(world), static_cast<int32_t>(rank),
      static_cast<int32_t>(block_m), static_cast<int32_t>(epoch));
  CHORD_CUDA(cudaGetLastError());
  int64_t blocks = (routes + 7) / 8;
  if (blocks > 4ll * dev.sm_count) blocks = 4ll * dev.sm_count;
  chord::ep_dispatch_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), topk_ids, send_pos, static_cast<int32_t>(routes),
      static_cast<int32_t>(top_k), static_cast<int32_t>(hidden), static_cast<int32_t>(experts_per_rank),
      static_cast<int32_t>(world), static_cast<int32_t>(rank), static_cast<chord::EpState*>(state),
      reinterpret_cast<chord::EpState* const*>(peer_state),
      reinterpret_cast<__nv_bfloat16* const*>(peer_recv_x), reinterpret_cast<int32_t* const*>(peer_recv_tag),
      static_cast<int32_t>(capacity), static_cast<int32_t>(epoch));
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

int chord_b200_ep_align(void* state, const int32_t* recv_tag, int64_t capacity, int64_t world, int64_t rank,
                        int64_t num_local_experts, int64_t block_m, int32_t* sorted_ids, int64_t sorted_cap,
                        int32_t* expert_ids, int64_t expert_cap, int32_t* num_tokens_padded,
                        int32_t* recv_count, void* const* peer_routed, int64_t routed_rows_per_rank,
                        int64_t hidden, void** row_ptr, int64_t epoch, void* stream) {
  CHORD_REQUIRE(state != nullptr && recv_tag != nullptr && sorted_ids != nullptr && expert_ids != nullptr &&
                    num_tokens_padded != nullptr && recv_count != nullptr && peer_routed != nullptr &&
                    row_ptr != nullptr,
                "null pointer");
  CHORD_REQUIRE(world >= 1 && world <= chord::kEpMaxRanks && rank >= 0 && rank < world, "bad rank");
  CHORD_REQUIRE(num_local_experts > 0 && world * num_local_experts <= chord::kEpMaxExperts,
                "num_local_experts=%lld: at most %d experts over all ranks",
                static_cast<long long>(num_local_experts), chord::kEpMaxExperts);
  CHORD_REQUIRE(block_m > 0 && block_m % 8 == 0, "block_m must be a positive multiple of 8");
  CHORD_REQUIRE(capacity > 0 && capacity < (1ll << 30), "bad capacity");
  CHORD_REQUIRE(capacity % block_m == 0 && sorted_cap >= capacity && expert_cap >= capacity / block_m,
                "the receive capacity must be whole blocks and the routing buffers must cover it");
  chord::ep_align_kernel<<<1, chord::kAlignThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<chord::EpState*>(state), recv_tag, static_cast<int32_t>(capacity),
      static_cast<int32_t>(world), static_cast<int32_t>(rank), static_cast<int32_t>(num_local_experts),
      static_cast<int32_t>(block_m), sorted_ids, static_cast<int32_t>(sorted_cap), expert_ids,
      static_cast<int32_t>(expert_cap), num_tokens_padded, recv_count,
      reinterpret_cast<__nv_bfloat16* const*>(peer_routed), routed_rows_per_rank,
      static_cast<int32_t>(hidden), row_ptr, static_cast<int32_t>(epoch));
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

int chord_b200_ep_combine_signal(void* const* peer_state, int64_t world, int64_t rank, int64_t epoch,
                                 void* stream) {
  CHORD_REQUIRE(peer_state != nullptr && world >= 1 && world <= chord::kEpMaxRanks && rank >= 0 &&
                    rank < world,
                "bad arguments");
  chord::ep_signal_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<chord::EpState* const*>(peer_state), static_cast<int32_t>(world),
      static_cast<int32_t>(rank), static_cast<int32_t>(epoch));
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

int chord_b200_ep_combine_wait(void* state, int64_t world, int64_t epoch, void* stream) {
  CHORD_REQUIRE(state != nullptr && world >= 1 && world <= chord::kEpMaxRanks, "bad arguments");
  chord::ep_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<chord::EpState*>(state), static_cast<int32_t>(world), static_cast<int32_t>(epoch));
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

}  // extern "C"
