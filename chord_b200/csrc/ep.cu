// Expert-parallel exchange around the local expert GEMMs, as kernels over peer memory.
//
// The reference has no communication code ("EP routing may carry only this rank's
// routes", docs/getting_started.md:21); a deployment shards the experts over the GPUs
// of one NVSwitch domain and has to move every routed row to the GPU that owns its
// expert and the result back.  Here that exchange is done by this library's own
// kernels through peer pointers (one process per GPU, buffers mapped into every
// process by the host side), not by a collective library:
//
//   plan      one CTA: per destination rank, how many of this rank's routes go there and
//             each route's position among them (ascending route order); the counts row
//             is stored into every peer's count matrix, followed by a flag.
//   dispatch  waits (bounded) for every rank's counts row, derives this rank's base
//             offset in each destination's receive buffer (rows ordered by source rank,
//             then route), copies each route's activation row and its (local expert,
//             source rank, route) tag straight into the owner's buffers with 16-byte
//             peer stores, then flags every peer.
//   align     one CTA on the owner: waits (bounded) for every rank's rows, runs
//             moe_align_block_size over the received expert tags and fills, per received
//             row, the address of the row of the source rank's result tensor that the
//             down projection's epilogue will store to (the combine step is that store).
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
#include "routing.cuh"

namespace chord {
namespace {

constexpr int kEpMaxRanks = 64;
constexpr long long kEpWaitCycles = 10000000000ll;  // about five seconds of SM clock
constexpr int32_t kEpStatusCountsTimeout = 1 << 8;
constexpr int32_t kEpStatusDispatchTimeout = 1 << 9;
constexpr int32_t kEpStatusCombineTimeout = 1 << 10;
constexpr int32_t kEpStatusOverflow = 1 << 11;

// Per-rank exchange state, in memory every peer can write.
struct EpState {
  int32_t counts[kEpMaxRanks][kEpMaxRanks];  // counts[src][dst], row src written by rank src
  int32_t flag_counts[kEpMaxRanks];          // epoch of the last counts row that landed from src
  int32_t flag_dispatch[kEpMaxRanks];        // epoch of the last complete set of rows from src
  int32_t flag_combine[kEpMaxRanks];         // epoch of the last complete set of results from owner
  int32_t dispatch_ctas_done;                // local: CTAs of the running dispatch kernel that finished
  int32_t status;                            // local: bits of waits that ran out
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

constexpr int kPlanWarps = 32;

// grid 1 x (kPlanWarps * 32).  send_pos[i] = position of route i among this rank's routes
// to the same destination rank (ascending i), or -1 for an expert id outside
// [0, world * experts_per_rank).
__global__ void __launch_bounds__(kPlanWarps * 32)
ep_plan_kernel(const int32_t* __restrict__ topk_ids, int32_t routes, int32_t experts_per_rank,
               int32_t world, int32_t rank, int32_t* __restrict__ send_pos,
               EpState* const* __restrict__ peer_state, int32_t epoch) {
  __shared__ int32_t run[kPlanWarps][kEpMaxRanks];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kPlanWarps * kEpMaxRanks; i += blockDim.x) (&run[0][0])[i] = 0;
  __syncthreads();
  const int32_t per_warp = ((routes + kPlanWarps - 1) / kPlanWarps + 31) / 32 * 32;
  const int32_t begin = warp * per_warp;
  const int32_t end = min(routes, begin + per_warp);
  auto dest_of = [&](int32_t idx) {
    if (idx >= end) return -1;
    const int32_t e = __ldg(topk_ids + idx);
    const int32_t d = e >= 0 ? e / experts_per_rank : -1;
    return d < world ? d : -1;
  };
  for (int32_t i = begin; i < end; i += 32) {
    const int32_t d = dest_of(i + lane);
    const uint32_t same = __match_any_sync(0xffffffffu, d);
    if (d >= 0 && lane == __ffs(same) - 1) run[warp][d] += __popc(same);
  }
  __syncthreads();
  // per destination: totals, and per-warp counts turned into exclusive prefixes
  int32_t total = 0;
  if (threadIdx.x < world) {
    for (int w = 0; w < kPlanWarps; ++w) {
      const int32_t c = run[w][threadIdx.x];
      run[w][threadIdx.x] = total;
      total += c;
    }
  }
  __syncthreads();
  for (int32_t i = begin; i < end; i += 32) {
    const int32_t idx = i + lane;
    const int32_t d = dest_of(idx);
    const uint32_t same = __match_any_sync(0xffffffffu, d);
    if (idx < end) send_pos[idx] = d >= 0 ? run[warp][d] + __popc(same & ((1u << lane) - 1u)) : -1;
    __syncwarp();
    if (d >= 0 && lane == __ffs(same) - 1) run[warp][d] += __popc(same);
    __syncwarp();
  }
  // This rank's counts row goes to every peer (thread d holds the count for destination d),
  // then the flag that says so.
  if (threadIdx.x < world) {
    for (int p = 0; p < world; ++p) peer_state[p]->counts[rank][threadIdx.x] = total;
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x < world) st_release_sys(&peer_state[threadIdx.x]->flag_counts[rank], epoch);
}

// One warp per route.  x bf16 [tokens, hidden]; the owner's receive buffers hold
// `capacity` rows: recv_x bf16 [capacity, hidden], recv_tag int32 [2][capacity]
// (local expert, then source rank << 24 | route).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_ids,
                   const int32_t* __restrict__ send_pos, int32_t routes, int32_t top_k, int32_t hidden,
                   int32_t experts_per_rank, int32_t world, int32_t rank, EpState* state,
                   EpState* const* __restrict__ peer_state, __nv_bfloat16* const* __restrict__ peer_recv_x,
                   int32_t* const* __restrict__ peer_recv_tag, int32_t capacity, int32_t epoch) {
  __shared__ int32_t base[kEpMaxRanks];
  __shared__ int32_t ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world && !ep_wait_flag(&state->flag_counts[threadIdx.x], epoch)) {
    ok = 0;
    atomicOr(&state->status, kEpStatusCountsTimeout);
  }
  __syncthreads();
  if (threadIdx.x < world) {
    // rows in destination d are ordered by source rank: mine start after the lower ranks'
    int32_t acc = 0;
    for (int s = 0; s < rank; ++s) acc += __ldcg(&state->counts[s][threadIdx.x]);
    base[threadIdx.x] = acc;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  const int32_t vecs = hidden / 8;  // 16-byte pieces per row
  for (int32_t i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; ok && i < routes; i += warps) {
    const int32_t pos = __ldg(send_pos + i);
    if (pos < 0) continue;
    const int32_t e = __ldg(topk_ids + i);
    const int32_t d = e / experts_per_rank;
    const int32_t slot = base[d] + pos;
    if (slot >= capacity) {
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
    if (lane == 0) {
      peer_recv_tag[d][slot] = e - d * experts_per_rank;
      peer_recv_tag[d][capacity + slot] = (rank << 24) | i;
    }
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

// grid 1 x (kAlignWarps * 32): routing of the received rows + result addresses.
__global__ void __launch_bounds__(kAlignWarps * 32)
ep_align_kernel(EpState* state, const int32_t* recv_tag, int32_t capacity, int32_t world, int32_t rank,
                int32_t num_local_experts, int32_t block_m, int32_t* __restrict__ sorted_ids,
                int32_t sorted_cap, int32_t* __restrict__ expert_ids, int32_t expert_cap,
                int32_t* __restrict__ num_tokens_padded, int32_t* __restrict__ recv_count,
                __nv_bfloat16* const* __restrict__ peer_routed, int64_t routed_rows_per_rank, int32_t hidden,
                void** __restrict__ row_ptr, int32_t epoch) {
  __shared__ int32_t total_rows;
  if (threadIdx.x < world && !ep_wait_flag(&state->flag_dispatch[threadIdx.x], epoch)) {
    atomicOr(&state->status, kEpStatusDispatchTimeout);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t acc = 0;
    for (int s = 0; s < world; ++s) acc += __ldcg(&state->counts[s][rank]);
    total_rows = acc < capacity ? acc : capacity;
    *recv_count = total_rows;
  }
  __syncthreads();
  const int32_t total = total_rows;
  for (int32_t i = threadIdx.x; i < total; i += blockDim.x) {
    const int32_t tag = __ldcg(recv_tag + capacity + i);
    const int32_t src = (tag >> 24) & 0xFF, route = tag & 0xFFFFFF;
    const bool valid = src < world && route < routed_rows_per_rank;
    row_ptr[i] = valid ? peer_routed[src] + static_cast<size_t>(route) * hidden : nullptr;
  }
  moe_align_block(recv_tag, total, capacity, 0, num_local_experts, block_m, sorted_ids, sorted_cap,
                  expert_ids, expert_cap, num_tokens_padded);
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
  CHORD_REQUIRE(experts_per_rank > 0, "experts_per_rank must be positive");
  chord::ep_plan_kernel<<<1, chord::kPlanWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, static_cast<int32_t>(routes), static_cast<int32_t>(experts_per_rank),
      static_cast<int32_t>(world), static_cast<int32_t>(rank), send_pos,
      reinterpret_cast<chord::EpState* const*>(peer_state), static_cast<int32_t>(epoch));
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

int chord_b200_ep_dispatch(const void* x, const int32_t* topk_ids, const int32_t* send_pos, int64_t routes,
                           int64_t top_k, int64_t hidden, int64_t experts_per_rank, int64_t world,
                           int64_t rank, void* state, void* const* peer_state, void* const* peer_recv_x,
                           void* const* peer_recv_tag, int64_t capacity, int64_t epoch, void* stream) {
  CHORD_REQUIRE(x != nullptr && topk_ids != nullptr && send_pos != nullptr && state != nullptr &&
                    peer_state != nullptr && peer_recv_x != nullptr && peer_recv_tag != nullptr,
                "null pointer");
  CHORD_REQUIRE(routes > 0 && routes < (1ll << 24) && top_k > 0 && routes % top_k == 0,
                "routes=%lld must be a positive multiple of top_k below 2^24", static_cast<long long>(routes));
  CHORD_REQUIRE(hidden > 0 && hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0,
                "rows must be 16-byte aligned multiples of 8 BF16");
  CHORD_REQUIRE(world >= 1 && world <= chord::kEpMaxRanks && rank >= 0 && rank < world, "bad rank");
  CHORD_REQUIRE(capacity > 0 && capacity < (1ll << 31), "bad capacity");
  chord::DeviceInfo dev;
  if (int rc = chord::current_device_info(&dev)) return rc;
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
  CHORD_REQUIRE(num_local_experts > 0 && num_local_experts <= 2048, "num_local_experts must be in [1, 2048]");
  CHORD_REQUIRE(block_m > 0 && block_m % 8 == 0, "block_m must be a positive multiple of 8");
  CHORD_REQUIRE(capacity > 0 && capacity < (1ll << 30), "bad capacity");
  const int64_t worst = capacity + num_local_experts * (block_m - 1);
  CHORD_REQUIRE(sorted_cap >= worst / block_m * block_m && expert_cap >= worst / block_m,
                "routing buffers are below the worst case of %lld ids", static_cast<long long>(worst));
  const size_t smem = chord::moe_align_smem_bytes(num_local_experts);
  static bool attr_set[64] = {};
  int device = 0;
  CHORD_CUDA(cudaGetDevice(&device));
  if (smem > 48 * 1024 && !attr_set[device & 63]) {
    CHORD_CUDA(cudaFuncSetAttribute(chord::ep_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    160 * 1024));
    attr_set[device & 63] = true;
  }
  chord::ep_align_kernel<<<1, chord::kAlignWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
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
