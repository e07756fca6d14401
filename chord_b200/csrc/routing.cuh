// Routing alignment (moe_align_block_size) as a device routine shared by the
// stand-alone kernel and the expert-parallel receive step.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace chord {

constexpr int kAlignWarps = 16;

// Dynamic shared memory the routine needs for `num_experts` experts.
inline size_t moe_align_smem_bytes(int64_t num_experts) {
  return (static_cast<size_t>(kAlignWarps) * num_experts + num_experts + 1) * 4;
}

// One CTA of kAlignWarps warps (CUDA form of the reference's align_routing_blocks,
// tests/generators.py:192-230).  Pass 1 counts routes per (warp, expert); the per-expert
// totals give the padded block layout; pass 2 replays the same walk and places every id
// at expert offset + routes of lower warps + routes seen so far by this warp, so ids
// inside an expert stay ascending and the result is deterministic.  `sentinel` pads the
// blocks (any value >= the number of routed rows the GEMM is told about).  Entries are
// read past L1, so ids another GPU wrote before a flag this CTA has acquired are seen.
__device__ __forceinline__ void moe_align_block(const int32_t* topk_ids, int32_t numel, int32_t sentinel,
                                                int32_t expert_base, int32_t num_experts,
                                                int32_t block_m, int32_t* sorted_ids,
                                                int32_t sorted_cap, int32_t* expert_ids,
                                                int32_t expert_cap, int32_t* num_tokens_padded) {
  extern __shared__ int32_t align_smem[];
  int32_t* counts = align_smem;                              // [kAlignWarps][num_experts]
  int32_t* offsets = align_smem + kAlignWarps * num_experts;  // [num_experts + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kAlignWarps * num_experts; i += blockDim.x) counts[i] = 0;
  __syncthreads();

  const int32_t per_warp = ((numel + kAlignWarps - 1) / kAlignWarps + 31) / 32 * 32;
  const int32_t begin = warp * per_warp;
  const int32_t end = min(numel, begin + per_warp);
  for (int32_t i = begin; i < end; i += 32) {
    const int32_t idx = i + lane;
    int32_t e = -1;
    if (idx < end) {
      e = __ldcg(topk_ids + idx) - expert_base;
      if (e < 0 || e >= num_experts) e = -1;
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && lane == __ffs(peers) - 1) counts[warp * num_experts + e] += __popc(peers);
  }
  __syncthreads();

  // Per expert: totals, and per-warp counts turned into exclusive prefixes.
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    int32_t run = 0;
    for (int w = 0; w < kAlignWarps; ++w) {
      const int32_t c = counts[w * num_experts + e];
      counts[w * num_experts + e] = run;
      run += c;
    }
    offsets[e] = (run + block_m - 1) / block_m * block_m;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t acc = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int32_t padded = offsets[e];
      offsets[e] = acc;
      acc += padded;
    }
    offsets[num_experts] = acc;
    *num_tokens_padded = acc < sorted_cap ? acc : sorted_cap / block_m * block_m;
  }
  __syncthreads();
  const int32_t total = min(offsets[num_experts], sorted_cap / block_m * block_m);
  for (int32_t i = threadIdx.x; i < total; i += blockDim.x) sorted_ids[i] = sentinel;
  for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
    for (int32_t b = offsets[e] / block_m; b < offsets[e + 1] / block_m; ++b) {
      if (b < expert_cap) expert_ids[b] = e;
    }
  }
  __syncthreads();

  for (int32_t i = begin; i < end; i += 32) {
    const int32_t idx = i + lane;
    int32_t e = -1;
    if (idx < end) {
      e = __ldcg(topk_ids + idx) - expert_base;
      if (e < 0 || e >= num_experts) e = -1;
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, e);
    if (e >= 0) {
      const int32_t rank = __popc(peers & ((1u << lane) - 1u));
      const int32_t pos = offsets[e] + counts[warp * num_experts + e] + rank;
      if (pos < total) sorted_ids[pos] = idx;
    }
    __syncwarp();
    if (e >= 0 && lane == __ffs(peers) - 1) counts[warp * num_experts + e] += __popc(peers);
    __syncwarp();
  }
}

}  // namespace chord
