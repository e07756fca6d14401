// The steps either side of the expert GEMMs: SiLU*mul between gate_up and
// down, and the routing alignment (moe_align_block_size) that produces the
// sorted_ids / expert_ids / num_tokens_padded contract `indexed` consumes.
#include <cuda_bf16.h>

#include "../../include/chord_b200.h"
#include "common.h"
#include "ptx.cuh"
#include "routing.cuh"

namespace chord {
namespace {

__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }

// Eight outputs per thread: out[r, c..c+7] = silu(in[r, c..]) * in[r, inter + c..].
__device__ __forceinline__ void silu_mul_vec8(const __nv_bfloat16* in_row, __nv_bfloat16* out_row,
                                              int64_t inter, int64_t c) {
  const uint4 g = __ldg(reinterpret_cast<const uint4*>(in_row + c));
  const uint4 u = __ldg(reinterpret_cast<const uint4*>(in_row + inter + c));
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
  const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t ow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 gf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
    const float2 uf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
    const __nv_bfloat162 o = __floats2bfloat162_rn(silu(gf.x) * uf.x, silu(gf.y) * uf.y);
    ow[i] = *reinterpret_cast<const uint32_t*>(&o);
  }
  *reinterpret_cast<uint4*>(out_row + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                int64_t rows, int64_t inter) {
  ptx::grid_dependency_wait();
  const int64_t vec_per_row = inter / 8;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * 8;
    silu_mul_vec8(in + r * 2 * inter, out + r * inter, inter, c);
  }
}

__global__ void __launch_bounds__(256)
silu_mul_routed_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                       const int32_t* __restrict__ sorted_ids, int64_t sorted_len,
                       const int32_t* __restrict__ num_tokens_padded, int64_t row_limit,
                       int64_t inter) {
  ptx::grid_dependency_wait();
  int64_t count = __ldg(num_tokens_padded);
  count = count < 0 ? 0 : (count > sorted_len ? sorted_len : count);
  for (int64_t slot = blockIdx.x; slot < count; slot += gridDim.x) {
    const int64_t r = __ldg(sorted_ids + slot);
    if (r < 0 || r >= row_limit) continue;
    for (int64_t c = threadIdx.x * 8; c < inter; c += blockDim.x * 8) {
      silu_mul_vec8(in + r * 2 * inter, out + r * inter, inter, c);
    }
  }
}

__global__ void __launch_bounds__(kAlignWarps * 32)
moe_align_kernel(const int32_t* __restrict__ topk_ids, int32_t numel, int32_t expert_base,
                 int32_t num_experts, int32_t block_m, int32_t* __restrict__ sorted_ids,
                 int32_t sorted_cap, int32_t* __restrict__ expert_ids, int32_t expert_cap,
                 int32_t* __restrict__ num_tokens_padded) {
  moe_align_block(topk_ids, numel, numel, expert_base, num_experts, block_m, sorted_ids, sorted_cap,
                  expert_ids, expert_cap, num_tokens_padded);
}

}  // namespace
}  // namespace chord

extern "C" {

int chord_b200_silu_mul(const void* in, void* out, int64_t rows, int64_t inter, void* stream) {
  CHORD_REQUIRE(in != nullptr && out != nullptr, "null tensor pointer");
  CHORD_REQUIRE(rows >= 0 && inter > 0 && inter % 8 == 0,
                "need rows >= 0 and a positive intermediate size divisible by 8");
  CHORD_REQUIRE(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0,
                "in and out must be 16-byte aligned");
  if (rows == 0) return chord::kOk;
  const int64_t total = rows * (inter / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  CHORD_CUDA(chord::launch_kernel(chord::silu_mul_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0,
                                  static_cast<cudaStream_t>(stream), chord::options().pdl != 0,
                                  static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out),
                                  rows, inter));
  return chord::kOk;
}

int chord_b200_silu_mul_routed(const void* in, void* out, const int32_t* sorted_ids,
                               int64_t sorted_len, const int32_t* num_tokens_padded,
                               int64_t row_limit, int64_t inter, void* stream) {
  CHORD_REQUIRE(in != nullptr && out != nullptr && sorted_ids != nullptr &&
                    num_tokens_padded != nullptr,
                "null tensor pointer");
  CHORD_REQUIRE(inter > 0 && inter % 8 == 0, "intermediate size must be a positive multiple of 8");
  CHORD_REQUIRE(((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0,
                "in and out must be 16-byte aligned");
  if (sorted_len <= 0) return chord::kOk;
  const int64_t blocks = sorted_len < 148 * 8 ? sorted_len : 148 * 8;
  CHORD_CUDA(chord::launch_kernel(chord::silu_mul_routed_kernel, dim3(static_cast<unsigned>(blocks)),
                                  dim3(256), 0, static_cast<cudaStream_t>(stream),
                                  chord::options().pdl != 0, static_cast<const __nv_bfloat16*>(in),
                                  static_cast<__nv_bfloat16*>(out), sorted_ids, sorted_len,
                                  num_tokens_padded, row_limit, inter));
  return chord::kOk;
}

int chord_b200_moe_align_block_size(const int32_t* topk_ids, int64_t numel, int64_t expert_base,
                                    int64_t num_experts, int64_t block_m, int32_t* sorted_ids,
                                    int64_t sorted_cap, int32_t* expert_ids, int64_t expert_cap,
                                    int32_t* num_tokens_padded, void* stream) {
  CHORD_REQUIRE(sorted_ids != nullptr && expert_ids != nullptr && num_tokens_padded != nullptr,
                "null routing pointer");
  CHORD_REQUIRE(numel >= 0 && numel < (1ll << 30), "numel out of range");
  CHORD_REQUIRE(numel == 0 || topk_ids != nullptr, "null topk_ids");
  CHORD_REQUIRE(num_experts > 0 && num_experts <= 2048, "num_experts must be in [1, 2048]");
  CHORD_REQUIRE(block_m > 0 && block_m % 8 == 0, "block_m must be a positive multiple of 8");
  const int64_t worst = numel + num_experts * (block_m - 1);
  const int64_t need = (worst < numel * block_m ? worst : numel * block_m);
  CHORD_REQUIRE(sorted_cap >= need / block_m * block_m,
                "sorted_ids capacity %lld is below the worst case %lld",
                static_cast<long long>(sorted_cap), static_cast<long long>(need / block_m * block_m));
  CHORD_REQUIRE(expert_cap >= need / block_m, "expert_ids capacity %lld is below the worst case %lld",
                static_cast<long long>(expert_cap), static_cast<long long>(need / block_m));
  const size_t smem = (static_cast<size_t>(chord::kAlignWarps) * num_experts + num_experts + 1) * 4;
  static bool attr_set[64] = {};
  int device = 0;
  CHORD_CUDA(cudaGetDevice(&device));
  if (smem > 48 * 1024 && !attr_set[device & 63]) {
    CHORD_CUDA(cudaFuncSetAttribute(chord::moe_align_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    attr_set[device & 63] = true;
  }
  chord::moe_align_kernel<<<1, chord::kAlignWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, static_cast<int32_t>(numel), static_cast<int32_t>(expert_base),
      static_cast<int32_t>(num_experts), static_cast<int32_t>(block_m), sorted_ids,
      static_cast<int32_t>(sorted_cap < (1ll << 30) ? sorted_cap : (1ll << 30)), expert_ids,
      static_cast<int32_t>(expert_cap < (1ll << 30) ? expert_cap : (1ll << 30)),
      num_tokens_padded);
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

}  // extern "C"
