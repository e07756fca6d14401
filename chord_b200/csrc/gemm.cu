// Host side of the W4A16 GEMMs: argument checks, TMA descriptors, launch.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "../../include/chord_b200.h"
#include "common.h"
#include "w4a16_decode.cuh"
#include "w4a16_gemm.cuh"

namespace chord {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      ptr = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t dim0, dim1;
  uint32_t box0, box1;
  int dtype, swizzle;
  bool operator==(const MapKey& o) const {
    return base == o.base && dim0 == o.dim0 && dim1 == o.dim1 && box0 == o.box0 &&
           box1 == o.box1 && dtype == o.dtype && swizzle == o.swizzle;
  }
};

struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.dim0);
    mix(k.dim1);
    mix(k.box0);
    mix(k.box1);
    mix(static_cast<uint64_t>(k.dtype) * 16 + k.swizzle);
    return h;
  }
};

// Row-major 2-D tensor [dim1 rows, dim0 columns] of 2- or 4-byte elements.
// Descriptors depend only on (pointer, shape, box), so they are memoised: a
// decode loop reuses the same weight tensors on every step.
int make_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, uint32_t elem_bytes,
                uint64_t dim0, uint64_t dim1, uint32_t box0, uint32_t box1,
                CUtensorMapSwizzle swizzle) {
  static std::mutex mutex;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{base, dim0, dim1, box0, box1, static_cast<int>(dtype),
                   static_cast<int>(swizzle)};
  {
    std::lock_guard<std::mutex> guard(mutex);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return kOk;
    }
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return fail(kCudaError, "cuTensorMapEncodeTiled is not available");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    return fail(kInvalidArgument, "tensor base address must be 16-byte aligned");
  }
  const cuuint64_t dims[2] = {dim0, dim1};
  const cuuint64_t strides[1] = {dim0 * elem_bytes};
  const cuuint32_t box[2] = {box0, box1};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult rc =
      encode(out, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
             CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    return fail(kCudaError, "cuTensorMapEncodeTiled failed with CUresult %d (dims %llu x %llu, box %u x %u)",
                static_cast<int>(rc), static_cast<unsigned long long>(dim0),
                static_cast<unsigned long long>(dim1), box0, box1);
  }
  std::lock_guard<std::mutex> guard(mutex);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return kOk;
}

int grid_size(const DeviceInfo& dev) {
  const int limit = options().grid_limit;
  return (limit > 0 && limit < dev.sm_count) ? limit : dev.sm_count;
}

int round_up16(int64_t v) { return static_cast<int>((v + 15) / 16 * 16); }

size_t fixed_smem_bytes() { return sizeof(GemmShared) + 1024; }

size_t x_stage_bytes(int mma_n) { return static_cast<size_t>(mma_n) * 256; }

// Clusters of two CTAs of the general kernel that the device keeps resident at once (one
// per TPC when every TPC has both SMs), looked up once per device and group count.
template <int kGroups>
int resident_pairs(size_t smem) {
  static std::mutex mutex;
  static int cached[64];
  static bool have[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> guard(mutex);
  if (!have[device & 63]) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2);
    config.blockDim = dim3(32 * (12 + 4 * kGroups));
    config.dynamicSmemBytes = smem;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    int clusters = 0;
    cudaFuncSetAttribute(w4a16_gemm_kernel<kGroups, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(smem));
    if (cudaOccupancyMaxActiveClusters(&clusters, w4a16_gemm_kernel<kGroups, true>, &config) != cudaSuccess) {
      cudaGetLastError();
      clusters = 0;
    }
    cached[device & 63] = clusters;
    have[device & 63] = true;
  }
  return cached[device & 63];
}

// Depth of the activation ring: small tiles get a deep ring cheaply, large
// ones are limited to what leaves room for the weight ring.
int pick_x_stages(int mma_n) {
  int stages = mma_n <= 32 ? 8 : mma_n <= 64 ? 6 : mma_n <= 128 ? 3 : 2;
  const int cap = options().max_stages;
  if (cap > 0 && stages > cap) stages = cap < 2 ? 2 : cap;
  return stages;
}

// The weight/scale ring takes the rest of shared memory.
int pick_w_stages(const DeviceInfo& dev, int mma_n, int x_stages) {
  const size_t used = fixed_smem_bytes() + static_cast<size_t>(x_stages) * x_stage_bytes(mma_n);
  if (used >= static_cast<size_t>(dev.max_smem_optin)) return 0;
  const size_t budget = static_cast<size_t>(dev.max_smem_optin) - used;
  int stages = static_cast<int>(budget / (kWStageBytes + kSStageBytes));
  if (stages > kMaxWStages) stages = kMaxWStages;
  const int cap = options().max_stages;
  if (cap > 0 && stages > cap) stages = cap < 2 ? 2 : cap;
  return stages;
}

template <int kGroups>
int launch_with_groups(const CUtensorMap& tm_w, const CUtensorMap& tm_s, const CUtensorMap& tm_x,
                       const GemmParams& p, int grid, size_t smem, cudaStream_t stream) {
  static std::once_flag flags[64];
  static cudaError_t attr_result[64];
  int device = 0;
  CHORD_CUDA(cudaGetDevice(&device));
  std::call_once(flags[device & 63], [&] {
    DeviceInfo dev;
    int max_optin = 227 * 1024;
    if (current_device_info(&dev) == kOk) max_optin = dev.max_smem_optin;
    attr_result[device & 63] = cudaFuncSetAttribute(
        w4a16_gemm_kernel<kGroups, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_optin);
    if (attr_result[device & 63] == cudaSuccess) {
      attr_result[device & 63] = cudaFuncSetAttribute(
          w4a16_gemm_kernel<kGroups, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_optin);
    }
  });
  if (attr_result[device & 63] != cudaSuccess) {
    return fail(kCudaError, "cudaFuncSetAttribute failed: %s",
                cudaGetErrorString(attr_result[device & 63]));
  }
  const int threads = 32 * (12 + 4 * kGroups);
  if (p.pair) {
    // every CTA has to be resident (stream-K owners wait for their contributors)
    CHORD_CUDA(launch_kernel_pairs(w4a16_gemm_kernel<kGroups, true>, dim3(grid), dim3(threads), smem, stream,
                                   p.pdl != 0, tm_w, tm_s, tm_x, p));
    return kOk;
  }
  CHORD_CUDA(launch_kernel(w4a16_gemm_kernel<kGroups, false>, dim3(grid), dim3(threads), smem, stream,
                           p.pdl != 0, tm_w, tm_s, tm_x, p));
  return kOk;
}

// `indexed` with routing blocks of 64 rows or more: the routed activation rows are first
// copied into slot order (row s of the copy = the row sorted_ids[s] names, zeros for a
// sentinel), so that the GEMM loads them as TMA boxes like `contiguous` does.  Two
// gathering warps cannot feed 64..256-row tiles: at 85 rows per tile they were the
// bottleneck (2400 of 2600 cycles per stage), at 256 rows seven times slower than the
// MMAs.  The copy costs one read and one write of the routed rows (HBM-bound, <2 % of
// the GEMM's time at these sizes).  One warp per slot.
__global__ void __launch_bounds__(256)
gather_routed_rows_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ sorted_ids,
                          const int32_t* __restrict__ num_tokens_padded, __nv_bfloat16* __restrict__ out,
                          int32_t sorted_len, int32_t x_rows, int32_t out_rows, int32_t top_k, int32_t k) {
  int32_t padded = __ldg(num_tokens_padded);
  padded = padded < 0 ? 0 : (padded > sorted_len ? sorted_len : padded);
  const int32_t lane = threadIdx.x & 31;
  const int32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (int32_t slot = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; slot < padded; slot += warps) {
    const int32_t id = __ldg(sorted_ids + slot);
    const int32_t row = (id >= 0 && id < out_rows) ? id / top_k : x_rows;
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(slot) * k);
    if (row < x_rows) {
      const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * k);
      for (int32_t i = lane; i < k / 8; i += 32) dst[i] = __ldg(src + i);
    } else {
      for (int32_t i = lane; i < k / 8; i += 32) dst[i] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Workspace of an `indexed` launch: the stream-K partials, then (1024-byte aligned) the
// slot-ordered copy of the activations when the routing blocks are large enough for it.
int64_t stream_k_bytes(int grid, int mma_n) {
  // one FP32 slot of 128 x mma_n per CTA; tiles of at most 128 tokens may span two weight
  // blocks (two accumulators), which doubles the slot
  const int64_t general = static_cast<int64_t>(grid) * kBlockN * mma_n * 4 * (mma_n <= 128 ? 2 : 1);
  return (general + 1023) / 1024 * 1024;
}

// CTA pairs pay off on tiles of more than 128 tokens: a pair MMA costs its issuing thread
// about 130 cycles whatever its N (measured at 85 and 128 rows per expert: 490 / 505 us on
// pairs against 388 / 419 us on the two-issuer layout; at 256 and 512 rows: 591 / 1131 us
// against 720 / 1386 us).  The single 256-column accumulator is drained between tiles with
// the tensor core idle, so very short K loops are left to single CTAs.
bool pair_applies(int mma_n, int n, int k) {
  return options().pair != 0 && mma_n > 128 && k >= 2048 && (n / kBlockN) % 2 == 0;
}

bool pregather_applies(int mma_n) { return options().pregather != 0 && mma_n >= 64; }

// Token tiles of at most 32 rows (indexed, masked) have a kernel of their own, in which
// every warpgroup of a CTA is an independent worker with a lock word and a scratch
// slot of its own: four times as many of each as the general kernel needs.
bool decode_kernel_applies(const GemmParams& p) {
  return options().decode_kernel != 0 && p.mode != kModeContiguous && p.mma_n <= kDecMaxTokens;
}

int decode_workers(int grid) { return grid * kDecWorkers; }

int64_t decode_workspace_bytes(int grid, int mma_n) {
  return static_cast<int64_t>(decode_workers(grid)) * kBlockN * mma_n * 4;
}

int launch_decode(GemmParams p, const DeviceInfo& dev, const int32_t* packed, const void* scale,
                  int grid, cudaStream_t stream) {
  // Shared memory: one ring of 128-wide K stages per worker, as deep as fits next to the
  // barriers and the epilogue buffers (four stages for 16-token tiles, three for 32).
  const size_t fixed = sizeof(DecodeShared) + 1024;
  const size_t stage_bytes = decode_stage_bytes(p.mma_n);
  int stages = static_cast<int>((static_cast<size_t>(dev.max_smem_optin) - fixed) / kDecWorkers / stage_bytes);
  if (stages > kDecMaxStages) stages = kDecMaxStages;
  const int cap = options().max_stages;
  if (cap > 0 && stages > cap) stages = cap < 3 ? 3 : cap;
  CHORD_REQUIRE(stages >= 3, "internal: decode ring too shallow (%d stages)", stages);
  p.w_stages = stages;
  p.x_stages = stages;
  CUtensorMap tm_w, tm_s;
  if (int rc = make_map_2d(&tm_w, packed, CU_TENSOR_MAP_DATA_TYPE_INT32, 4,
                           static_cast<uint64_t>(p.n) * 2,
                           static_cast<uint64_t>(p.num_experts) * (p.k / 16), 256, kDecStageK / 16,
                           CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (int rc = make_map_2d(&tm_s, scale, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           static_cast<uint64_t>(p.n),
                           static_cast<uint64_t>(p.num_experts) * (p.k / 32), kBlockN,
                           kDecStageK / 32, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  const size_t smem = kDecWorkers * static_cast<size_t>(stages) * stage_bytes + fixed;
  static std::once_flag flags[64];
  static cudaError_t attr_result[64];
  int device = 0;
  CHORD_CUDA(cudaGetDevice(&device));
  std::call_once(flags[device & 63], [&] {
    attr_result[device & 63] = cudaFuncSetAttribute(
        w4a16_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.max_smem_optin);
    if (attr_result[device & 63] == cudaSuccess) {
      attr_result[device & 63] = cudaFuncSetAttribute(
          w4a16_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dev.max_smem_optin);
    }
  });
  if (attr_result[device & 63] != cudaSuccess) {
    return fail(kCudaError, "cudaFuncSetAttribute failed: %s",
                cudaGetErrorString(attr_result[device & 63]));
  }
  if (p.fuse_silu) {
    CHORD_CUDA(launch_kernel(w4a16_decode_kernel<true>, dim3(grid), dim3(kDecThreads), smem, stream,
                             p.pdl != 0, tm_w, tm_s, p));
  } else {
    CHORD_CUDA(launch_kernel(w4a16_decode_kernel<false>, dim3(grid), dim3(kDecThreads), smem, stream,
                             p.pdl != 0, tm_w, tm_s, p));
  }
  return kOk;
}

// Common tail of the three operators: weight/scale/activation descriptors,
// pipeline depth, scratch checks, launch.
int launch_gemm(GemmParams p, const void* x, const int32_t* packed, const void* scale,
                int64_t num_locks, int64_t workspace_bytes, void* stream) {
  OptionsReadLock options_guard(options_mutex());
  CHORD_REQUIRE(p.n > 0 && p.n % kBlockN == 0, "N=%d must be a positive multiple of 128", p.n);
  CHORD_REQUIRE(p.k > 0 && p.k % 64 == 0, "K=%d must be a positive multiple of 64", p.k);
  CHORD_REQUIRE(p.num_experts > 0, "num_experts must be positive");
  CHORD_REQUIRE(p.tile_tokens > 0 && p.tile_tokens <= kMaxTileTokens,
                "token tile %d must be in [1, %d]", p.tile_tokens, kMaxTileTokens);
  CHORD_REQUIRE(x != nullptr && packed != nullptr && scale != nullptr &&
                    (p.out != nullptr || p.out_row_ptr != nullptr),
                "null tensor pointer");
  CHORD_REQUIRE((reinterpret_cast<uintptr_t>(p.out) & 15u) == 0,
                "the output tensor must be 16-byte aligned");
  CHORD_REQUIRE(static_cast<int64_t>(p.num_experts) * (p.k / 16) < (1ll << 31) &&
                    static_cast<int64_t>(p.x_rows) < (1ll << 31) - 1,
                "tensor too large for 32-bit TMA coordinates");

  // Both kernels read activation rows in 16-byte pieces (cp.async, TMA) and write the
  // FP32 partial sums as words.
  CHORD_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15u) == 0,
                "the activation tensor must be 16-byte aligned");
  CHORD_REQUIRE((reinterpret_cast<uintptr_t>(p.workspace) & 15u) == 0,
                "the workspace must be 16-byte aligned");
  // The row gathers (decode kernel, in-kernel gather of `indexed`) address activations
  // by 32-bit element offsets; tiled TMA loads use row coordinates and have no such limit.
  const bool offsets_fit = static_cast<int64_t>(p.x_rows) * p.k < (1ll << 31);
  DeviceInfo dev;
  if (int rc = current_device_info(&dev)) return rc;
  if (int rc = require_blackwell(dev)) return rc;
  const int grid = grid_size(dev);
  p.mma_n = round_up16(p.tile_tokens);
  p.lock_spins = options().lock_spins;
  if (options().pdl != 0) p.pdl = 1;
  // The decode kernel runs when the caller's locks and scratch are large enough for
  // one per warpgroup; with the smaller buffers of the general kernel, that one runs.
  // SiLU*mul fused into the gate_up epilogue: on the decode kernel for 16-token tiles (two
  // accumulators of 16 columns: twice the scratch slot), on the general kernel for tiles that
  // span a gate and an up block (`npair` layout).
  const bool fused_decode_ok = p.mma_n == 16 && p.k % kDecStageK == 0;
  if (decode_kernel_applies(p) && offsets_fit && p.locks != nullptr && p.workspace != nullptr &&
      (!p.fuse_silu || fused_decode_ok) && num_locks >= decode_workers(grid) &&
      workspace_bytes >= decode_workspace_bytes(grid, p.mma_n) * (p.fuse_silu ? 2 : 1)) {
    p.num_locks = static_cast<int32_t>(num_locks);
    return launch_decode(p, dev, packed, scale, grid, static_cast<cudaStream_t>(stream));
  }
  p.x_load = p.mode == kModeIndexed ? (options().x_load == 1 ? kXLoadGather4 : kXLoadCpAsync)
                                    : kXLoadTiled;
  // Large routing blocks: slot-ordered copy of the activations behind the stream-K
  // partials, if the caller's workspace has room for it (chord_b200_indexed_workspace_bytes).
  __nv_bfloat16* gathered = nullptr;
  if (p.mode == kModeIndexed && p.slot_ordered) {
    p.x_load = kXLoadTiled;
  } else if (p.mode == kModeIndexed && pregather_applies(p.mma_n) && p.sorted_len > 0) {
    const int64_t offset = stream_k_bytes(grid, p.mma_n);
    const int64_t bytes = static_cast<int64_t>(p.sorted_len) * p.k * 2;
    if (workspace_bytes >= offset + bytes) {
      gathered = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(p.workspace) + offset);
      p.x_load = kXLoadTiled;
    }
  }
  CHORD_REQUIRE(p.x_load == kXLoadTiled || offsets_fit,
                "activation tensor too large for the 32-bit element offsets of the row gather");
  p.x_stages = pick_x_stages(p.mma_n);
  p.w_stages = pick_w_stages(dev, p.mma_n, p.x_stages);
  CHORD_REQUIRE(p.w_stages >= 2, "token tile %d leaves room for fewer than two pipeline stages",
                p.tile_tokens);
  // Consecutive rows take one tiled box per K half; routed rows are gathered.
  // Small token tiles are issue-bound with one MMA issuer: use one per dequant group.
  // The accumulators (issuers x buffers x mma_n columns, double-buffered where they
  // fit) take 128 of the 512 TMEM columns for decode-sized tiles and 256 otherwise;
  // the dequantised-operand ring gets the rest.
  const int groups = options().dequant_groups == 4 ? 4 : 2;
  p.issuers = p.mma_n <= 16 ? groups : (p.mma_n <= 64 ? 2 : 1);
  if (options().issuers > 0 && options().issuers * p.mma_n <= 256) p.issuers = options().issuers;
  // Single-issuer layouts with consecutive activation rows get a second issuer for the
  // second K half of tiles of at most 128 tokens (two 128-column accumulators in the
  // same 256 columns).  Not where two warps gather the rows: there the 128-token layout
  // keeps its double-buffered accumulator instead, which measured 7 % faster.
  p.ksplit = (p.issuers == 1 && options().ksplit != 0 && p.x_load == kXLoadTiled) ? 1 : 0;
  // Tiles of at most 128 tokens with consecutive activation rows take two neighbouring
  // 128-row weight blocks each (one issuer, dequant group and accumulator per block), so
  // that an activation stage is fetched from L2 once per 256 weight rows.  Needs the
  // doubled scratch slot; a caller that sized its workspace for single-block tiles (the
  // built-in 5 MiB scratch with 64-row blocks) gets those.
  const int64_t slot_bytes = static_cast<int64_t>(grid) * kBlockN * p.mma_n * 4;
  const int64_t behind_partials = gathered != nullptr ? static_cast<int64_t>(p.sorted_len) * p.k * 2 : 0;
  p.npair = ((options().npair != 0 || p.fuse_silu) && p.x_load == kXLoadTiled && p.mma_n <= 128 &&
             (p.n / kBlockN) % 2 == 0 &&
             workspace_bytes >= (gathered != nullptr ? stream_k_bytes(grid, p.mma_n) + behind_partials
                                                     : 2 * slot_bytes)) ? 1 : 0;
  if (p.npair) {
    p.issuers = 2;
    p.ksplit = 0;
  }
  // Clusters of two CTAs (option "pair") take the same tiles, and 256-token ones, where the
  // rows are consecutive: one CTA per weight block, half of the token rows each.  Every CTA
  // must be resident (stream-K owners wait for their contributors), so the grid is cut to
  // the clusters the device holds at once.
  int launch_grid = grid;
  if (pair_applies(p.mma_n, p.n, p.k) && !p.fuse_silu && p.x_load == kXLoadTiled && grid >= 2) {
    const size_t optin = static_cast<size_t>(dev.max_smem_optin);
    const int pairs = groups == 4 ? resident_pairs<4>(optin) : resident_pairs<2>(optin);
    if (pairs >= 1) {
      p.pair = 1;
      p.npair = 0;
      p.ksplit = 0;
      p.issuers = 1;
      launch_grid = 2 * (pairs < grid / 2 ? pairs : grid / 2);
    }
  }
  CHORD_REQUIRE(!p.fuse_silu || p.npair,
                "gate_up with fused SiLU*mul needs routing blocks of at most 16 rows, or of 64 to 128 "
                "rows with the full workspace of chord_b200_indexed_workspace_bytes(); got block_m=%d",
                p.tile_tokens);
  const int acc_cols = p.ksplit ? 256 : p.issuers * p.mma_n;
  p.a_stages = 2 * acc_cols <= 128 ? 6 : 4;
  if (options().a_stages > 0 && (512 - 64 * options().a_stages) >= acc_cols) {
    p.a_stages = options().a_stages;
  }
  // Ring depths are multiples of the number of warp groups (or issuers) that take
  // turns on a ring, so that successive uses of one barrier are always awaited by the
  // same threads in program order.  Otherwise a party that runs ahead could ask for
  // phase u+1 of a barrier still in phase u-1 and be let through (mbarrier waits only
  // know the phase parity).
  const int turn = groups > p.issuers ? groups : p.issuers;  // both are powers of two
  p.a_stages -= p.a_stages % turn;
  p.w_stages -= p.w_stages % groups;
  if (p.pair) {
    // half a token tile per CTA: a ring twice as deep in the same shared memory
    p.x_stages = p.mma_n <= 64 ? 8 : (p.mma_n <= 128 ? 6 : 4);
    p.w_stages = pick_w_stages(dev, p.mma_n / 2, p.x_stages);
    p.w_stages -= p.w_stages % groups;
  } else if (p.npair) {
    // both issuers consume every activation stage (nobody takes turns on that ring), and
    // with two weight stages per activation stage a deeper activation ring is affordable
    p.x_stages = p.mma_n <= 64 ? 6 : 4;
    p.w_stages = pick_w_stages(dev, p.mma_n, p.x_stages);
    p.w_stages -= p.w_stages % groups;
  } else {
    p.x_stages -= p.x_stages % p.issuers;
  }
  CHORD_REQUIRE(p.a_stages >= turn && p.w_stages >= groups && p.x_stages >= p.issuers,
                "internal: ring depths %d/%d/%d too small for %d groups and %d issuers",
                p.a_stages, p.w_stages, p.x_stages, groups, p.issuers);
  p.num_locks = static_cast<int32_t>(num_locks);
  CHORD_REQUIRE(p.locks != nullptr && num_locks >= grid,
                "stream-K needs a zeroed locks buffer of at least %d lock words, got %lld", grid,
                static_cast<long long>(num_locks));
  const int64_t need = slot_bytes * (p.npair ? 2 : 1);
  CHORD_REQUIRE(p.workspace != nullptr && workspace_bytes >= need,
                "workspace must hold %lld bytes, got %lld", static_cast<long long>(need),
                static_cast<long long>(workspace_bytes));

  // 256-token layouts load consecutive rows as boxes of 128 (sub-slot ring of the kernel).
  p.x_box_rows = (p.mode == kModeContiguous || p.mma_n == 256) ? 128 : p.mma_n;
  if (p.x_load != kXLoadTiled) p.x_box_rows = p.mma_n;
  if (p.pair) {
    // boxes of this CTA's half tile; whole boxes must fit the half (mma_n / 2 rows per K half)
    const int half = p.mma_n / 2;
    p.x_box_rows = half <= 64 ? half : (half % 64 == 0 ? 64 : (half % 32 == 0 ? 32 : (half % 16 == 0 ? 16 : 8)));
  }
  CUtensorMap tm_w, tm_s, tm_x;
  if (int rc = make_map_2d(&tm_w, packed, CU_TENSOR_MAP_DATA_TYPE_INT32, 4,
                           static_cast<uint64_t>(p.n) * 2,
                           static_cast<uint64_t>(p.num_experts) * (p.k / 16), 256, kBlockK / 16,
                           CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (int rc = make_map_2d(&tm_s, scale, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           static_cast<uint64_t>(p.n),
                           static_cast<uint64_t>(p.num_experts) * (p.k / 32), kBlockN,
                           kBlockK / 32, CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (gathered != nullptr) {
    const int warps_needed = p.sorted_len;
    const int blocks = warps_needed / 8 + 1 < 8 * dev.sm_count ? warps_needed / 8 + 1 : 8 * dev.sm_count;
    gather_routed_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        p.x, p.sorted_ids, p.num_tokens_padded, gathered, p.sorted_len, p.x_rows, p.out_rows, p.top_k,
        p.k);
    CHORD_CUDA(cudaGetLastError());
  }
  const void* x_base = gathered != nullptr ? static_cast<const void*>(gathered) : x;
  const uint64_t x_map_rows = gathered != nullptr ? static_cast<uint64_t>(p.sorted_len)
                                                  : static_cast<uint64_t>(p.x_rows);
  if (int rc = make_map_2d(&tm_x, x_base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                           static_cast<uint64_t>(p.k), x_map_rows, 64,
                           p.x_load == kXLoadTiled ? static_cast<uint32_t>(p.x_box_rows) : 1u,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;

  const size_t smem = static_cast<size_t>(p.x_stages) * x_stage_bytes(p.pair ? p.mma_n / 2 : p.mma_n) +
                      static_cast<size_t>(p.w_stages) * (kWStageBytes + kSStageBytes) +
                      fixed_smem_bytes();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (options().dequant_groups == 4) return launch_with_groups<4>(tm_w, tm_s, tm_x, p, launch_grid, smem, s);
  return launch_with_groups<2>(tm_w, tm_s, tm_x, p, launch_grid, smem, s);
}

// Stream-K scratch that lives in the library image instead of in an allocation:
// one FP32 slot of 128 x kStaticScratchTokens per CTA for up to kStaticScratchCtas
// CTAs (5 MiB).  Every GPU that loads the library holds it until the process exits.
constexpr int kStaticScratchTokens = 64;
constexpr int kStaticScratchCtas = 160;
static __device__ __align__(256) float
    static_stream_k_scratch[kStaticScratchCtas * kBlockN * kStaticScratchTokens];

// Device address of the array above on the current device.  In host code the array's
// name is only a handle for the runtime, not an address a kernel could use, so the
// address is looked up once per device (with that device current) and remembered.
int static_scratch_address(float** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mutex;
  static float* address[kMaxDevices] = {};
  int device = 0;
  CHORD_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return fail(kCudaError, "device index %d out of range", device);
  std::lock_guard<std::mutex> guard(mutex);
  if (address[device] == nullptr) {
    void* ptr = nullptr;
    CHORD_CUDA(cudaGetSymbolAddress(&ptr, static_stream_k_scratch));
    if (ptr == nullptr) return fail(kCudaError, "cudaGetSymbolAddress returned a null address");
    address[device] = static_cast<float*>(ptr);
  }
  *out = address[device];
  return kOk;
}

}  // namespace
}  // namespace chord

extern "C" {

int chord_b200_indexed_block_m(int64_t n, int64_t k, int64_t num_experts, int64_t routed_m) {
  (void)n;
  (void)k;
  if (num_experts <= 0 || routed_m < 0) return 16;
  // Rows per local expert if the routes spread evenly; the tile's token
  // dimension is the MMA N, whose minimum is 16, so smaller blocks buy nothing.
  const double avg = static_cast<double>(routed_m) / static_cast<double>(num_experts);
  if (avg <= 8.0) return 16;
  if (avg <= 20.0) return 32;
  if (avg <= 44.0) return 64;
  if (avg <= 100.0) return 128;
  return 256;
}

int chord_b200_masked_tile_m(int64_t expected_m) {
  // A group with more rows than the tile costs a second pass over its weights, so the
  // tile leaves room for the spread around the expected count (measured on 24 groups of
  // 4096 x 7168 with Poisson row counts: at 32 expected rows 64-token tiles take 170 us
  // against 200 us for 32-token tiles, at 64 rows 128-token tiles 182 us against 236 us,
  // at 128 rows 128-token tiles 254 us against 279 us for 256-token tiles on CTA pairs,
  // at 200 rows 350 us against 295 us).
  if (expected_m <= 8) return 16;
  if (expected_m <= 20) return 32;
  if (expected_m <= 48) return 64;
  if (expected_m <= 144) return 128;
  return 256;
}

int64_t chord_b200_gemm_workspace_bytes(int64_t tile_tokens) {
  chord::OptionsReadLock options_guard(chord::options_mutex());
  chord::DeviceInfo dev;
  if (chord::current_device_info(&dev)) return -1;
  if (tile_tokens <= 0 || tile_tokens > chord::kMaxTileTokens) {
    chord::fail(chord::kInvalidArgument, "token tile %lld must be in [1, %d]",
                static_cast<long long>(tile_tokens), chord::kMaxTileTokens);
    return -1;
  }
  const int grid = chord::grid_size(dev);
  const int mma_n = chord::round_up16(tile_tokens);
  if (mma_n <= chord::kDecMaxTokens) return chord::decode_workspace_bytes(grid, mma_n);
  return chord::stream_k_bytes(grid, mma_n);
}

int64_t chord_b200_gate_up_silu_workspace_bytes(int64_t block_m, int64_t sorted_len, int64_t k) {
  const int64_t plain = chord_b200_indexed_workspace_bytes(block_m, sorted_len, k);
  if (plain < 0) return plain;
  // 16-token tiles keep two accumulators per worker: twice the scratch slot
  return chord::round_up16(block_m) <= chord::kDecMaxTokens ? 2 * plain : plain;
}

int64_t chord_b200_indexed_workspace_bytes(int64_t block_m, int64_t sorted_len, int64_t k) {
  chord::OptionsReadLock options_guard(chord::options_mutex());
  chord::DeviceInfo dev;
  if (chord::current_device_info(&dev)) return -1;
  if (block_m <= 0 || block_m > chord::kMaxTileTokens || sorted_len < 0 || k <= 0) {
    chord::fail(chord::kInvalidArgument, "bad workspace query");
    return -1;
  }
  const int grid = chord::grid_size(dev);
  const int mma_n = chord::round_up16(block_m);
  if (mma_n <= chord::kDecMaxTokens) return chord::decode_workspace_bytes(grid, mma_n);
  int64_t bytes = chord::stream_k_bytes(grid, mma_n);
  if (chord::pregather_applies(mma_n)) bytes += sorted_len * k * 2;
  return bytes;
}

int chord_b200_gemm_lock_words(void) {
  chord::OptionsReadLock options_guard(chord::options_mutex());
  chord::DeviceInfo dev;
  if (chord::current_device_info(&dev)) return -1;
  return chord::decode_workers(chord::grid_size(dev));
}

int64_t chord_b200_schedule_segments(int64_t tiles, int64_t k, int64_t grid, int64_t cta,
                                     int32_t* out, int64_t capacity) {
  if (tiles < 0 || k <= 0 || k % 64 || grid <= 0 || cta < 0 || cta >= grid ||
      tiles > (1ll << 30)) {
    chord::fail(chord::kInvalidArgument, "bad schedule query");
    return -1;
  }
  chord::SegmentIterator it;
  it.init(static_cast<int32_t>(tiles), static_cast<int32_t>((k + chord::kBlockK - 1) / chord::kBlockK),
          static_cast<int32_t>(grid), static_cast<int32_t>(cta));
  chord::Segment seg;
  int64_t count = 0;
  while (it.next(seg)) {
    if (out != nullptr && count < capacity) {
      int32_t* rec = out + count * 5;
      rec[0] = seg.tile;
      rec[1] = seg.kb;
      rec[2] = seg.ke;
      rec[3] = seg.type;
      rec[4] = seg.peer;
    }
    ++count;
  }
  return count;
}

static int indexed_launch(const void* x, const int32_t* packed, const void* scale,
                          const int32_t* sorted_ids, int64_t sorted_len, const int32_t* expert_ids,
                          int64_t expert_len, const int32_t* num_tokens_padded, void* out,
                          void* const* out_rows, int32_t* locks, int64_t num_locks, void* workspace,
                          int64_t workspace_bytes, int32_t* status, int64_t m, int64_t n, int64_t k,
                          int64_t num_experts, int64_t top_k, int64_t block_m, void* stream,
                          int fuse_silu = 0, int slot_ordered = 0) {
  CHORD_REQUIRE(m > 0, "inputs must be non-empty, got m=%lld", static_cast<long long>(m));
  CHORD_REQUIRE(top_k > 0, "top_k must be positive, got %lld", static_cast<long long>(top_k));
  CHORD_REQUIRE(block_m > 0 && block_m % 8 == 0 && block_m <= chord::kMaxTileTokens,
                "routing block_m must be a positive multiple of 8 no larger than %d, got %lld",
                chord::kMaxTileTokens, static_cast<long long>(block_m));
  CHORD_REQUIRE(sorted_ids != nullptr && expert_ids != nullptr && num_tokens_padded != nullptr,
                "null routing pointer");
  CHORD_REQUIRE(sorted_len >= 0 && expert_len >= 0, "negative routing length");
  CHORD_REQUIRE(m * top_k < (1ll << 31), "m * top_k overflows int32");
  chord::GemmParams p{};
  p.mode = chord::kModeIndexed;
  p.n = static_cast<int32_t>(n);
  p.k = static_cast<int32_t>(k);
  p.num_experts = static_cast<int32_t>(num_experts);
  p.x_rows = static_cast<int32_t>(m);
  p.out_rows = static_cast<int32_t>(m * top_k);
  p.tile_tokens = static_cast<int32_t>(block_m);
  p.top_k = static_cast<int32_t>(top_k);
  p.sorted_len = static_cast<int32_t>(sorted_len < (1ll << 30) ? sorted_len : (1ll << 30));
  p.expert_len = static_cast<int32_t>(expert_len < (1ll << 30) ? expert_len : (1ll << 30));
  p.sorted_ids = sorted_ids;
  p.expert_ids = expert_ids;
  p.num_tokens_padded = num_tokens_padded;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_ptr = out_rows;
  p.fuse_silu = fuse_silu;
  p.slot_ordered = slot_ordered;
  p.workspace = static_cast<float*>(workspace);
  p.locks = locks;
  p.status = status;
  return chord::launch_gemm(p, x, packed, scale, num_locks, workspace_bytes, stream);
}

int chord_b200_indexed_slots(const void* x, const int32_t* packed, const void* scale,
                             const int32_t* sorted_ids, int64_t sorted_len, const int32_t* expert_ids,
                             int64_t expert_len, const int32_t* num_tokens_padded, void* out,
                             void* const* out_rows, int32_t* locks, int64_t num_locks, void* workspace,
                             int64_t workspace_bytes, int32_t* status, int64_t m, int64_t n, int64_t k,
                             int64_t num_experts, int64_t block_m, int fuse_silu, void* stream) {
  CHORD_REQUIRE(out != nullptr || out_rows != nullptr, "null output pointer and null row-address table");
  CHORD_REQUIRE(sorted_len <= m, "slot-ordered rows: x must hold a row for every routing slot");
  return indexed_launch(x, packed, scale, sorted_ids, sorted_len, expert_ids, expert_len,
                        num_tokens_padded, out, out_rows, locks, num_locks, workspace, workspace_bytes,
                        status, m, n, k, num_experts, 1, block_m, stream, fuse_silu != 0, 1);
}

int chord_b200_indexed(const void* x, const int32_t* packed, const void* scale,
                       const int32_t* sorted_ids, int64_t sorted_len, const int32_t* expert_ids,
                       int64_t expert_len, const int32_t* num_tokens_padded, void* out,
                       int32_t* locks, int64_t num_locks, void* workspace, int64_t workspace_bytes,
                       int32_t* status, int64_t m, int64_t n, int64_t k, int64_t num_experts,
                       int64_t top_k, int64_t block_m, void* stream) {
  CHORD_REQUIRE(out != nullptr, "null output pointer");
  return indexed_launch(x, packed, scale, sorted_ids, sorted_len, expert_ids, expert_len,
                        num_tokens_padded, out, nullptr, locks, num_locks, workspace, workspace_bytes,
                        status, m, n, k, num_experts, top_k, block_m, stream);
}

int chord_b200_indexed_rows(const void* x, const int32_t* packed, const void* scale,
                            const int32_t* sorted_ids, int64_t sorted_len, const int32_t* expert_ids,
                            int64_t expert_len, const int32_t* num_tokens_padded, void* const* out_rows,
                            int32_t* locks, int64_t num_locks, void* workspace, int64_t workspace_bytes,
                            int32_t* status, int64_t m, int64_t n, int64_t k, int64_t num_experts,
                            int64_t top_k, int64_t block_m, void* stream) {
  CHORD_REQUIRE(out_rows != nullptr, "null row-address table");
  return indexed_launch(x, packed, scale, sorted_ids, sorted_len, expert_ids, expert_len,
                        num_tokens_padded, nullptr, out_rows, locks, num_locks, workspace,
                        workspace_bytes, status, m, n, k, num_experts, top_k, block_m, stream);
}

int chord_b200_indexed_gate_up_silu(const void* x, const int32_t* packed, const void* scale,
                                    const int32_t* sorted_ids, int64_t sorted_len,
                                    const int32_t* expert_ids, int64_t expert_len,
                                    const int32_t* num_tokens_padded, void* out, int32_t* locks,
                                    int64_t num_locks, void* workspace, int64_t workspace_bytes,
                                    int32_t* status, int64_t m, int64_t n, int64_t k,
                                    int64_t num_experts, int64_t top_k, int64_t block_m, void* stream) {
  CHORD_REQUIRE(out != nullptr, "null output pointer");
  CHORD_REQUIRE(n > 0 && n % (2 * chord::kBlockN) == 0,
                "fused gate_up needs N=%lld to be a multiple of 256 (gate rows, then as many up rows)",
                static_cast<long long>(n));
  return indexed_launch(x, packed, scale, sorted_ids, sorted_len, expert_ids, expert_len,
                        num_tokens_padded, out, nullptr, locks, num_locks, workspace, workspace_bytes,
                        status, m, n, k, num_experts, top_k, block_m, stream, /*fuse_silu=*/1);
}

int chord_b200_gate_up_silu_supported(int64_t n, int64_t k, int64_t block_m) {
  if (n <= 0 || n % (2 * chord::kBlockN) != 0 || k <= 0 || k % 64 != 0 || block_m <= 0) return 0;
  const int mma_n = chord::round_up16(block_m);
  chord::OptionsReadLock options_guard(chord::options_mutex());
  if (mma_n == 16) return chord::options().decode_kernel != 0 && k % chord::kDecStageK == 0;
  return mma_n >= 64 && mma_n <= 128 && chord::options().pregather != 0;
}

int chord_b200_indexed_static_scratch(const void* x, const int32_t* packed, const void* scale,
                                      const int32_t* sorted_ids, int64_t sorted_len,
                                      const int32_t* expert_ids, int64_t expert_len,
                                      const int32_t* num_tokens_padded, void* out, int32_t* locks,
                                      int64_t num_locks, int32_t* status, int64_t m, int64_t n,
                                      int64_t k, int64_t num_experts, int64_t top_k,
                                      int64_t block_m, void* stream) {
  CHORD_REQUIRE(block_m > 0 && block_m <= chord::kStaticScratchTokens,
                "the built-in scratch holds token blocks of at most %d rows, got block_m=%lld; "
                "use chord_b200_indexed with a caller-provided workspace for larger blocks",
                chord::kStaticScratchTokens, static_cast<long long>(block_m));
  chord::DeviceInfo dev;
  if (int rc = chord::current_device_info(&dev)) return rc;
  int grid = 0;
  {
    chord::OptionsReadLock options_guard(chord::options_mutex());
    grid = chord::grid_size(dev);
  }
  CHORD_REQUIRE(grid <= chord::kStaticScratchCtas,
                "the built-in scratch serves at most %d CTAs, this GPU would launch %d; "
                "use chord_b200_indexed with a caller-provided workspace",
                chord::kStaticScratchCtas, grid);
  float* scratch = nullptr;
  if (int rc = chord::static_scratch_address(&scratch)) return rc;
  const int64_t scratch_bytes = static_cast<int64_t>(chord::kStaticScratchCtas) * chord::kBlockN *
                                chord::kStaticScratchTokens * 4;
  // Nothing in the scratch has to start at zero: a slot is written in full by the CTA
  // that owns it before the reducing CTA reads it, so the last call's contents are harmless.
  return chord_b200_indexed(x, packed, scale, sorted_ids, sorted_len, expert_ids, expert_len,
                            num_tokens_padded, out, locks, num_locks, scratch, scratch_bytes, status,
                            m, n, k, num_experts, top_k, block_m, stream);
}

int chord_b200_contiguous(const void* x, const int32_t* packed, const void* scale,
                          const int32_t* m_indices, void* out, int32_t* locks, int64_t num_locks,
                          void* workspace, int64_t workspace_bytes, int32_t* status, int64_t m,
                          int64_t n, int64_t k, int64_t num_experts, int enable_pdl, void* stream) {
  CHORD_REQUIRE(m > 0 && m % 128 == 0,
                "contiguous m=%lld must be a positive multiple of 128 (per-expert padded)",
                static_cast<long long>(m));
  CHORD_REQUIRE(m_indices != nullptr, "null m_indices");
  chord::GemmParams p{};
  p.mode = chord::kModeContiguous;
  p.n = static_cast<int32_t>(n);
  p.k = static_cast<int32_t>(k);
  p.num_experts = static_cast<int32_t>(num_experts);
  p.x_rows = static_cast<int32_t>(m);
  p.out_rows = static_cast<int32_t>(m);
  CHORD_REQUIRE(m / 128 <= chord::kMaxMTiles && num_experts <= 0x7FFF,
                "contiguous supports at most %d rows and %d experts", chord::kMaxMTiles * 128, 0x7FFF);
  // Token tiles are the 128-row blocks, each spanning two 128-row weight blocks
  // (`npair`).  Where that layout does not apply (option npair = 0, an odd number of
  // weight blocks) or with option contiguous_tile = 256, neighbouring blocks of one
  // expert are merged into 256-token tiles over one weight block instead.
  bool two_launches = false;
  {
    chord::OptionsReadLock options_guard(chord::options_mutex());
    const chord::Options& o = chord::options();
    const bool even_blocks = (n / chord::kBlockN) % 2 == 0;
    const bool pairs = o.npair != 0 && even_blocks;
    p.tile_tokens = o.contiguous_tile == 128 || (o.contiguous_tile == 0 && pairs) ? 128 : 256;
    // With CTA pairs enabled, experts of more than one 128-row block take 256-token tiles
    // on CTA pairs in a second launch; single-block experts stay on 128-token tiles.
    two_launches = o.contiguous_tile == 0 && pairs && chord::pair_applies(256, static_cast<int>(n), static_cast<int>(k));
  }
  p.top_k = 1;
  p.m_blocks = static_cast<int32_t>(m / 128);
  p.pdl = enable_pdl != 0;
  p.m_indices = m_indices;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.workspace = static_cast<float*>(workspace);
  p.locks = locks;
  p.status = status;
  if (two_launches) {
    // Each expert's run of 128-row blocks is cut into pairs; the blocks left over (single-
    // block experts, the last block of an odd run) take 128-token tiles in the first launch,
    // the pairs 256-token tiles on CTA pairs in the second.  The launches write disjoint
    // rows and use the scratch and the locks one after the other (the second launch's
    // kernel waits for the first before it touches either).
    p.run_part = 1;
    if (int rc = chord::launch_gemm(p, x, packed, scale, num_locks, workspace_bytes, stream)) return rc;
    p.tile_tokens = 256;
    p.run_part = 2;
  }
  return chord::launch_gemm(p, x, packed, scale, num_locks, workspace_bytes, stream);
}

int chord_b200_masked(const void* x, const int32_t* packed, const void* scale,
                      const int32_t* masked_m, void* out, int32_t* locks, int64_t num_locks,
                      void* workspace, int64_t workspace_bytes, int32_t* status,
                      int64_t num_groups, int64_t max_m, int64_t n, int64_t k, int64_t tile_m,
                      int enable_pdl, void* stream) {
  CHORD_REQUIRE(num_groups > 0 && num_groups <= chord::kMaxGroups,
                "num_groups=%lld must be in [1, %d]", static_cast<long long>(num_groups),
                chord::kMaxGroups);
  CHORD_REQUIRE(max_m > 0, "max_m must be positive");
  CHORD_REQUIRE(masked_m != nullptr, "null masked_m");
  CHORD_REQUIRE(tile_m > 0 && tile_m <= chord::kMaxTileTokens, "tile_m=%lld must be in [1, %d]",
                static_cast<long long>(tile_m), chord::kMaxTileTokens);
  CHORD_REQUIRE(num_groups * max_m < (1ll << 31) - 1, "num_groups * max_m overflows int32");
  chord::GemmParams p{};
  p.mode = chord::kModeMasked;
  p.n = static_cast<int32_t>(n);
  p.k = static_cast<int32_t>(k);
  p.num_experts = static_cast<int32_t>(num_groups);
  p.x_rows = static_cast<int32_t>(num_groups * max_m);
  p.out_rows = p.x_rows;
  p.tile_tokens = static_cast<int32_t>(tile_m);
  p.top_k = 1;
  p.max_m = static_cast<int32_t>(max_m);
  p.pdl = enable_pdl != 0;
  p.masked_m = masked_m;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.workspace = static_cast<float*>(workspace);
  p.locks = locks;
  p.status = status;
  return chord::launch_gemm(p, x, packed, scale, num_locks, workspace_bytes, stream);
}

}  // extern "C"
