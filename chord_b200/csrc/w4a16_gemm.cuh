// W4A16 grouped GEMM for sm_100a: BF16 activations x INT4 weights with one
// BF16 scale per 32-element K group, FP32 accumulation in tensor memory.
//
// One kernel serves the three operators of the reference library
// (chord_kernels/ops.py:8-90): `indexed` (routed rows named by sorted_ids /
// expert_ids / num_tokens_padded), `contiguous` (128-row expert runs named by
// m_indices) and `masked` (per-group valid-row counts).  They differ only in
// how a tile finds its expert, its activation rows and its output rows.
//
// Orientation ("swap-AB"): the 128 weight rows of a tile are the MMA's M
// dimension and the tile's tokens (16..256) are its N dimension, so
//     D[128 weight rows, tokens] += Wdeq[128, 16] * X[tokens, 16]^T
// per K16 step.  The dequantised weights never touch shared memory: dequant
// warps read the packed words the TMA brought in, expand them to BF16 in
// registers and store them straight into tensor memory, from where
// tcgen05.mma takes its A operand.  Activations arrive K-major with the
// 128-byte swizzle, either by TMA tile::gather4 (four arbitrary rows per
// instruction - the routed-row gather) or, as a selectable variant, by
// per-thread cp.async.
//
// Warp roles (one CTA per SM, persistent):
//   warp 0            producer: TMA for packed weights, scales, activations
//   warp 1            MMA issuer (one thread)
//   warp 2            tensor-memory allocator
//   warps 4..4+4G-1   G dequant groups of four warps (one per TMEM lane quarter)
//   last four warps   epilogue: TMEM -> registers -> BF16 -> global, plus the
//                     stream-K reduction through `locks` and the FP32 workspace
//
// Scheduling follows the reference's scheme (humming/scheduler.cuh:73-101):
// whole tiles are dealt round-robin to the CTAs while full waves last; the
// remaining tiles are flattened into (tile, k-block) units and split evenly
// over the grid (stream-K).  A tile split this way is finished by the CTA that
// holds its k=0 slice: the other slices write FP32 partials to their workspace
// slot and bump the owner's lock word; the owner waits for the count, adds the
// partials in CTA order (deterministic), rounds once to BF16 and resets the
// lock to zero (reference protocol: humming/epilogue/pipeline.cuh:132-163).
//
// Numerics match the reference's kernels (humming/arith/mainloop_arith.cuh:66-101,
// deep_gemm/ptx/ld_st.cuh:15-40): weight = RN_bf16((code - 8) * scale), products
// and sums in FP32, one rounding to BF16 at the end.
#pragma once

#include <cuda.h>

#include "ptx.cuh"

namespace chord {

enum GemmMode : int32_t { kModeIndexed = 0, kModeContiguous = 1, kModeMasked = 2 };
enum XLoadMode : int32_t { kXLoadGather4 = 0, kXLoadCpAsync = 1 };

// Device status bits (OR-ed into *status by a kernel that gave up on a wait).
enum StatusBits : int32_t {
  kStatusProducerTimeout = 1,
  kStatusMmaTimeout = 2,
  kStatusDequantTimeout = 4,
  kStatusEpilogueTimeout = 8,
  kStatusLockTimeout = 16,
};

constexpr int kBlockN = 128;      // weight rows per tile (MMA M)
constexpr int kBlockK = 64;       // K elements per pipeline stage
constexpr int kMaxStages = 12;
constexpr int kASlots = 4;        // tensor-memory ring for the dequantised A operand
constexpr int kAColsPerSlot = kBlockK / 2;
constexpr int kDCol0 = kASlots * kAColsPerSlot;  // 128
constexpr int kTmemCols = 512;
constexpr int kMaxTileTokens = 256;
constexpr int kMaxGroups = 1024;  // masked: prefix table capacity
constexpr int kWStageBytes = (kBlockK / 16) * 1024;
constexpr int kSStageBytes = (kBlockK / 32) * 256;

struct GemmParams {
  int32_t mode;
  int32_t x_load;
  int32_t n;            // weight rows per expert
  int32_t k;
  int32_t num_experts;
  int32_t x_rows;       // rows of the activation tensor
  int32_t out_rows;     // rows of the output tensor
  int32_t tile_tokens;  // indexed: block_m; contiguous: 128; masked: tokens per M tile
  int32_t mma_n;        // tile_tokens rounded up to 16
  int32_t top_k;        // indexed
  int32_t max_m;        // masked
  int32_t m_blocks;     // contiguous: m / 128
  int32_t sorted_len;   // indexed: capacity of sorted_ids
  int32_t expert_len;   // indexed: capacity of expert_ids
  int32_t stages;
  int32_t num_locks;
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_tokens_padded;
  const int32_t* m_indices;
  const int32_t* masked_m;
  const __nv_bfloat16* x;
  __nv_bfloat16* out;
  float* workspace;     // grid * 128 * mma_n floats
  int32_t* locks;
  int32_t* status;
};

struct TileInfo {
  int32_t n0;      // first weight row
  int32_t expert;
  int32_t ntok;    // valid token slots in the tile
  int32_t base;    // indexed: first sorted_ids slot; contiguous: first row; masked: first row of the group
  int32_t m0;      // masked: first row inside the group
  int32_t limit;   // masked: masked_m of the group
  bool valid;
};

enum SegType : int32_t { kSegFull = 0, kSegOwner = 1, kSegContrib = 2 };

struct Segment {
  int32_t tile;
  int32_t kb, ke;  // k-block range [kb, ke)
  int32_t type;
  int32_t peer;    // owner: number of contributors; contributor: owner CTA
};

// Enumerates the work of one CTA; every warp role walks the same sequence.
struct SegmentIterator {
  int32_t grid, cta, ki;
  int32_t dp_waves, dp_tiles, wave;
  int64_t units, u0, u1;
  int32_t geff;

  __device__ void init(int32_t tiles, int32_t k_iters, int32_t grid_, int32_t cta_) {
    grid = grid_;
    cta = cta_;
    ki = k_iters;
    dp_waves = tiles / grid;
    int32_t sk_tiles = tiles - dp_waves * grid;
    // A short tail would be cut into slivers: fold one full wave into it.
    if (dp_waves > 0 && sk_tiles > 0 && static_cast<int64_t>(sk_tiles) * ki < 8ll * grid) {
      dp_waves -= 1;
      sk_tiles += grid;
    }
    dp_tiles = dp_waves * grid;
    wave = 0;
    units = static_cast<int64_t>(sk_tiles) * ki;
    geff = units < grid ? static_cast<int32_t>(units) : grid;
    if (cta < geff) {
      u0 = cta * units / geff;
      u1 = (cta + 1) * units / geff;
    } else {
      u0 = u1 = 0;
    }
  }

  __device__ int32_t cta_of_unit(int64_t u) const {
    return static_cast<int32_t>(((u + 1) * geff - 1) / units);
  }

  __device__ bool next(Segment& s) {
    if (wave < dp_waves) {
      s.tile = wave * grid + cta;
      s.kb = 0;
      s.ke = ki;
      s.type = kSegFull;
      s.peer = 0;
      ++wave;
      return true;
    }
    if (u0 >= u1) return false;
    const int64_t t = u0 / ki;
    const int32_t kb = static_cast<int32_t>(u0 - t * ki);
    const int64_t room = u1 - u0;
    const int32_t ke = (ki - kb) < room ? ki : static_cast<int32_t>(kb + room);
    s.tile = dp_tiles + static_cast<int32_t>(t);
    s.kb = kb;
    s.ke = ke;
    if (kb == 0 && ke == ki) {
      s.type = kSegFull;
      s.peer = 0;
    } else if (kb == 0) {
      s.type = kSegOwner;
      s.peer = cta_of_unit(t * ki + ki - 1) - cta;
    } else {
      s.type = kSegContrib;
      s.peer = cta_of_unit(t * ki);
    }
    u0 += ke - kb;
    return true;
  }
};

struct __align__(16) GemmShared {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t afull[kASlots];
  uint64_t aempty[kASlots];
  uint64_t dfull[2];
  uint64_t dempty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  int32_t m_blocks;
  volatile uint32_t epilogue_failed;
  int32_t out_row[kMaxTileTokens];   // epilogue: output row per token slot, -1 = skip
  int32_t x_row[kMaxTileTokens];     // producer (cp.async variant): activation row per slot
  int32_t group_prefix[kMaxGroups + 1];  // masked: first M tile of each group
};

__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, const GemmShared& sh,
                                                int32_t tile) {
  TileInfo t;
  const int32_t n_blocks = p.n / kBlockN;
  const int32_t mb = tile / n_blocks;
  t.n0 = (tile - mb * n_blocks) * kBlockN;
  t.m0 = 0;
  t.limit = 0;
  if (p.mode == kModeIndexed) {
    t.expert = __ldg(p.expert_ids + mb);
    t.ntok = p.tile_tokens;
    t.base = mb * p.tile_tokens;
  } else if (p.mode == kModeContiguous) {
    t.expert = __ldg(p.m_indices + mb * p.tile_tokens);
    t.ntok = p.tile_tokens;
    t.base = mb * p.tile_tokens;
  } else {
    // Largest g with group_prefix[g] <= mb.
    int32_t lo = 0, hi = p.num_experts;
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (sh.group_prefix[mid] <= mb) lo = mid; else hi = mid;
    }
    t.expert = lo;
    t.m0 = (mb - sh.group_prefix[lo]) * p.tile_tokens;
    int32_t mm = __ldg(p.masked_m + lo);
    mm = mm < 0 ? 0 : (mm > p.max_m ? p.max_m : mm);
    t.limit = mm;
    const int32_t left = mm - t.m0;
    t.ntok = left < p.tile_tokens ? left : p.tile_tokens;
    t.base = lo * p.max_m;
  }
  t.valid = t.expert >= 0 && t.expert < p.num_experts && t.ntok > 0;
  return t;
}

// Activation row feeding token slot `slot` of a tile; `p.x_rows` (one past the
// end) for a slot that carries no token, which the TMA reads as zeros.
__device__ __forceinline__ int32_t x_row_of(const GemmParams& p, const TileInfo& t, int32_t slot) {
  if (p.mode == kModeIndexed) {
    const int32_t id = __ldg(p.sorted_ids + t.base + slot);
    const int32_t row = id / p.top_k;
    return (id >= 0 && row < p.x_rows) ? row : p.x_rows;
  }
  if (p.mode == kModeContiguous) return t.base + slot;
  return (t.m0 + slot < t.limit) ? t.base + t.m0 + slot : p.x_rows;
}

// Output row written by token slot `slot`, or -1.
__device__ __forceinline__ int32_t out_row_of(const GemmParams& p, const TileInfo& t, int32_t slot) {
  if (slot >= t.ntok) return -1;
  if (p.mode == kModeIndexed) {
    const int32_t id = __ldg(p.sorted_ids + t.base + slot);
    return (id >= 0 && id < p.out_rows) ? id : -1;
  }
  if (p.mode == kModeContiguous) return t.base + slot;
  return (t.m0 + slot < t.limit) ? t.base + t.m0 + slot : -1;
}

__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Expands one packed word (rows r and r+8, K offsets {2q, 2q+1, 2q+8, 2q+9} of a
// K16 block; humming/kernel/repack.cuh:8-33) into four BF16 pairs
// RN((code - 8) * scale), in tensor-memory store order:
//   out[0] = (row r,   K 2q..2q+1)     out[1] = (row r+8, K 2q..2q+1)
//   out[2] = (row r,   K 2q+8..2q+9)   out[3] = (row r+8, K 2q+8..2q+9)
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t scale_lo, uint32_t scale_hi,
                                             uint32_t* out) {
  constexpr uint32_t kMask = 0x000F000Fu;
  constexpr uint32_t kMagic = 0x43004300u;   // BF16 128.0 in both halves
  constexpr uint32_t kBias = 0x43084308u;    // BF16 136.0 in both halves
  uint32_t v0, v1, v2, v3;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v0) : "r"(w), "r"(kMask), "r"(kMagic));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v1) : "r"(w >> 4), "r"(kMask), "r"(kMagic));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v2) : "r"(w >> 8), "r"(kMask), "r"(kMagic));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v3) : "r"(w >> 12), "r"(kMask), "r"(kMagic));
  out[0] = bf16x2_mul(bf16x2_sub(v0, kBias), scale_lo);  // rows r,   K-half 0
  out[2] = bf16x2_mul(bf16x2_sub(v1, kBias), scale_lo);  // rows r,   K-half 1
  out[1] = bf16x2_mul(bf16x2_sub(v2, kBias), scale_hi);  // rows r+8, K-half 0
  out[3] = bf16x2_mul(bf16x2_sub(v3, kBias), scale_hi);  // rows r+8, K-half 1
}

template <int kDequantGroups>
__global__ void __launch_bounds__(32 * (8 + 4 * kDequantGroups), 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_s,
                  const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Dynamic shared memory: [X stages | W stages | S stages | GemmShared], 1024-aligned.
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t x_stage_bytes = static_cast<uint32_t>(p.mma_n) * 128u;
  const uint32_t stages = static_cast<uint32_t>(p.stages);
  uint8_t* smem_x = smem;
  uint8_t* smem_w = smem_x + stages * x_stage_bytes;
  uint8_t* smem_s = smem_w + stages * kWStageBytes;
  GemmShared& sh = *reinterpret_cast<GemmShared*>(smem_s + stages * kSStageBytes);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  constexpr uint32_t kFirstDequantWarp = 4;
  constexpr uint32_t kFirstEpilogueWarp = 4 + 4 * kDequantGroups;
  const uint32_t d_bufs = p.mma_n <= 128 ? 2u : 1u;
  const uint32_t d_stride = p.mma_n <= 128 ? 128u : 256u;
  const int32_t k_iters = p.k / kBlockK;

  // ------------------------------------------------------------------ setup --
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_s);
    ptx::prefetch_tensormap(&tm_x);
    const uint32_t full_count = p.x_load == kXLoadCpAsync ? 33u : 1u;
    for (uint32_t s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sh.full[s]), full_count);
      ptx::mbar_init(ptx::smem_u32(&sh.empty[s]), 5);
    }
    for (uint32_t a = 0; a < kASlots; ++a) {
      ptx::mbar_init(ptx::smem_u32(&sh.afull[a]), 4);
      ptx::mbar_init(ptx::smem_u32(&sh.aempty[a]), 1);
    }
    for (uint32_t d = 0; d < 2; ++d) {
      ptx::mbar_init(ptx::smem_u32(&sh.dfull[d]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh.dempty[d]), 4);
    }
    sh.abort_flag = 0;
    sh.epilogue_failed = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(&sh.tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  // Token slots no load ever fills must not hold NaN patterns.
  for (uint32_t i = threadIdx.x; i < stages * x_stage_bytes / 16; i += blockDim.x) {
    reinterpret_cast<uint4*>(smem_x)[i] = make_uint4(0, 0, 0, 0);
  }
  // Number of M tiles.
  if (p.mode == kModeMasked) {
    if (threadIdx.x == 0) {
      int32_t acc = 0;
      for (int32_t g = 0; g < p.num_experts; ++g) {
        sh.group_prefix[g] = acc;
        int32_t mm = __ldg(p.masked_m + g);
        mm = mm < 0 ? 0 : (mm > p.max_m ? p.max_m : mm);
        acc += (mm + p.tile_tokens - 1) / p.tile_tokens;
      }
      sh.group_prefix[p.num_experts] = acc;
      sh.m_blocks = acc;
    }
  } else if (p.mode == kModeIndexed) {
    if (threadIdx.x == 0) {
      int32_t padded = __ldg(p.num_tokens_padded);
      padded = padded < 0 ? 0 : (padded > p.sorted_len ? p.sorted_len : padded);
      int32_t blocks = padded / p.tile_tokens;
      sh.m_blocks = blocks > p.expert_len ? p.expert_len : blocks;
    }
  } else {
    if (threadIdx.x == 0) sh.m_blocks = p.m_blocks;
  }
  ptx::fence_proxy_async();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  const uint32_t tmem_base = sh.tmem_base;
  volatile uint32_t* abort_flag = &sh.abort_flag;
  const int32_t tiles = sh.m_blocks * (p.n / kBlockN);
  SegmentIterator iter;
  iter.init(tiles, k_iters, static_cast<int32_t>(gridDim.x), static_cast<int32_t>(blockIdx.x));
  Segment seg;

  if (warp == 0) {
    // -------------------------------------------------------------- producer --
    uint32_t it = 0;
    bool ok = true;
    while (ok && iter.next(seg)) {
      const TileInfo t = decode_tile(p, sh, seg.tile);
      if (!t.valid) continue;
      // Token slots loaded per stage: whole groups of four rows.
      const int32_t load_groups = (t.ntok + 3) >> 2;
      int32_t rows[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int32_t gi = static_cast<int32_t>(lane) + 32 * h;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int32_t slot = gi * 4 + j;
          rows[h][j] = (gi < load_groups && slot < t.ntok) ? x_row_of(p, t, slot) : p.x_rows;
        }
      }
      if (p.x_load == kXLoadCpAsync) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int32_t gi = static_cast<int32_t>(lane) + 32 * h;
          if (gi < load_groups) {
#pragma unroll
            for (int j = 0; j < 4; ++j) sh.x_row[gi * 4 + j] = rows[h][j];
          }
        }
        __syncwarp();
      }
      const uint32_t tx_bytes = kWStageBytes + kSStageBytes +
                                (p.x_load == kXLoadGather4 ? load_groups * 512u : 0u);
      for (int32_t kb = seg.kb; kb < seg.ke; ++kb, ++it) {
        const uint32_t s = it % stages;
        const uint32_t ph = (it / stages) & 1u;
        if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.empty[s]), ph ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        const uint32_t full = ptx::smem_u32(&sh.full[s]);
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(full, tx_bytes);
          ptx::tma_load_2d(ptx::smem_u32(smem_w + s * kWStageBytes), &tm_w, full, 2 * t.n0,
                           t.expert * (p.k / 16) + kb * (kBlockK / 16));
          ptx::tma_load_2d(ptx::smem_u32(smem_s + s * kSStageBytes), &tm_s, full, t.n0,
                           t.expert * (p.k / 32) + kb * (kBlockK / 32));
        }
        __syncwarp();
        const uint32_t xs = ptx::smem_u32(smem_x + s * x_stage_bytes);
        if (p.x_load == kXLoadGather4) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int32_t gi = static_cast<int32_t>(lane) + 32 * h;
            if (gi < load_groups) {
              ptx::tma_gather4(xs + gi * 512u, &tm_x, full, kb * kBlockK, rows[h][0], rows[h][1],
                               rows[h][2], rows[h][3]);
            }
          }
        } else {
          // 8 sixteen-byte chunks per row, XOR-swizzled by (row & 7) like the TMA would.
          const int32_t chunks = load_groups * 4 * 8;
          for (int32_t c = lane; c < chunks; c += 32) {
            const int32_t r = c >> 3, ch = c & 7;
            const int32_t row = sh.x_row[r];
            const bool valid = row < p.x_rows;
            const __nv_bfloat16* src =
                p.x + static_cast<size_t>(valid ? row : 0) * p.k + kb * kBlockK + ch * 8;
            ptx::cp_async_16(xs + r * 128u + ((ch ^ (r & 7)) << 4), src, valid);
          }
          ptx::cp_async_wait_all();
          ptx::fence_proxy_async();
          ptx::mbar_arrive(full);
        }
      }
    }
    if (!ok && lane == 0) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, kStatusProducerTimeout);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer --
    if (lane == 0) {
      const uint32_t idesc = ptx::idesc_bf16_f32(kBlockN, static_cast<uint32_t>(p.mma_n));
      uint32_t it = 0, segc = 0;
      bool ok = true;
      while (ok && iter.next(seg)) {
        const TileInfo t = decode_tile(p, sh, seg.tile);
        if (!t.valid) continue;
        const uint32_t d = segc % d_bufs;
        const uint32_t dph = (segc / d_bufs) & 1u;
        if (!ptx::mbar_wait(ptx::smem_u32(&sh.dempty[d]), dph ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_addr = tmem_base + kDCol0 + d * d_stride;
        for (int32_t kb = seg.kb; kb < seg.ke; ++kb, ++it) {
          const uint32_t s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          const uint32_t a = it % kASlots;
          const uint32_t aph = (it / kASlots) & 1u;
          if (!ptx::mbar_wait(ptx::smem_u32(&sh.full[s]), ph, abort_flag) ||
              !ptx::mbar_wait(ptx::smem_u32(&sh.afull[a]), aph, abort_flag)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t a_addr = tmem_base + a * kAColsPerSlot;
          const uint32_t xs = ptx::smem_u32(smem_x + s * x_stage_bytes);
#pragma unroll
          for (int j = 0; j < kBlockK / 16; ++j) {
            ptx::mma_ts(d_addr, a_addr + 8 * j, ptx::smem_desc_k_sw128(xs + 32 * j), idesc,
                        (kb > seg.kb || j > 0) ? 1u : 0u);
          }
          ptx::mma_commit(ptx::smem_u32(&sh.empty[s]));
          ptx::mma_commit(ptx::smem_u32(&sh.aempty[a]));
        }
        if (!ok) break;
        ptx::mma_commit(ptx::smem_u32(&sh.dfull[d]));
        ++segc;
      }
      if (!ok) {
        sh.abort_flag = 1;
        if (p.status) atomicOr(p.status, kStatusMmaTimeout);
      }
    }
    __syncwarp();
  } else if (warp >= kFirstDequantWarp && warp < kFirstEpilogueWarp) {
    // --------------------------------------------------------------- dequant --
    const uint32_t group = (warp - kFirstDequantWarp) >> 2;
    const uint32_t q = warp & 3;  // TMEM lane quarter == 32 weight rows
    // Byte offset of this thread's two packed words (slabs 2(q&1), 2(q&1)+1 of the
    // 64-row chunk q>>1) inside one K16 row of the stage, and of its four scales.
    const uint32_t w_off = (q >> 1) * 512u + lane * 16u + (q & 1) * 8u;
    const uint32_t s_off = (q >> 1) * 128u + (lane >> 2) * 16u + (q & 1) * 8u;
    uint32_t it = 0;
    bool ok = true;
    while (ok && iter.next(seg)) {
      const TileInfo t = decode_tile(p, sh, seg.tile);
      if (!t.valid) continue;
      for (int32_t kb = seg.kb; kb < seg.ke; ++kb, ++it) {
        if (it % kDequantGroups != group) continue;
        const uint32_t s = it % stages;
        const uint32_t ph = (it / stages) & 1u;
        const uint32_t a = it % kASlots;
        const uint32_t aph = (it / kASlots) & 1u;
        if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.full[s]), ph, abort_flag)) {
          ok = false;
          break;
        }
        uint2 words[kBlockK / 16];
        uint2 scales[kBlockK / 32];
        const uint8_t* wsrc = smem_w + s * kWStageBytes + w_off;
        const uint8_t* ssrc = smem_s + s * kSStageBytes + s_off;
#pragma unroll
        for (int j = 0; j < kBlockK / 16; ++j) {
          words[j] = *reinterpret_cast<const uint2*>(wsrc + j * 1024);
        }
#pragma unroll
        for (int g = 0; g < kBlockK / 32; ++g) {
          scales[g] = *reinterpret_cast<const uint2*>(ssrc + g * 256);
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sh.empty[s]));

        uint32_t lo[16], hi[16];  // lanes 0-15 (first slab) and 16-31 (second slab) of the quarter
#pragma unroll
        for (int j = 0; j < kBlockK / 16; ++j) {
          const uint2 sc = scales[j >> 1];
          // sc.x = {slab A row r, slab A row r+8}; sc.y = same for slab B.
          const uint32_t a_lo = __byte_perm(sc.x, 0, 0x1010);
          const uint32_t a_hi = __byte_perm(sc.x, 0, 0x3232);
          const uint32_t b_lo = __byte_perm(sc.y, 0, 0x1010);
          const uint32_t b_hi = __byte_perm(sc.y, 0, 0x3232);
          dequant_word(words[j].x, a_lo, a_hi, lo + 4 * j);
          dequant_word(words[j].y, b_lo, b_hi, hi + 4 * j);
        }
        if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.aempty[a]), aph ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t a_addr = tmem_base + ((q * 32u) << 16) + a * kAColsPerSlot;
        ptx::tmem_st_16x128b_x8(a_addr, lo);
        ptx::tmem_st_16x128b_x8(a_addr + (16u << 16), hi);
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sh.afull[a]));
      }
    }
    if (!ok && lane == 0) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, kStatusDequantTimeout);
    }
  } else if (warp >= kFirstEpilogueWarp) {
    // -------------------------------------------------------------- epilogue --
    const uint32_t q = warp & 3;
    const uint32_t et = threadIdx.x - kFirstEpilogueWarp * 32;  // 0..127 == TMEM lane
    const uint32_t row_in_tile = q * 32 + lane;                 // == et
    uint32_t segc = 0;
    bool ok = true;
    const size_t ws_slot = static_cast<size_t>(kBlockN) * p.mma_n;
    while (ok && iter.next(seg)) {
      const TileInfo t = decode_tile(p, sh, seg.tile);
      if (!t.valid) continue;
      const uint32_t d = segc % d_bufs;
      const uint32_t dph = (segc / d_bufs) & 1u;
      ptx::named_bar_sync(1, 128);  // previous segment's out_row readers are done
      for (int32_t c = et; c < p.mma_n; c += 128) sh.out_row[c] = out_row_of(p, t, c);
      int32_t lock_ok = 1;
      if (seg.type == kSegOwner && et == 0) {
        // Wait (bounded) until every other slice of this tile has published its partial.
        const int* lock = p.locks + blockIdx.x;
        lock_ok = 0;
        for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
          if (ptx::ld_acquire(lock) >= seg.peer) {
            lock_ok = 1;
            break;
          }
          __nanosleep(64);
        }
        if (!lock_ok && p.status) atomicOr(p.status, kStatusLockTimeout);
      }
      // The four warps must agree on the outcome before any of them leaves the loop,
      // or the named barriers below would wait for warps that are gone.
      if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.dfull[d]), dph, abort_flag) && lane == 0) {
        sh.epilogue_failed = 1;
      }
      ptx::tc_fence_after();
      ptx::named_bar_sync(1, 128);  // out_row filled, lock observed, verdict published
      if (sh.epilogue_failed != 0) {
        ok = false;
        break;
      }
      const uint32_t d_addr = tmem_base + ((q * 32u) << 16) + kDCol0 + d * d_stride;
      __nv_bfloat16* out_col = p.out + t.n0 + row_in_tile;
      for (int32_t c0 = 0; c0 < p.mma_n; c0 += 16) {
        uint32_t v[16];
        ptx::tmem_ld_32x32b_x16(d_addr + c0, v);
        ptx::tmem_wait_ld();
        if (seg.type == kSegContrib) {
          float* dst = p.workspace + blockIdx.x * ws_slot + static_cast<size_t>(c0) * kBlockN + et;
#pragma unroll
          for (int j = 0; j < 16; ++j) __stcg(dst + j * kBlockN, __uint_as_float(v[j]));
          continue;
        }
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(v[j]);
        if (seg.type == kSegOwner) {
          for (int32_t peer = 1; peer <= seg.peer; ++peer) {
            const float* src = p.workspace + (blockIdx.x + peer) * ws_slot +
                               static_cast<size_t>(c0) * kBlockN + et;
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] += __ldcg(src + j * kBlockN);
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int32_t row = sh.out_row[c0 + j];
          if (row >= 0) out_col[static_cast<size_t>(row) * p.n] = __float2bfloat16_rn(acc[j]);
        }
      }
      // Release the accumulator buffer to the MMA issuer.
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sh.dempty[d]));
      if (seg.type == kSegContrib) {
        __threadfence();
        ptx::named_bar_sync(1, 128);
        if (et == 0) ptx::red_release_add(p.locks + seg.peer, 1);
      } else if (seg.type == kSegOwner) {
        ptx::named_bar_sync(1, 128);
        if (et == 0) p.locks[blockIdx.x] = 0;
      }
      ++segc;
    }
    if (!ok && lane == 0) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, kStatusEpilogueTimeout);
    }
  }

  // --------------------------------------------------------------- teardown --
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace chord
