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
// 128-byte swizzle: one tiled TMA box per K half where a tile's rows are
// consecutive, a cp.async gather by two helper warps (or, selectable, TMA
// tile::gather4) where sorted_ids names them.
//
// Two shared-memory rings decouple the HBM stream from the token side: a
// weight/scale stage is free again as soon as the dequant warps have read it
// into registers (its content lives on in tensor memory), so that ring can be
// deep enough (20+ stages of 9 KB) to cover HBM latency, while an activation
// stage stays until the MMAs that read it have completed.
//
// The single-thread issue loops (TMA, MMA) are kept free of divisions and
// descriptor rebuilds: one lone thread retires a dependent instruction only
// every few cycles, and at decode sizes a K16 MMA has roughly 45 cycles of HBM
// time to hide behind.
//
// Warp roles (one CTA per SM, persistent):
//   warp 0            producer: TMA for packed weights
//   warp 1            producer: TMA for scales
//   warps 2-3         activations: tiled TMA (one thread), cp.async gather (64 threads)
//                     or TMA gather4 (one warp); warp 2 also allocates tensor memory
//   warps 4-7         MMA issuers, one thread each; issuer i takes the stages
//                     with index = i modulo the issuer count and owns one accumulator
//   warps 8..8+4G-1   G dequant groups of four warps (one per TMEM lane quarter)
//   last four warps   epilogue: TMEM -> registers -> BF16 -> global, plus the
//                     stream-K reduction through `locks` and the FP32 workspace
//
// Why several issuers: one thread can issue a tcgen05.mma only every ~56 cycles
// (measured), while a 128x16 tile of packed weights arrives from HBM every ~45
// cycles per SM.  With small token tiles (decode) the stages are therefore
// dealt to 2 or 4 issuers in different warps, each accumulating into its own
// TMEM columns; the epilogue adds the accumulators in issuer order, so the
// result does not depend on timing.  Large token tiles use a single issuer.
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
// How activation rows reach shared memory.  Consecutive rows (contiguous,
// masked) always use one tiled TMA box per 64-wide K half; the routed rows of
// `indexed` are gathered by two helper warps with cp.async (default) or by the
// producer with TMA tile::gather4.
enum XLoadMode : int32_t { kXLoadCpAsync = 0, kXLoadGather4 = 1, kXLoadTiled = 2 };

// Device status bits (OR-ed into *status by a kernel that gave up on a wait).
enum StatusBits : int32_t {
  kStatusProducerTimeout = 1,
  kStatusMmaTimeout = 2,
  kStatusDequantTimeout = 4,
  kStatusEpilogueTimeout = 8,
  kStatusLockTimeout = 16,
};

constexpr int kBlockN = 128;      // weight rows per tile (MMA M)
constexpr int kBlockK = 128;      // K elements per pipeline stage (two 64-wide swizzle atoms)
constexpr int kMaxWStages = 24;   // ring of packed-weight + scale stages
constexpr int kMaxXStages = 8;    // ring of activation stages
// Tensor-memory ring for the dequantised A operand: `a_stages` stages of 64 columns,
// each handed over in two halves of one 64-wide K half (32 columns), so that the
// MMAs of a stage's first half are issued while its second half is still being
// dequantised.  The ring takes the columns the accumulators leave free (4 stages next
// to 256 accumulator columns, 6 next to 128): the deeper it is, the further the
// dequant warps run ahead of the MMA issuers, which hides the barrier round trips
// between them.
constexpr int kMaxAStages = 8;
constexpr int kAColsPerStage = kBlockK / 2;
constexpr int kHelperThreads = 64;  // warps 2-3: activation gather for `indexed`
constexpr int kTmemCols = 512;
constexpr int kMaxTileTokens = 256;
constexpr int kMaxGroups = 512;   // masked: prefix table capacity
constexpr int kMaxMTiles = 2048;  // contiguous: 128-row blocks of the activation tensor
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
  int32_t run_part;     // contiguous: 0 = every block; 1 = only the blocks left over when each expert's run of consecutive 128-row blocks is cut into pairs (single-block experts, last block of an odd run); 2 = only the pairs
  int32_t x_box_rows;   // tiled activation loads: rows per TMA box
  int32_t sorted_len;   // indexed: capacity of sorted_ids
  int32_t expert_len;   // indexed: capacity of expert_ids
  int32_t w_stages;     // depth of the weight/scale ring
  int32_t x_stages;     // depth of the activation ring
  int32_t issuers;      // 1, 2 or 4 MMA issuers (and accumulators)
  int32_t ksplit;       // single-issuer layouts: a second issuer takes the second K half of tiles of <= 128 tokens
  int32_t fuse_silu;    // 1 = gate_up with SiLU*mul in the epilogue: a tile is gate block j and up block j (row N/2 + 128 j), out is [rows, N/2]
  int32_t npair;        // 1 = a tile is two neighbouring 128-row weight blocks sharing one activation stage (tiles of <= 128 tokens)
  int32_t pair;         // 1 = launched as clusters of two CTAs: a tile is two neighbouring 128-row weight blocks, one per CTA, multiplied by one tcgen05.mma.cta_group::2 stream; each CTA loads half of the tile's token rows
  int32_t a_stages;     // depth of the TMEM A ring; accumulators start at column 64 * a_stages
  int32_t num_locks;
  int32_t slot_ordered; // host side only (indexed): row s of x is the row of routing slot s, so the rows load as consecutive boxes without a copy
  int32_t pdl;          // host side only: launch with the programmatic stream-serialization attribute
  int32_t lock_spins;   // polls (64 ns apart) a stream-K owner spends on its lock word before it gives up
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_tokens_padded;
  const int32_t* m_indices;
  const int32_t* masked_m;
  const __nv_bfloat16* x;
  __nv_bfloat16* out;
  void* const* out_row_ptr;  // optional (indexed): out_row_ptr[id] = address of the row that receives routed id's result
  float* workspace;     // grid * 128 * mma_n floats
  int32_t* locks;
  int32_t* status;
};

struct TileInfo {
  int32_t n0;      // first weight row
  int32_t expert;
  int32_t ntok;    // token slots of the tile that carry a row (one past the last one)
  int32_t rows;    // token slots whose output rows the tile writes (contiguous: whole blocks)
  int32_t base;    // indexed: first sorted_ids slot; contiguous: first row; masked: first row of the group
  int32_t m0;      // masked: first row inside the group
  int32_t limit;   // masked: masked_m of the group
  int32_t mma_n;   // MMA N of this tile: ntok rounded up to 16
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

  __host__ __device__ void init(int32_t tiles, int32_t k_iters, int32_t grid_, int32_t cta_) {
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
    // No slice shorter than eight k-blocks (unless the whole tail is): a finer split costs
    // more in partial sums and per-slice set-up than the extra parallelism returns.
    const int64_t slices = units / 8 > 0 ? units / 8 : (units > 0 ? 1 : 0);
    geff = slices < grid ? static_cast<int32_t>(slices) : grid;
    if (cta < geff) {
      u0 = cta * units / geff;
      u1 = (cta + 1) * units / geff;
    } else {
      u0 = u1 = 0;
    }
  }

  __host__ __device__ int32_t cta_of_unit(int64_t u) const {
    return static_cast<int32_t>(((u + 1) * geff - 1) / units);
  }

  __host__ __device__ bool next(Segment& s) {
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
  uint64_t wfull[kMaxWStages];   // weights + scales landed        (2 producer arrivals + bytes)
  uint64_t wempty[kMaxWStages];  // dequant warps have read them   (4 arrivals)
  uint64_t xfull[kMaxXStages];   // activations landed
  uint64_t xempty[kMaxXStages];  // the stage's MMAs have completed (1 commit)
  uint64_t afull[2 * kMaxAStages];   // per K half: dequantised operand stored (4 arrivals)
  uint64_t aempty[2 * kMaxAStages];  // per K half: its MMAs have completed (1 commit)
  uint64_t dfull[2];
  uint64_t dempty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  int32_t m_blocks;
  volatile uint32_t epilogue_failed;
  int32_t x_slots;                   // helpers: token slots of the current tile that carry a row
  int32_t out_row[kMaxTileTokens];   // epilogue: output row per token slot, -1 = skip
  __align__(16) __nv_bfloat16 stage[8][16][32];  // epilogue: per-warp transpose buffer (second set: the pair kernel's second epilogue group)
  int32_t x_row[kMaxTileTokens];     // producer (cp.async variant): activation row per slot
  int32_t group_prefix[kMaxGroups + 1];  // masked: first M tile of each group
  // contiguous: M tiles after merging neighbouring 128-row blocks of one expert:
  // expert | first block << 15 | (256 rows ? 1 : 0) << 31
  uint32_t mtile[kMaxMTiles];
  // contiguous, indexed: token slots of each M tile that carry a row (padding rows at
  // the end of an expert's run, sentinels at the end of a routing block, do not): the
  // tile's MMA runs with N = that count rounded up to 16, not with the full block.
  uint16_t tile_rows[kMaxMTiles];
  int32_t have_tile_rows;
};

__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, const GemmShared& sh,
                                                int32_t tile, uint32_t rank = 0) {
  TileInfo t;
  // With `npair` a tile spans two neighbouring 128-row weight blocks (n0 and n0 + 128).
  // With fused SiLU*mul the two blocks are gate block n0 and up block N/2 + n0.
  // With `pair` the two blocks belong to the two CTAs of the cluster: n0 is this CTA's.
  const int32_t wide = p.npair | p.pair;
  const int32_t n_blocks = p.fuse_silu ? (p.n >> 1) / kBlockN : p.n / (kBlockN << wide);
  const int32_t mb = tile / n_blocks;
  t.n0 = (tile - mb * n_blocks) * (p.fuse_silu ? kBlockN : (kBlockN << wide)) +
         static_cast<int32_t>(rank) * kBlockN;
  t.m0 = 0;
  t.limit = 0;
  t.mma_n = p.mma_n;
  if (p.mode == kModeIndexed) {
    t.expert = __ldg(p.expert_ids + mb);
    t.ntok = sh.have_tile_rows ? static_cast<int32_t>(sh.tile_rows[mb]) : p.tile_tokens;
    t.rows = t.ntok;
    t.base = mb * p.tile_tokens;
  } else if (p.mode == kModeContiguous) {
    const uint32_t info = sh.mtile[mb];
    t.expert = static_cast<int32_t>(info & 0x7FFFu);
    t.rows = (info >> 31) ? 256 : 128;
    t.ntok = static_cast<int32_t>(sh.tile_rows[mb]);
    t.base = static_cast<int32_t>((info >> 15) & 0xFFFFu) * 128;
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
    t.rows = t.ntok;
    t.base = lo * p.max_m;
  }
  t.mma_n = (t.ntok + 15) & ~15;
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
  if (slot >= t.rows) return -1;
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

// First half of dequant_word: the four BF16 pairs (code - 8), exact, in the same order;
// the multiplication by the scales is left to tmem_st_16x128b_x8_scaled.
__device__ __forceinline__ void unbias_word(uint32_t w, uint32_t* out) {
  constexpr uint32_t kMask = 0x000F000Fu;
  constexpr uint32_t kMagic = 0x43004300u;
  constexpr uint32_t kBias = 0x43084308u;
  uint32_t v0, v1, v2, v3;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v0) : "r"(w), "r"(kMask), "r"(kMagic));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v1) : "r"(w >> 4), "r"(kMask), "r"(kMagic));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v2) : "r"(w >> 8), "r"(kMask), "r"(kMagic));
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v3) : "r"(w >> 12), "r"(kMask), "r"(kMagic));
  out[0] = bf16x2_sub(v0, kBias);
  out[2] = bf16x2_sub(v1, kBias);
  out[1] = bf16x2_sub(v2, kBias);
  out[3] = bf16x2_sub(v3, kBias);
}

// Ring position advanced without divisions (a lone issuing thread pays ~100
// cycles for an integer division by a runtime value).
struct StageCursor {
  uint32_t s = 0, ph = 0;
  __device__ __forceinline__ void advance(uint32_t stages) {
    if (++s == stages) {
      s = 0;
      ph ^= 1u;
    }
  }
  // Any distance, without a division (a few subtractions per tile at most).
  __device__ __forceinline__ void advance_by(uint32_t n, uint32_t stages) {
    s += n;
    while (s >= stages) {
      s -= stages;
      ph ^= 1u;
    }
  }
};

// Activation ring cut into sub-slots of 128 token rows (both 64-wide K halves, 32 KB).
// A stage of a tile of at most 128 tokens takes one sub-slot, a 256-token stage an
// aligned pair (one sub-slot may be skipped to align), so that a launch mixing small and
// large tiles gives the small ones a ring twice as deep.  Every party keeps a cursor
// and one phase bit per sub-slot barrier of its own; all walk the same tile sequence.
// A pair is tracked by the barriers of its even sub-slot alone (the MMA issuer is the
// critical path of large tiles: no second wait or commit for it); the odd sub-slot's
// barriers keep the state of its last use on its own, which the loader checks without
// consuming it before it overwrites the memory.  That use is never outstanding when the
// odd sub-slot is next taken on its own, because the ring always passes through the even
// one (and so waits for the pair) first.
struct XSubRing {
  uint32_t next = 0;
  uint32_t phases = 0;
  __device__ __forceinline__ uint32_t take(bool pair, uint32_t count) {
    if (pair && (next & 1u)) next = next + 1u == count ? 0u : next + 1u;
    const uint32_t first = next;
    next += pair ? 2u : 1u;
    if (next >= count) next -= count;
    return first;
  }
  __device__ __forceinline__ uint32_t phase(uint32_t slot) const { return (phases >> slot) & 1u; }
  __device__ __forceinline__ void flip(uint32_t slot) { phases ^= 1u << slot; }
};

template <int kDequantGroups, bool kPair>
__global__ void __launch_bounds__(32 * (12 + 4 * kDequantGroups), 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_s,
                  const __grid_constant__ CUtensorMap tm_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Dynamic shared memory: [X ring | W ring | S ring | GemmShared], 1024-aligned.
  // One X stage holds two K halves, each mma_n rows of 128 bytes.
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  // `pair`: this CTA is rank 0 (leader: issues the MMAs for both) or 1 of a cluster of two
  // and holds half of a tile's token rows.
  // (A kernel that contains cta_group::2 instructions can only be launched as clusters of
  // two, hence an instantiation of its own.)
  constexpr bool pair = kPair;
  uint32_t rank = 0;
  if constexpr (kPair) rank = ptx::cluster_ctarank();
  const uint32_t x_half_bytes = (static_cast<uint32_t>(p.mma_n) >> p.pair) * 128u;
  const uint32_t x_stage_bytes = 2u * x_half_bytes;
  const uint32_t w_stages = static_cast<uint32_t>(p.w_stages);
  const uint32_t x_stages = static_cast<uint32_t>(p.x_stages);
  uint8_t* smem_x = smem;
  uint8_t* smem_w = smem_x + x_stages * x_stage_bytes;
  uint8_t* smem_s = smem_w + w_stages * kWStageBytes;
  GemmShared& sh = *reinterpret_cast<GemmShared*>(smem_s + w_stages * kSStageBytes);

  // Read back through a shuffle so that the compiler knows the warp index (and what is
  // derived from it: roles, ring positions, barrier and tensor-memory addresses) to be
  // the same in all lanes and keeps them in uniform registers.
  const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const uint32_t lane = threadIdx.x & 31;
  constexpr uint32_t kFirstIssuerWarp = 4;
  constexpr uint32_t kFirstDequantWarp = 8;
  constexpr uint32_t kFirstEpilogueWarp = 8 + 4 * kDequantGroups;
  // Accumulators: `ni` issuers x `d_bufs` buffers of `d_cols` columns each in the
  // 256 TMEM columns after the A ring; buffer d of issuer i starts at column
  // 64 * a_stages + (d * ni + i) * d_cols.
  // With `ksplit` (layouts whose token tile exceeds 64) there are two issuers that do
  // not take turns: on tiles of at most 128 tokens issuer 0 takes the first 64-wide K
  // half of every stage and issuer 1 the second, each into its own 128-column
  // accumulator; on larger tiles issuer 0 does both halves into all 256 columns and
  // issuer 1 only keeps the barriers' phases moving.  One tcgen05.mma costs its issuing
  // thread ~100 cycles on a busy SM whatever its size, so a lone issuer caps small
  // tiles at ~900 cycles per stage.
  const bool ksplit = p.ksplit != 0;
  // `npair`: two issuers as well, but issuer i (with dequant group i) owns the weight block
  // n0 + 128 i of the tile: weight/scale stages alternate between the two blocks, one
  // activation stage serves both, and the two accumulators are two output blocks instead
  // of two partial sums.  An activation tile then crosses from L2 to the SM once per 256
  // weight rows instead of once per 128: with 128-row tiles the kernel was bound by that
  // traffic (about 10 TB/s between L2 and the SMs), not by the tensor pipe.
  const bool npair = p.npair != 0;
  const int32_t w_per_kb = npair ? 2 : 1;  // weight/scale ring entries per K block
  // 256-token layouts with consecutive activation rows: sub-slot ring (see XSubRing).
  const bool subslots = ksplit && p.x_load == kXLoadTiled && p.mma_n == 256;
  constexpr uint32_t kSubBytes = 128u * 256u;
  const uint32_t ni = ksplit ? 2u : static_cast<uint32_t>(p.issuers);
  const uint32_t d_cols = ksplit ? 128u : static_cast<uint32_t>(p.mma_n);
  const uint32_t a_stages = static_cast<uint32_t>(p.a_stages);
  const uint32_t d_col0 = a_stages * kAColsPerStage;
  const uint32_t d_bufs = 2u * ni * d_cols <= kTmemCols - d_col0 ? 2u : 1u;
  const int32_t k_iters = (p.k + kBlockK - 1) / kBlockK;
  const bool k_tail_half = (p.k % kBlockK) != 0;  // last stage carries 64 K values only
  // Consecutive activation rows need one loading thread (warp 2) instead of two gathering
  // warps, and at most two issuers: warp 0 then feeds both the weight and the scale ring,
  // the issuers sit in warps 1 and 3, and warps 4-7 are a second group of epilogue warps
  // taking every other 16-column chunk.  Accumulators of 128 columns and more are
  // single-buffered, so the tensor core idles while a tile is drained: with K = 2048 the
  // four-warp drain was a quarter of the time of a two-block tile.
  const bool tiled_roles = kPair || (p.x_load == kXLoadTiled && ni <= 2u);
  const uint32_t epi_threads = tiled_roles ? 256u : 128u;

  // ------------------------------------------------------------------ setup --
  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_w);
    ptx::prefetch_tensormap(&tm_s);
    ptx::prefetch_tensormap(&tm_x);
    for (uint32_t s = 0; s < w_stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sh.wfull[s]), 2);
      ptx::mbar_init(ptx::smem_u32(&sh.wempty[s]), 4);
    }
    // One arrival per gathering warp, or one transaction-count arrival.
    const uint32_t xfull_count = p.x_load == kXLoadCpAsync ? kHelperThreads / 32 : 1u;
    for (uint32_t s = 0; s < (subslots ? 2u * x_stages : x_stages); ++s) {
      ptx::mbar_init(ptx::smem_u32(&sh.xfull[s]), xfull_count);
      ptx::mbar_init(ptx::smem_u32(&sh.xempty[s]), (ksplit || npair) ? 2 : 1);
    }
    // `pair`: the leader's afull / dempty collect the arrivals of both CTAs' warps (four
    // dequant warps per stage, eight epilogue warps per CTA); the leader's commits reach
    // xempty / aempty / dfull of both CTAs.
    for (uint32_t a = 0; a < 2 * a_stages; ++a) {
      ptx::mbar_init(ptx::smem_u32(&sh.afull[a]), pair ? 8 : 4);
      ptx::mbar_init(ptx::smem_u32(&sh.aempty[a]), 1);
    }
    for (uint32_t d = 0; d < 2; ++d) {
      ptx::mbar_init(ptx::smem_u32(&sh.dfull[d]), ni);
      ptx::mbar_init(ptx::smem_u32(&sh.dempty[d]), (tiled_roles ? 8u : 4u) << p.pair);
    }
    sh.abort_flag = 0;
    sh.epilogue_failed = 0;
    ptx::fence_barrier_init();
  }
  if (warp == 2) {
    if constexpr (kPair) {
      ptx::tmem_alloc_pair(ptx::smem_u32(&sh.tmem_base), kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(&sh.tmem_base), kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  // Token slots no load ever fills must not hold NaN patterns.
  for (uint32_t i = threadIdx.x; i < x_stages * x_stage_bytes / 16; i += blockDim.x) {
    reinterpret_cast<uint4*>(smem_x)[i] = make_uint4(0, 0, 0, 0);
  }
  // Up to here nothing an earlier kernel of the stream may still be writing has been
  // read: with programmatic dependent launch the set-up above overlaps that kernel's tail.
  ptx::grid_dependency_wait();
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
      sh.have_tile_rows = sh.m_blocks <= kMaxMTiles ? 1 : 0;
    }
    __syncthreads();
    // One warp per routing block: one past the last slot whose id names a row.
    if (sh.have_tile_rows) {
      for (int32_t b = static_cast<int32_t>(warp); b < sh.m_blocks; b += static_cast<int32_t>(blockDim.x >> 5)) {
        int32_t last = 0;
        for (int32_t i = static_cast<int32_t>(lane); i < p.tile_tokens; i += 32) {
          const int32_t id = __ldg(p.sorted_ids + b * p.tile_tokens + i);
          if (id >= 0 && id < p.out_rows && id / p.top_k < p.x_rows) last = i + 1;
        }
        last = __reduce_max_sync(0xffffffffu, last);
        if (lane == 0) sh.tile_rows[b] = static_cast<uint16_t>(last);
      }
    }
  } else {
    // Expert of every 128-row block (its first row names it), then one thread merges
    // neighbouring blocks of one expert into 256-token tiles (the MMA runs at full
    // rate only with N = 256) and drops padding blocks.  In place: the write position
    // never passes the read position.
    for (int32_t i = threadIdx.x; i < p.m_blocks; i += blockDim.x) {
      sh.mtile[i] = static_cast<uint32_t>(__ldg(p.m_indices + i * 128));
    }
    // One warp per block: one past its last row that belongs to an expert.
    for (int32_t b = static_cast<int32_t>(warp); b < p.m_blocks; b += static_cast<int32_t>(blockDim.x >> 5)) {
      int32_t last = 0;
#pragma unroll
      for (int32_t j = 0; j < 4; ++j) {
        const int32_t i = 32 * j + static_cast<int32_t>(lane);
        if (__ldg(p.m_indices + b * 128 + i) >= 0) last = i + 1;
      }
      last = __reduce_max_sync(0xffffffffu, last);
      if (lane == 0) sh.tile_rows[b] = static_cast<uint16_t>(last);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int32_t count = 0;
      int32_t run_start = 0, run_end = 0;  // the current expert's run of blocks
      for (int32_t i = 0; i < p.m_blocks;) {
        const int32_t e = static_cast<int32_t>(sh.mtile[i]);
        if (e < 0 || e >= p.num_experts) {
          ++i;
          continue;
        }
        if (i >= run_end) {
          run_start = i;
          run_end = i + 1;
          while (run_end < p.m_blocks && static_cast<int32_t>(sh.mtile[run_end]) == e) ++run_end;
        }
        if (p.run_part != 0) {
          // Pairs are counted from the start of the run; an odd run leaves its last block.
          const bool in_pair = i - run_start < ((run_end - run_start) & ~1);
          if (in_pair != (p.run_part == 2)) {
            i += in_pair ? 2 : 1;
            continue;
          }
        }
        const bool merged = p.tile_tokens == 256 && i + 1 < run_end;
        sh.tile_rows[count] = merged ? static_cast<uint16_t>(128 + sh.tile_rows[i + 1]) : sh.tile_rows[i];
        sh.mtile[count++] = static_cast<uint32_t>(e) | (static_cast<uint32_t>(i) << 15) |
                            (merged ? 0x80000000u : 0u);
        i += merged ? 2 : 1;
      }
      sh.m_blocks = count;
    }
  }
  ptx::fence_proxy_async();
  ptx::tc_fence_before();
  __syncthreads();
  // the peer's barriers must be initialised before anything arrives on them
  if constexpr (kPair) ptx::cluster_sync();
  ptx::tc_fence_after();
  ptx::grid_launch_dependents();

  const uint32_t tmem_base = __shfl_sync(0xffffffffu, sh.tmem_base, 0);  // uniform, see `warp`
  volatile uint32_t* abort_flag = &sh.abort_flag;
  // Offset that turns a shared-memory address of this CTA into the cluster address of the
  // same location in the leader (rank 0).
  const uint32_t sh_addr = ptx::smem_u32(&sh);
  uint32_t to_leader = 0;
  if constexpr (kPair) to_leader = ptx::map_to_cta(sh_addr, 0) - sh_addr;
  const int32_t tiles = __shfl_sync(0xffffffffu, sh.m_blocks, 0) *
                        (p.fuse_silu ? (p.n >> 1) / kBlockN : p.n / (kBlockN << (p.npair | p.pair)));
  // Both CTAs of a pair walk the same sequence of tiles.
  SegmentIterator iter;
  iter.init(tiles, k_iters, static_cast<int32_t>(gridDim.x >> p.pair),
            static_cast<int32_t>(blockIdx.x >> p.pair));
  Segment seg;

  if (warp == 0 && tiled_roles) {
    // ------------------------------ producer of both rings (packed weights, scales) --
    if (lane == 0) {
      StageCursor cur;
      bool ok = true;
      while (ok && iter.next(seg)) {
        const TileInfo t = decode_tile(p, sh, seg.tile, rank);
        if (!t.valid) continue;
        // to the tile's second weight block: the next 128 rows, or the up rows of a fused gate_up
        const int32_t block_step = p.fuse_silu ? (p.n >> 1) : kBlockN;
        int32_t w_row = t.expert * (p.k / 16) + seg.kb * (kBlockK / 16);
        int32_t s_row = t.expert * (p.k / 32) + seg.kb * (kBlockK / 32);
        for (int32_t kb = seg.kb; ok && kb < seg.ke; ++kb) {
          for (int32_t sub = 0; sub < w_per_kb; ++sub) {
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.wempty[cur.s]), cur.ph ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            const uint32_t full = ptx::smem_u32(&sh.wfull[cur.s]);
            ptx::mbar_arrive_expect_tx(full, kWStageBytes);
            ptx::tma_load_2d(ptx::smem_u32(smem_w + cur.s * kWStageBytes), &tm_w, full,
                             2 * (t.n0 + sub * block_step), w_row);
            ptx::mbar_arrive_expect_tx(full, kSStageBytes);
            ptx::tma_load_2d(ptx::smem_u32(smem_s + cur.s * kSStageBytes), &tm_s, full,
                             t.n0 + sub * block_step, s_row);
            cur.advance(w_stages);
          }
          w_row += kBlockK / 16;
          s_row += kBlockK / 32;
        }
      }
      if (!ok) {
        sh.abort_flag = 1;
        if (p.status) atomicOr(p.status, kStatusProducerTimeout);
      }
    }
    __syncwarp();
  } else if (!tiled_roles && (warp == 0 || warp == 1)) {
    // ------------------------- producers: packed weights (warp 0), scales (warp 1) --
    if (lane == 0) {
      const bool weights = warp == 0;
      const CUtensorMap* map = weights ? &tm_w : &tm_s;
      uint8_t* ring = weights ? smem_w : smem_s;
      const uint32_t stage_bytes = weights ? kWStageBytes : kSStageBytes;
      const int32_t rows_per_stage = weights ? kBlockK / 16 : kBlockK / 32;
      const int32_t rows_per_expert = weights ? p.k / 16 : p.k / 32;
      StageCursor cur;
      bool ok = true;
      while (ok && iter.next(seg)) {
        const TileInfo t = decode_tile(p, sh, seg.tile, rank);
        if (!t.valid) continue;
        const int32_t col = weights ? 2 * t.n0 : t.n0;
        // to the tile's second weight block: the next 128 rows, or the up rows of a fused gate_up
        const int32_t block_step = p.fuse_silu ? (p.n >> 1) : kBlockN;
        const int32_t col_step = weights ? 2 * block_step : block_step;
        int32_t row = t.expert * rows_per_expert + seg.kb * rows_per_stage;
        for (int32_t kb = seg.kb; ok && kb < seg.ke; ++kb) {
          for (int32_t sub = 0; sub < w_per_kb; ++sub) {
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.wempty[cur.s]), cur.ph ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            const uint32_t full = ptx::smem_u32(&sh.wfull[cur.s]);
            ptx::mbar_arrive_expect_tx(full, stage_bytes);
            ptx::tma_load_2d(ptx::smem_u32(ring + cur.s * stage_bytes), map, full, col + sub * col_step, row);
            cur.advance(w_stages);
          }
          row += rows_per_stage;
        }
      }
      if (!ok) {
        sh.abort_flag = 1;
        if (p.status) atomicOr(p.status, kStatusProducerTimeout);
      }
    }
    __syncwarp();
  } else if (warp == 2 || (warp == 3 && !tiled_roles)) {
    // ------------------------------------------------ warps 2-3: activations --
    StageCursor cur;
    XSubRing xring;
    bool ok = true;
    if (p.x_load == kXLoadTiled) {
      // Consecutive rows: one box per 64-wide K half, issued by one thread.
      while (ok && threadIdx.x == 64 && iter.next(seg)) {
        const TileInfo t = decode_tile(p, sh, seg.tile, rank);
        if (!t.valid) continue;
        int32_t k_col = seg.kb * kBlockK;
        // `pair`: this CTA's half of the tile's token rows
        const int32_t tile_rows_here = t.mma_n >> p.pair;
        const int32_t x_row0 = t.base + t.m0 + static_cast<int32_t>(rank) * tile_rows_here;
        const int32_t boxes = (tile_rows_here + p.x_box_rows - 1) / p.x_box_rows;
        const bool two_slots = t.mma_n > 128;
        for (int32_t kb = seg.kb; kb < seg.ke; ++kb) {
          if (subslots) {
            const uint32_t s0 = xring.take(two_slots, 2u * x_stages);
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.xempty[s0]), xring.phase(s0) ^ 1u, abort_flag) ||
                (two_slots && !ptx::mbar_wait(ptx::smem_u32(&sh.xempty[s0 + 1]), xring.phase(s0 + 1) ^ 1u,
                                              abort_flag))) {  // odd half: checked, not consumed
              ok = false;
              break;
            }
            const uint32_t full = ptx::smem_u32(&sh.xfull[s0]);
            const uint32_t xs = ptx::smem_u32(smem_x + s0 * kSubBytes);
            const uint32_t half = two_slots ? kSubBytes : kSubBytes / 2;  // bytes of one K half
            ptx::mbar_arrive_expect_tx(full, static_cast<uint32_t>(boxes) * kSubBytes);
            for (int32_t b = 0; b < boxes; ++b) {
              const uint32_t off = static_cast<uint32_t>(b) * (kSubBytes / 2);
              ptx::tma_load_2d(xs + off, &tm_x, full, k_col, x_row0 + b * 128);
              ptx::tma_load_2d(xs + half + off, &tm_x, full, k_col + 64, x_row0 + b * 128);
            }
            xring.flip(s0);
            k_col += kBlockK;
            continue;
          }
          if (!ptx::mbar_wait(ptx::smem_u32(&sh.xempty[cur.s]), cur.ph ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&sh.xfull[cur.s]);
          const uint32_t xs = ptx::smem_u32(smem_x + cur.s * x_stage_bytes);
          if constexpr (kPair) {
            // Both CTAs' boxes are counted on the leader's barrier, which expects the bytes
            // of both halves.  (A box of the peer that lands before the leader's arrival
            // only drives the transaction count negative for a moment: the phase cannot
            // complete before that arrival.)
            if (rank == 0) {
              ptx::mbar_arrive_expect_tx(full, 2u * static_cast<uint32_t>(boxes * p.x_box_rows) * 256u);
            }
            for (int32_t b = 0; b < boxes; ++b) {
              const uint32_t off = static_cast<uint32_t>(b * p.x_box_rows) * 128u;
              ptx::tma_load_2d_pair(xs + off, &tm_x, full + to_leader, k_col, x_row0 + b * p.x_box_rows);
              ptx::tma_load_2d_pair(xs + x_half_bytes + off, &tm_x, full + to_leader, k_col + 64,
                                    x_row0 + b * p.x_box_rows);
            }
            k_col += kBlockK;
            cur.advance(x_stages);
            continue;
          }
          ptx::mbar_arrive_expect_tx(full, static_cast<uint32_t>(boxes * p.x_box_rows) * 256u);
          for (int32_t b = 0; b < boxes; ++b) {
            const uint32_t off = static_cast<uint32_t>(b * p.x_box_rows) * 128u;
            ptx::tma_load_2d(xs + off, &tm_x, full, k_col, x_row0 + b * p.x_box_rows);
            ptx::tma_load_2d(xs + x_half_bytes + off, &tm_x, full, k_col + 64,
                             x_row0 + b * p.x_box_rows);
          }
          k_col += kBlockK;
          cur.advance(x_stages);
        }
      }
    } else if (p.x_load == kXLoadGather4) {
      // Routed rows by TMA: four rows per instruction, lanes of warp 2 own the row
      // groups lane and lane + 32.
      while (ok && warp == 2 && iter.next(seg)) {
        const TileInfo t = decode_tile(p, sh, seg.tile, rank);
        if (!t.valid) continue;
        int32_t rows[2][4];
        const int32_t load_groups = (t.ntok + 3) >> 2;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int32_t gi = static_cast<int32_t>(lane) + 32 * h;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int32_t slot = gi * 4 + j;
            rows[h][j] = (gi < load_groups && slot < t.ntok) ? x_row_of(p, t, slot) : p.x_rows;
          }
        }
        const uint32_t tx_bytes = static_cast<uint32_t>(load_groups) * 1024u;
        int32_t k_col = seg.kb * kBlockK;
        for (int32_t kb = seg.kb; kb < seg.ke; ++kb) {
          if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.xempty[cur.s]), cur.ph ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&sh.xfull[cur.s]);
          const uint32_t xs = ptx::smem_u32(smem_x + cur.s * x_stage_bytes);
          if (lane == 0) ptx::mbar_arrive_expect_tx(full, tx_bytes);
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int32_t gi = static_cast<int32_t>(lane) + 32 * h;
            if (gi < load_groups) {
              ptx::tma_gather4(xs + gi * 512u, &tm_x, full, k_col, rows[h][0], rows[h][1],
                               rows[h][2], rows[h][3]);
              ptx::tma_gather4(xs + x_half_bytes + gi * 512u, &tm_x, full, k_col + 64, rows[h][0],
                               rows[h][1], rows[h][2], rows[h][3]);
            }
          }
          k_col += kBlockK;
          cur.advance(x_stages);
        }
      }
    } else {
      // Routed rows by cp.async: thread = (16-byte chunk of the 256-byte stage row,
      // row modulo 4).
      const uint32_t ht = threadIdx.x - 64;
      const uint32_t ch = ht & 15;
      const uint32_t half = ch >> 3, ch8 = ch & 7;
      const uint32_t r0 = ht >> 4;
      // A stage is published (one arrival per warp: 32 lanes arriving on one mbarrier
      // would serialise) once its copies have landed, which is checked `depth` stages
      // later so that the copies of several stages stay in flight.
      const int32_t depth = x_stages >= 4 ? 2 : 1;
      StageCursor done;
      int32_t pending = 0;
      // A warp whose bounded wait ran out stops copying but keeps walking the tiles, so
      // that its sibling never waits alone at the three barriers below.
      while (iter.next(seg)) {
        const TileInfo t = decode_tile(p, sh, seg.tile, rank);
        if (!t.valid) continue;
        ptx::named_bar_sync(2, kHelperThreads);  // readers of the previous tile's rows are done
        // Element offset of each slot's activation row, or -1 for a slot without a token;
        // x_slots = one past the last slot that carries a token.  Slots beyond it keep
        // whatever an earlier tile left there: they only feed accumulator columns that
        // are never stored.
        if (ht == 0) sh.x_slots = 0;
        ptx::named_bar_sync(2, kHelperThreads);
        for (int32_t slot = ht; slot < t.ntok; slot += kHelperThreads) {
          const int32_t row = x_row_of(p, t, slot);
          sh.x_row[slot] = row < p.x_rows ? row * p.k : -1;
          if (row < p.x_rows) atomicMax(&sh.x_slots, slot + 1);
        }
        ptx::named_bar_sync(2, kHelperThreads);
        if (!ok) continue;
        const int32_t x_slots = sh.x_slots;
        int32_t k_col = seg.kb * kBlockK + static_cast<int32_t>(ch) * 8;
        // Decode-sized tiles (at most 16 rows with a token): each thread owns at most
        // four copies per stage, whose addresses live in registers for the whole tile.
        const bool few_rows = x_slots <= 16;
        const __nv_bfloat16* fsrc[4];
        uint32_t fdst[4];
        bool fact[4], fval[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t rr = r0 + 4 * b;
          fact[b] = few_rows && static_cast<int32_t>(rr) < x_slots;
          const int32_t off = fact[b] ? sh.x_row[rr] : -1;
          fval[b] = off >= 0;
          fsrc[b] = p.x + (fval[b] ? off : 0) + k_col;
          fdst[b] = half * x_half_bytes + rr * 128u + ((ch8 ^ (rr & 7u)) << 4);
        }
        for (int32_t kb = seg.kb; kb < seg.ke; ++kb) {
          if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.xempty[cur.s]), cur.ph ^ 1u, abort_flag)) {
            ok = false;
            if (lane == 0) sh.abort_flag = 1;  // the sibling's waits end soon too
            break;
          }
          const uint32_t xs = ptx::smem_u32(smem_x + cur.s * x_stage_bytes);
          const bool col_ok = k_col + 8 <= p.k;
          if (few_rows) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              if (fact[b]) ptx::cp_async_16(xs + fdst[b], fsrc[b], fval[b] && col_ok);
              fsrc[b] += kBlockK;
            }
          } else {
            const __nv_bfloat16* xk = p.x + k_col;
            // Four rows per round: the offset loads go first so that the copies that
            // follow do not each wait on a shared-memory round trip.
            for (int32_t r = r0; r < x_slots; r += 16) {
              int32_t off[4];
#pragma unroll
              for (int b = 0; b < 4; ++b) off[b] = (r + 4 * b < x_slots) ? sh.x_row[r + 4 * b] : -1;
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const uint32_t rr = static_cast<uint32_t>(r + 4 * b);
                if (static_cast<int32_t>(rr) < x_slots) {
                  const bool valid = col_ok && off[b] >= 0;
                  ptx::cp_async_16(xs + half * x_half_bytes + rr * 128u + ((ch8 ^ (rr & 7u)) << 4),
                                   xk + (valid ? off[b] : 0), valid);
                }
              }
            }
          }
          ptx::cp_async_commit();
          if (++pending > depth) {
            // The MMA issuer adds the generic-to-async proxy fence after its wait.
            if (depth == 2) ptx::cp_async_wait_group<2>(); else ptx::cp_async_wait_group<1>();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sh.xfull[done.s]));
            done.advance(x_stages);
            --pending;
          }
          k_col += kBlockK;
          cur.advance(x_stages);
        }
      }
      // Drain: publish what is still in flight (also when leaving on a timeout).
      ptx::cp_async_wait_all();
      __syncwarp();
      for (; pending > 0; --pending) {
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sh.xfull[done.s]));
        done.advance(x_stages);
      }
    }
    __syncwarp();
    if (!ok && lane == 0) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, kStatusProducerTimeout);
    }
  } else if (tiled_roles ? (warp == 1 || warp == 3) : (warp >= kFirstIssuerWarp && warp < kFirstDequantWarp)) {
    // ----------------------------------------------------------- MMA issuers --
    const uint32_t me = tiled_roles ? (warp >> 1) : warp - kFirstIssuerWarp;
    if (me < ni && lane == 0 && rank == 0) {
      const uint64_t xdesc0 = ptx::smem_desc_k_sw128(ptx::smem_u32(smem_x));
      const uint64_t xdesc_stage = x_stage_bytes >> 4;  // descriptor address units are 16 bytes
      const uint64_t xdesc_half = x_half_bytes >> 4;
      uint64_t xdesc = xdesc0;
      StageCursor cur, acur;
      XSubRing xring;
      uint32_t it = 0, segc = 0;
      bool ok = true;
      while (ok && iter.next(seg)) {
        const TileInfo t = decode_tile(p, sh, seg.tile, rank);
        if (!t.valid) continue;
        const uint32_t d = d_bufs == 2 ? (segc & 1u) : 0u;
        const uint32_t dph = d_bufs == 2 ? ((segc >> 1) & 1u) : (segc & 1u);
        if (!ptx::mbar_wait(ptx::smem_u32(&sh.dempty[d]), dph ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_addr = tmem_base + d_col0 + (d * ni + me) * d_cols;
        const uint32_t idesc = ptx::idesc_bf16_f32(kBlockN << p.pair, static_cast<uint32_t>(t.mma_n));
        uint32_t acc = 0;
        const bool split = ksplit && t.mma_n <= 128;
        for (int32_t kb = seg.kb; kb < seg.ke; ++kb, ++it) {
          if constexpr (kPair) {
            // One MMA stream for both CTAs; every commit arrives on the barrier of each.
            const uint32_t a = acur.s << 1;
            const uint32_t aph = acur.ph;
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.xfull[cur.s]), cur.ph, abort_flag)) {
              ok = false;
              break;
            }
            const uint32_t a_addr = tmem_base + acur.s * kAColsPerStage;
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a]), aph, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            ptx::mma_ts_k64_pair(d_addr, a_addr, xdesc, idesc, acc);
            const uint32_t ae = ptx::smem_u32(&sh.aempty[a]);
            ptx::mma_commit_pair(ae);
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a + 1]), aph, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            if (!(k_tail_half && kb == k_iters - 1)) {
              ptx::mma_ts_k64_pair(d_addr, a_addr + 32, xdesc + xdesc_half, idesc, 1);
            }
            acc = 1;
            ptx::mma_commit_pair(ae + 8u);
            ptx::mma_commit_pair(ptx::smem_u32(&sh.xempty[cur.s]));
          } else if (npair) {
            // The K block's two operand-ring entries belong to the tile's two weight blocks;
            // this issuer takes the one of its block, with both K halves, into its accumulator.
            uint32_t as = acur.s + me, aph = acur.ph;
            if (as >= a_stages) {
              as -= a_stages;
              aph ^= 1u;
            }
            const uint32_t a = as << 1;
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.xfull[cur.s]), cur.ph, abort_flag)) {
              ok = false;
              break;
            }
            const uint32_t a_addr = tmem_base + as * kAColsPerStage;
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a]), aph, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            ptx::mma_ts_k64(d_addr, a_addr, xdesc, idesc, acc);
            ptx::mma_commit(ptx::smem_u32(&sh.aempty[a]));
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a + 1]), aph, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            if (!(k_tail_half && kb == k_iters - 1)) {
              ptx::mma_ts_k64(d_addr, a_addr + 32, xdesc + xdesc_half, idesc, 1);
            }
            acc = 1;
            ptx::mma_commit(ptx::smem_u32(&sh.aempty[a + 1]));
            ptx::mma_commit(ptx::smem_u32(&sh.xempty[cur.s]));
            acur.advance(a_stages);  // the other block's entry; the common advance below takes this one
          } else if (ksplit) {
            const uint32_t a = acur.s << 1;
            const uint32_t aph = acur.ph;
            uint32_t xslot = cur.s;       // barrier (and, with sub-slots, buffer) of this stage
            uint64_t xd = xdesc, xd_half = xdesc_half;
            const bool two_slots = subslots && t.mma_n > 128;
            if (subslots) {
              xslot = xring.take(two_slots, 2u * x_stages);
              xd = xdesc0 + xslot * (kSubBytes >> 4);
              xd_half = two_slots ? (kSubBytes >> 4) : (kSubBytes >> 5);
              if (!ptx::mbar_wait(ptx::smem_u32(&sh.xfull[xslot]), xring.phase(xslot), abort_flag)) {
                ok = false;
                break;
              }
              xring.flip(xslot);
            } else if (!ptx::mbar_wait(ptx::smem_u32(&sh.xfull[cur.s]), cur.ph, abort_flag)) {
              ok = false;
              break;
            }
            if (p.x_load == kXLoadCpAsync) ptx::fence_proxy_async();
            const uint32_t a_addr = tmem_base + acur.s * kAColsPerStage;
            const bool tail = k_tail_half && kb == k_iters - 1;
            if (me == 0) {
              if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a]), aph, abort_flag)) {
                ok = false;
                break;
              }
              ptx::tc_fence_after();
              ptx::mma_ts(d_addr, a_addr, xd, idesc, acc);
              ptx::mma_ts(d_addr, a_addr + 8, xd + 2, idesc, 1);
              ptx::mma_ts(d_addr, a_addr + 16, xd + 4, idesc, 1);
              ptx::mma_ts(d_addr, a_addr + 24, xd + 6, idesc, 1);
              acc = 1;
              ptx::mma_commit(ptx::smem_u32(&sh.aempty[a]));
            }
            if (me == 0 ? !split : split) {
              if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a + 1]), aph, abort_flag)) {
                ok = false;
                break;
              }
              ptx::tc_fence_after();
              if (!tail) {
                const uint64_t xd1 = xd + xd_half;
                ptx::mma_ts(d_addr, a_addr + 32, xd1, idesc, acc);
                ptx::mma_ts(d_addr, a_addr + 40, xd1 + 2, idesc, 1);
                ptx::mma_ts(d_addr, a_addr + 48, xd1 + 4, idesc, 1);
                ptx::mma_ts(d_addr, a_addr + 56, xd1 + 6, idesc, 1);
                acc = 1;
              }
              ptx::mma_commit(ptx::smem_u32(&sh.aempty[a + 1]));
            }
            // Both issuers account for the activation stage: a commit after MMAs of one's
            // own, a plain arrival otherwise.
            if (me == 0 || split) ptx::mma_commit(ptx::smem_u32(&sh.xempty[xslot]));
            else ptx::mbar_arrive(ptx::smem_u32(&sh.xempty[xslot]));
          } else if ((it & (ni - 1)) == me) {
            const uint32_t a = acur.s << 1;  // barrier of the first K half; the second is a + 1
            const uint32_t aph = acur.ph;
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.xfull[cur.s]), cur.ph, abort_flag)) {
              ok = false;
              break;
            }
            if (p.x_load == kXLoadCpAsync) ptx::fence_proxy_async();
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a]), aph, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t a_addr = tmem_base + acur.s * kAColsPerStage;
            ptx::mma_ts(d_addr, a_addr, xdesc, idesc, acc);
            ptx::mma_ts(d_addr, a_addr + 8, xdesc + 2, idesc, 1);
            ptx::mma_ts(d_addr, a_addr + 16, xdesc + 4, idesc, 1);
            ptx::mma_ts(d_addr, a_addr + 24, xdesc + 6, idesc, 1);
            ptx::mma_commit(ptx::smem_u32(&sh.aempty[a]));
            if (!ptx::mbar_wait(ptx::smem_u32(&sh.afull[a + 1]), aph, abort_flag)) {
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            if (!(k_tail_half && kb == k_iters - 1)) {
              const uint64_t xd1 = xdesc + xdesc_half;
              ptx::mma_ts(d_addr, a_addr + 32, xd1, idesc, 1);
              ptx::mma_ts(d_addr, a_addr + 40, xd1 + 2, idesc, 1);
              ptx::mma_ts(d_addr, a_addr + 48, xd1 + 4, idesc, 1);
              ptx::mma_ts(d_addr, a_addr + 56, xd1 + 6, idesc, 1);
            }
            acc = 1;
            ptx::mma_commit(ptx::smem_u32(&sh.aempty[a + 1]));
            ptx::mma_commit(ptx::smem_u32(&sh.xempty[cur.s]));
          }
          xdesc += xdesc_stage;
          cur.advance(x_stages);
          acur.advance(a_stages);
          if (cur.s == 0) xdesc = xdesc0;
        }
        if (!ok) break;
        // One arrival per issuer and segment, also from an issuer that had no stage in it.
        if constexpr (kPair) {
          ptx::mma_commit_pair(ptx::smem_u32(&sh.dfull[d]));
        } else if (acc != 0) {
          ptx::mma_commit(ptx::smem_u32(&sh.dfull[d]));
        } else {
          ptx::mbar_arrive(ptx::smem_u32(&sh.dfull[d]));
        }
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
    StageCursor cur, acur;
    uint32_t it = 0;
    bool ok = true;
    // A stored K half is published to the MMA issuer one compute step later (after
    // the next half has been dequantised), so that the latency of the tensor-memory
    // store and of the barrier round trip hides behind ALU work.  `pending` is the
    // slot whose store has been issued but not yet published.
    int32_t pending = -1;
    auto publish = [&]() {
      if (pending >= 0) {
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          // `pair`: the leader's barrier counts the warps of both CTAs
          if constexpr (kPair) ptx::mbar_arrive_cluster(ptx::smem_u32(&sh.afull[pending]) + to_leader);
          else ptx::mbar_arrive(ptx::smem_u32(&sh.afull[pending]));
        }
        pending = -1;
      }
    };
    auto load_half = [&](const uint8_t* wsrc, const uint8_t* ssrc, int h, uint2 (&words)[4],
                         uint2 (&scales)[2]) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        words[j] = *reinterpret_cast<const uint2*>(wsrc + (4 * h + j) * 1024);
      }
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        scales[g] = *reinterpret_cast<const uint2*>(ssrc + (2 * h + g) * 256);
      }
    };
    auto dequant_half = [&](const uint2 (&words)[4], const uint2 (&scales)[2], uint32_t (&lo)[16],
                            uint32_t (&hi)[16]) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint2 sc = scales[j >> 1];
        // sc.x = {slab A row r, slab A row r+8}; sc.y = same for slab B.
        const uint32_t a_lo = __byte_perm(sc.x, 0, 0x1010);
        const uint32_t a_hi = __byte_perm(sc.x, 0, 0x3232);
        const uint32_t b_lo = __byte_perm(sc.y, 0, 0x1010);
        const uint32_t b_hi = __byte_perm(sc.y, 0, 0x3232);
        dequant_word(words[j].x, a_lo, a_hi, lo + 4 * j);
        dequant_word(words[j].y, b_lo, b_hi, hi + 4 * j);
      }
    };
    // Waits for the slot to be free, then stores one K half: lo to TMEM lanes 0-15 of
    // the quarter (first slab), hi to lanes 16-31 (second slab).
    auto store_half = [&](uint32_t slot, uint32_t aph, const uint32_t (&lo)[16],
                          const uint32_t (&hi)[16]) -> bool {
      if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.aempty[slot]), aph ^ 1u, abort_flag)) return false;
      ptx::tc_fence_after();
      const uint32_t a_addr = tmem_base + ((q * 32u) << 16) + slot * (kAColsPerStage / 2);
      ptx::tmem_st_16x128b_x8(a_addr, lo);
      ptx::tmem_st_16x128b_x8(a_addr + (16u << 16), hi);
      pending = static_cast<int32_t>(slot);
      return true;
    };
    while (ok && iter.next(seg)) {
      const TileInfo t = decode_tile(p, sh, seg.tile, rank);
      if (!t.valid) continue;
      // This group owns the stages whose running index is `group` modulo the number
      // of groups: step over the others without visiting them.
      const uint32_t seg_len = static_cast<uint32_t>((seg.ke - seg.kb) * w_per_kb);  // ring entries
      const uint32_t first = (group - it) & (kDequantGroups - 1);
      const uint32_t it_end = it + seg_len;
      if (first >= seg_len) {
        it = it_end;
        cur.advance_by(seg_len, w_stages);
        acur.advance_by(seg_len, a_stages);
        continue;
      }
      it += first;
      cur.advance_by(first, w_stages);
      acur.advance_by(first, a_stages);
      for (; it < it_end; it += kDequantGroups, cur.advance_by(kDequantGroups, w_stages),
                          acur.advance_by(kDequantGroups, a_stages)) {
        const uint32_t a = acur.s << 1;  // half-slots a (first K half) and a + 1 (second)
        const uint32_t aph = acur.ph;
        if (!ptx::mbar_wait_warp(ptx::smem_u32(&sh.wfull[cur.s]), cur.ph, abort_flag)) {
          ok = false;
          break;
        }
        const uint8_t* wsrc = smem_w + cur.s * kWStageBytes + w_off;
        const uint8_t* ssrc = smem_s + cur.s * kSStageBytes + s_off;
        uint2 words[4], scales[2];
        uint32_t lo[16], hi[16];
        load_half(wsrc, ssrc, 0, words, scales);
        dequant_half(words, scales, lo, hi);
        // Second half's words are fetched before the first half is stored, and the
        // stage goes back to the producers as soon as they are in registers.
        load_half(wsrc, ssrc, 1, words, scales);
        publish();  // previous stage's second half
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sh.wempty[cur.s]));
        if (!store_half(a, aph, lo, hi)) {
          ok = false;
          break;
        }
        dequant_half(words, scales, lo, hi);
        publish();  // this stage's first half
        if (!store_half(a + 1, aph, lo, hi)) {
          ok = false;
          break;
        }
      }
      // `it` overshoots the segment's end by less than one stride: bring the cursor back.
      if (ok) {
        const uint32_t over = it - it_end;
        it = it_end;
        cur.advance_by(w_stages - over, w_stages);
        cur.ph ^= 1u;
        acur.advance_by(a_stages - over, a_stages);
        acur.ph ^= 1u;
      }
    }
    publish();
    if (!ok && lane == 0) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, kStatusDequantTimeout);
    }
  } else {
    // -------------------------------------------------------------- epilogue --
    // Four warps, one per tensor-memory lane quarter; with `tiled_roles` a second group of
    // four (warps 4-7) takes every other 16-column chunk.
    const uint32_t q = warp & 3;
    const uint32_t kEpiThreads = epi_threads;
    const uint32_t egroup = warp < kFirstDequantWarp ? 1u : 0u;
    const uint32_t et = threadIdx.x - (egroup ? kFirstIssuerWarp : kFirstEpilogueWarp) * 32;  // 0..127 == TMEM lane
    const uint32_t efill = egroup * 128u + et;  // index among all epilogue threads
    uint32_t segc = 0, it0 = 0;
    bool ok = true;
    const size_t ws_block = static_cast<size_t>(kBlockN) * p.mma_n;  // partial sums of one weight block
    const size_t ws_slot = ws_block * w_per_kb;
    while (ok && iter.next(seg)) {
      const TileInfo t = decode_tile(p, sh, seg.tile, rank);
      if (!t.valid) continue;
      const uint32_t d = d_bufs == 2 ? (segc & 1u) : 0u;
      const uint32_t dph = d_bufs == 2 ? ((segc >> 1) & 1u) : (segc & 1u);
      ptx::named_bar_sync(1, kEpiThreads);  // previous segment's out_row readers are done
      const int32_t row_slots = (t.rows + 15) & ~15;  // >= t.mma_n; beyond it: rows written as zeros
      for (int32_t c = efill; c < row_slots; c += kEpiThreads) sh.out_row[c] = out_row_of(p, t, c);
      bool lock_ok = true;
      if (seg.type == kSegOwner && efill == 0) {
        // Wait (bounded) until every other slice of this tile has published its partial.
        const int* lock = p.locks + blockIdx.x;  // (`pair`: one word per CTA; the slices of its rows come from CTAs of its own rank)
        lock_ok = false;
        for (int32_t spin = 0; spin < p.lock_spins; ++spin) {
          if (ptx::ld_acquire(lock) >= seg.peer) {
            lock_ok = true;
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
      ptx::named_bar_sync(1, kEpiThreads);  // out_row filled, lock observed, verdict published
      if (sh.epilogue_failed != 0) {
        ok = false;
        break;
      }
      const uint32_t d_addr = tmem_base + ((q * 32u) << 16) + d_col0 + d * ni * d_cols;
      // Issuer i accumulated the stages it0 + j with (it0 + j) % ni == i; it took part
      // in this segment only if one of them falls inside it.  (With `npair` accumulator
      // `sub` is the tile's weight block `sub` instead, and nothing is summed.)
      const uint32_t seg_len = static_cast<uint32_t>(seg.ke - seg.kb);
      // Fused SiLU*mul: one pass, which reads both accumulators (gate, up), combines them
      // and writes a [rows, N/2] tensor.
      const bool fuse = p.fuse_silu != 0;
      const int32_t ldn = fuse ? (p.n >> 1) : p.n;
      for (int32_t sub = 0; sub < (fuse ? 1 : w_per_kb); ++sub) {
      const int32_t n_sub = t.n0 + sub * kBlockN + static_cast<int32_t>(q) * 32;
      __nv_bfloat16* out_tile = p.out + n_sub;
      const size_t ws_sub = static_cast<size_t>(sub) * ws_block;
      for (int32_t c0 = static_cast<int32_t>(egroup) * 16; c0 < row_slots; c0 += tiled_roles ? 32 : 16) {
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
        // Slots past the tile's MMA N hold padding rows of a contiguous block: the product
        // of their all-zero activations is written without having been computed.
        const bool computed = c0 < t.mma_n;
        if (!computed && seg.type == kSegContrib) continue;
        for (uint32_t i = 0; computed && i < ni; ++i) {
          if (npair) {
            if (static_cast<int32_t>(i) != sub) continue;
          } else if (ksplit) {
            // issuer 1 holds the second K halves of tiles of at most 128 tokens, unless the
            // segment is nothing but the half-filled last stage
            if (i == 1 && (t.mma_n > 128 || seg_len == (k_tail_half && seg.ke == k_iters ? 1u : 0u))) continue;
          } else if (((i - it0) & (ni - 1)) >= seg_len) {
            continue;
          }
          uint32_t v[16];
          ptx::tmem_ld_32x32b_x16(d_addr + i * d_cols + c0, v);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] += __uint_as_float(v[j]);
        }
        float up[16];
        if (fuse) {
#pragma unroll
          for (int j = 0; j < 16; ++j) up[j] = 0.0f;
          if (computed) {
            uint32_t v[16];
            ptx::tmem_ld_32x32b_x16(d_addr + d_cols + c0, v);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) up[j] = __uint_as_float(v[j]);
          }
        }
        if (seg.type == kSegContrib) {
          float* dst = p.workspace + blockIdx.x * ws_slot + ws_sub + static_cast<size_t>(c0) * kBlockN + et;
#pragma unroll
          for (int j = 0; j < 16; ++j) __stcg(dst + j * kBlockN, acc[j]);
          if (fuse) {
#pragma unroll
            for (int j = 0; j < 16; ++j) __stcg(dst + ws_block + j * kBlockN, up[j]);
          }
          continue;
        }
        if (seg.type == kSegOwner && computed) {
          for (int32_t peer = 1; peer <= seg.peer; ++peer) {
            const float* src = p.workspace + (blockIdx.x + (peer << p.pair)) * ws_slot + ws_sub +
                               static_cast<size_t>(c0) * kBlockN + et;
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] += __ldcg(src + j * kBlockN);
            if (fuse) {
#pragma unroll
              for (int j = 0; j < 16; ++j) up[j] += __ldcg(src + ws_block + j * kBlockN);
            }
          }
        }
        if (fuse) {
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = acc[j] / (1.0f + __expf(-acc[j])) * up[j];
        }
        // Transpose through shared memory so that global stores are 16 bytes wide: the
        // warp holds 32 weight rows x 16 tokens (one token per register); staged as
        // [token][row], each lane then stores two 8-row pieces of a token's 64 bytes.
        __nv_bfloat16* stage = &sh.stage[egroup * 4u + q][0][0];
#pragma unroll
        for (int j = 0; j < 16; ++j) stage[j * 32 + lane] = __float2bfloat16_rn(acc[j]);
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t idx = lane + 32 * i;
          const uint32_t tj = idx >> 2, piece = idx & 3;
          const int32_t row = sh.out_row[c0 + tj];
          const uint4 v = *reinterpret_cast<const uint4*>(stage + tj * 32 + piece * 8);
          if (row >= 0) {
            if (p.out_row_ptr != nullptr) {
              // the row lives wherever the caller's table says (possibly on another GPU)
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(
                  __ldg(reinterpret_cast<const unsigned long long*>(p.out_row_ptr) + row));
              if (dst != nullptr) *reinterpret_cast<uint4*>(dst + n_sub + piece * 8) = v;
            } else {
              *reinterpret_cast<uint4*>(out_tile + static_cast<size_t>(row) * ldn + piece * 8) = v;
            }
          }
        }
        __syncwarp();
      }
      }
      // Release the accumulator buffer to the MMA issuer.
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) ptx::mbar_arrive_cluster(ptx::smem_u32(&sh.dempty[d]) + to_leader);
        else ptx::mbar_arrive(ptx::smem_u32(&sh.dempty[d]));
      }
      if (seg.type == kSegContrib) {
        __threadfence();
        ptx::named_bar_sync(1, kEpiThreads);
        // the owner of this CTA's rows: the CTA of the same rank in the owning pair
        if (efill == 0) ptx::red_release_add(p.locks + ((seg.peer << p.pair) + static_cast<int32_t>(rank)), 1);
      } else if (seg.type == kSegOwner) {
        ptx::named_bar_sync(1, kEpiThreads);
        // After a timeout the word is left as it is: contributors that arrive late would
        // otherwise leave it non-zero behind a reset, and the caller has to clear the
        // buffer anyway once the status word reports the failure.
        if (efill == 0 && lock_ok) p.locks[blockIdx.x] = 0;
      }
      ++segc;
      it0 += seg_len;
    }
    if (!ok && lane == 0) {
      sh.abort_flag = 1;
      if (p.status) atomicOr(p.status, kStatusEpilogueTimeout);
    }
  }

  // --------------------------------------------------------------- teardown --
  ptx::tc_fence_before();
  __syncthreads();
  // `pair`: neither CTA may leave (or free tensor memory) while the other can still
  // signal its barriers or have MMAs reading its shared and tensor memory.
  if constexpr (kPair) ptx::cluster_sync();
  if (warp == 2) {
    ptx::tc_fence_after();
    if constexpr (kPair) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    else ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace chord
