// Decode-sized variant of the W4A16 grouped GEMM (token tiles of at most 32 rows).
//
// Same data formats, numerics, scheduling and stream-K protocol as
// w4a16_gemm_kernel (w4a16_gemm.cuh); what changes is who does what.  With a
// handful of tokens per tile the MMAs are tiny and the kernel is bound by the number
// of instructions it spends per weight byte (the integer pipe that pulls the nibbles
// apart runs at half rate), so every barrier round trip between specialised warps and
// every address computation counts.  Here each of the four warpgroups of a CTA is a
// self-contained worker with a feeder warp and an MMA issuer warp of its own:
//
//   * it has its own slice of the work (the grid of workers is 4 x the grid of CTAs),
//     its own shared-memory ring and its own 128 tensor-memory columns
//     (three 32-column operand slots + up to 32 accumulator columns);
//   * a ring stage holds everything one 64-wide K step needs: 4 KB of packed weights
//     and 512 B of scales (two TMA boxes) and the step's activation rows
//     (cp.async gather, 128-byte swizzle).  The worker's feeder warp fills it:
//     lane 0 issues the TMA, all 32 lanes gather the activation rows.  The weight half
//     of a stage is handed back as soon as the warps have read it, so the HBM stream
//     runs a full ring ahead; the activation half waits for the MMAs that read it;
//   * per step each of the worker's four warps reads its packed words, dequantises
//     them and stores them to one of three operand slots in tensor memory; the
//     worker's issuer warp then issues the step's four tcgen05.mma, whose completion
//     frees the activation half of the stage and the operand slot.  The four warps do
//     not wait for one another inside a tile;
//   * after the last step of a tile the same four warps run the epilogue.
#pragma once

#include <type_traits>

#include "w4a16_gemm.cuh"

namespace chord {

constexpr int kDecStepK = 64;                        // K elements per step (one operand slot, four MMAs)
constexpr int kDecStageK = 2 * kDecStepK;            // K elements per ring stage (two steps)
constexpr int kDecWBytes = (kDecStageK / 16) * 1024;  // packed weights per stage
constexpr int kDecSBytes = (kDecStageK / 32) * 256;   // scales per stage
constexpr int kDecWSBytes = kDecWBytes + kDecSBytes;  // 9 KB: keeps stages 1024-aligned
constexpr int kDecMaxStages = 6;
constexpr int kDecMaxTokens = 32;
constexpr int kDecWorkers = 4;                       // warpgroups per CTA
constexpr int kDecThreads = 32 * (2 * kDecWorkers + 4 * kDecWorkers);  // feeders, issuers, workers
constexpr int kDecSlots = 3;                         // operand slots (32 TMEM columns each) per worker
constexpr int kDecDCol = 32 * kDecSlots;             // the worker's accumulator follows its operand slots

struct __align__(16) DecodeWorkerShared {
  uint64_t wfull[kDecMaxStages];   // weights and scales landed (1 arrival + TMA bytes)
  uint64_t wempty[kDecMaxStages];  // the four warps have them in registers (4 arrivals)
  uint64_t xfull[kDecMaxStages];   // activation rows landed and visible to the tensor core (1 arrival)
  uint64_t xempty[kDecMaxStages];  // the MMAs reading them have completed (1 commit)
  uint64_t afree[kDecSlots];      // the MMAs reading the operand slot have completed (1 commit)
  uint64_t afull[kDecSlots];      // operand slot stored by the four warps (4 arrivals)
  __align__(16) __nv_bfloat16 stage[4][8][32];   // epilogue transpose buffers, one per warp
};

struct __align__(16) DecodeShared {
  DecodeWorkerShared worker[kDecWorkers];
  uint32_t tmem_base;
  uint32_t abort_flag;
  int32_t m_blocks;
  int32_t pad;
  int32_t group_prefix[kMaxGroups + 1];  // masked: first M tile of each group
};

// Bytes of one ring stage: the activation rows of both 64-wide K halves first
// (1024-aligned for the swizzle), then packed weights and scales.
__host__ __device__ inline uint32_t decode_stage_bytes(int mma_n) {
  return static_cast<uint32_t>(mma_n) * 256u + kDecWSBytes;
}

// decode_tile() of the general kernel without its contiguous branch (not served here),
// plus the tile's own MMA N: 16 when no token slot beyond the sixteenth carries a row,
// which is the common case at decode sizes whatever block size the routing was
// aligned to.  A tile without any row is not valid (nothing to compute).  Must be
// called by all 32 lanes of a warp.
__device__ __forceinline__ TileInfo decode_tile_small(const GemmParams& p, const int32_t* group_prefix,
                                                      int32_t tile) {
  TileInfo t;
  const int32_t n_blocks = (p.n >> p.fuse_silu) / kBlockN;  // fused SiLU*mul: one tile per gate block
  const int32_t mb = tile / n_blocks;
  t.n0 = (tile - mb * n_blocks) * kBlockN;
  t.m0 = 0;
  t.limit = 0;
  t.mma_n = p.mma_n;
  if (p.mode == kModeIndexed) {
    // (through a shuffle: a loaded value is not known to be the same in all lanes)
    t.expert = __shfl_sync(0xffffffffu, __ldg(p.expert_ids + mb), 0);
    t.ntok = p.tile_tokens;
    t.base = mb * p.tile_tokens;
    const int32_t lane = static_cast<int32_t>(threadIdx.x & 31u);
    const int32_t id = lane < p.tile_tokens ? __ldg(p.sorted_ids + t.base + lane) : -1;
    const uint32_t rows = __ballot_sync(0xffffffffu, id >= 0 && id < p.out_rows && id / p.top_k < p.x_rows);
    t.ntok = 32 - __clz(static_cast<int32_t>(rows));  // one past the last slot that carries a row
    t.mma_n = t.ntok <= 16 ? 16 : 32;
  } else {
    int32_t lo = 0, hi = p.num_experts;
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (group_prefix[mid] <= mb) lo = mid; else hi = mid;
    }
    lo = __shfl_sync(0xffffffffu, lo, 0);
    t.expert = lo;
    t.m0 = __shfl_sync(0xffffffffu, (mb - group_prefix[lo]) * p.tile_tokens, 0);
    int32_t mm = __shfl_sync(0xffffffffu, __ldg(p.masked_m + lo), 0);
    mm = mm < 0 ? 0 : (mm > p.max_m ? p.max_m : mm);
    t.limit = mm;
    const int32_t left = mm - t.m0;
    t.ntok = left < p.tile_tokens ? left : p.tile_tokens;
    t.base = lo * p.max_m;
    t.mma_n = t.ntok <= 16 ? 16 : 32;
  }
  t.rows = t.ntok;
  t.valid = t.expert >= 0 && t.expert < p.num_experts && t.ntok > 0;
  return t;
}

// The steps (tile, 64-wide K block) of one worker in order, one at a time.
struct StepStream {
  SegmentIterator iter;
  Segment seg;
  TileInfo t;
  int32_t kb;
  bool live;

  __device__ void init(int32_t tiles, int32_t k_steps, int32_t workers, int32_t worker) {
    iter.init(tiles, k_steps, workers, worker);
    live = false;
    kb = 0;
  }

  // Moves to the next step; `first` tells whether it opens a new segment.
  __device__ bool next(const GemmParams& p, const int32_t* group_prefix, bool& first) {
    if (live && ++kb < seg.ke) {
      first = false;
      return true;
    }
    while (iter.next(seg)) {
      t = decode_tile_small(p, group_prefix, seg.tile);
      if (!t.valid) continue;
      kb = seg.kb;
      live = true;
      first = true;
      return true;
    }
    live = false;
    return false;
  }
};

// Accumulator -> BF16 -> global for one warp's 32 weight rows of one segment.  Lane l
// holds the output row of token slot l (`rows`).  A whole tile needs nothing from the
// worker's other three warps; a stream-K slice does (lock, partials), and only then do
// the four warps meet at named barriers.  Kept out of line: it runs once per tile, and
// inlined into the dequantisation loop it took registers from that loop.
static __device__ __noinline__ void decode_drain(uint32_t d_addr, __nv_bfloat16* out_tile,
                                                 void* const* out_rows, int32_t col0, int32_t ldn,
                                          int32_t rows, int32_t mma_n, int32_t seg_type, int32_t seg_peer,
                                          float* workspace, size_t ws_slot, int32_t worker_id,
                                          int32_t* locks, int32_t lock_spins, int32_t* status,
                                          __nv_bfloat16* stage, uint32_t bar_id, uint32_t wt, bool ok) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t q = (threadIdx.x >> 5) & 3u;
  ptx::tc_fence_after();
  const bool shared_tile = seg_type != kSegFull;
  bool lock_ok = true;
  if (shared_tile) {
    if (ok && seg_type == kSegOwner && wt == 0) {
      const int* lock = locks + worker_id;
      lock_ok = false;
      for (int32_t spin = 0; spin < lock_spins; ++spin) {
        if (ptx::ld_acquire(lock) >= seg_peer) {
          lock_ok = true;
          break;
        }
        __nanosleep(64);
      }
      if (!lock_ok && status) atomicOr(status, kStatusLockTimeout);
    }
    ptx::named_bar_sync(bar_id, 128);  // lock observed
  }
  if (ok) {
    for (int32_t c0 = 0; c0 < mma_n; c0 += 16) {
      uint32_t v[16];
      ptx::tmem_ld_32x32b_x16(d_addr + c0, v);
      ptx::tmem_wait_ld();
      float accv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) accv[i] = __uint_as_float(v[i]);
      if (seg_type == kSegContrib) {
        float* dst = workspace + worker_id * ws_slot + static_cast<size_t>(c0) * kBlockN + q * 32 + lane;
#pragma unroll
        for (int i = 0; i < 16; ++i) __stcg(dst + i * kBlockN, accv[i]);
        continue;
      }
      if (seg_type == kSegOwner) {
        // Partials are added in worker order (deterministic); two slices' loads are in
        // flight at a time, each a round trip to L2.
        const float* part = workspace + (worker_id + 1) * ws_slot + static_cast<size_t>(c0) * kBlockN +
                            q * 32 + lane;
        int32_t peer = 1;
        for (; peer + 1 <= seg_peer; peer += 2, part += 2 * ws_slot) {
          float p0[16], p1[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) p0[i] = __ldcg(part + i * kBlockN);
#pragma unroll
          for (int i = 0; i < 16; ++i) p1[i] = __ldcg(part + ws_slot + i * kBlockN);
#pragma unroll
          for (int i = 0; i < 16; ++i) accv[i] = (accv[i] + p0[i]) + p1[i];
        }
        if (peer <= seg_peer) {
#pragma unroll
          for (int i = 0; i < 16; ++i) accv[i] += __ldcg(part + i * kBlockN);
        }
      }
      // Transpose through shared memory so that global stores are 16 bytes wide: eight
      // tokens at a time (32 weight rows x 8 tokens = one 16-byte piece per lane).
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int i = 0; i < 8; ++i) stage[i * 32 + lane] = __float2bfloat16_rn(accv[8 * half + i]);
        __syncwarp();
        const uint32_t tj = lane >> 2, pc = lane & 3;
        const int32_t row = __shfl_sync(0xffffffffu, rows, c0 + 8 * half + static_cast<int32_t>(tj));
        const uint4 val = *reinterpret_cast<const uint4*>(stage + tj * 32 + pc * 8);
        if (row >= 0) {
          if (out_rows != nullptr) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(
                __ldg(reinterpret_cast<const unsigned long long*>(out_rows) + row));
            if (dst != nullptr) *reinterpret_cast<uint4*>(dst + col0 + pc * 8) = val;
          } else {
            *reinterpret_cast<uint4*>(out_tile + static_cast<size_t>(row) * ldn + pc * 8) = val;
          }
        }
        __syncwarp();
      }
    }
    ptx::tc_fence_before();
    if (seg_type == kSegContrib) __threadfence();
  }
  if (shared_tile) {
    ptx::named_bar_sync(bar_id, 128);  // all four warps' partials are written / read
    if (wt == 0) {
      // A contributor completes the handshake even after a failure, so that no owner
      // spins on a lock that would never move; the status word tells the host.  An owner
      // whose wait ran out leaves its word as it is (late contributors would make it
      // non-zero again behind a reset).
      if (seg_type == kSegContrib) ptx::red_release_add(locks + seg_peer, 1);
      else if (lock_ok) locks[worker_id] = 0;
    }
  }
}

__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + __expf(-v)); }

// decode_drain() for a gate_up tile with SiLU*mul fused in: the worker's accumulator holds
// the gate block in columns 0-15 and the up block in columns 16-31 (16-token tiles); a
// stream-K slice publishes or collects both, and the warp stores
// bf16(silu(gate) * up) for its 32 rows of the block into a [rows, N/2] tensor (`ldn`).
// `covered` bit b says whether the segment had any stage of block b: a one-stage slice
// touches only one of the two accumulators, and the other then counts as zero.
static __device__ __noinline__ void decode_drain_silu(uint32_t d_addr, __nv_bfloat16* out_tile,
                                                      void* const* out_rows, int32_t col0, int32_t ldn,
                                                      int32_t rows, uint32_t covered, int32_t seg_type,
                                                      int32_t seg_peer, float* workspace, size_t ws_slot,
                                                      int32_t worker_id, int32_t* locks, int32_t lock_spins,
                                                      int32_t* status, __nv_bfloat16* stage,
                                                      uint32_t bar_id, uint32_t wt, bool ok) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t q = (threadIdx.x >> 5) & 3u;
  ptx::tc_fence_after();
  const bool shared_tile = seg_type != kSegFull;
  bool lock_ok = true;
  if (shared_tile) {
    if (ok && seg_type == kSegOwner && wt == 0) {
      const int* lock = locks + worker_id;
      lock_ok = false;
      for (int32_t spin = 0; spin < lock_spins; ++spin) {
        if (ptx::ld_acquire(lock) >= seg_peer) {
          lock_ok = true;
          break;
        }
        __nanosleep(64);
      }
      if (!lock_ok && status) atomicOr(status, kStatusLockTimeout);
    }
    ptx::named_bar_sync(bar_id, 128);  // lock observed
  }
  if (ok) {
    float gate[16], up[16];
    {
      uint32_t v[16];
      ptx::tmem_ld_32x32b_x16(d_addr, v);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) gate[i] = (covered & 1u) ? __uint_as_float(v[i]) : 0.0f;
      ptx::tmem_ld_32x32b_x16(d_addr + 16, v);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 16; ++i) up[i] = (covered & 2u) ? __uint_as_float(v[i]) : 0.0f;
    }
    if (seg_type == kSegContrib) {
      float* dst = workspace + worker_id * ws_slot + q * 32 + lane;
#pragma unroll
      for (int i = 0; i < 16; ++i) __stcg(dst + i * kBlockN, gate[i]);
#pragma unroll
      for (int i = 0; i < 16; ++i) __stcg(dst + (16 + i) * kBlockN, up[i]);
    } else {
      if (seg_type == kSegOwner) {
        // partials are added in worker order (deterministic)
        const float* part = workspace + (worker_id + 1) * ws_slot + q * 32 + lane;
        for (int32_t peer = 1; peer <= seg_peer; ++peer, part += ws_slot) {
          float pg[16], pu[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pg[i] = __ldcg(part + i * kBlockN);
#pragma unroll
          for (int i = 0; i < 16; ++i) pu[i] = __ldcg(part + (16 + i) * kBlockN);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            gate[i] += pg[i];
            up[i] += pu[i];
          }
        }
      }
      // eight tokens at a time through shared memory, as in decode_drain()
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          stage[i * 32 + lane] = __float2bfloat16_rn(silu_f32(gate[8 * half + i]) * up[8 * half + i]);
        }
        __syncwarp();
        const uint32_t tj = lane >> 2, pc = lane & 3;
        const int32_t row = __shfl_sync(0xffffffffu, rows, 8 * half + static_cast<int32_t>(tj));
        const uint4 val = *reinterpret_cast<const uint4*>(stage + tj * 32 + pc * 8);
        if (row >= 0) {
          if (out_rows != nullptr) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(
                __ldg(reinterpret_cast<const unsigned long long*>(out_rows) + row));
            if (dst != nullptr) *reinterpret_cast<uint4*>(dst + col0 + pc * 8) = val;
          } else {
            *reinterpret_cast<uint4*>(out_tile + static_cast<size_t>(row) * ldn + pc * 8) = val;
          }
        }
        __syncwarp();
      }
    }
    ptx::tc_fence_before();
    if (seg_type == kSegContrib) __threadfence();
  }
  if (shared_tile) {
    ptx::named_bar_sync(bar_id, 128);  // all four warps' partials are written / read
    if (wt == 0) {
      if (seg_type == kSegContrib) ptx::red_release_add(locks + seg_peer, 1);
      else if (lock_ok) locks[worker_id] = 0;
    }
  }
}

// kFuse: gate_up with SiLU*mul in the epilogue (its own instantiation, so that the plain
// kernel's loops carry none of it).
template <bool kFuse>
__global__ void __launch_bounds__(kDecThreads, 1)
w4a16_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_s,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Dynamic shared memory, 1024-aligned: one ring per worker, then DecodeShared.
  const uint32_t raw_addr = ptx::smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const uint32_t stages = static_cast<uint32_t>(p.w_stages);
  const uint32_t x_half_bytes = static_cast<uint32_t>(p.mma_n) * 128u;  // one K half of the activation rows
  const uint32_t x_bytes = 2u * x_half_bytes;
  const uint32_t stage_bytes = x_bytes + kDecWSBytes;
  const uint32_t worker_bytes = stages * stage_bytes;
  DecodeShared& sh = *reinterpret_cast<DecodeShared*>(smem + kDecWorkers * worker_bytes);

  // Read back through a shuffle so that the compiler knows the warp index (and every
  // ring position, barrier and tensor-memory address derived from it) to be the same in
  // all lanes and keeps them in uniform registers.
  const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const uint32_t lane = threadIdx.x & 31;
  // With SiLU*mul fused into the epilogue a tile is a gate block and its up block (weight
  // rows n0.. and N/2 + n0..): its ring stages alternate between the two (even stage = gate,
  // odd = up, both of K block stage / 2), each block accumulates into its own 16 columns,
  // and the epilogue combines them.  (Host side: only for 16-token tiles and K % 128 == 0.)
  constexpr int32_t fuse = kFuse ? 1 : 0;
  const int32_t k_steps = ((p.k + kDecStageK - 1) / kDecStageK) << fuse;  // ring stages per tile
  const bool k_tail_half = (p.k % kDecStageK) != 0;             // last stage: first K half only

  // Set-up is on the critical path of a small launch (a batch of one token is a
  // 25 us kernel): one thread per worker initialises that worker's barriers.
  if (warp >= 4 && warp < 8 && lane == 0) {
    const uint32_t w = warp - 4;
    if (w == 0) {
      ptx::prefetch_tensormap(&tm_w);
      ptx::prefetch_tensormap(&tm_s);
      sh.abort_flag = 0;
    }
    for (uint32_t s = 0; s < stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&sh.worker[w].wfull[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh.worker[w].wempty[s]), 4);
      ptx::mbar_init(ptx::smem_u32(&sh.worker[w].xfull[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&sh.worker[w].xempty[s]), 1);
    }
    for (int j = 0; j < kDecSlots; ++j) {
      ptx::mbar_init(ptx::smem_u32(&sh.worker[w].afull[j]), 4);
      ptx::mbar_init(ptx::smem_u32(&sh.worker[w].afree[j]), 1);
    }
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&sh.tmem_base), kTmemCols);
    ptx::tmem_relinquish();
  }
  // Activation rows no gather ever fills must not hold NaN patterns: zero the activation
  // part of every stage (the weight part is always written in full by the TMA).
  {
    const uint32_t x_vecs = x_bytes / 16;
    const uint32_t total = kDecWorkers * stages * x_vecs;
    for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
      const uint32_t stage_index = i / x_vecs;
      reinterpret_cast<uint4*>(smem + stage_index * stage_bytes)[i - stage_index * x_vecs] =
          make_uint4(0, 0, 0, 0);
    }
  }
  // Up to here nothing an earlier kernel of the stream may still be writing has been
  // read: with programmatic dependent launch the set-up above overlaps that kernel's tail.
  ptx::grid_dependency_wait();
  if (threadIdx.x == 0) {
    if (p.mode == kModeMasked) {
      int32_t acc = 0;
      for (int32_t g = 0; g < p.num_experts; ++g) {
        sh.group_prefix[g] = acc;
        int32_t mm = __ldg(p.masked_m + g);
        mm = mm < 0 ? 0 : (mm > p.max_m ? p.max_m : mm);
        acc += (mm + p.tile_tokens - 1) / p.tile_tokens;
      }
      sh.group_prefix[p.num_experts] = acc;
      sh.m_blocks = acc;
    } else {
      int32_t padded = __ldg(p.num_tokens_padded);
      padded = padded < 0 ? 0 : (padded > p.sorted_len ? p.sorted_len : padded);
      const int32_t blocks = padded / p.tile_tokens;
      sh.m_blocks = blocks > p.expert_len ? p.expert_len : blocks;
    }
  }
  ptx::fence_proxy_async();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  ptx::grid_launch_dependents();

  const uint32_t tmem_base = __shfl_sync(0xffffffffu, sh.tmem_base, 0);  // uniform, see `warp`
  const uint32_t abort_addr = ptx::smem_u32(&sh.abort_flag);  // raised by any wait that gives up
  const int32_t tiles = __shfl_sync(0xffffffffu, sh.m_blocks, 0) * ((p.n >> fuse) / kBlockN);
  // warps 0-3 feed, warps 4-7 issue the MMAs, warps 8-23 are the four workers
  const uint32_t wk = warp < 8 ? (warp & 3u) : (warp - 8) >> 2;
  // Worker ids interleave the CTAs (worker w of CTA c is c + w * grid), so that a launch
  // with fewer slices than workers spreads them over all SMs first.
  const int32_t worker_id = static_cast<int32_t>(wk * gridDim.x + blockIdx.x);
  SegmentIterator iter;
  iter.init(tiles, k_steps, static_cast<int32_t>(gridDim.x) * kDecWorkers, worker_id);
  Segment seg;
  DecodeWorkerShared& ws = sh.worker[wk];
  const uint32_t ring = ptx::smem_u32(smem + wk * worker_bytes);  // shared address of stage 0
  const uint32_t wfull0 = ptx::smem_u32(&ws.wfull[0]);
  const uint32_t wempty0 = ptx::smem_u32(&ws.wempty[0]);
  const uint32_t xfull0 = ptx::smem_u32(&ws.xfull[0]);
  const uint32_t xempty0 = ptx::smem_u32(&ws.xempty[0]);
  const uint32_t afree0 = ptx::smem_u32(&ws.afree[0]);
  const uint32_t afull0 = ptx::smem_u32(&ws.afull[0]);
  const uint32_t col0 = wk * 128u;  // this worker's tensor-memory columns

  if (warp < 4) {
    // ------------------------- feeder of worker `warp`: weights, scales, activations --
    // The two halves of a stage have different lifetimes: the packed weights and scales
    // are free again as soon as the worker's warps hold them in registers, the
    // activation rows only when the MMAs that read them have completed.  The feeder
    // therefore walks the worker's stage sequence twice: `wsm` (lane 0: two TMA boxes per
    // stage) runs stages - 2 stages ahead of `xsm` (all lanes: cp.async gather, lane l
    // fetching the 16-byte piece l % 8 of rows l / 8 + 4 b, b < mma_n / 4, of both K halves).  In steady
    // state both waits below are over when they are reached, and the weight stream stays
    // a full ring ahead of the workers.
    const uint32_t piece = lane & 7u;
    const uint32_t r0 = lane >> 3;
    uint32_t dst_off[2];
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const uint32_t r = r0 + 4u * b;
      dst_off[b] = r * 128u + ((piece ^ (r & 7u)) << 4);
    }
    StepStream wsm, xsm;
    wsm.init(tiles, k_steps, static_cast<int32_t>(gridDim.x) * kDecWorkers, worker_id);
    xsm = wsm;
    StageCursor wcur, xcur, xdone;
    bool x_pending = false;
    const int32_t w_lead = static_cast<int32_t>(stages) - 2;
    int32_t w_ahead = 0;
    bool w_more = true;
    uint32_t bad = 0;
    int32_t w_row = 0, s_row = 0, w_col = 0;
    int32_t x_off[8];
    uint32_t active = 0;  // bit b: some lane has a row to fetch in round b
    const __nv_bfloat16* src = p.x;
    while (bad == 0) {
      while (w_more && w_ahead <= w_lead) {
        bool first = false;
        if (!wsm.next(p, sh.group_prefix, first)) {
          w_more = false;
          break;
        }
        if (fuse) {
          // stage u of the tile: K block u / 2 of the gate (u even) or up (u odd) block
          w_row = wsm.t.expert * (p.k / 16) + (wsm.kb >> 1) * (kDecStageK / 16);
          s_row = wsm.t.expert * (p.k / 32) + (wsm.kb >> 1) * (kDecStageK / 32);
          w_col = wsm.t.n0 + (wsm.kb & 1) * (p.n >> 1);
        } else if (first) {
          w_row = wsm.t.expert * (p.k / 16) + wsm.kb * (kDecStageK / 16);
          s_row = wsm.t.expert * (p.k / 32) + wsm.kb * (kDecStageK / 32);
          w_col = wsm.t.n0;
        }
        ptx::mbar_wait_sticky(wempty0 + wcur.s * 8u, wcur.ph ^ 1u, abort_addr, bad);
        if (bad != 0) break;
        if (lane == 0) {
          const uint32_t st = ring + wcur.s * stage_bytes + x_bytes;
          const uint32_t full = wfull0 + wcur.s * 8u;
          ptx::mbar_arrive_expect_tx(full, kDecWSBytes);
          ptx::tma_load_2d(st, &tm_w, full, 2 * w_col, w_row);
          ptx::tma_load_2d(st + kDecWBytes, &tm_s, full, w_col, s_row);
        }
        __syncwarp();
        w_row += kDecStageK / 16;
        s_row += kDecStageK / 32;
        wcur.advance(stages);
        ++w_ahead;
      }
      if (bad != 0) break;
      bool first = false;
      if (!xsm.next(p, sh.group_prefix, first)) break;
      if (first) {
        active = 0;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          const int32_t slot = static_cast<int32_t>(r0) + 4 * b;
          int32_t off = -1;
          if (slot < xsm.t.ntok) {
            const int32_t row = x_row_of(p, xsm.t, slot);
            if (row < p.x_rows) off = row * p.k;
          }
          x_off[b] = off;
          if (__ballot_sync(0xffffffffu, off >= 0) != 0) active |= 1u << b;
        }
        src = p.x + xsm.kb * kDecStageK + piece * 8;
      }
      if (fuse) src = p.x + (xsm.kb >> 1) * kDecStageK + piece * 8;  // both blocks read the same K block
      ptx::mbar_wait_sticky(xempty0 + xcur.s * 8u, xcur.ph ^ 1u, abort_addr, bad);
      if (bad != 0) break;
      const uint32_t xs = ring + xcur.s * stage_bytes;
      const bool second_half = !(k_tail_half && xsm.kb == k_steps - 1);
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        if (((active >> b) & 1u) && x_off[b] >= 0) {
          const uint32_t dst = xs + dst_off[b & 1] + (b >> 1) * 1024u;
          ptx::cp_async_16(dst, src + x_off[b], true);
          if (second_half) ptx::cp_async_16(dst + x_half_bytes, src + x_off[b] + kDecStepK, true);
        }
      }
      ptx::cp_async_commit();
      // The previous step's rows have landed by now: make them visible to the tensor
      // core (they were written through the generic proxy) and publish them.  (Publishing
      // two steps late instead, to keep the wait off the feeder's path, measured 2 % slower.)
      if (x_pending) {
        ptx::cp_async_wait_group<1>();
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(xfull0 + xdone.s * 8u);
        xdone.advance(stages);
      }
      x_pending = true;
      src += kDecStageK;
      xcur.advance(stages);
      --w_ahead;
    }
    // Publish the last step (also when leaving on a timeout: nothing may stay in
    // flight towards shared memory when the CTA retires).
    ptx::cp_async_wait_all();
    ptx::fence_proxy_async();
    __syncwarp();
    if (x_pending && lane == 0) ptx::mbar_arrive(xfull0 + xdone.s * 8u);
    if (bad != 0 && lane == 0 && p.status) atomicOr(p.status, kStatusProducerTimeout);
    __syncwarp();
  } else if (warp < 8) {
    // ------------------------------------------------- MMA issuer of worker `warp - 4` --
    // One tcgen05.mma costs its issuing thread some tens of cycles whatever its size, and
    // a 64-wide step needs four: kept off the warps that dequantise.  A stage carries two
    // steps (one operand slot each); the activation half of the stage goes back to the
    // feeder with the second one.
    // This warp's loop is the critical path of the kernel (measured: the workers' warps
    // wait for free operand slots a fifth of their time while this loop takes as long per
    // step as the whole step), and what it costs is a chain of dependent scalar
    // instructions on a scheduler it shares with four dequantising warps: so the operand
    // descriptor is formed once and advanced by additions, the four MMAs of a step are one
    // statement, and nothing else is computed between the wait and the issue.
    const uint32_t d_tm = tmem_base + col0 + kDecDCol;
    const uint32_t a_tm0 = tmem_base + col0;
    const uint64_t xdesc_ring = ptx::smem_desc_k_sw128(ring);  // activation rows of stage 0, first K half
    const uint32_t stage_units = stage_bytes >> 4, half_units = x_half_bytes >> 4;  // descriptor units: 16 bytes
    StageCursor cur, slot;
    uint32_t cur_units = 0;  // cur.s * stage_units
    uint32_t bad = 0;
    while (bad == 0 && iter.next(seg)) {
      const TileInfo t = decode_tile_small(p, sh.group_prefix, seg.tile);
      if (!t.valid) continue;
      const uint32_t idesc = ptx::idesc_bf16_f32(kBlockN, static_cast<uint32_t>(t.mma_n));
      uint32_t acc = 0;
      uint32_t started = 0;  // fused SiLU*mul: bit b = block b's accumulator holds a sum already
      for (int32_t kb = seg.kb; bad == 0 && kb < seg.ke; ++kb) {
        // No wait is needed for the accumulator: the first store of a segment follows
        // its warp's share of the previous segment's epilogue.
        const int32_t halves = (k_tail_half && kb == k_steps - 1) ? 1 : 2;
        uint32_t d_blk = d_tm;
        if (fuse) {
          const uint32_t blk = static_cast<uint32_t>(kb) & 1u;
          d_blk = d_tm + blk * 16u;
          acc = (started >> blk) & 1u;
          started |= 1u << blk;
        }
        uint64_t xdesc = xdesc_ring + cur_units;
        for (int32_t h = 0; h < halves; ++h) {
          ptx::mbar_wait_sticky(afull0 + slot.s * 8u, slot.ph, abort_addr, bad);
          if (h == 0) ptx::mbar_wait_sticky(xfull0 + cur.s * 8u, cur.ph, abort_addr, bad);
          ptx::tc_fence_after();
          if (bad == 0 && ptx::elect_one()) {  // (elected, not `lane == 0`: measured 1.5 % faster)
            ptx::mma_ts_k64(d_blk, a_tm0 + slot.s * 32u, xdesc, idesc, acc);
            if (h == halves - 1) ptx::mma_commit(xempty0 + cur.s * 8u);
            ptx::mma_commit(afree0 + slot.s * 8u);
          }
          __syncwarp();
          acc = 1;
          xdesc += half_units;
          slot.advance(kDecSlots);
        }
        cur.advance(stages);
        cur_units = cur.s == 0 ? 0u : cur_units + stage_units;
      }
    }
    if (bad != 0 && lane == 0 && p.status) atomicOr(p.status, kStatusMmaTimeout);
    __syncwarp();
  } else {
    // ------------------------------------------------------------- worker warps --
    // Inside a segment the four warps run independently: each waits for the stage,
    // dequantises its 32 weight rows, waits for a free operand slot, stores, and tells
    // the issuer.  They meet (named barriers) only in the epilogue of a stream-K slice.
    // A warp whose bounded wait gave up keeps `bad` set (and the CTA's abort flag raised,
    // so that the others' waits give up quickly too), leaves the stage loop at the end
    // of that stage and does no more work, but still walks the remaining segments and
    // meets its siblings at those barriers.
    const uint32_t q = warp & 3;                          // TMEM lane quarter == 32 weight rows
    const uint32_t wt = threadIdx.x - (8 + 4 * wk) * 32;  // 0..127 inside the worker
    const uint32_t bar_id = 1 + wk;
    // This thread's two packed words per K16 row (slabs 2(q&1), 2(q&1)+1 of the 64-row
    // chunk q>>1) and its four scales per K32 group, as offsets into a stage.
    const uint32_t w_off = x_bytes + (q >> 1) * 512u + lane * 16u + (q & 1) * 8u;
    const uint32_t s_off = x_bytes + kDecWBytes + (q >> 1) * 128u + (lane >> 2) * 16u + (q & 1) * 8u;
    const uint32_t a_lane = tmem_base + ((q * 32u) << 16) + col0;
    // Ring positions as running byte offsets (no multiplications in the loop): `stage_off`
    // into the ring, `stage_bar` into the per-stage barrier arrays (8 bytes each),
    // `slot_bar` into the per-slot barrier arrays; one phase bit each.
    const uint32_t ring_bytes = stages * stage_bytes;
    uint32_t stage_off = 0, stage_bar = 0, stage_ph = 0, slot_bar = 0, slot_ph = 0;
    uint32_t bad = 0;  // sticky: set by the first bounded wait that gives up
    const size_t ws_slot = (static_cast<size_t>(kBlockN) * p.mma_n) << fuse;

    auto drain = [&](const Segment& sg, int32_t rows, int32_t n0, uint32_t dcol, int32_t mma_n) {
      if (fuse) {
        // blocks the segment's stages touched: even stages are the gate block, odd ones the up block
        const uint32_t covered = (sg.ke - sg.kb >= 2) ? 3u : (1u << (sg.kb & 1));
        decode_drain_silu(tmem_base + ((q * 32u) << 16) + dcol, p.out + n0 + q * 32, p.out_row_ptr,
                          n0 + static_cast<int32_t>(q) * 32, p.n >> 1, rows, covered, sg.type, sg.peer,
                          p.workspace, ws_slot, worker_id, p.locks, p.lock_spins, p.status,
                          &ws.stage[q][0][0], bar_id, wt, bad == 0);
        return;
      }
      decode_drain(tmem_base + ((q * 32u) << 16) + dcol, p.out + n0 + q * 32, p.out_row_ptr,
                   n0 + static_cast<int32_t>(q) * 32, p.n, rows, mma_n, sg.type,
                   sg.peer, p.workspace, ws_slot, worker_id, p.locks, p.lock_spins, p.status,
                   &ws.stage[q][0][0], bar_id, wt, bad == 0);
    };
    while (iter.next(seg)) {
      const TileInfo t = decode_tile_small(p, sh.group_prefix, seg.tile);
      if (!t.valid) continue;
      // The segment's last stage holds one K half only when K is an odd multiple of 64.
      const bool tail = k_tail_half && seg.ke == k_steps;
      const int32_t n_full = seg.ke - seg.kb - (tail ? 1 : 0);
      // Output row of token slot `lane`: loaded now, used in the epilogue.
      const int32_t my_out_row = out_row_of(p, t, static_cast<int32_t>(lane));
      // One 64-wide step (K half `h` of the stage at `st`), straight-line: the waits
      // record a failure in `bad` and the code runs on (on stale data, within this
      // worker's own shared and tensor memory); `bad` is tested once per stage.
      auto step = [&](auto half, uint32_t st, bool release_weights) {
        constexpr int h = decltype(half)::value;
        // four K16 rows of packed words, two K32 groups of scales
        uint2 words[4], scales[2];
        words[0] = ptx::lds64<4096 * h + 0>(st + w_off);
        words[1] = ptx::lds64<4096 * h + 1024>(st + w_off);
        words[2] = ptx::lds64<4096 * h + 2048>(st + w_off);
        words[3] = ptx::lds64<4096 * h + 3072>(st + w_off);
        scales[0] = ptx::lds64<512 * h + 0>(st + s_off);
        scales[1] = ptx::lds64<512 * h + 256>(st + s_off);
        if (release_weights) {
          // The weight half of the stage goes back to the feeder as soon as its last
          // words are in registers.
          __syncwarp();
          ptx::mbar_arrive_lane0(wempty0 + stage_bar, lane);
        }
        // The operand slot is free once the MMAs of its previous use have completed.
        // Waited for here, before the dequantised values exist.
        const uint32_t afree = afree0 + slot_bar;
        ptx::mbar_wait_sticky(afree, slot_ph ^ 1u, abort_addr, bad);
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          unbias_word(words[i].x, lo + 4 * i);
          unbias_word(words[i].y, hi + 4 * i);
        }
        // scales[g].x = {slab A row r, slab A row r+8} of K32 group g; .y = same for slab B.
        ptx::tc_fence_after();
        const uint32_t a_addr = a_lane + slot_bar * 4u;  // 32 columns per slot
        ptx::tmem_st_16x128b_x8_scaled(a_addr, lo, scales[0].x, scales[1].x);
        ptx::tmem_st_16x128b_x8_scaled(a_addr + (16u << 16), hi, scales[0].y, scales[1].y);
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        // (the wait above is warp-wide: every lane's stores are complete when lane 0 arrives)
        ptx::mbar_arrive_lane0(afull0 + slot_bar, lane);
        slot_bar += 8u;
        if (slot_bar == 8u * kDecSlots) {
          slot_bar = 0;
          slot_ph ^= 1u;
        }
      };
      auto next_stage = [&]() {
        stage_off += stage_bytes;
        stage_bar += 8u;
        if (stage_off == ring_bytes) {
          stage_off = 0;
          stage_bar = 0;
          stage_ph ^= 1u;
        }
      };
      if (bad == 0) {
        for (int32_t j = 0; j < n_full; ++j) {
          const uint32_t st = ring + stage_off;
          ptx::mbar_wait_sticky(wfull0 + stage_bar, stage_ph, abort_addr, bad);
          step(std::integral_constant<int, 0>{}, st, false);
          step(std::integral_constant<int, 1>{}, st, true);
          next_stage();
          if (bad != 0) break;
        }
        if (tail && bad == 0) {
          ptx::mbar_wait_sticky(wfull0 + stage_bar, stage_ph, abort_addr, bad);
          step(std::integral_constant<int, 0>{}, ring + stage_off, true);
          next_stage();
        }
        // ---- end of the segment: wait for its last MMAs.
        // (the slot stored last is the one before the current ring position)
        const uint32_t last_bar = slot_bar == 0 ? 8u * (kDecSlots - 1) : slot_bar - 8u;
        const uint32_t last_ph = slot_bar == 0 ? slot_ph ^ 1u : slot_ph;
        ptx::mbar_wait_sticky(afree0 + last_bar, last_ph, abort_addr, bad);
      }
      // Drain the accumulator.  A warp that has given up skips the work but still meets
      // its siblings at the named barriers of a stream-K slice, here and for every
      // segment that follows.
      drain(seg, my_out_row, t.n0, col0 + kDecDCol, t.mma_n);
    }
    if (bad != 0 && lane == 0 && p.status) atomicOr(p.status, kStatusDequantTimeout);
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace chord
