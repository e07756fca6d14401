// Weight packer and scale permutation (load-time, integer / data-movement only).
//
// Output format, bit-exact with the reference's repack kernel
// (chord_kernels/operator/include/humming/kernel/repack.cuh:8-121 launched with
// interleave_mode 3, chord_kernels/operator/kernel/repack_weight.py:41-77):
//   packed int32 [E, K/16, 2N]; for word c of row kb let nb = c / 128,
//   t = (c % 128) / 4, s = c % 4; for rh, kh, kk in {0, 1} the 4-bit code of
//   weight (n, k) = (64 nb + 16 s + 8 rh + t / 4, 16 kb + 8 kh + 2 (t % 4) + kk)
//   sits at bit 4 (2 rh + kh) + 16 kk.
// The kernels below are organised around the output: one thread assembles one
// 16-byte vector (the four slabs s = 0..3 of one (kb, nb, t)), so stores are
// fully coalesced, and a CTA stages its 64-row x kTileK input tile in shared
// memory as nibbles with coalesced vector loads.
#include "../../include/chord_b200.h"
#include "common.h"

namespace chord {
namespace {

constexpr int kRows = 64;  // weight rows per CTA tile (one 64-row chunk)

// Shared tile: kRows rows of kTileK nibbles, eight nibbles per word
// (little-endian, i.e. the checkpoint form), one pad word per row against bank
// conflicts.
template <int kTileK, bool kPackedInput>
__global__ void __launch_bounds__(256)
repack_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int n, int k,
              int32_t* __restrict__ range_flag) {
  constexpr int kWordsPerRow = kTileK / 8;
  __shared__ uint32_t tile[kRows][kWordsPerRow + 1];
  const int nb = blockIdx.x;
  const int k0 = blockIdx.y * kTileK;
  const int e = blockIdx.z;
  const int tid = threadIdx.x;
  const int k_here = min(kTileK, k - k0);  // multiple of 16

  if constexpr (kPackedInput) {
    const size_t row_words = static_cast<size_t>(k) / 8;
    const uint32_t* src = in + (static_cast<size_t>(e) * n + static_cast<size_t>(nb) * kRows) * row_words + k0 / 8;
    for (int i = tid; i < kRows * kWordsPerRow; i += blockDim.x) {
      const int r = i / kWordsPerRow, w = i % kWordsPerRow;
      tile[r][w] = (w * 8 < k_here) ? __ldg(src + r * row_words + w) : 0u;
    }
  } else {
    const uint32_t* src = in + (static_cast<size_t>(e) * n + static_cast<size_t>(nb) * kRows) * k + k0;
    bool bad = false;
    for (int i = tid; i < kRows * kWordsPerRow; i += blockDim.x) {
      const int r = i / kWordsPerRow, w = i % kWordsPerRow;
      uint32_t word = 0;
      if (w * 8 < k_here) {
        const uint4* p = reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * k + w * 8);
        const uint4 a = __ldg(p), b = __ldg(p + 1);
        const uint32_t c[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          bad |= c[j] > 15u;
          word |= (c[j] & 15u) << (4 * j);
        }
      }
      tile[r][w] = word;
    }
    if (bad && range_flag != nullptr) atomicOr(range_flag, 1);
  }
  __syncthreads();

  // One uint4 per (kb, t): words s = 0..3 of packed row kb, columns 128 nb + 4 t + s.
  const int kb_count = k_here / 16;
  for (int i = tid; i < kb_count * 32; i += blockDim.x) {
    const int kbl = i >> 5, t = i & 31;
    const int r8 = t >> 2, q = t & 3;
    uint32_t words[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      uint32_t word = 0;
#pragma unroll
      for (int rh = 0; rh < 2; ++rh) {
        const int row = 16 * s + 8 * rh + r8;
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
          // K offsets 16 kbl + 8 kh + 2 q + {0, 1}: two adjacent nibbles of one tile word.
          const uint32_t src = tile[row][2 * kbl + kh];
          const uint32_t pair = (src >> (8 * q)) & 0xFFu;
          word |= (pair & 0xFu) << (4 * (2 * rh + kh));
          word |= (pair >> 4) << (4 * (2 * rh + kh) + 16);
        }
      }
      words[s] = word;
    }
    const size_t out_row = static_cast<size_t>(e) * (k / 16) + (k0 / 16) + kbl;
    uint4* dst = reinterpret_cast<uint4*>(out + out_row * (2 * static_cast<size_t>(n)) + 128 * nb + 4 * t);
    *dst = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

// out[e, g, 64 c + j] = in[e, 64 c + 8 (j % 8) + j / 8, g]
__global__ void __launch_bounds__(256)
permute_scale_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int n, int groups) {
  // 64 rows (one chunk) x 64 groups per CTA, transposed through shared memory.
  __shared__ uint16_t tile[64][64 + 2];
  const int c = blockIdx.x, g0 = blockIdx.y * 64, e = blockIdx.z;
  const int tid = threadIdx.x;
  const uint16_t* src = in + (static_cast<size_t>(e) * n + static_cast<size_t>(c) * 64) * groups;
  for (int i = tid; i < 64 * 64; i += blockDim.x) {
    const int r = i >> 6, g = i & 63;
    if (g0 + g < groups) tile[r][g] = src[static_cast<size_t>(r) * groups + g0 + g];
  }
  __syncthreads();
  for (int i = tid; i < 64 * 64; i += blockDim.x) {
    const int g = i >> 6, j = i & 63;
    if (g0 + g < groups) {
      const int row = 8 * (j & 7) + (j >> 3);
      out[(static_cast<size_t>(e) * groups + g0 + g) * n + static_cast<size_t>(c) * 64 + j] = tile[row][g];
    }
  }
}

}  // namespace
}  // namespace chord

extern "C" {

int chord_b200_repack_w4a16(const int32_t* in, int32_t* out, int64_t num_experts, int64_t n,
                            int64_t k, int packed_input, int32_t* range_flag, void* stream) {
  CHORD_REQUIRE(in != nullptr && out != nullptr, "null tensor pointer");
  CHORD_REQUIRE(num_experts > 0 && n > 0 && k > 0, "weight dimensions must be non-zero");
  CHORD_REQUIRE(n % 128 == 0, "shape_n must be divisible by 128, got %lld", static_cast<long long>(n));
  CHORD_REQUIRE(k % 64 == 0, "shape_k must be divisible by 64, got %lld", static_cast<long long>(k));
  CHORD_REQUIRE(num_experts <= 65535 && n * 2 < (1ll << 31) && k < (1ll << 31), "weight too large");
  CHORD_REQUIRE((reinterpret_cast<uintptr_t>(in) & 15u) == 0 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0,
                "weight tensors must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t* src = reinterpret_cast<const uint32_t*>(in);
  uint32_t* dst = reinterpret_cast<uint32_t*>(out);
  if (packed_input) {
    constexpr int kTileK = 256;
    const dim3 grid(static_cast<unsigned>(n / 64), static_cast<unsigned>((k + kTileK - 1) / kTileK),
                    static_cast<unsigned>(num_experts));
    chord::repack_kernel<kTileK, true><<<grid, 256, 0, s>>>(src, dst, static_cast<int>(n),
                                                           static_cast<int>(k), nullptr);
  } else {
    constexpr int kTileK = 64;
    const dim3 grid(static_cast<unsigned>(n / 64), static_cast<unsigned>(k / kTileK),
                    static_cast<unsigned>(num_experts));
    chord::repack_kernel<kTileK, false><<<grid, 256, 0, s>>>(src, dst, static_cast<int>(n),
                                                            static_cast<int>(k), range_flag);
  }
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

int chord_b200_permute_scale(const void* in, void* out, int64_t num_experts, int64_t n, int64_t k,
                             void* stream) {
  CHORD_REQUIRE(in != nullptr && out != nullptr, "null tensor pointer");
  CHORD_REQUIRE(num_experts > 0 && n > 0 && k > 0, "scale dimensions must be non-zero");
  CHORD_REQUIRE(n % 64 == 0 && k % 32 == 0, "need N %% 64 == 0 and K %% 32 == 0");
  CHORD_REQUIRE(num_experts <= 65535, "too many experts");
  const int groups = static_cast<int>(k / 32);
  const dim3 grid(static_cast<unsigned>(n / 64), static_cast<unsigned>((groups + 63) / 64),
                  static_cast<unsigned>(num_experts));
  chord::permute_scale_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out), static_cast<int>(n), groups);
  CHORD_CUDA(cudaGetLastError());
  return chord::kOk;
}

}  // extern "C"
