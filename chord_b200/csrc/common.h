// Host-side helpers shared by the C-ABI translation units: error reporting,
// argument checks, per-device properties.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <shared_mutex>
#include <string>

namespace chord {

// Return codes of every extern "C" entry point.
enum Status : int {
  kOk = 0,
  kInvalidArgument = 1,   // binder maps to ValueError
  kUnsupportedDevice = 2, // binder maps to RuntimeError
  kCudaError = 3,         // binder maps to RuntimeError
};

std::string& last_error_storage();

inline int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error_storage() = buf;
  return code;
}

#define CHORD_REQUIRE(cond, ...)                                   \
  do {                                                             \
    if (!(cond)) return ::chord::fail(::chord::kInvalidArgument, __VA_ARGS__); \
  } while (0)

#define CHORD_CUDA(call)                                                              \
  do {                                                                                \
    cudaError_t err__ = (call);                                                       \
    if (err__ != cudaSuccess)                                                         \
      return ::chord::fail(::chord::kCudaError, "%s failed: %s", #call,               \
                           cudaGetErrorString(err__));                                \
  } while (0)

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
  int max_smem_optin = 0;
};

// Properties of the current device (cached per device).  Returns nonzero and
// sets the last error on failure.
int current_device_info(DeviceInfo* info);

// Requires compute capability 10.x; the kernels are built for sm_100a only.
int require_blackwell(const DeviceInfo& info);

// Tuning knobs settable through chord_b200_set_option().
struct Options {
  int x_load = 0;          // indexed activation gather: 0 = cp.async helper warps, 1 = TMA gather4
  int dequant_groups = 2;  // 2 or 4 groups of four dequant warps
  int issuers = 0;         // 0 = automatic; 1, 2 or 4 MMA issuers
  int contiguous_tile = 0; // 0 / 256 = merge neighbouring 128-row blocks of one expert; 128 = do not
  int a_stages = 0;        // 0 = automatic; depth of the TMEM operand ring (2..7)
  int pregather = 1;       // 1 = `indexed` with blocks of >= 64 rows copies the routed rows into slot order first
  int pair = 1;            // 1 = tiles of more than 128 tokens with consecutive activation rows and K >= 2048 run on clusters of two CTAs (tcgen05.mma.cta_group::2)
  int npair = 1;           // 1 = tiles of <= 128 tokens with consecutive activation rows span two 128-row weight blocks
  int ksplit = 1;          // 1 = layouts with one MMA issuer split small tiles' K halves over two issuers
  int decode_kernel = 1;   // 1 = token tiles of <= 32 rows (indexed, masked) use the warpgroup-per-worker kernel; 0 = never
  int max_stages = 0;      // 0 = as many as fit
  int grid_limit = 0;      // 0 = one CTA per SM
  int pdl = 0;             // 1 = `indexed` launches carry the programmatic stream-serialization attribute
  int lock_spins = 1 << 22;  // polls (64 ns apart) of a stream-K owner on its lock word before it gives up
};
Options& options();

// Kernel launch with, optionally, the programmatic stream-serialization attribute
// (programmatic dependent launch): the kernel may then become resident while its
// predecessor in the stream drains, and synchronises with it through
// griddepcontrol.wait.  The reference sets the same attribute for `enable_pdl`
// (chord_kernels/operator/csrc/launcher/launcher.cpp:440-451).
template <typename... Params, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, bool pdl, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// The same launch as clusters of two CTAs along x (grid.x even).
template <typename... Params, typename... Args>
inline cudaError_t launch_kernel_pairs(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, bool pdl, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
// chord_b200_set_option() writes the options under the exclusive lock; every entry
// point that reads them holds the shared lock for the length of its host-side work, so
// a launch sees one consistent set.
std::shared_mutex& options_mutex();
using OptionsReadLock = std::shared_lock<std::shared_mutex>;

}  // namespace chord
