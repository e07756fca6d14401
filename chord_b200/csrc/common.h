// Host-side helpers shared by the C-ABI translation units: error reporting,
// argument checks, per-device properties.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
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
  int ksplit = 1;          // 1 = layouts with one MMA issuer split small tiles' K halves over two issuers
  int decode_kernel = 1;   // 1 = token tiles of <= 32 rows (indexed, masked) use the warpgroup-per-worker kernel; 0 = never
  int max_stages = 0;      // 0 = as many as fit
  int grid_limit = 0;      // 0 = one CTA per SM
  int ablate = 0;          // CHORD_PROFILE builds: bit mask of work to skip in timing studies
  long long profile_buffer = 0;  // device pointer for per-CTA cycle counters (CHORD_PROFILE builds)
};
Options& options();

}  // namespace chord
