// Error reporting, device queries and options behind the C ABI.
#include <cstring>
#include <mutex>

#include "../../include/chord_b200.h"
#include "common.h"

namespace chord {

std::string& last_error_storage() {
  thread_local std::string message;
  return message;
}

Options& options() {
  static Options opts;
  return opts;
}

std::shared_mutex& options_mutex() {
  static std::shared_mutex mutex;
  return mutex;
}

int current_device_info(DeviceInfo* info) {
  constexpr int kMaxDevices = 64;
  static DeviceInfo cache[kMaxDevices];
  static std::mutex mutex;
  int device = 0;
  CHORD_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) {
    return fail(kCudaError, "device index %d out of range", device);
  }
  std::lock_guard<std::mutex> guard(mutex);
  if (cache[device].device != device) {
    DeviceInfo d;
    d.device = device;
    CHORD_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
    CHORD_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, device));
    CHORD_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, device));
    CHORD_CUDA(
        cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    cache[device] = d;
  }
  *info = cache[device];
  return kOk;
}

int require_blackwell(const DeviceInfo& info) {
  if (info.cc_major != 10) {
    return fail(kUnsupportedDevice,
                "chord_b200 kernels are built for sm_100a and need a compute capability 10.x GPU, "
                "got %d.%d on device %d",
                info.cc_major, info.cc_minor, info.device);
  }
  return kOk;
}

}  // namespace chord

extern "C" {

const char* chord_b200_last_error(void) { return chord::last_error_storage().c_str(); }

const char* chord_b200_version(void) { return "chord_b200 sm_100a"; }

int chord_b200_set_option(const char* name, int64_t value) {
  using chord::fail;
  using chord::kInvalidArgument;
  if (name == nullptr) return fail(kInvalidArgument, "option name is null");
  std::unique_lock<std::shared_mutex> guard(chord::options_mutex());
  chord::Options& o = chord::options();
  if (!std::strcmp(name, "x_load")) {
    if (value != 0 && value != 1) return fail(kInvalidArgument, "x_load must be 0 or 1");
    o.x_load = static_cast<int>(value);
  } else if (!std::strcmp(name, "dequant_groups")) {
    if (value != 2 && value != 4) return fail(kInvalidArgument, "dequant_groups must be 2 or 4");
    o.dequant_groups = static_cast<int>(value);
  } else if (!std::strcmp(name, "issuers")) {
    if (value != 0 && value != 1 && value != 2 && value != 4)
      return fail(kInvalidArgument, "issuers must be 0, 1, 2 or 4");
    o.issuers = static_cast<int>(value);
  } else if (!std::strcmp(name, "contiguous_tile")) {
    if (value != 0 && value != 128 && value != 256)
      return fail(kInvalidArgument, "contiguous_tile must be 0, 128 or 256");
    o.contiguous_tile = static_cast<int>(value);
  } else if (!std::strcmp(name, "pregather")) {
    if (value != 0 && value != 1) return fail(kInvalidArgument, "pregather must be 0 or 1");
    o.pregather = static_cast<int>(value);
  } else if (!std::strcmp(name, "ksplit")) {
    if (value != 0 && value != 1) return fail(kInvalidArgument, "ksplit must be 0 or 1");
    o.ksplit = static_cast<int>(value);
  } else if (!std::strcmp(name, "pair")) {
    if (value != 0 && value != 1) return fail(kInvalidArgument, "pair must be 0 or 1");
    o.pair = static_cast<int>(value);
  } else if (!std::strcmp(name, "npair")) {
    if (value != 0 && value != 1) return fail(kInvalidArgument, "npair must be 0 or 1");
    o.npair = static_cast<int>(value);
  } else if (!std::strcmp(name, "decode_kernel")) {
    if (value != 0 && value != 1) return fail(kInvalidArgument, "decode_kernel must be 0 or 1");
    o.decode_kernel = static_cast<int>(value);
  } else if (!std::strcmp(name, "a_stages")) {
    if (value != 0 && (value < 2 || value > 7)) return fail(kInvalidArgument, "a_stages must be 0 or 2..7");
    o.a_stages = static_cast<int>(value);
  } else if (!std::strcmp(name, "max_stages")) {
    if (value < 0 || value > 64) return fail(kInvalidArgument, "max_stages must be in [0, 64]");
    o.max_stages = static_cast<int>(value);
  } else if (!std::strcmp(name, "grid_limit")) {
    if (value < 0) return fail(kInvalidArgument, "grid_limit must be >= 0");
    o.grid_limit = static_cast<int>(value);
  } else if (!std::strcmp(name, "pdl")) {
    if (value != 0 && value != 1) return fail(kInvalidArgument, "pdl must be 0 or 1");
    o.pdl = static_cast<int>(value);
  } else if (!std::strcmp(name, "lock_spins")) {
    if (value < 1 || value > (1 << 24)) return fail(kInvalidArgument, "lock_spins must be in [1, 2^24]");
    o.lock_spins = static_cast<int>(value);
  } else {
    return fail(kInvalidArgument, "unknown option '%s'", name);
  }
  return chord::kOk;
}

}  // extern "C"
