// Host-side helpers: tensor-map construction through the driver entry point (no link-time
// dependency on libcuda), argument checks, the per-device status word.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nsa {

// Error codes returned by every extern "C" entry point.
//   0                ok
//   -1               invalid argument (null pointer, bad size, misaligned stride)
//   -2               unsupported configuration (head_dim, group size, block size ...)
//   -3               scratch / workspace too small
//   -4               device reported a bounded-wait timeout or a bad index (see nsa_last_device_status)
//   1000 + cudaError a CUDA runtime call failed
enum : int { kOk = 0, kInvalid = -1, kUnsupported = -2, kWorkspace = -3, kDeviceStatus = -4 };

inline int cuda_rc(cudaError_t e) { return e == cudaSuccess ? 0 : 1000 + static_cast<int>(e); }

// 3-D tensor map over a [n2][n1][n0] array of 16-bit elements (n0 contiguous).
// stride1/stride2 in ELEMENTS.  Box = (b0, b1, b2), 128-byte swizzle when b0*2 == 128, none otherwise.
int make_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t n0, uint64_t n1, uint64_t n2,
                 uint64_t stride1, uint64_t stride2, uint32_t b0, uint32_t b1, uint32_t b2);

// 4-D variant over [n3][n2][n1][n0]; box (b0, 1, b2, b3).
int make_tmap_4d(CUtensorMap* out, CUtensorMapDataType dt, const void* base, uint64_t n0, uint64_t n1, uint64_t n2,
                 uint64_t n3, uint64_t stride1, uint64_t stride2, uint64_t stride3, uint32_t b0, uint32_t b2,
                 uint32_t b3 = 1);

// device status word of the current device (allocated on first use, zero-initialised)
int* status_word();
// read-and-clear; returns the OR of error bits raised by kernels since the last call
int read_status(cudaStream_t stream);

// Launch accounting.  Every kernel launch of the library sits inside a LaunchScope: it always bumps a
// process-wide launch counter and, when profiling is enabled (nsa_profile_enable), brackets the launch
// with CUDA events on the launching stream so that per-kernel device time can be read back.
void launch_begin(const char* tag, cudaStream_t stream);
void launch_end(cudaStream_t stream);
struct LaunchScope {
  cudaStream_t s;
  LaunchScope(const char* tag, cudaStream_t stream) : s(stream) { launch_begin(tag, stream); }
  ~LaunchScope() { launch_end(s); }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace nsa
