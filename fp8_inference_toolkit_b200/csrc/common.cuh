// Shared host/device helpers for the int4tc_b200 library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/int4tc_b200.h"

namespace i4tc {

// ---- per-thread error message ------------------------------------------------
inline char* err_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int cuda_fail(cudaError_t e, const char* what) {
  snprintf(err_buf(), 512, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return (int)e;
}

#define I4TC_CUDA(expr)                                   \
  do {                                                    \
    cudaError_t _e = (expr);                              \
    if (_e != cudaSuccess) return ::i4tc::cuda_fail(_e, #expr); \
  } while (0)

#define I4TC_REQUIRE(cond, code, ...)                     \
  do {                                                    \
    if (!(cond)) return ::i4tc::fail((code), __VA_ARGS__); \
  } while (0)

// Makes `device` current for the scope of one C-ABI call and restores the previous one.
struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int device) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != device) {
      err = cudaSetDevice(device);
      changed = (err == cudaSuccess);
    }
  }
  ~DeviceGuard() {
    if (changed) cudaSetDevice(prev);
  }
};

struct DeviceInfo {
  bool valid = false;
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
  int max_smem_optin = 0;
  unsigned int* status = nullptr;  // device status word written by bounded waits
};

// Cached per-device properties; allocates the status word on first use.
int device_info(int device, const DeviceInfo** out);
// Returns the library-owned split-K workspace of (`device`, `stream`), at least `bytes` large.  A buffer that was
// handed out is never freed or moved: when a stream needs more than it has, a larger buffer is allocated beside
// the old one (which stays valid for launches and CUDA graphs that already hold it).
int split_workspace(int device, cudaStream_t stream, size_t bytes, float** out);

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Vectorised clipped-symmetric / asymmetric per-group quantiser (quant.cu); the caller has validated the sizes and
// holds the device.  grouped_ext_fast_ok: the pointers and the row stride allow its 128-bit accesses.
bool grouped_ext_fast_ok(const void* x, int64_t ldx, const uint8_t* packed);
int launch_grouped_ext(bool asym, const void* x, int dtype, int64_t rows, int64_t K, int64_t ldx, int gs, float clip,
                       uint8_t* packed, float* scale, float* azp_adj, cudaStream_t st);

// ---- device helpers ------------------------------------------------------------
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(float v) { return v; }

// clamp(rint(x / s), -8, 7) with IEEE division and round-half-even; returns the 4-bit code.
__device__ __forceinline__ uint32_t code4(float x, float s) {
  float q = rintf(__fdiv_rn(x, s));
  q = fminf(fmaxf(q, -8.0f), 7.0f);
  return static_cast<uint32_t>(static_cast<int>(q)) & 0xFu;
}

}  // namespace i4tc
