// Shared host/device helpers of the hybrid-cache kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/aptserve_b200.h"

namespace aps {

// ---- error reporting -------------------------------------------------------
char* last_error_buffer();  // thread-local, defined in c_api.cu

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define APS_REQUIRE(cond, code, ...) \
  do {                               \
    if (!(cond)) return ::aps::fail((code), __VA_ARGS__); \
  } while (0)

#define APS_CUDA(expr)                                                          \
  do {                                                                          \
    cudaError_t e__ = (expr);                                                   \
    if (e__ != cudaSuccess)                                                     \
      return ::aps::fail(APS_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

inline int launch_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(APS_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  return APS_OK;
}

inline int dtype_size(int dtype) {
  switch (dtype) {
    case APS_F32: return 4;
    case APS_F16: return 2;
    case APS_BF16: return 2;
    default: return 0;
  }
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Number of SMs of the current device (cached per device).
int sm_count();

// Optional timing hooks (see aps_set_profile_events): events recorded around the
// K/V streaming kernel (which = 0) and the re-projection kernel (which = 1).
struct ProfileEvents { cudaEvent_t start, stop; };
ProfileEvents* profile_events(int which);

struct ScopedProfile {
  ProfileEvents* ev; cudaStream_t stream;
  ScopedProfile(int which, cudaStream_t s) : ev(profile_events(which)), stream(s) {
    if (ev->start) cudaEventRecord(ev->start, stream);
  }
  ~ScopedProfile() { if (ev->stop) cudaEventRecord(ev->stop, stream); }
};

// ---- device helpers ----------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_float(float x) { return x; }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_float(float x) { return __float2half_rn(x); }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float x) { return __float2bfloat16_rn(x); }
};

// Unpack one 16-byte vector of T into floats (8 for 2-byte types, 4 for float).
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};
template <> struct Vec16<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

}  // namespace aps
