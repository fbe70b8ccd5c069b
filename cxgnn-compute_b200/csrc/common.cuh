// Shared helpers of the sm_100a kernels: error reporting for the C ABI, index
// loads of either width, 128-bit feature vectors in fp32 / bf16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/cxgnn_b200.h"

namespace cxg {

// Number of SMs the grids are sized for (B200: 2 dies x 74).
constexpr int kNumSM = 148;

int set_error(int code, const char *fmt, ...);
int check_launch(const char *what);
// Adds n to the process-wide count of kernels this library has launched.
void count_launches(int n);
// Cycle limit of one bounded device-side wait (cxg_set_wait_limit_cycles; default about a second).
long long wait_limit_cycles();

#define CXG_REQUIRE(cond, code, ...)                   \
  do {                                                 \
    if (!(cond)) return cxg::set_error(code, __VA_ARGS__); \
  } while (0)

static inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ptr entries are read twice per row, so their width is a run-time switch.
__device__ __forceinline__ int64_t load_ptr(const void *ptr, int64_t i, int ptr_bytes) {
  return ptr_bytes == 8 ? __ldg(reinterpret_cast<const int64_t *>(ptr) + i)
                        : static_cast<int64_t>(__ldg(reinterpret_cast<const int32_t *>(ptr) + i));
}

// 16-byte feature vector: 4 floats or 8 bf16, accumulated in fp32.
template <typename T>
struct Vec;

template <>
struct Vec<float> {
  static constexpr int kElems = 4;
  using Raw = float4;
  __device__ __forceinline__ static Raw load(const float *p) {
    return __ldg(reinterpret_cast<const float4 *>(p));
  }
  __device__ __forceinline__ static void add(float *acc, const Raw &v) {
    acc[0] += v.x;
    acc[1] += v.y;
    acc[2] += v.z;
    acc[3] += v.w;
  }
  __device__ __forceinline__ static void fma(float *acc, const Raw &v, float s) {
    acc[0] = fmaf(v.x, s, acc[0]);
    acc[1] = fmaf(v.y, s, acc[1]);
    acc[2] = fmaf(v.z, s, acc[2]);
    acc[3] = fmaf(v.w, s, acc[3]);
  }
  __device__ __forceinline__ static void to_float(float *out, const Raw &v) {
    out[0] = v.x;
    out[1] = v.y;
    out[2] = v.z;
    out[3] = v.w;
  }
  __device__ __forceinline__ static Raw from_float(const float *a) {
    return make_float4(a[0], a[1], a[2], a[3]);
  }
  __device__ __forceinline__ static void store_stream(float *p, const Raw &v) {
    __stcs(reinterpret_cast<float4 *>(p), v);
  }
  __device__ __forceinline__ static Raw load_plain(const float *p) {
    return *reinterpret_cast<const float4 *>(p);
  }
};

template <>
struct Vec<__nv_bfloat16> {
  static constexpr int kElems = 8;
  using Raw = uint4;
  __device__ __forceinline__ static Raw load(const __nv_bfloat16 *p) {
    return __ldg(reinterpret_cast<const uint4 *>(p));
  }
  // bf16 -> fp32 is a 16-bit shift of the bit pattern.
  __device__ __forceinline__ static void to_float(float *out, const Raw &v) {
    out[0] = __uint_as_float(v.x << 16);
    out[1] = __uint_as_float(v.x & 0xffff0000u);
    out[2] = __uint_as_float(v.y << 16);
    out[3] = __uint_as_float(v.y & 0xffff0000u);
    out[4] = __uint_as_float(v.z << 16);
    out[5] = __uint_as_float(v.z & 0xffff0000u);
    out[6] = __uint_as_float(v.w << 16);
    out[7] = __uint_as_float(v.w & 0xffff0000u);
  }
  __device__ __forceinline__ static void add(float *acc, const Raw &v) {
    float f[8];
    to_float(f, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += f[i];
  }
  __device__ __forceinline__ static void fma(float *acc, const Raw &v, float s) {
    float f[8];
    to_float(f, v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(f[i], s, acc[i]);
  }
  __device__ __forceinline__ static Raw from_float(const float *a) {
    uint4 r;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(a[0], a[1]);
    r.x = *reinterpret_cast<uint32_t *>(&t);
    t = __floats2bfloat162_rn(a[2], a[3]);
    r.y = *reinterpret_cast<uint32_t *>(&t);
    t = __floats2bfloat162_rn(a[4], a[5]);
    r.z = *reinterpret_cast<uint32_t *>(&t);
    t = __floats2bfloat162_rn(a[6], a[7]);
    r.w = *reinterpret_cast<uint32_t *>(&t);
    return r;
  }
  __device__ __forceinline__ static void store_stream(__nv_bfloat16 *p, const Raw &v) {
    __stcs(reinterpret_cast<uint4 *>(p), v);
  }
  __device__ __forceinline__ static Raw load_plain(const __nv_bfloat16 *p) {
    return *reinterpret_cast<const uint4 *>(p);
  }
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// One scalar element per lane: rows whose width is not a multiple of a 16-byte
// vector (F = 47, 1, 33 ...).
template <typename T>
struct Scalar {
  static constexpr int kElems = 1;
  using Raw = T;
  __device__ __forceinline__ static Raw load(const T *p) { return __ldg(p); }
  __device__ __forceinline__ static void add(float *acc, const Raw &v) { acc[0] += to_f32(v); }
  __device__ __forceinline__ static void fma(float *acc, const Raw &v, float s) {
    acc[0] = fmaf(to_f32(v), s, acc[0]);
  }
  __device__ __forceinline__ static void to_float(float *out, const Raw &v) { out[0] = to_f32(v); }
  __device__ __forceinline__ static Raw from_float(const float *a) { return from_f32<T>(a[0]); }
  __device__ __forceinline__ static void store_stream(T *p, const Raw &v) { *p = v; }
  __device__ __forceinline__ static Raw load_plain(const T *p) { return *p; }
};


}  // namespace cxg
