// Shared host/device helpers of the nb200 kernel library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "nb200.h"

namespace nb200 {

// ---- host-side error reporting -------------------------------------------------------------
// Thread-local text returned by nb200_last_error(); defined in api.cu.
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define NB200_CHECK_CUDA(expr)                                                                   \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess)                                                                       \
      return ::nb200::fail(NB200_ERR_LAUNCH, "%s failed: %s", #expr, cudaGetErrorString(_e));    \
  } while (0)

#define NB200_REQUIRE(cond, code, ...)                                                           \
  do {                                                                                           \
    if (!(cond)) return ::nb200::fail(code, __VA_ARGS__);                                        \
  } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- storage element traits ----------------------------------------------------------------
template <int DT> struct Elem;
template <> struct Elem<NB200_F16> {
  using type = __half;
  using type2 = __half2;
};
template <> struct Elem<NB200_BF16> {
  using type = __nv_bfloat16;
  using type2 = __nv_bfloat162;
};

// Unpack two 16-bit floats held in one 32-bit word to fp32.
template <int DT> __device__ __forceinline__ float2 unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 unpack2<NB200_BF16>(uint32_t w) {
  // a bf16 is the upper half of an fp32
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack2<NB200_F16>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}

// Round two fp32 to the storage type and pack them (lo in the low half).
template <int DT> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<NB200_BF16>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
template <> __device__ __forceinline__ uint32_t pack2<NB200_F16>(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <int DT> __device__ __forceinline__ float load1(const void *p, size_t i);
template <> __device__ __forceinline__ float load1<NB200_BF16>(const void *p, size_t i) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
}
template <> __device__ __forceinline__ float load1<NB200_F16>(const void *p, size_t i) {
  return __half2float(reinterpret_cast<const __half *>(p)[i]);
}
template <> __device__ __forceinline__ float load1<NB200_F32>(const void *p, size_t i) {
  return reinterpret_cast<const float *>(p)[i];
}

template <int DT> __device__ __forceinline__ void store1(void *p, size_t i, float x);
template <> __device__ __forceinline__ void store1<NB200_BF16>(void *p, size_t i, float x) {
  reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(x);
}
template <> __device__ __forceinline__ void store1<NB200_F16>(void *p, size_t i, float x) {
  reinterpret_cast<__half *>(p)[i] = __float2half_rn(x);
}
template <> __device__ __forceinline__ void store1<NB200_F32>(void *p, size_t i, float x) {
  reinterpret_cast<float *>(p)[i] = x;
}

// 2^x on the special-function unit.
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed pair of fp32 in one 64-bit register (Blackwell f32x2 arithmetic).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float2 f2_unpack(uint64_t v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// Three-input maximum (one instruction on sm_100).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

}  // namespace nb200
