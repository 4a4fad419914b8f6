// Device-side pieces of the peer-memory merge of sharded-decode partials, shared by the stand-alone merge kernel
// and by the tail of the fused sharded decode kernel: buffer layout, push of one rank's partial into the peers'
// gather areas, the bounded wait for everybody's arrival, and the log-sum-exp combine over the gathered slots.
// No multicast anywhere: plain stores to one peer at a time, loads of local memory only.
#pragma once

#include "nb200_common.cuh"

namespace nb200 {
namespace peer {

constexpr int kMaxWorld = 16;
constexpr int kD = 128;
constexpr int kErrWait = 31;

struct Ptrs {
  float *buf[kMaxWorld];
};

// A rank's symmetric buffer: two gather areas [world][rows][D + 2] floats (alternating with the call's generation),
// then, 128-byte aligned, two sets of kMaxWorld arrival flags.
__host__ __device__ inline size_t area_floats(int rows, int world) { return (size_t)world * rows * (kD + 2); }
__host__ __device__ inline size_t flags_offset_floats(int rows, int world) { return (2 * area_floats(rows, world) + 31) / 32 * 32; }
__host__ __device__ inline size_t buffer_floats(int rows, int world) { return flags_offset_floats(rows, world) + 2 * kMaxWorld; }

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Threads tid, tid + nthreads, ... of the caller copy this rank's partial (rows * (D + 2) floats, L2-coherent
// loads) into slot `rank` of rank p's area for p in [p_begin, p_end).  The caller then fences (system scope),
// synchronises its threads and calls release_flags.
__device__ __forceinline__ void push(const float *local_partial, const Ptrs &peers, int rows, int world, int rank,
                                     unsigned generation, int p_begin, int p_end, int tid, int nthreads) {
  const int set = static_cast<int>(generation & 1u);
  const size_t slot = (size_t)rows * (kD + 2);
  const float4 *src = reinterpret_cast<const float4 *>(local_partial);
  for (int p = p_begin; p < p_end; ++p) {
    float4 *dst = reinterpret_cast<float4 *>(peers.buf[p] + set * area_floats(rows, world) + rank * slot);
    for (int i = tid; i < static_cast<int>(slot / 4); i += nthreads) dst[i] = __ldcg(src + i);
  }
}
__device__ __forceinline__ void release_flag(const Ptrs &peers, int rows, int world, int rank, unsigned generation, int p) {
  unsigned *flags = reinterpret_cast<unsigned *>(peers.buf[p] + flags_offset_floats(rows, world));
  st_release_sys(flags + (generation & 1u) * kMaxWorld + rank, generation);
}

// Called by thread `r` (< world): waits until rank r's partial of this generation has arrived in this rank's own
// buffer; false after wait_ns, with the status words saying who was missing.
__device__ __forceinline__ bool wait_arrival(const Ptrs &peers, int rows, int world, int rank, unsigned generation, int r,
                                             long long wait_ns, int *status) {
  const unsigned *flag = reinterpret_cast<const unsigned *>(peers.buf[rank] + flags_offset_floats(rows, world)) +
                         (generation & 1u) * kMaxWorld + r;
  const unsigned long long t0 = timer_ns();
  while (ld_acquire_sys(flag) != generation) {
    if (timer_ns() - t0 > static_cast<unsigned long long>(wait_ns)) {
      if (status && atomicCAS(status, 0, kErrWait) == 0) {
        status[1] = static_cast<int>(blockIdx.x);
        status[2] = r;                             // the rank whose partial never arrived
        status[3] = static_cast<int>(generation);
      }
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

// One warp: output row `row` from the `world` gathered slots ([world][rows][D + 2], slot stride in floats).
template <int ODT>
__device__ __forceinline__ void combine_row(const float *gathered, size_t slot, int world, int row, void *out, int lane) {
  const float *base = gathered + (size_t)row * (kD + 2);
  float M = -INFINITY;
  for (int r = 0; r < world; ++r) M = fmaxf(M, __ldcg(base + r * slot + kD));
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
  for (int r = 0; r < world; ++r) {
    const float *ps = base + r * slot;
    const float w = ex2(__ldcg(ps + kD) - Ms);
    const float2 o01 = __ldcg(reinterpret_cast<const float2 *>(ps + lane * 4));
    const float2 o23 = __ldcg(reinterpret_cast<const float2 *>(ps + lane * 4 + 2));
    acc.x += w * o01.x;
    acc.y += w * o01.y;
    acc.z += w * o23.x;
    acc.w += w * o23.y;
    lsum += w * __ldcg(ps + kD + 1);
  }
  if constexpr (ODT == NB200_F32) {
    float *dst = reinterpret_cast<float *>(out) + (size_t)row * (kD + 2);
    dst[lane * 4 + 0] = acc.x;
    dst[lane * 4 + 1] = acc.y;
    dst[lane * 4 + 2] = acc.z;
    dst[lane * 4 + 3] = acc.w;
    if (lane == 0) {
      dst[kD] = M;
      dst[kD + 1] = lsum;
    }
  } else {
    const float inv = lsum == 0.f ? 0.f : 1.f / lsum;
    uint2 w2;
    w2.x = pack2<ODT>(acc.x * inv, acc.y * inv);
    w2.y = pack2<ODT>(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(out) + (size_t)row * kD + lane * 4) = w2;
  }
}

}  // namespace peer
}  // namespace nb200
