// Mamba-1 selective scan forward.
//
//   h[b,d,n] <- exp(delta*A[d,n]) h + delta*Bm[b,n,t]*u ;  y = sum_n Cm[b,n,t] h + Dskip[d] u ;
//   out = y * silu(z)
//
// The recurrence is sequential in t, so the parallelism is the (b, d, n) index space.  Algorithmic
// HBM traffic is tiny next to the arithmetic (one exp per state update), so the kernel is organised
// around the special-function and fp32 pipes while keeping every global access a full coalesced
// row segment:
//   * one CTA = one sequence b and 32 channels d; 64 threads = 32 channels x 2 groups of 8 states;
//     a thread keeps its 8 states and 8 decay rates in registers for the whole sequence (8 rather
//     than 4 states per thread spreads the per-step scalar work over more updates: 5 % faster);
//   * u, delta, z, Bm, Cm are staged through shared memory in chunks of 32 time steps with
//     cp.async (16-byte, double-buffered), rows padded by 16 bytes so that the per-thread 128-bit
//     reads are bank-conflict free; Bm/Cm are converted once per chunk to fp32 [t][n];
//   * the state update runs on packed f32x2 FMAs; exp(delta*A) is one ex2 per update with A
//     pre-multiplied by log2(e);
//   * the sum over n is finished by the two lanes of a channel swapping halves (4 shuffles per 8
//     time steps), which leaves each lane four adjacent time steps, for which it applies the skip
//     term and the SiLU gate and writes two packed pairs into the output tile, stored to global
//     memory as full rows.
#include "nb200_common.cuh"

namespace nb200 {
namespace {

constexpr int kScanThreads = 64;
constexpr int kNPT = 8;                       // states per thread (two threads per channel)
constexpr int kDB = 32;                       // channels per CTA
constexpr int kLC = 32;                       // time steps per staged chunk
constexpr int kRowBytes = kLC * 2 + 16;       // padded row of a 16-bit tile
constexpr int kStates = 16;
constexpr float kLog2e = 1.4426950408889634f;

struct __align__(16) ScanStage {
  unsigned char u[kDB * kRowBytes];
  unsigned char dl[kDB * kRowBytes];
  unsigned char z[kDB * kRowBytes];
  unsigned char braw[kStates * kLC * 2];
  unsigned char craw[kStates * kLC * 2];
};

struct __align__(16) ScanSmem {
  ScanStage stage[2];
  float bf[kLC][kStates];
  float cf[kLC][kStates];
  unsigned char out[kDB * kRowBytes];
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int DT>
__global__ void __launch_bounds__(kScanThreads, 7)
selective_scan_kernel(const uint16_t *__restrict__ u, const uint16_t *__restrict__ delta,
                      const float *__restrict__ A, const uint16_t *__restrict__ Bm,
                      const uint16_t *__restrict__ Cm, const float *__restrict__ Dskip,
                      const uint16_t *__restrict__ z, uint16_t *__restrict__ out, int Dm, int L) {
  __shared__ ScanSmem sm;
  const int tid = threadIdx.x;
  const int b = blockIdx.y;
  const int d0 = blockIdx.x * kDB;
  const int dl = tid >> 1, ng = tid & 1;
  const int d = d0 + dl;

  // decay rates of this thread's 4 states, in the exp2 domain, as two packed pairs
  const float4 a4 = *reinterpret_cast<const float4 *>(A + (size_t)d * kStates + ng * kNPT);
  const float4 a5 = *reinterpret_cast<const float4 *>(A + (size_t)d * kStates + ng * kNPT + 4);
  const uint64_t A2[4] = {f2_pack(a4.x * kLog2e, a4.y * kLog2e), f2_pack(a4.z * kLog2e, a4.w * kLog2e),
                          f2_pack(a5.x * kLog2e, a5.y * kLog2e), f2_pack(a5.z * kLog2e, a5.w * kLog2e)};
  const float dskip = Dskip[d];
  uint64_t h2[4] = {0ull, 0ull, 0ull, 0ull};

  const size_t row_base = ((size_t)b * Dm + d0) * L;        // element offset of row d0 of this sequence
  const size_t bc_base = (size_t)b * kStates * L;
  const int nchunks = L / kLC;

  auto issue_loads = [&](int chunk, int buf) {
    ScanStage &s = sm.stage[buf];
    const int t0 = chunk * kLC;
#pragma unroll
    for (int k = 0; k < 2; ++k) {  // u / delta / z : 32 rows x 4 segments of 16 bytes -> two per thread per tensor
      const int idx = tid + k * kScanThreads, row = idx >> 2, seg = idx & 3;
      const size_t g = row_base + (size_t)row * L + t0 + seg * 8;
      cp_async16(s.u + row * kRowBytes + seg * 16, u + g);
      cp_async16(s.dl + row * kRowBytes + seg * 16, delta + g);
      cp_async16(s.z + row * kRowBytes + seg * 16, z + g);
    }
    {  // Bm and Cm: 16 rows x 4 segments each -> one of each per thread
      const int row = tid >> 2, seg = tid & 3;
      const size_t g = bc_base + (size_t)row * L + t0 + seg * 8;
      cp_async16(s.braw + row * (kLC * 2) + seg * 16, Bm + g);
      cp_async16(s.craw + row * (kLC * 2) + seg * 16, Cm + g);
    }
    cp_async_commit();
  };

  issue_loads(0, 0);
  for (int chunk = 0; chunk < nchunks; ++chunk) {
    const int buf = chunk & 1;
    if (chunk + 1 < nchunks) {
      issue_loads(chunk + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    ScanStage &s = sm.stage[buf];

    {  // Bm/Cm of this chunk -> fp32 [t][n]; thread = (n, group of 8 time steps)
      const int n = tid >> 2, tq = tid & 3;
      const uint4 bw = *reinterpret_cast<const uint4 *>(s.braw + n * (kLC * 2) + tq * 16);
      const uint4 cw = *reinterpret_cast<const uint4 *>(s.craw + n * (kLC * 2) + tq * 16);
      const uint32_t bs[4] = {bw.x, bw.y, bw.z, bw.w}, cs[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 bb = unpack2<DT>(bs[e]), cc = unpack2<DT>(cs[e]);
        sm.bf[tq * 8 + 2 * e][n] = bb.x;
        sm.bf[tq * 8 + 2 * e + 1][n] = bb.y;
        sm.cf[tq * 8 + 2 * e][n] = cc.x;
        sm.cf[tq * 8 + 2 * e + 1][n] = cc.y;
      }
    }
    __syncthreads();

#pragma unroll 1
    for (int t8 = 0; t8 < kLC / 8; ++t8) {
      const uint4 uw = *reinterpret_cast<const uint4 *>(s.u + dl * kRowBytes + t8 * 16);
      const uint4 dw = *reinterpret_cast<const uint4 *>(s.dl + dl * kRowBytes + t8 * 16);
      const uint32_t us[4] = {uw.x, uw.y, uw.z, uw.w};
      const uint32_t ds[4] = {dw.x, dw.y, dw.z, dw.w};
      float y8[8];
#pragma unroll
      for (int tp = 0; tp < 4; ++tp) {
        const float2 uf = unpack2<DT>(us[tp]);
        const float2 df = unpack2<DT>(ds[tp]);
        const float uu[2] = {uf.x, uf.y}, dd[2] = {df.x, df.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = t8 * 8 + tp * 2 + e;
          const uint64_t dt2 = f2_pack(dd[e], dd[e]);
          const float dtu = dd[e] * uu[e];
          const uint64_t dtu2 = f2_pack(dtu, dtu);
          const ulonglong2 bv = *reinterpret_cast<const ulonglong2 *>(&sm.bf[t][ng * kNPT]);
          const ulonglong2 bw = *reinterpret_cast<const ulonglong2 *>(&sm.bf[t][ng * kNPT + 4]);
          const ulonglong2 cv = *reinterpret_cast<const ulonglong2 *>(&sm.cf[t][ng * kNPT]);
          const ulonglong2 cw = *reinterpret_cast<const ulonglong2 *>(&sm.cf[t][ng * kNPT + 4]);
          const uint64_t b2[4] = {bv.x, bv.y, bw.x, bw.y}, c2[4] = {cv.x, cv.y, cw.x, cw.y};
          uint64_t y2 = 0ull;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 x = f2_unpack(f2_mul(dt2, A2[i]));
            const uint64_t a2 = f2_pack(ex2(x.x), ex2(x.y));
            h2[i] = f2_fma(a2, h2[i], f2_mul(dtu2, b2[i]));
            y2 = f2_fma(c2[i], h2[i], y2);
          }
          const float2 yy = f2_unpack(y2);
          y8[tp * 2 + e] = yy.x + yy.y;
        }
      }
      // The two lanes of a channel exchange halves: lane ng ends with t = 4*ng .. 4*ng+3.
      float r4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float keep = ng ? y8[4 + i] : y8[i];
        const float send = ng ? y8[i] : y8[4 + i];
        r4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
      }
      // skip term and SiLU gate for this lane's four time steps
      const int off = dl * kRowBytes + t8 * 16 + ng * 8;
      const uint2 uw2 = *reinterpret_cast<const uint2 *>(s.u + off);
      const uint2 zw2 = *reinterpret_cast<const uint2 *>(s.z + off);
      const float2 ua = unpack2<DT>(uw2.x), ub = unpack2<DT>(uw2.y), za = unpack2<DT>(zw2.x), zb = unpack2<DT>(zw2.y);
      const float uu4[4] = {ua.x, ua.y, ub.x, ub.y}, zz4[4] = {za.x, za.y, zb.x, zb.y};
      float o4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float yv = fmaf(dskip, uu4[i], r4[i]);
        o4[i] = yv * zz4[i] * __frcp_rn(1.f + ex2(-zz4[i] * kLog2e));
      }
      *reinterpret_cast<uint2 *>(sm.out + off) = make_uint2(pack2<DT>(o4[0], o4[1]), pack2<DT>(o4[2], o4[3]));
    }
    __syncthreads();

#pragma unroll
    for (int k = 0; k < 2; ++k) {  // output tile -> global, two 16-byte segments per thread (rows are 64 contiguous bytes)
      const int idx = tid + k * kScanThreads, row = idx >> 2, seg = idx & 3;
      const uint4 w = *reinterpret_cast<const uint4 *>(sm.out + row * kRowBytes + seg * 16);
      *reinterpret_cast<uint4 *>(out + row_base + (size_t)row * L + chunk * kLC + seg * 8) = w;
    }
    // The next iteration's first barrier orders these reads of sm.out before its next writes, and
    // its cp.async into stage[buf] is issued after the barrier above, i.e. after every read of it.
  }
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" int nb200_selective_scan_fwd(const void *u, const void *delta, const float *A, const void *Bm,
                                        const void *Cm, const float *Dskip, const void *z, void *out,
                                        int B, int Dm, int L, int N, int dtype, void *stream) {
  NB200_REQUIRE(u && delta && A && Bm && Cm && Dskip && z && out, NB200_ERR_BAD_ARG,
                "selective_scan: null pointer");
  NB200_REQUIRE(B > 0 && Dm > 0 && L > 0, NB200_ERR_BAD_ARG, "selective_scan: non-positive extent");
  NB200_REQUIRE(aligned16(u) && aligned16(delta) && aligned16(z) && aligned16(out) && aligned16(Bm) &&
                    aligned16(Cm) && aligned16(A),
                NB200_ERR_BAD_ARG, "selective_scan: tensors must be 16-byte aligned");
  NB200_REQUIRE(N == kStates, NB200_ERR_UNSUPPORTED, "selective_scan: d_state = %d, only 16 is implemented", N);
  NB200_REQUIRE(L % 64 == 0 && Dm % kDB == 0, NB200_ERR_UNSUPPORTED,
                "selective_scan: L must be a multiple of 64 and D_inner a multiple of %d", kDB);
  NB200_REQUIRE(B <= 65535, NB200_ERR_UNSUPPORTED, "selective_scan: batch too large");
  auto st = static_cast<cudaStream_t>(stream);
  const dim3 grid(Dm / kDB, B), block(kScanThreads);
#define NB200_SCAN_ARGS                                                                              \
  static_cast<const uint16_t *>(u), static_cast<const uint16_t *>(delta), A,                         \
      static_cast<const uint16_t *>(Bm), static_cast<const uint16_t *>(Cm), Dskip,                   \
      static_cast<const uint16_t *>(z), static_cast<uint16_t *>(out), Dm, L
  if (dtype == NB200_BF16) selective_scan_kernel<NB200_BF16><<<grid, block, 0, st>>>(NB200_SCAN_ARGS);
  else if (dtype == NB200_F16) selective_scan_kernel<NB200_F16><<<grid, block, 0, st>>>(NB200_SCAN_ARGS);
  else return fail(NB200_ERR_UNSUPPORTED, "selective_scan: dtype %d (f16 and bf16 only)", dtype);
#undef NB200_SCAN_ARGS
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}
