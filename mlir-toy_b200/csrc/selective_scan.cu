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
#include <cstdlib>

#include "nb200_common.cuh"

namespace nb200 {
namespace {

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
__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// NPT = states per thread (8, 4 or 2), so 16 / NPT threads share a channel and a CTA of 32 channels has
// 512 / NPT threads.  8 states per thread is the cheapest per update (the per-step scalar work is spread over
// more states) and is used when the problem fills the GPU; smaller problems take 4 or 2, which multiplies the
// number of warps: a lone warp per scheduler is held by its own exp2 issue rate (one warp instruction per
// 8 cycles), so the time of a small problem is set by the states per thread, not by the work.
template <int NPT> constexpr int scan_min_ctas() { return NPT == 8 ? 7 : (NPT == 4 ? 4 : 2); }

template <int DT, int NPT>
__global__ void __launch_bounds__(512 / NPT, scan_min_ctas<NPT>())
selective_scan_kernel(const uint16_t *__restrict__ u, const uint16_t *__restrict__ delta,
                      const float *__restrict__ A, const uint16_t *__restrict__ Bm,
                      const uint16_t *__restrict__ Cm, const float *__restrict__ Dskip,
                      const uint16_t *__restrict__ z, uint16_t *__restrict__ out, int Dm, int L) {
  constexpr int TPC = kStates / NPT;          // threads per channel: 2, 4 or 8
  constexpr int T = kDB * TPC;                // threads per CTA
  constexpr int NP = NPT / 2;                 // packed pairs of states per thread
  constexpr int TS = 8 / TPC;                 // time steps of an 8-step group that a lane finishes: 4, 2 or 1
  __shared__ ScanSmem sm;
  const int tid = threadIdx.x;
  const int b = blockIdx.y;
  const int d0 = blockIdx.x * kDB;
  const int dl = tid / TPC, ng = tid % TPC;
  const int d = d0 + dl;

  // decay rates of this thread's states, in the exp2 domain, as packed pairs
  uint64_t A2[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const float2 a = *reinterpret_cast<const float2 *>(A + (size_t)d * kStates + ng * NPT + 2 * i);
    A2[i] = f2_pack(a.x * kLog2e, a.y * kLog2e);
  }
  const float dskip = Dskip[d];
  uint64_t h2[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) h2[i] = 0ull;

  const size_t row_base = ((size_t)b * Dm + d0) * L;        // element offset of row d0 of this sequence
  const size_t bc_base = (size_t)b * kStates * L;
  const int nchunks = L / kLC;

  auto issue_loads = [&](int chunk, int buf) {
    ScanStage &s = sm.stage[buf];
    const int t0 = chunk * kLC;
    for (int idx = tid; idx < kDB * 4; idx += T) {  // u / delta / z : 32 rows x 4 segments of 16 bytes
      const int row = idx >> 2, seg = idx & 3;
      const size_t g = row_base + (size_t)row * L + t0 + seg * 8;
      cp_async16(s.u + row * kRowBytes + seg * 16, u + g);
      cp_async16(s.dl + row * kRowBytes + seg * 16, delta + g);
      cp_async16(s.z + row * kRowBytes + seg * 16, z + g);
    }
    for (int idx = tid; idx < kStates * 4; idx += T) {  // Bm and Cm: 16 rows x 4 segments each
      const int row = idx >> 2, seg = idx & 3;
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

    for (int idx = tid; idx < kStates * 4; idx += T) {  // Bm/Cm of this chunk -> fp32 [t][n]; item = (n, group of 8 time steps)
      const int n = idx >> 2, tq = idx & 3;
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
          uint64_t b2[NP], c2[NP];
          if constexpr (NPT >= 4) {
#pragma unroll
            for (int q = 0; q < NPT / 4; ++q) {
              const ulonglong2 bv = *reinterpret_cast<const ulonglong2 *>(&sm.bf[t][ng * NPT + 4 * q]);
              const ulonglong2 cv = *reinterpret_cast<const ulonglong2 *>(&sm.cf[t][ng * NPT + 4 * q]);
              b2[2 * q] = bv.x;
              b2[2 * q + 1] = bv.y;
              c2[2 * q] = cv.x;
              c2[2 * q + 1] = cv.y;
            }
          } else {
            b2[0] = *reinterpret_cast<const uint64_t *>(&sm.bf[t][ng * NPT]);
            c2[0] = *reinterpret_cast<const uint64_t *>(&sm.cf[t][ng * NPT]);
          }
          uint64_t y2 = 0ull;
#pragma unroll
          for (int i = 0; i < NP; ++i) {
            const float2 x = f2_unpack(f2_mul(dt2, A2[i]));
            const uint64_t a2 = f2_pack(ex2(x.x), ex2(x.y));
            h2[i] = f2_fma(a2, h2[i], f2_mul(dtu2, b2[i]));
            y2 = f2_fma(c2[i], h2[i], y2);
          }
          const float2 yy = f2_unpack(y2);
          y8[tp * 2 + e] = yy.x + yy.y;
        }
      }
      // Sum over the lanes of a channel by recursive halving: at distance dist a lane keeps the half of its
      // time steps that its bit selects and receives the partner's sums for them, so that lane ng ends with
      // the complete sums of time steps ng*TS .. ng*TS + TS - 1 of the group.
#pragma unroll
      for (int dist = TPC / 2, n = 8; dist >= 1; dist >>= 1, n >>= 1) {
        const bool upper = (ng & dist) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
          const float keep = upper ? y8[n / 2 + i] : y8[i];
          const float send = upper ? y8[i] : y8[n / 2 + i];
          y8[i] = keep + __shfl_xor_sync(0xffffffffu, send, dist);
        }
      }
      // skip term and SiLU gate for this lane's TS time steps
      const int off = dl * kRowBytes + t8 * 16 + ng * (TS * 2);
      float uu4[TS], zz4[TS], o4[TS];
      if constexpr (TS == 4) {
        const uint2 uw2 = *reinterpret_cast<const uint2 *>(s.u + off);
        const uint2 zw2 = *reinterpret_cast<const uint2 *>(s.z + off);
        const float2 ua = unpack2<DT>(uw2.x), ub = unpack2<DT>(uw2.y), za = unpack2<DT>(zw2.x), zb = unpack2<DT>(zw2.y);
        uu4[0] = ua.x; uu4[1] = ua.y; uu4[2] = ub.x; uu4[3] = ub.y;
        zz4[0] = za.x; zz4[1] = za.y; zz4[2] = zb.x; zz4[3] = zb.y;
      } else if constexpr (TS == 2) {
        const float2 ua = unpack2<DT>(*reinterpret_cast<const uint32_t *>(s.u + off));
        const float2 za = unpack2<DT>(*reinterpret_cast<const uint32_t *>(s.z + off));
        uu4[0] = ua.x; uu4[1] = ua.y;
        zz4[0] = za.x; zz4[1] = za.y;
      } else {
        uu4[0] = load1<DT>(s.u + off, 0);
        zz4[0] = load1<DT>(s.z + off, 0);
      }
#pragma unroll
      for (int i = 0; i < TS; ++i) {
        const float yv = fmaf(dskip, uu4[i], y8[i]);
        // silu(z) = z * sigmoid(z) = z * (0.5 + 0.5 tanh(z / 2)): one special-function result instead of two
        o4[i] = yv * zz4[i] * fmaf(0.5f, tanh_approx(0.5f * zz4[i]), 0.5f);
      }
      if constexpr (TS == 4) {
        *reinterpret_cast<uint2 *>(sm.out + off) = make_uint2(pack2<DT>(o4[0], o4[1]), pack2<DT>(o4[2], o4[3]));
      } else if constexpr (TS == 2) {
        *reinterpret_cast<uint32_t *>(sm.out + off) = pack2<DT>(o4[0], o4[1]);
      } else {
        store1<DT>(sm.out + off, 0, o4[0]);
      }
    }
    __syncthreads();

    for (int idx = tid; idx < kDB * 4; idx += T) {  // output tile -> global in 16-byte segments (rows are 64 contiguous bytes)
      const int row = idx >> 2, seg = idx & 3;
      const uint4 w = *reinterpret_cast<const uint4 *>(sm.out + row * kRowBytes + seg * 16);
      *reinterpret_cast<uint4 *>(out + row_base + (size_t)row * L + chunk * kLC + seg * 8) = w;
    }
    // The next iteration's first barrier orders these reads of sm.out before its next writes, and
    // its cp.async into stage[buf] is issued after the barrier above, i.e. after every read of it.
  }
}

template <int DT, int NPT>
void launch_scan(const void *u, const void *delta, const float *A, const void *Bm, const void *Cm, const float *Dskip,
                 const void *z, void *out, int B, int Dm, int L, cudaStream_t st) {
  const dim3 grid(Dm / kDB, B), block(512 / NPT);
  selective_scan_kernel<DT, NPT><<<grid, block, 0, st>>>(
      static_cast<const uint16_t *>(u), static_cast<const uint16_t *>(delta), A, static_cast<const uint16_t *>(Bm),
      static_cast<const uint16_t *>(Cm), Dskip, static_cast<const uint16_t *>(z), static_cast<uint16_t *>(out), Dm, L);
}

// States per thread for a problem of `ctas` CTAs on a GPU of `sms` SMs.  Measured on 148 SMs (D = 4096, L = 4096,
// time in ms for 8 / 4 / 2 states per thread, before the gate went to tanh.approx; after it 1024 CTAs take
// 0.71 / 0.79): 1024 CTAs 0.80 / 0.84 / -, 512 CTAs 0.48 / 0.48 / 0.61,
// 256 CTAs 0.37 / 0.29 / 0.31, 128 CTAs 0.35 / 0.22 / 0.21.
int states_per_thread(long long ctas, int sms) {
  if (const char *e = getenv("NB200_SCAN_STATES")) {   // 8, 4 or 2: forces the choice (tests and tuning)
    const int v = atoi(e);
    if (v == 8 || v == 4 || v == 2) return v;
  }
  const long long want = 3ll * 4 * sms;   // about three warps of 8 states per scheduler
  if (ctas * 2 >= want) return 8;
  if (ctas * 8 >= want) return 4;
  return 2;
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
  int dev = 0, sms = 0;
  NB200_CHECK_CUDA(cudaGetDevice(&dev));
  NB200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int npt = states_per_thread((long long)B * (Dm / kDB), sms);
#define NB200_SCAN(DTV)                                                                         \
  switch (npt) {                                                                                \
    case 8: launch_scan<DTV, 8>(u, delta, A, Bm, Cm, Dskip, z, out, B, Dm, L, st); break;       \
    case 4: launch_scan<DTV, 4>(u, delta, A, Bm, Cm, Dskip, z, out, B, Dm, L, st); break;       \
    default: launch_scan<DTV, 2>(u, delta, A, Bm, Cm, Dskip, z, out, B, Dm, L, st); break;      \
  }
  if (dtype == NB200_BF16) { NB200_SCAN(NB200_BF16) }
  else if (dtype == NB200_F16) { NB200_SCAN(NB200_F16) }
  else return fail(NB200_ERR_UNSUPPORTED, "selective_scan: dtype %d (f16 and bf16 only)", dtype);
#undef NB200_SCAN
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}
