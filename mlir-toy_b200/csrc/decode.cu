// Split-K flash-decoding with grouped-query attention, and the log-sum-exp combine.
//
// The path is HBM-bound (about 4 FLOP per byte of KV cache), so the kernel is built around
// streaming K and V exactly once with 128-bit coalesced loads:
//   * one CTA per (split, kv head, sequence); the G query heads that share a kv head are all
//     evaluated by the same CTA, so each K/V row is read once and used G times;
//   * a K/V row of 128 elements is 16 lanes x 16 bytes; a warp therefore reads two rows per load
//     instruction, 8 rows per warp iteration.  For splits of 256 rows or more the rows come through
//     a ring of shared-memory stages filled by TMA bulk copies (decode_splitk_ring_kernel);
//     otherwise by 128-bit global loads, four of K and four of V in flight per lane;
//   * the 16-lane dot-product reduction is a butterfly that leaves head g's score on lanes whose
//     bits 3:2 equal g (5 shuffles for G = 4 instead of 16), the online softmax runs on those lanes,
//     and the probabilities are broadcast back for the PV accumulation;
//   * all arithmetic is fp32 (packed f32x2 FMAs), scores in the exp2 domain.
// Per (row, split) the kernel writes the un-normalised output, the running maximum and the sum,
// which nb200_decode_combine merges.
#include <mutex>

#include "nb200_common.cuh"
#include "peer_merge.cuh"
#include "sm100_primitives.cuh"

namespace nb200 {
namespace {

constexpr int kDecodeThreads = 256;
constexpr int kDecodeWarps = kDecodeThreads / 32;
constexpr int kHeadDim = 128;
constexpr int kPairs = 4;                               // row pairs per warp iteration
constexpr int kRowsPerIter = kDecodeWarps * kPairs * 2;  // 64 rows per CTA iteration

__device__ __forceinline__ uint4 ldg_stream(const void *p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

template <int DT, int G>
__global__ void __launch_bounds__(kDecodeThreads, (G >= 8 ? 1 : 2))
decode_splitk_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k,
                     const uint16_t *__restrict__ v, float *__restrict__ partials, int Hkv, int Lkv,
                     int n_splits, float scale_log2) {
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int Hq = Hkv * G;
  // split s covers rows [floor(s*L/n), floor((s+1)*L/n)): equal parts when n divides L, else parts that
  // differ by one row, so that the caller can choose n for the machine (one CTA per resident slot)
  const int t0 = static_cast<int>((long long)split * Lkv / n_splits);
  const int T = static_cast<int>((long long)(split + 1) * Lkv / n_splits) - t0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, c = lane & 15;

  // q for the G heads of this kv head, this lane's 8 elements, pre-multiplied by the scale.
  uint64_t q2[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 w = *reinterpret_cast<const uint4 *>(q + ((size_t)b * Hq + hkv * G + g) * kHeadDim + c * 8);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float2 f = unpack2<DT>(ws[p]);
      q2[g][p] = f2_pack(f.x * scale_log2, f.y * scale_log2);
    }
  }

  const size_t kv_base = (((size_t)b * Hkv + hkv) * Lkv + (size_t)t0) * kHeadDim + c * 8;
  const uint16_t *kp = k + kv_base;
  const uint16_t *vp = v + kv_base;

  uint64_t o2[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int p = 0; p < 4; ++p) o2[g][p] = 0ull;
  // Running max / sum of the head this lane owns after the butterfly (head index = lane bits 3:2
  // for G = 4; for other G every lane tracks all heads through the generic path below).
  float m_run[G == 4 ? 1 : G], l_run[G == 4 ? 1 : G];
#pragma unroll
  for (int g = 0; g < (G == 4 ? 1 : G); ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
  }

  for (int r0 = warp * (kPairs * 2); r0 < T; r0 += kRowsPerIter) {
    uint4 kr[kPairs], vr[kPairs];
    bool valid[kPairs];
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const int r = r0 + 2 * i + half;
      valid[i] = r < T;
      if (valid[i]) {
        kr[i] = ldg_stream(kp + (size_t)r * kHeadDim);
        vr[i] = ldg_stream(vp + (size_t)r * kHeadDim);
      } else {
        kr[i] = make_uint4(0, 0, 0, 0);
        vr[i] = make_uint4(0, 0, 0, 0);
      }
    }

    // ---- scores: partial dot products over this lane's 8 elements ----
    float part[kPairs][G];
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const uint32_t ws[4] = {kr[i].x, kr[i].y, kr[i].z, kr[i].w};
      uint64_t k2[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 f = unpack2<DT>(ws[p]);
        k2[p] = f2_pack(f.x, f.y);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        uint64_t acc = f2_mul(q2[g][0], k2[0]);
#pragma unroll
        for (int p = 1; p < 4; ++p) acc = f2_fma(q2[g][p], k2[p], acc);
        const float2 a = f2_unpack(acc);
        part[i][g] = a.x + a.y;
      }
    }

    float pg[kPairs][G];  // probabilities of every head for this lane's rows
    float alpha[G];
    if constexpr (G == 4) {
      // Butterfly over the 16 lanes of a row: afterwards lanes with bits 3:2 == g hold head g.
      const bool b3 = lane & 8, b2 = lane & 4;
      float s[kPairs];
#pragma unroll
      for (int i = 0; i < kPairs; ++i) {
        float a0 = b3 ? part[i][2] : part[i][0];
        float a1 = b3 ? part[i][3] : part[i][1];
        const float s0 = b3 ? part[i][0] : part[i][2];
        const float s1 = b3 ? part[i][1] : part[i][3];
        a0 += __shfl_xor_sync(0xffffffffu, s0, 8);
        a1 += __shfl_xor_sync(0xffffffffu, s1, 8);
        float x = b2 ? a1 : a0;
        const float sx = b2 ? a0 : a1;
        x += __shfl_xor_sync(0xffffffffu, sx, 4);
        x += __shfl_xor_sync(0xffffffffu, x, 2);
        x += __shfl_xor_sync(0xffffffffu, x, 1);
        s[i] = valid[i] ? x : -INFINITY;
      }
      float mb = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
      mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
      const float m_new = fmaxf(m_run[0], mb);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float a = ex2(m_run[0] - m_safe);
      float p[kPairs], psum = 0.f;
#pragma unroll
      for (int i = 0; i < kPairs; ++i) {
        p[i] = ex2(s[i] - m_safe);
        psum += p[i];
      }
      l_run[0] = l_run[0] * a + psum;
      m_run[0] = m_new;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        alpha[g] = __shfl_sync(0xffffffffu, a, g << 2);
#pragma unroll
        for (int i = 0; i < kPairs; ++i) pg[i][g] = __shfl_sync(0xffffffffu, p[i], (lane & 16) | (g << 2));
      }
    } else {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s[kPairs];
#pragma unroll
        for (int i = 0; i < kPairs; ++i) {
          float x = part[i][g];
          x += __shfl_xor_sync(0xffffffffu, x, 8);
          x += __shfl_xor_sync(0xffffffffu, x, 4);
          x += __shfl_xor_sync(0xffffffffu, x, 2);
          x += __shfl_xor_sync(0xffffffffu, x, 1);
          s[i] = valid[i] ? x : -INFINITY;
        }
        float mb = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
        mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
        const float m_new = fmaxf(m_run[g], mb);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[g] = ex2(m_run[g] - m_safe);
        float psum = 0.f;
#pragma unroll
        for (int i = 0; i < kPairs; ++i) {
          pg[i][g] = ex2(s[i] - m_safe);
          psum += pg[i][g];
        }
        l_run[g] = l_run[g] * alpha[g] + psum;
        m_run[g] = m_new;
      }
    }

    // ---- o = o * alpha + sum_i p_i v_i ----
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const uint64_t a2 = f2_pack(alpha[g], alpha[g]);
#pragma unroll
      for (int p = 0; p < 4; ++p) o2[g][p] = f2_mul(o2[g][p], a2);
    }
#pragma unroll
    for (int i = 0; i < kPairs; ++i) {
      const uint32_t ws[4] = {vr[i].x, vr[i].y, vr[i].z, vr[i].w};
      uint64_t v2[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 f = unpack2<DT>(ws[p]);
        v2[p] = f2_pack(f.x, f.y);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const uint64_t p2 = f2_pack(pg[i][g], pg[i][g]);
#pragma unroll
        for (int p = 0; p < 4; ++p) o2[g][p] = f2_fma(p2, v2[p], o2[g][p]);
      }
    }
  }

  // ---- merge the two row halves of the warp, then the warps of the CTA ----
  __shared__ float sm_o[kDecodeWarps][G][kHeadDim];
  __shared__ float sm_m[kDecodeWarps][G], sm_l[kDecodeWarps][G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      float2 f = f2_unpack(o2[g][p]);
      f.x += __shfl_xor_sync(0xffffffffu, f.x, 16);
      f.y += __shfl_xor_sync(0xffffffffu, f.y, 16);
      if (half == 0) {
        sm_o[warp][g][c * 8 + 2 * p] = f.x;
        sm_o[warp][g][c * 8 + 2 * p + 1] = f.y;
      }
    }
  }
  if constexpr (G == 4) {
    const float l_tot = l_run[0] + __shfl_xor_sync(0xffffffffu, l_run[0], 16);
    if (half == 0 && (lane & 3) == 0) {
      sm_m[warp][lane >> 2] = m_run[0];
      sm_l[warp][lane >> 2] = l_tot;
    }
  } else {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float l_tot = l_run[g] + __shfl_xor_sync(0xffffffffu, l_run[g], 16);
      if (lane == 0) {
        sm_m[warp][g] = m_run[g];
        sm_l[warp][g] = l_tot;
      }
    }
  }
  __syncthreads();

  for (int idx = threadIdx.x; idx < G * kHeadDim; idx += kDecodeThreads) {
    const int g = idx / kHeadDim, d = idx % kHeadDim;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, sm_m[w][g]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float wgt = ex2(sm_m[w][g] - Ms);
      acc += wgt * sm_o[w][g][d];
      lsum += wgt * sm_l[w][g];
    }
    float *dst = partials + (((size_t)b * Hq + hkv * G + g) * n_splits + split) * (kHeadDim + 2);
    dst[d] = acc;
    if (d == 0) {
      dst[kHeadDim] = M;
      dst[kHeadDim + 1] = lsum;
    }
  }
}

// ---- K/V staged by bulk copies --------------------------------------------------------------------
// Same arithmetic as decode_splitk_kernel, but the K and V rows of a split arrive through a ring of
// shared-memory stages filled by TMA bulk copies (one producer thread, mbarrier completion) instead of
// per-lane global loads.  With plain loads a warp has one iteration (4 KB) in flight and none while it
// computes; halving the resident warps cost 60 % of the bandwidth, i.e. the kernel was bound by bytes in
// flight.  The ring keeps three 32 KB stages (64 rows of K and of V) per CTA in flight whatever the warps do.
constexpr int kRingStages = 3;
constexpr int kStageRows = 64;
constexpr int kStageBytes = kStageRows * kHeadDim * 2;                 // 16 KB per operand
constexpr int kRingThreads = kDecodeThreads + 32;                      // 8 consumer warps + the producer warp
constexpr int kRingSmem = kRingStages * 2 * kStageBytes + 128;         // stages, then the barriers

struct RingBarriers {
  uint64_t full[kRingStages], empty[kRingStages];
  int abort_flag;
  int stage_rows[kRingStages];   // dynamic deal only: rows in the stage, 0 = no more stages
};
constexpr int kChunkRows = 2 * kStageRows;   // dynamic deal: rows a CTA takes from its head's counter at a time
                                             // (64 to 256 measured within 1 % of each other from 32 K to 256 K rows; 512 is slower)

// Codes the ring kernel records in status[0] (block, detail and thread follow in status[1..3]).
enum : int { kErrDecodeWait = 21, kErrDecodeBadPage = 22 };

__device__ __forceinline__ void decode_report(int *status, int code, int detail) {
  if (status && atomicCAS(status, 0, code) == 0) {
    status[1] = static_cast<int>(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    status[2] = detail;
    status[3] = static_cast<int>(threadIdx.x);
  }
}

__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void *gsrc, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}

// ---- the sharded single-sequence decode as ONE kernel -------------------------------------------------------
// When one sequence's cache is split along its length over the GPUs of a node, every GPU reduces its slice with the
// split-K kernel above and the per-GPU results are merged.  With TAIL the ring kernel does all of it in one launch,
// the hand-overs made by "the last CTA to finish does the next stage" tickets, so that no CTA ever waits for
// another CTA of the launch:
//   1. every CTA writes its split's partial, then takes a ticket of its kv head; the CTA that takes the head's last
//      ticket combines the head's splits into this GPU's partial (o, m, l) for the G query heads of the group;
//   2. it then takes a ticket of the launch; the CTA that takes the last one pushes the GPU's whole partial
//      [Hq][D + 2] into every peer's gather area (plain stores over NVLink), releases the arrival flags, waits
//      (bounded) for the other GPUs' partials in its own area and writes the merged, normalised output.
// With world == 1 step 2 is only the normalisation, which makes the same launch a single-kernel decode of one
// sequence on one GPU.  The ticket counters ([Hkv + 1] ints, zeroed once by the caller) are reset by the last CTA.
struct DecodeTail {
  float *local;            // [Hq][D + 2] fp32 scratch: this GPU's partial
  int *counters;           // [Hkv + 1] tickets, then [Hkv] chunk counters; zero between launches
  peer::Ptrs peers;        // symmetric buffers of all ranks (unused when world == 1)
  void *out;               // [Hq][D] in out_dtype (or [Hq][D + 2] fp32)
  int world, rank, out_dtype;
  unsigned generation;
  long long wait_ns;
  int *status;
};

template <int G>
__device__ __forceinline__ void decode_tail(const DecodeTail &t, const float *partials, int Hkv, int n_splits, int hkv,
                                            unsigned char *scratch) {
  constexpr int kW = kDecodeWarps;                 // the eight consumer warps do the arithmetic
  constexpr int kWarpsPerRow = kW / G;             // G <= 8
  float(*sm_acc)[kHeadDim] = reinterpret_cast<float(*)[kHeadDim]>(scratch);
  float *sm_l = reinterpret_cast<float *>(scratch + kW * kHeadDim * 4);
  int *sm_flag = reinterpret_cast<int *>(scratch + kW * kHeadDim * 4 + 64);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Hq = Hkv * G;

  __threadfence();                                 // this CTA's partial is visible before its ticket is
  __syncthreads();
  if (tid == 0) sm_flag[0] = (atomicAdd(t.counters + hkv, 1) == n_splits - 1) ? 1 : 0;
  __syncthreads();
  if (!sm_flag[0]) return;
  __threadfence();

  // ---- stage 1: this kv head's splits -> the GPU's partial for its G rows; kWarpsPerRow warps share a row
  if (warp < kW) {
    const int g = warp / kWarpsPerRow, part = warp % kWarpsPerRow;
    const float *base = partials + ((size_t)(hkv * G + g) * n_splits) * (kHeadDim + 2);
    float M = -INFINITY;
    for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, __ldcg(base + (size_t)s * (kHeadDim + 2) + kHeadDim));
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float lsum = 0.f;
    constexpr int kU = 4;
    for (int s0 = part; s0 < n_splits; s0 += kWarpsPerRow * kU) {
      float4 o[kU];
      float ms[kU], ls[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int sidx = s0 + u * kWarpsPerRow;
        const float *ps = base + (size_t)(sidx < n_splits ? sidx : s0) * (kHeadDim + 2);
        const float2 a = __ldcg(reinterpret_cast<const float2 *>(ps + lane * 4));
        const float2 b2 = __ldcg(reinterpret_cast<const float2 *>(ps + lane * 4 + 2));
        o[u] = make_float4(a.x, a.y, b2.x, b2.y);
        ms[u] = __ldcg(ps + kHeadDim);
        ls[u] = __ldcg(ps + kHeadDim + 1);
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (s0 + u * kWarpsPerRow < n_splits) {
          const float w = ex2(ms[u] - Ms);
          acc.x += w * o[u].x;
          acc.y += w * o[u].y;
          acc.z += w * o[u].z;
          acc.w += w * o[u].w;
          lsum += w * ls[u];
        }
      }
    }
    *reinterpret_cast<float4 *>(&sm_acc[warp][lane * 4]) = acc;
    if (lane == 0) sm_l[warp] = lsum;
    __syncwarp();
    asm volatile("bar.sync 2, %0;" ::"r"(kW * 32) : "memory");
    if (part == 0) {
      for (int w = 1; w < kWarpsPerRow; ++w) {
        const float4 a = *reinterpret_cast<const float4 *>(&sm_acc[warp + w][lane * 4]);
        acc.x += a.x;
        acc.y += a.y;
        acc.z += a.z;
        acc.w += a.w;
        lsum += sm_l[warp + w];
      }
      float *dst = t.local + (size_t)(hkv * G + g) * (kHeadDim + 2);
      *reinterpret_cast<float2 *>(dst + lane * 4) = make_float2(acc.x, acc.y);
      *reinterpret_cast<float2 *>(dst + lane * 4 + 2) = make_float2(acc.z, acc.w);
      if (lane == 0) {
        dst[kHeadDim] = M;
        dst[kHeadDim + 1] = lsum;
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) sm_flag[0] = (atomicAdd(t.counters + Hkv, 1) == Hkv - 1) ? 1 : 0;
  __syncthreads();
  if (!sm_flag[0]) return;
  __threadfence();

  // ---- stage 2: across the GPUs
  const float *gathered = t.local;                 // world == 1: the "gather" is the local partial itself
  if (t.world > 1) {
    peer::push(t.local, t.peers, Hq, t.world, t.rank, t.generation, 0, t.world, tid, blockDim.x);
    __threadfence_system();
    __syncthreads();
    if (tid < t.world) peer::release_flag(t.peers, Hq, t.world, t.rank, t.generation, tid);
    if (tid == 0) sm_flag[1] = 0;
    __syncthreads();
    if (tid < t.world && !peer::wait_arrival(t.peers, Hq, t.world, t.rank, t.generation, tid, t.wait_ns, t.status)) sm_flag[1] = 1;
    __syncthreads();
    gathered = t.peers.buf[t.rank] + (t.generation & 1u) * peer::area_floats(Hq, t.world);
  } else if (tid == 0) {
    sm_flag[1] = 0;
  }
  __syncthreads();
  if (!sm_flag[1]) {
    const size_t slot = (size_t)Hq * (kHeadDim + 2);
    for (int row = warp; row < Hq; row += blockDim.x / 32) {
      if (t.out_dtype == NB200_BF16) peer::combine_row<NB200_BF16>(gathered, slot, t.world, row, t.out, lane);
      else if (t.out_dtype == NB200_F16) peer::combine_row<NB200_F16>(gathered, slot, t.world, row, t.out, lane);
      else peer::combine_row<NB200_F32>(gathered, slot, t.world, row, t.out, lane);
    }
  }
  for (int i = tid; i <= 2 * Hkv; i += blockDim.x) t.counters[i] = 0;   // ready for the next launch (also after an expired wait)
}

// DYN (one sequence, dense cache, with the fused tail): a 1-D grid of n_splits * Hkv CTAs, CTA l working for kv head
// (l % Hkv + l / Hkv) % Hkv.  Instead of a fixed range of rows a CTA takes chunks of kChunkRows rows from its head's counter (the
// first one is its own index, so nothing waits at the start).  Two CTAs share an SM and the one launched first gets
// the larger share of it: with fixed ranges the first 148 CTAs of a one-wave launch finished at 152 us and the
// other 148 at 178 us (measured), the GPU half idle in between.  Interleaving the heads over the launch order gives
// every head both kinds of CTA, and the counters let the faster ones take more chunks.
template <int DT, int G, bool TAIL = false, bool DYN = false>
__global__ void __launch_bounds__(kRingThreads, (G >= 8 ? 1 : 2))
decode_splitk_ring_kernel(const uint16_t *__restrict__ q, const uint16_t *__restrict__ k,
                          const uint16_t *__restrict__ v, float *__restrict__ partials, int Hkv, int Lkv,
                          int n_splits, float scale_log2, const int *__restrict__ block_table,
                          const int *__restrict__ seq_lens, int max_pages, int num_pages, int *status,
                          const DecodeTail tail = DecodeTail{}) {
  extern __shared__ __align__(128) unsigned char ring[];
  RingBarriers *bars = reinterpret_cast<RingBarriers *>(ring + kRingStages * 2 * kStageBytes);
  volatile int *abort_flag = &bars->abort_flag;
  const uint32_t ring_base = sm100::smem_u32(ring);
  const uint32_t b_full = sm100::smem_u32(&bars->full[0]), b_empty = sm100::smem_u32(&bars->empty[0]);

  const int split = DYN ? static_cast<int>(blockIdx.x) / Hkv : static_cast<int>(blockIdx.x);
  // DYN: row `split` of the launch order is a rotation of the heads, so that a head's CTAs fall on even and odd SMs and
  // on both resident slots alike (the odd SM of a pair, like the second CTA of an SM, gets the smaller share)
  const int hkv = DYN ? (static_cast<int>(blockIdx.x) % Hkv + split) % Hkv : static_cast<int>(blockIdx.y);
  const int b = DYN ? 0 : static_cast<int>(blockIdx.z);
  const int Hq = Hkv * G;
  // Dense cache: split s covers rows [floor(s*L/n), floor((s+1)*L/n)) of a [B, Hkv, L, D] tensor.
  // Paged cache (block_table != nullptr): a sequence of seq_lens[b] rows lives in pages of 64 rows, page p of it
  // at pages[block_table[b][p]][hkv]; split s covers whole pages [floor(s*np/n), floor((s+1)*np/n)), and a page is
  // exactly one stage of the ring.
  const bool paged = block_table != nullptr;
  int t0, T;
  if (paged) {
    // the table row has max_pages entries: a length beyond that (or a negative one) is cut to what the row can address
    const int len = max(0, min(seq_lens[b], max_pages * kStageRows));
    const int np = (len + kStageRows - 1) / kStageRows;
    const int p0 = static_cast<int>((long long)split * np / n_splits);
    const int p1 = static_cast<int>((long long)(split + 1) * np / n_splits);
    t0 = p0 * kStageRows;
    T = max(0, min(len, p1 * kStageRows) - t0);
  } else {
    t0 = static_cast<int>((long long)split * Lkv / n_splits);
    T = static_cast<int>((long long)(split + 1) * Lkv / n_splits) - t0;
  }
  const int n_iter = (T + kStageRows - 1) / kStageRows;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, c = lane & 15;

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    for (int s = 0; s < kRingStages; ++s) {
      sm100::mbar_init(b_full + 8 * s, 1);
      sm100::mbar_init(b_empty + 8 * s, kDecodeWarps);
    }
    sm100::fence_barrier_init();
  }
  __syncthreads();

  uint64_t o2[G][4];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int p = 0; p < 4; ++p) o2[g][p] = 0ull;
  // Running max / sum: for G = 4 of the head this lane owns after the butterfly (head = lane bits 3:2);
  // for other G every lane tracks all heads.
  float m_run[G == 4 ? 1 : G], l_run[G == 4 ? 1 : G];
#pragma unroll
  for (int g = 0; g < (G == 4 ? 1 : G); ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
  }
  bool ok = true;

  if (warp == kDecodeWarps) {
    // ================================ producer ================================
    if (lane == 0 && DYN) {
      const size_t head_base = ((size_t)b * Hkv + hkv) * Lkv * kHeadDim;
      const int n_chunks = (Lkv + kChunkRows - 1) / kChunkRows;
      int *counter = tail.counters + Hkv + 1 + hkv;
      int it = 0;
      bool gave_up = false;
      int chunk = split;
      while (chunk < n_chunks && !gave_up) {
        const int next = n_splits + atomicAdd(counter, 1);   // asked for now, needed when this chunk's copies are out
        const int row0 = chunk * kChunkRows;
        const int rows_c = min(kChunkRows, Lkv - row0);
        for (int r = 0; r < rows_c; r += kStageRows, ++it) {
          const int st = it % kRingStages;
          if (it >= kRingStages && !sm100::mbar_wait(b_empty + 8 * st, ((it / kRingStages) & 1) ^ 1, abort_flag)) {
            decode_report(status, kErrDecodeWait, it);
            gave_up = true;
            break;
          }
          const int rows = min(kStageRows, rows_c - r);
          const uint32_t bytes = static_cast<uint32_t>(rows) * kHeadDim * 2;
          bars->stage_rows[st] = rows;
          sm100::mbar_arrive_expect_tx(b_full + 8 * st, 2 * bytes);
          const size_t off = head_base + (size_t)(row0 + r) * kHeadDim;
          bulk_load(ring_base + st * 2 * kStageBytes, k + off, bytes, b_full + 8 * st);
          bulk_load(ring_base + st * 2 * kStageBytes + kStageBytes, v + off, bytes, b_full + 8 * st);
        }
        chunk = next;
      }
      if (!gave_up) {   // the end marker: a stage of no rows
        const int st = it % kRingStages;
        if (it >= kRingStages && !sm100::mbar_wait(b_empty + 8 * st, ((it / kRingStages) & 1) ^ 1, abort_flag)) {
          decode_report(status, kErrDecodeWait, it);
          gave_up = true;
        } else {
          bars->stage_rows[st] = 0;
          sm100::mbar_arrive(b_full + 8 * st);
        }
      }
      if (gave_up) {  // let the copies in flight land before the CTA's shared memory goes away
        for (int spin = 0; spin < 100000; ++spin) {
          bool done = true;
          for (int n = 0; n < kRingStages; ++n) {
            const int j = it - 1 - n;
            if (j >= 0) done = done && sm100::mbar_try_wait(b_full + 8 * (j % kRingStages), (j / kRingStages) & 1);
          }
          if (done) break;
          __nanosleep(100);
        }
      }
    } else if (lane == 0) {
      const size_t kv_base = (((size_t)b * Hkv + hkv) * Lkv + (size_t)t0) * kHeadDim;
      int issued = 0;
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % kRingStages;
        if (it >= kRingStages && !sm100::mbar_wait(b_empty + 8 * st, ((it / kRingStages) & 1) ^ 1, abort_flag)) {
          decode_report(status, kErrDecodeWait, it);
          break;
        }
        const int rows = min(kStageRows, T - it * kStageRows);
        const uint32_t bytes = static_cast<uint32_t>(rows) * kHeadDim * 2;
        sm100::mbar_arrive_expect_tx(b_full + 8 * st, 2 * bytes);
        size_t off = kv_base + (size_t)it * kStageRows * kHeadDim;
        if (paged) {
          const int page = block_table[(size_t)b * max_pages + t0 / kStageRows + it];
          if (page < 0 || page >= num_pages) {
            // a table entry outside the pool: no copy is issued from it; the consumers see the abort flag, the
            // partial is poisoned and the status words say which entry it was
            decode_report(status, kErrDecodeBadPage, page);
            *abort_flag = 1;
            break;
          }
          off = ((size_t)page * Hkv + hkv) * kStageRows * kHeadDim;
        }
        bulk_load(ring_base + st * 2 * kStageBytes, k + off, bytes, b_full + 8 * st);
        bulk_load(ring_base + st * 2 * kStageBytes + kStageBytes, v + off, bytes, b_full + 8 * st);
        ++issued;
      }
      if (issued < n_iter) {  // gave up: let the copies in flight land before the CTA's shared memory goes away
        for (int spin = 0; spin < 100000; ++spin) {
          bool done = true;
          for (int n = 0; n < kRingStages; ++n) {
            const int it = issued - 1 - n;
            if (it >= 0) done = done && sm100::mbar_try_wait(b_full + 8 * (it % kRingStages), (it / kRingStages) & 1);
          }
          if (done) break;
          __nanosleep(100);
        }
      }
    }
  } else {
    // ================================ consumers ===============================
    // q for the G heads of this kv head, this lane's 8 elements, pre-multiplied by the scale.
    uint64_t q2[G][4];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const uint4 w = *reinterpret_cast<const uint4 *>(q + ((size_t)b * Hq + hkv * G + g) * kHeadDim + c * 8);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 f = unpack2<DT>(ws[p]);
        q2[g][p] = f2_pack(f.x * scale_log2, f.y * scale_log2);
      }
    }
    const bool b3 = lane & 8, b2 = lane & 4;
    for (int it = 0; DYN || it < n_iter; ++it) {
      const int st = it % kRingStages;
      ok = __all_sync(0xffffffffu, sm100::mbar_wait(b_full + 8 * st, (it / kRingStages) & 1, abort_flag));
      if (!ok) {
        if (lane == 0) decode_report(status, kErrDecodeWait, 1000000 + it);   // no-op if the producer already said why
        break;
      }
      const unsigned char *sk = ring + st * 2 * kStageBytes + (warp * (kPairs * 2) + half) * (kHeadDim * 2) + c * 16;
      const unsigned char *sv = sk + kStageBytes;
      const int srows = DYN ? *reinterpret_cast<volatile int *>(&bars->stage_rows[st]) : 0;
      if (DYN && srows == 0) break;   // the end marker
      // row of this lane's first pair and the limit it is compared with: inside the stage, or inside the split
      const int r0 = (DYN ? 0 : it * kStageRows) + warp * (kPairs * 2) + half;
      const int r_end = DYN ? srows : T;

      // ---- scores: partial dot products over this lane's 8 elements ----
      bool valid[kPairs];
      float part[kPairs][G];
#pragma unroll
      for (int i = 0; i < kPairs; ++i) {
        valid[i] = r0 + 2 * i < r_end;
        uint4 kr = *reinterpret_cast<const uint4 *>(sk + i * (2 * kHeadDim * 2));
        if (!valid[i]) kr = make_uint4(0, 0, 0, 0);   // rows past the end of the split were not copied
        const uint32_t ws[4] = {kr.x, kr.y, kr.z, kr.w};
        uint64_t k2[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float2 f = unpack2<DT>(ws[p]);
          k2[p] = f2_pack(f.x, f.y);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          uint64_t acc = f2_mul(q2[g][0], k2[0]);
#pragma unroll
          for (int p = 1; p < 4; ++p) acc = f2_fma(q2[g][p], k2[p], acc);
          const float2 a = f2_unpack(acc);
          part[i][g] = a.x + a.y;
        }
      }
      float pg[kPairs][G];  // probabilities of every head for this lane's rows
      float alpha[G];
      if constexpr (G == 4) {
        // Butterfly over the 16 lanes of a row: afterwards lanes with bits 3:2 == g hold head g.
        float sc[kPairs];
#pragma unroll
        for (int i = 0; i < kPairs; ++i) {
          float a0 = b3 ? part[i][2] : part[i][0];
          float a1 = b3 ? part[i][3] : part[i][1];
          const float s0 = b3 ? part[i][0] : part[i][2];
          const float s1 = b3 ? part[i][1] : part[i][3];
          a0 += __shfl_xor_sync(0xffffffffu, s0, 8);
          a1 += __shfl_xor_sync(0xffffffffu, s1, 8);
          float x = b2 ? a1 : a0;
          const float sx = b2 ? a0 : a1;
          x += __shfl_xor_sync(0xffffffffu, sx, 4);
          x += __shfl_xor_sync(0xffffffffu, x, 2);
          x += __shfl_xor_sync(0xffffffffu, x, 1);
          sc[i] = valid[i] ? x : -INFINITY;
        }
        float mb = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
        const float m_new = fmaxf(m_run[0], mb);
        const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
        const float a = ex2(m_run[0] - m_safe);
        float pr[kPairs], psum = 0.f;
#pragma unroll
        for (int i = 0; i < kPairs; ++i) {
          pr[i] = ex2(sc[i] - m_safe);
          psum += pr[i];
        }
        l_run[0] = l_run[0] * a + psum;
        m_run[0] = m_new;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          alpha[g] = __shfl_sync(0xffffffffu, a, g << 2);
#pragma unroll
          for (int i = 0; i < kPairs; ++i) pg[i][g] = __shfl_sync(0xffffffffu, pr[i], (lane & 16) | (g << 2));
        }
      } else {
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float sc[kPairs];
#pragma unroll
          for (int i = 0; i < kPairs; ++i) {
            float x = part[i][g];
            x += __shfl_xor_sync(0xffffffffu, x, 8);
            x += __shfl_xor_sync(0xffffffffu, x, 4);
            x += __shfl_xor_sync(0xffffffffu, x, 2);
            x += __shfl_xor_sync(0xffffffffu, x, 1);
            sc[i] = valid[i] ? x : -INFINITY;
          }
          float mb = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
          mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 16));
          const float m_new = fmaxf(m_run[g], mb);
          const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
          alpha[g] = ex2(m_run[g] - m_safe);
          float psum = 0.f;
#pragma unroll
          for (int i = 0; i < kPairs; ++i) {
            pg[i][g] = ex2(sc[i] - m_safe);
            psum += pg[i][g];
          }
          l_run[g] = l_run[g] * alpha[g] + psum;
          m_run[g] = m_new;
        }
      }

      // ---- o = o * alpha + sum_i p_i v_i ----
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const uint64_t a2 = f2_pack(alpha[g], alpha[g]);
#pragma unroll
        for (int p = 0; p < 4; ++p) o2[g][p] = f2_mul(o2[g][p], a2);
      }
#pragma unroll
      for (int i = 0; i < kPairs; ++i) {
        uint4 vr = *reinterpret_cast<const uint4 *>(sv + i * (2 * kHeadDim * 2));
        if (!valid[i]) vr = make_uint4(0, 0, 0, 0);
        const uint32_t ws[4] = {vr.x, vr.y, vr.z, vr.w};
        uint64_t v2[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          const float2 f = unpack2<DT>(ws[p]);
          v2[p] = f2_pack(f.x, f.y);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const uint64_t p2 = f2_pack(pg[i][g], pg[i][g]);
#pragma unroll
          for (int p = 0; p < 4; ++p) o2[g][p] = f2_fma(p2, v2[p], o2[g][p]);
        }
      }
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(b_empty + 8 * st);   // this warp is done with its rows of the stage
    }
  }

  // ---- merge the two row halves of a warp, then the warps of the CTA (the ring is dead: reuse it) ----
  __syncthreads();
  float(*sm_o)[G][kHeadDim] = reinterpret_cast<float(*)[G][kHeadDim]>(ring);
  float(*sm_m)[G] = reinterpret_cast<float(*)[G]>(ring + kDecodeWarps * G * kHeadDim * 4);
  float(*sm_l)[G] = sm_m + kDecodeWarps;
  if (warp < kDecodeWarps) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        float2 f = f2_unpack(o2[g][p]);
        f.x += __shfl_xor_sync(0xffffffffu, f.x, 16);
        f.y += __shfl_xor_sync(0xffffffffu, f.y, 16);
        if (half == 0) {
          sm_o[warp][g][c * 8 + 2 * p] = f.x;
          sm_o[warp][g][c * 8 + 2 * p + 1] = f.y;
        }
      }
    }
    // a wait that expired poisons the partial: the combine then yields NaN instead of a wrong number
    if constexpr (G == 4) {
      const float l_tot = l_run[0] + __shfl_xor_sync(0xffffffffu, l_run[0], 16);
      if (half == 0 && (lane & 3) == 0) {
        sm_m[warp][lane >> 2] = ok ? m_run[0] : 0.f;
        sm_l[warp][lane >> 2] = ok ? l_tot : __int_as_float(0x7fc00000);
      }
    } else {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float l_tot = l_run[g] + __shfl_xor_sync(0xffffffffu, l_run[g], 16);
        if (lane == 0) {
          sm_m[warp][g] = ok ? m_run[g] : 0.f;
          sm_l[warp][g] = ok ? l_tot : __int_as_float(0x7fc00000);
        }
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * kHeadDim; idx += kRingThreads) {
    const int g = idx / kHeadDim, d = idx % kHeadDim;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) M = fmaxf(M, sm_m[w][g]);
    const float Ms = (M == -INFINITY) ? 0.f : M;
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float wgt = ex2(sm_m[w][g] - Ms);
      acc += wgt * sm_o[w][g][d];
      lsum += wgt * sm_l[w][g];
    }
    float *dst = partials + (((size_t)b * Hq + hkv * G + g) * n_splits + split) * (kHeadDim + 2);
    dst[d] = acc;
    if (d == 0) {
      dst[kHeadDim] = M;
      dst[kHeadDim + 1] = lsum;
    }
  }
  if constexpr (TAIL) {
    __syncthreads();   // the merge scratch in `ring` is read no more
    decode_tail<G>(tail, partials, Hkv, n_splits, hkv, ring);
  }
}

// One CTA of four warps per output row.  The partials of a row sit in memory that nothing has touched since the
// split-K kernel wrote it, so every load costs a full memory latency: the kernel is organised to have them all in
// flight at once instead of one per split.  Each warp first finds the row maximum with its lanes reading
// different splits' maxima in parallel; then warp w accumulates splits w, w + 4, ... (lane = 4 of the 128
// elements), four splits' loads issued before any is used; the four partial sums meet in shared memory.
constexpr int kCombineWarps = 4;
template <int ODT>
__global__ void __launch_bounds__(kCombineWarps * 32)
decode_combine_kernel(const float *__restrict__ partials, void *__restrict__ out, int rows, int n_splits,
                      long long row_stride, long long split_stride) {
  __shared__ float sm_acc[kCombineWarps][kHeadDim];
  __shared__ float sm_l[kCombineWarps];
  const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float *base = partials + (size_t)row * row_stride;
  float M = -INFINITY;
  for (int s = lane; s < n_splits; s += 32) M = fmaxf(M, base[(size_t)s * split_stride + kHeadDim]);
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, d));
  const float Ms = (M == -INFINITY) ? 0.f : M;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
  constexpr int kU = 4;
  for (int s0 = warp; s0 < n_splits; s0 += kCombineWarps * kU) {
    float2 o01[kU], o23[kU];
    float ms[kU], ls[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int s = s0 + u * kCombineWarps;
      const float *ps = base + (size_t)(s < n_splits ? s : s0) * split_stride;
      o01[u] = *reinterpret_cast<const float2 *>(ps + lane * 4);
      o23[u] = *reinterpret_cast<const float2 *>(ps + lane * 4 + 2);
      ms[u] = ps[kHeadDim];
      ls[u] = ps[kHeadDim + 1];
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (s0 + u * kCombineWarps < n_splits) {
        const float w = ex2(ms[u] - Ms);
        acc.x += w * o01[u].x;
        acc.y += w * o01[u].y;
        acc.z += w * o23[u].x;
        acc.w += w * o23[u].y;
        lsum += w * ls[u];
      }
    }
  }
  *reinterpret_cast<float4 *>(&sm_acc[warp][lane * 4]) = acc;
  if (lane == 0) sm_l[warp] = lsum;
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int w = 1; w < kCombineWarps; ++w) {
    const float4 a = *reinterpret_cast<const float4 *>(&sm_acc[w][lane * 4]);
    acc.x += a.x;
    acc.y += a.y;
    acc.z += a.z;
    acc.w += a.w;
    lsum += sm_l[w];
  }
  if constexpr (ODT == NB200_F32) {
    float *dst = reinterpret_cast<float *>(out) + (size_t)row * (kHeadDim + 2);
    dst[lane * 4 + 0] = acc.x;
    dst[lane * 4 + 1] = acc.y;
    dst[lane * 4 + 2] = acc.z;
    dst[lane * 4 + 3] = acc.w;
    if (lane == 0) {
      dst[kHeadDim] = M;
      dst[kHeadDim + 1] = lsum;
    }
  } else {
    const float inv = lsum == 0.f ? 0.f : 1.f / lsum;  // a sequence of length 0 (paged cache) yields zeros; a NaN-poisoned partial stays NaN
    uint2 w;
    w.x = pack2<ODT>(acc.x * inv, acc.y * inv);
    w.y = pack2<ODT>(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(out) + (size_t)row * kHeadDim + lane * 4) = w;
  }
}

template <int DT>
int launch_splitk(const void *q, const void *k, const void *v, float *partials, int B, int Hq, int Hkv,
                  int Lkv, int n_splits, float scale_log2, int *status, cudaStream_t st,
                  const int *block_table = nullptr, const int *seq_lens = nullptr, int max_pages = 0,
                  int num_pages = 0) {
  const dim3 grid(n_splits, Hkv, B), block(kDecodeThreads);
  const auto *qp = static_cast<const uint16_t *>(q);
  const auto *kp = static_cast<const uint16_t *>(k);
  const auto *vp = static_cast<const uint16_t *>(v);
  // long splits: K/V through the ring of bulk copies; short ones: per-lane loads
  const bool ring = Lkv / n_splits >= 4 * kStageRows;
#define NB200_DECODE_CASE(GV)                                                                                          \
  case GV:                                                                                                             \
    if (block_table != nullptr || (ring && GV <= 4)) { /* dense G = 8: 128 accumulator registers, per-lane loads spill less */ \
      NB200_CHECK_CUDA(cudaFuncSetAttribute(decode_splitk_ring_kernel<DT, GV>,                                         \
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSmem));                  \
      NB200_CHECK_CUDA(cudaFuncSetAttribute(decode_splitk_ring_kernel<DT, GV>,                                         \
                                            cudaFuncAttributePreferredSharedMemoryCarveout,                            \
                                            cudaSharedmemCarveoutMaxShared));                                          \
      decode_splitk_ring_kernel<DT, GV><<<grid, dim3(kRingThreads), kRingSmem, st>>>(                                  \
          qp, kp, vp, partials, Hkv, Lkv, n_splits, scale_log2, block_table, seq_lens, max_pages, num_pages, status); \
    } else {                                                                                                           \
      decode_splitk_kernel<DT, GV><<<grid, block, 0, st>>>(qp, kp, vp, partials, Hkv, Lkv, n_splits, scale_log2);      \
    }                                                                                                                  \
    break;
  switch (Hq / Hkv) {
    NB200_DECODE_CASE(1)
    NB200_DECODE_CASE(2)
    NB200_DECODE_CASE(4)
    NB200_DECODE_CASE(8)
    default: return fail(NB200_ERR_UNSUPPORTED, "decode: Hq/Hkv = %d not in {1,2,4,8}", Hq / Hkv);
  }
#undef NB200_DECODE_CASE
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_decode_workspace_bytes(int B, int Hq, int D, int n_splits) {
  if (B <= 0 || Hq <= 0 || D <= 0 || n_splits <= 0) return 0;
  return (size_t)B * Hq * n_splits * (D + 2) * sizeof(float);
}

extern "C" int nb200_decode_auto_splits(int B, int Hkv, int Lkv, int max_splits) {
  if (B <= 0 || Hkv <= 0 || Lkv <= 0 || max_splits < 0) return 0;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return 0;
  // One CTA per (split, kv head, sequence), two CTAs resident per SM.  The time of a launch is about
  // waves * (rows per split + a fixed cost per CTA): pick the split count that minimises it.  The fixed cost
  // (prologue, cross-warp merge, write of the partial) is worth about 128 rows of streaming at one CTA's
  // share of the bandwidth.  Splits stay at 256 rows or more (from there K/V stream through the ring of bulk
  // copies) unless that leaves CTA slots empty, in which case they may shrink to 64 rows.
  const long long slots = 2ll * sms, units = (long long)B * Hkv;
  const long long cap = max_splits > 0 ? max_splits : (1ll << 30);
  long long best = 1;
  double best_cost = 0.0;
  for (long long n = 1; n <= cap && n <= Lkv && n <= 4096; ++n) {
    const long long rows = Lkv / n;
    if (n > 1 && rows < 4 * kStageRows && ((n - 1) * units >= slots || rows < kStageRows)) break;
    const long long waves = (n * units + slots - 1) / slots;
    const double cost = static_cast<double>(waves) * static_cast<double>((Lkv + n - 1) / n + 128);
    if (n == 1 || cost < best_cost * 0.995) {   // a clearly better count only: more splits cost combine work
      best = n;
      best_cost = cost;
    }
  }
  if (best > Lkv) best = Lkv;
  return static_cast<int>(best);
}

extern "C" int nb200_decode_splitk(const void *q, const void *k, const void *v, float *partials, int B,
                                   int Hq, int Hkv, int Lkv, int D, int n_splits, int dtype,
                                   float scale_log2, int *status, void *stream) {
  NB200_REQUIRE(q && k && v && partials, NB200_ERR_BAD_ARG, "decode_splitk: null pointer");
  NB200_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Lkv > 0 && n_splits > 0, NB200_ERR_BAD_ARG,
                "decode_splitk: non-positive extent");
  NB200_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v), NB200_ERR_BAD_ARG,
                "decode_splitk: q/k/v must be 16-byte aligned");
  NB200_REQUIRE(D == kHeadDim, NB200_ERR_UNSUPPORTED, "decode_splitk: D = %d, only 128 is implemented", D);
  NB200_REQUIRE(Hq % Hkv == 0, NB200_ERR_UNSUPPORTED, "decode_splitk: Hq %% Hkv != 0");
  NB200_REQUIRE(n_splits <= Lkv, NB200_ERR_UNSUPPORTED, "decode_splitk: more splits (%d) than KV rows (%d)",
                n_splits, Lkv);
  NB200_REQUIRE(Hkv <= 65535 && B <= 65535, NB200_ERR_UNSUPPORTED, "decode_splitk: grid too large");
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == NB200_BF16) return launch_splitk<NB200_BF16>(q, k, v, partials, B, Hq, Hkv, Lkv, n_splits, scale_log2, status, st);
  if (dtype == NB200_F16) return launch_splitk<NB200_F16>(q, k, v, partials, B, Hq, Hkv, Lkv, n_splits, scale_log2, status, st);
  return fail(NB200_ERR_UNSUPPORTED, "decode_splitk: dtype %d (f16 and bf16 only)", dtype);
}

namespace {

size_t sharded_local_offset(int Hkv) { return ((size_t)(2 * Hkv + 1) * sizeof(int) + 255) / 256 * 256; }
size_t sharded_partials_offset(int Hq, int Hkv) {
  return sharded_local_offset(Hkv) + ((size_t)Hq * (kHeadDim + 2) * sizeof(float) + 255) / 256 * 256;
}

template <int DT, int GV>
int launch_sharded(const void *q, const void *k, const void *v, float *partials, int Hkv, int Lkv, int n_splits,
                   float scale_log2, int *status, const DecodeTail &tail, cudaStream_t st) {
  NB200_CHECK_CUDA(cudaFuncSetAttribute(decode_splitk_ring_kernel<DT, GV, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSmem));
  NB200_CHECK_CUDA(cudaFuncSetAttribute(decode_splitk_ring_kernel<DT, GV, true, true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
  decode_splitk_ring_kernel<DT, GV, true, true><<<dim3(n_splits * Hkv), dim3(kRingThreads), kRingSmem, st>>>(
      static_cast<const uint16_t *>(q), static_cast<const uint16_t *>(k), static_cast<const uint16_t *>(v), partials, Hkv, Lkv,
      n_splits, scale_log2, nullptr, nullptr, 0, 0, status, tail);
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

}  // namespace

extern "C" size_t nb200_decode_sharded_workspace_bytes(int Hq, int Hkv, int D, int n_splits) {
  if (Hq <= 0 || Hkv <= 0 || D != kHeadDim || n_splits <= 0 || Hq % Hkv != 0) return 0;
  return sharded_partials_offset(Hq, Hkv) + (size_t)Hq * n_splits * (kHeadDim + 2) * sizeof(float);
}

extern "C" int nb200_decode_sharded_fwd(const void *q, const void *k, const void *v, void *workspace,
                                        void *const *peer_buffers, void *out, int Hq, int Hkv, int Lkv, int D,
                                        int n_splits, int dtype, float scale_log2, int world, int rank,
                                        unsigned generation, int out_dtype, long long wait_ns, int *status,
                                        void *stream) {
  NB200_REQUIRE(q && k && v && workspace && out, NB200_ERR_BAD_ARG, "decode_sharded_fwd: null pointer");
  NB200_REQUIRE(Hq > 0 && Hkv > 0 && Lkv > 0 && n_splits > 0 && world > 0 && rank >= 0 && rank < world, NB200_ERR_BAD_ARG,
                "decode_sharded_fwd: bad extent or rank");
  NB200_REQUIRE(D == kHeadDim, NB200_ERR_UNSUPPORTED, "decode_sharded_fwd: D = %d, only 128 is implemented", D);
  NB200_REQUIRE(Hq % Hkv == 0 && n_splits <= Lkv && Hkv <= 65535, NB200_ERR_UNSUPPORTED, "decode_sharded_fwd: Hq %% Hkv != 0, or more splits than rows");
  NB200_REQUIRE(world <= peer::kMaxWorld, NB200_ERR_UNSUPPORTED, "decode_sharded_fwd: at most %d ranks", peer::kMaxWorld);
  NB200_REQUIRE(world == 1 || (peer_buffers && generation != 0 && wait_ns > 0), NB200_ERR_BAD_ARG,
                "decode_sharded_fwd: several ranks need peer buffers, a generation >= 1 and a positive wait limit");
  NB200_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0 &&
                    (reinterpret_cast<uintptr_t>(out) & (out_dtype == NB200_F32 ? 3u : 7u)) == 0,
                NB200_ERR_BAD_ARG, "decode_sharded_fwd: q/k/v 16-byte, workspace 256-byte, out 8-byte aligned");
  NB200_REQUIRE(out_dtype == NB200_BF16 || out_dtype == NB200_F16 || out_dtype == NB200_F32, NB200_ERR_UNSUPPORTED,
                "decode_sharded_fwd: out_dtype %d", out_dtype);
  auto *ws = static_cast<unsigned char *>(workspace);
  DecodeTail tail{};
  tail.counters = reinterpret_cast<int *>(ws);
  tail.local = reinterpret_cast<float *>(ws + sharded_local_offset(Hkv));
  float *partials = reinterpret_cast<float *>(ws + sharded_partials_offset(Hq, Hkv));
  for (int r = 0; r < world && world > 1; ++r) {
    NB200_REQUIRE(peer_buffers[r] && aligned16(peer_buffers[r]), NB200_ERR_BAD_ARG,
                  "decode_sharded_fwd: buffer of rank %d is null or not 16-byte aligned", r);
    tail.peers.buf[r] = static_cast<float *>(peer_buffers[r]);
  }
  tail.out = out;
  tail.world = world;
  tail.rank = rank;
  tail.out_dtype = out_dtype;
  tail.generation = generation;
  tail.wait_ns = wait_ns;
  tail.status = status;
  auto st = static_cast<cudaStream_t>(stream);
#define NB200_SHARDED(DTV)                                                                                             \
  switch (Hq / Hkv) {                                                                                                  \
    case 1: return launch_sharded<DTV, 1>(q, k, v, partials, Hkv, Lkv, n_splits, scale_log2, status, tail, st);         \
    case 2: return launch_sharded<DTV, 2>(q, k, v, partials, Hkv, Lkv, n_splits, scale_log2, status, tail, st);         \
    case 4: return launch_sharded<DTV, 4>(q, k, v, partials, Hkv, Lkv, n_splits, scale_log2, status, tail, st);         \
    case 8: return launch_sharded<DTV, 8>(q, k, v, partials, Hkv, Lkv, n_splits, scale_log2, status, tail, st);         \
    default: return fail(NB200_ERR_UNSUPPORTED, "decode_sharded_fwd: Hq/Hkv = %d not in {1,2,4,8}", Hq / Hkv);         \
  }
  if (dtype == NB200_BF16) { NB200_SHARDED(NB200_BF16) }
  if (dtype == NB200_F16) { NB200_SHARDED(NB200_F16) }
#undef NB200_SHARDED
  return fail(NB200_ERR_UNSUPPORTED, "decode_sharded_fwd: dtype %d (f16 and bf16 only)", dtype);
}

extern "C" int nb200_decode_paged_splitk(const void *q, const void *k_pages, const void *v_pages,
                                         const int *block_table, const int *seq_lens, float *partials, int B,
                                         int Hq, int Hkv, int num_pages, int max_pages, int page_size, int D,
                                         int n_splits, int dtype, float scale_log2, int *status, void *stream) {
  NB200_REQUIRE(q && k_pages && v_pages && block_table && seq_lens && partials, NB200_ERR_BAD_ARG,
                "decode_paged_splitk: null pointer");
  NB200_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && num_pages > 0 && max_pages > 0 && n_splits > 0, NB200_ERR_BAD_ARG,
                "decode_paged_splitk: non-positive extent");
  NB200_REQUIRE((long long)max_pages * page_size < (1ll << 31), NB200_ERR_UNSUPPORTED,
                "decode_paged_splitk: max_pages * page_size does not fit 31 bits");
  NB200_REQUIRE(aligned16(q) && aligned16(k_pages) && aligned16(v_pages), NB200_ERR_BAD_ARG,
                "decode_paged_splitk: q and the page pools must be 16-byte aligned");
  NB200_REQUIRE(D == kHeadDim, NB200_ERR_UNSUPPORTED, "decode_paged_splitk: D = %d, only 128 is implemented", D);
  NB200_REQUIRE(page_size == kStageRows, NB200_ERR_UNSUPPORTED,
                "decode_paged_splitk: page_size = %d, only %d rows per page is implemented", page_size, kStageRows);
  NB200_REQUIRE(Hq % Hkv == 0, NB200_ERR_UNSUPPORTED, "decode_paged_splitk: Hq %% Hkv != 0");
  NB200_REQUIRE(Hkv <= 65535 && B <= 65535, NB200_ERR_UNSUPPORTED, "decode_paged_splitk: grid too large");
  auto st = static_cast<cudaStream_t>(stream);
  const int Lmax = max_pages * page_size;
  if (dtype == NB200_BF16)
    return launch_splitk<NB200_BF16>(q, k_pages, v_pages, partials, B, Hq, Hkv, Lmax, n_splits, scale_log2, status, st,
                                     block_table, seq_lens, max_pages, num_pages);
  if (dtype == NB200_F16)
    return launch_splitk<NB200_F16>(q, k_pages, v_pages, partials, B, Hq, Hkv, Lmax, n_splits, scale_log2, status, st,
                                    block_table, seq_lens, max_pages, num_pages);
  return fail(NB200_ERR_UNSUPPORTED, "decode_paged_splitk: dtype %d (f16 and bf16 only)", dtype);
}

extern "C" int nb200_decode_combine(const float *partials, void *out, int rows, int D, int n_splits,
                                    long long row_stride, long long split_stride, int out_dtype,
                                    void *stream) {
  NB200_REQUIRE(partials && out, NB200_ERR_BAD_ARG, "decode_combine: null pointer");
  NB200_REQUIRE(rows > 0 && n_splits > 0, NB200_ERR_BAD_ARG, "decode_combine: non-positive extent");
  NB200_REQUIRE(D == kHeadDim, NB200_ERR_UNSUPPORTED, "decode_combine: D = %d, only 128 is implemented", D);
  NB200_REQUIRE(row_stride % 2 == 0 && split_stride % 2 == 0 &&
                    (reinterpret_cast<uintptr_t>(partials) & 7u) == 0,
                NB200_ERR_BAD_ARG, "decode_combine: partials must be 8-byte aligned with even strides");
  // 16-bit outputs are written as 8-byte vectors (four elements per lane), fp32 partials as single floats
  NB200_REQUIRE((reinterpret_cast<uintptr_t>(out) & (out_dtype == NB200_F32 ? 3u : 7u)) == 0, NB200_ERR_BAD_ARG,
                "decode_combine: out must be %d-byte aligned", out_dtype == NB200_F32 ? 4 : 8);
  auto st = static_cast<cudaStream_t>(stream);
  const dim3 grid(rows), block(kCombineWarps * 32);
  switch (out_dtype) {
    case NB200_BF16: decode_combine_kernel<NB200_BF16><<<grid, block, 0, st>>>(partials, out, rows, n_splits, row_stride, split_stride); break;
    case NB200_F16: decode_combine_kernel<NB200_F16><<<grid, block, 0, st>>>(partials, out, rows, n_splits, row_stride, split_stride); break;
    case NB200_F32: decode_combine_kernel<NB200_F32><<<grid, block, 0, st>>>(partials, out, rows, n_splits, row_stride, split_stride); break;
    default: return fail(NB200_ERR_UNSUPPORTED, "decode_combine: out_dtype %d", out_dtype);
  }
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

// ---- decode without any allocation ---------------------------------------------------------------
// Scratch for nb200_decode_fwd_static: the split-K partials live in this fixed array instead of a
// caller-provided workspace.  Every GPU on which the library is loaded carries these 4 MiB until
// the process exits.  In host code the array's name only stands for the symbol; the address that a
// kernel can use comes from cudaGetSymbolAddress, looked up once per device below.
static __device__ __align__(256) unsigned char nb200_decode_static_scratch[NB200_DECODE_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_static_scratch_mutex;
float *g_static_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device (resolved on first use per device).
int static_scratch_address(float **out) {
  int dev = -1;
  NB200_CHECK_CUDA(cudaGetDevice(&dev));
  NB200_REQUIRE(dev >= 0 && dev < kMaxDevices, NB200_ERR_UNSUPPORTED, "decode_fwd_static: device index %d", dev);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void *p = nullptr;
    NB200_CHECK_CUDA(cudaGetSymbolAddress(&p, nb200_decode_static_scratch));
    NB200_REQUIRE(p != nullptr, NB200_ERR_LAUNCH, "decode_fwd_static: cudaGetSymbolAddress returned null");
    g_static_scratch_ptr[dev] = static_cast<float *>(p);
  }
  *out = g_static_scratch_ptr[dev];
  return NB200_OK;
}

}  // namespace

extern "C" int nb200_decode_fwd_static(const void *q, const void *k, const void *v, void *out, int B, int Hq,
                                       int Hkv, int Lkv, int D, int n_splits, int dtype, float scale_log2,
                                       void *stream) {
  NB200_REQUIRE(q && k && v && out, NB200_ERR_BAD_ARG, "decode_fwd_static: null pointer");
  NB200_REQUIRE(B > 0 && Hq > 0 && Hkv > 0 && Lkv > 0 && D > 0 && n_splits > 0, NB200_ERR_BAD_ARG,
                "decode_fwd_static: non-positive extent");
  // checked here as well as in the combine, so that a bad `out` is refused before anything is launched
  NB200_REQUIRE((reinterpret_cast<uintptr_t>(out) & 7u) == 0, NB200_ERR_BAD_ARG,
                "decode_fwd_static: out must be 8-byte aligned");
  const size_t need = (size_t)B * Hq * n_splits * ((size_t)D + 2) * sizeof(float);
  NB200_REQUIRE(need <= (size_t)NB200_DECODE_STATIC_SCRATCH_BYTES, NB200_ERR_UNSUPPORTED,
                "decode_fwd_static: B*Hq*n_splits*(D+2) floats = %zu bytes of partials do not fit the built-in "
                "%zu-byte scratch; call nb200_decode_splitk / nb200_decode_combine with your own workspace",
                need, (size_t)NB200_DECODE_STATIC_SCRATCH_BYTES);
  float *partials = nullptr;
  const int rc = static_scratch_address(&partials);
  if (rc != NB200_OK) return rc;
  // Split-K writes every (row, split) slot that the combine reads, so nothing left in the array by
  // an earlier call can leak into this one and nothing has to be cleared first.
  const int rc1 = nb200_decode_splitk(q, k, v, partials, B, Hq, Hkv, Lkv, D, n_splits, dtype, scale_log2, nullptr, stream);
  if (rc1 != NB200_OK) return rc1;
  return nb200_decode_combine(partials, out, B * Hq, D, n_splits, (long long)n_splits * (D + 2), D + 2, dtype,
                              stream);
}
