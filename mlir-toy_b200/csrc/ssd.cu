// Mamba-2 SSD scan forward, fused into one kernel with the state kept on chip.
//
//   S <- exp(dt*A) S + dt * x (outer) B ;   y = S . C        (S is P x N per (batch, head))
//
// One CTA owns TWO heads of one batch (a "lane" each) and walks a segment of the sequence in steps of 128
// rows; the fp32 state S (N x P = 128 x 64) of each head never leaves tensor memory, x is read once and y
// written once.  With cum_i = sum_{s<=i} dt_s*A inside a step (kept in the log2 domain) a step of one head is
//
//   G  = C . B^T                             both operands TMA tiles in shared memory; the heads of a group
//                                            share B and C, so the CTA computes G once for its two heads
//   Y  = C . S_in, then row i scaled by      B operand: S_in rounded to 16 bit in shared memory; the scaling is
//        e^cum_i in TMEM                     an element-wise pass over the 64 columns      (128x64x128)
//   S  = e^cum_last S + B^T . (w x)          w_j = e^(cum_last - cum_j) dt_j; both operands MN-major
//                                            shared-memory tiles, accumulator = the state  (128x64x128)
//   Y += (G o decay o mask) . x              decay_ij = e^(cum_i - cum_j) dt_j for j <= i; A operand: the
//                                            16-bit masked copy of G in TMEM               (128x64x128)
//
// Warps (15, one CTA per SM):
//   0-3, 4-7    element-wise warps of head 0 / head 1: thread i = row i of the step = TMEM lane i: the scaled
//               copies of x and S, the decay/mask pass over G (an exponential per element only in the
//               32-column chunk on the diagonal; chunks left of it take one factor per row and one per column),
//               the row scaling of C.S_in and the epilogue (Y -> 16 bit -> staging buffer)
//   8, 9        per-head TMA producer: x and dt tiles of the next step, and the TMA store of the finished Y tile
//   10, 11      per-head MMA issuer (warp 10 also issues the shared G product)
//   12, 13      per-head prefix warp: the scan of dt*A over the 128 rows of a step and everything derived from it
//               alone, written to a double-buffered table one to two steps ahead
//   14          TMA producer of the shared B and C tiles
//
// Shared memory: B and C tiles (32 KB each, shared by the two heads) and per head four 16 KB buffers that
// rotate through the roles x(s) / Y(s) staging, 16-bit copy of the incoming state, w*x(s), and x(s+1) in
// flight, so that no element-wise pass waits for a buffer: 208 KB.  Tensor memory (all 512 columns):
// G 0-127; per head the masked 16-bit product 64, Y 64 and the state 64 columns.
//
// A sequence can be cut into segments that run as separate CTAs: ssd_segment_state_kernel first leaves in global
// memory the state each segment but the last would reach from zero and its total decay; a CTA of segment k > 0
// then starts from the recurrence over the earlier segments' states.  That is how a problem with few
// (batch, head) pairs, e.g. one GPU's share of the heads, still fills the SMs.
//
// All exponents are <= 0 (A < 0), so nothing overflows.  Every barrier exists twice and alternates with the
// step, so a waiter can never be lapped; every wait is bounded and reports through the status words.
#include <cuda.h>

#include "nb200_common.cuh"
#include "sm100_primitives.cuh"
#include "tma_host.cuh"

namespace nb200 {
namespace {

using namespace sm100;

constexpr int kQ = 128;          // rows per step
constexpr int kP = 64;           // head dimension
constexpr int kN = 128;          // state dimension
constexpr int kBCBytes = kQ * kN * 2;      // 32 KB: two 64-column boxes of 16 KB
constexpr int kBCBox = kBCBytes / 2;
constexpr int kXBytes = kQ * kP * 2;       // 16 KB: one box
constexpr int kUBufs = 4;                  // rotating 16 KB buffers per head
constexpr int kDtBytes = kQ * 4 * 4;       // 128 rows x 4 heads of dt (fp32): the 16-byte minimum of a TMA box row
constexpr int kPfFloats = 4 * kQ;          // one prefix table: cum[128] | dt[128] | lb[128] | cf[128]
constexpr int kPfBytes = kPfFloats * 4;
constexpr int kLaneBytes = kUBufs * kXBytes + 2 * kPfBytes + 2 * kDtBytes;   // 72 KB per head
constexpr int kSsdThreads = 15 * 32;
constexpr int kSsdSmem = 2 * kBCBytes + 2 * kLaneBytes + 1024 /*barriers*/;
constexpr int kSsdTmemCols = 512;
constexpr int kStateFloats = kN * kP;
constexpr float kLog2e = 1.4426950408889634f;

enum : int { kErrSsdProducer = 11, kErrSsdMma = 12, kErrSsdCompute = 13, kErrSsdPrefix = 14, kErrSsdAlign = 15,
             kErrSsdShared = 16, kErrSegState = 17 };

// Per-head barriers; index [s & 1], parity (s >> 1) & 1 for local step s.
struct LaneBars {
  uint64_t x_full[2], dt_full[2], pf_full[2], pf_free[2], e1a[2], inter_done[2], e1b[2], z_done[2], m_ready[2],
      y_ready[2], y_staged[2], y_free[2];
};
struct SsdBarriers {
  LaneBars lane[2];
  uint64_t c_full[2], b_full[2], g_ready[2];
  uint32_t tmem_base;
  int abort_flag;
  int skip;
};
static_assert(sizeof(SsdBarriers) <= 1024, "barrier block");

__device__ __forceinline__ void ssd_report(int *status, int code, int detail) {
  if (status && atomicCAS(status, 0, code) == 0) {
    status[1] = static_cast<int>(blockIdx.x);
    status[2] = detail;
    status[3] = static_cast<int>(threadIdx.x);
  }
}

__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `c` of row `r` inside a 128-byte-swizzled box (rows of 128 bytes).
__device__ __forceinline__ uint32_t sw128(int r, int c) { return r * 128 + ((c ^ (r & 7)) << 4); }

__device__ __forceinline__ uint32_t bar2(const uint64_t (&b)[2], int s) { return smem_u32(&b[s & 1]); }
__device__ __forceinline__ uint32_t par2(int s) { return static_cast<uint32_t>(s >> 1) & 1u; }

// Work of one CTA: heads h0 .. h0 + lanes - 1 of batch b, steps [s_begin, s_end) of the sequence.
struct SsdWork {
  int b, h0, seg, s_begin, s_end;
};

template <int DT>
__global__ void __launch_bounds__(kSsdThreads, 1)
ssd_fused_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_y,
                 const __grid_constant__ CUtensorMap tm_dt, int dt_by_tma, const float *__restrict__ dt,
                 const float *__restrict__ A, int L, int H, int G, int lanes, int nseg, int steps_per_seg,
                 const float *__restrict__ seg_states, const float *__restrict__ seg_totals, int *status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t base = smem_u32(smem);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) ssd_report(status, kErrSsdAlign, static_cast<int>(base));
    return;
  }
  const uint32_t sB = base, sC = base + kBCBytes;
  SsdBarriers *bars = reinterpret_cast<SsdBarriers *>(smem + 2 * kBCBytes + 2 * kLaneBytes);
  volatile int *abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nsteps_total = L / kQ;
  // block -> (batch, segment, head group of `lanes` heads); CTAs that share B/C tiles are neighbours
  const int groups = H / lanes;
  const int hg = blockIdx.x % groups, seg = (blockIdx.x / groups) % nseg, b = blockIdx.x / (groups * nseg);
  const int s_begin = seg * steps_per_seg, s_end = min(nsteps_total, s_begin + steps_per_seg);
  const int nsteps = s_end - s_begin;
  const int h_first = hg * lanes;
  const int g = h_first / (H / G);

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    bars->skip = (status != nullptr && *reinterpret_cast<volatile int *>(status) != 0) ? 1 : 0;
    for (int q = 0; q < 2; ++q) {
      LaneBars &lb = bars->lane[q];
      for (int p = 0; p < 2; ++p) {
        mbar_init(smem_u32(&lb.x_full[p]), 1);
        mbar_init(smem_u32(&lb.dt_full[p]), 1);
        mbar_init(smem_u32(&lb.pf_full[p]), 1);
        mbar_init(smem_u32(&lb.pf_free[p]), 128);
        mbar_init(smem_u32(&lb.e1a[p]), 128);
        mbar_init(smem_u32(&lb.inter_done[p]), 1);
        mbar_init(smem_u32(&lb.e1b[p]), 128);
        mbar_init(smem_u32(&lb.z_done[p]), 1);
        mbar_init(smem_u32(&lb.m_ready[p]), 128);
        mbar_init(smem_u32(&lb.y_ready[p]), 1);
        mbar_init(smem_u32(&lb.y_staged[p]), 128);
        mbar_init(smem_u32(&lb.y_free[p]), 1);
      }
    }
    for (int p = 0; p < 2; ++p) {
      mbar_init(smem_u32(&bars->c_full[p]), 1);
      mbar_init(smem_u32(&bars->b_full[p]), 1);
      mbar_init(smem_u32(&bars->g_ready[p]), 1);
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (bars->skip) return;

  if (warp == 10) {
    tmem_alloc(smem_u32(&bars->tmem_base), kSsdTmemCols);
    tmem_relinquish();
  }
  if (warp == 14 && lane == 0) {
    tma_prefetch_desc(&tm_x);
    tma_prefetch_desc(&tm_b);
    tma_prefetch_desc(&tm_c);
    tma_prefetch_desc(&tm_y);
    if (dt_by_tma) tma_prefetch_desc(&tm_dt);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const uint32_t tG = tmem;

  // role -> head lane q (0 or 1)
  const int q = (warp < 8) ? (warp >> 2) : ((warp < 14) ? (warp & 1) : 0);
  const bool lane_active = q < lanes;
  const int h = h_first + q;
  LaneBars &LB = bars->lane[q];
  unsigned char *pLane = smem + 2 * kBCBytes + q * kLaneBytes;
  const uint32_t sLane = base + 2 * kBCBytes + q * kLaneBytes;
  const uint32_t sU = sLane;                                      // U[k] at + k * kXBytes
  float *pf_all = reinterpret_cast<float *>(pLane + kUBufs * kXBytes);
  const float *dt_tile = reinterpret_cast<const float *>(pLane + kUBufs * kXBytes + 2 * kPfBytes);
  const uint32_t sDt = sLane + kUBufs * kXBytes + 2 * kPfBytes;
  const uint32_t tM = tmem + 128 + 192 * q, tY = tM + 64, tS = tM + 128;

  if (warp == 14) {
    // ================================ producer of the shared B and C tiles ================================
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int s = 0; s < nsteps && ok; ++s) {
        const int row = b * L + (s_begin + s) * kQ;
        if (s > 0) {
          // C(s-1) is free once G(s-1) and both heads' C.S_in(s-1) have retired (G is issued before them by the
          // same thread, so the later commit covers it)
          for (int k = 0; k < lanes && ok; ++k)
            ok = mbar_wait(bar2(bars->lane[k].inter_done, s - 1), par2(s - 1), abort_flag);
          if (!ok) { ssd_report(status, kErrSsdShared, 4 * s); break; }
        }
        mbar_arrive_expect_tx(bar2(bars->c_full, s), kBCBytes);
        tma_load_2d(sC, &tm_c, g * kN, row, bar2(bars->c_full, s));
        tma_load_2d(sC + kBCBox, &tm_c, g * kN + 64, row, bar2(bars->c_full, s));
        if (s > 0) {
          for (int k = 0; k < lanes && ok; ++k)
            ok = mbar_wait(bar2(bars->lane[k].z_done, s - 1), par2(s - 1), abort_flag);
          if (!ok) { ssd_report(status, kErrSsdShared, 4 * s + 1); break; }
        }
        mbar_arrive_expect_tx(bar2(bars->b_full, s), kBCBytes);
        tma_load_2d(sB, &tm_b, g * kN, row, bar2(bars->b_full, s));
        tma_load_2d(sB + kBCBox, &tm_b, g * kN + 64, row, bar2(bars->b_full, s));
        ++issued;
      }
      if (!ok && issued > 0) {
        for (int spin = 0; spin < 100000; ++spin) {  // let the loads in flight land before smem goes away
          if (mbar_try_wait(bar2(bars->c_full, issued - 1), par2(issued - 1)) &&
              mbar_try_wait(bar2(bars->b_full, issued - 1), par2(issued - 1)))
            break;
          __nanosleep(100);
        }
      }
    }
    __syncwarp();
  } else if (warp == 8 || warp == 9) {
    // ================================ per-head producer: x, dt, and the Y store ===========================
    if (lane == 0 && lane_active) {
      bool ok = true;
      int issued_x = 0, issued_dt = 0;
      auto load_x = [&](int s) {
        mbar_arrive_expect_tx(bar2(LB.x_full, s), kXBytes);
        tma_load_2d(sU + (s & 3) * kXBytes, &tm_x, h * kP, b * L + (s_begin + s) * kQ, bar2(LB.x_full, s));
        ++issued_x;
      };
      // dt of one step for the four heads around h (a TMA box row cannot be narrower than 16 bytes)
      auto load_dt = [&](int s) {
        if (!dt_by_tma) return;
        mbar_arrive_expect_tx(bar2(LB.dt_full, s), kDtBytes);
        tma_load_2d(sDt + (s & 1) * kDtBytes, &tm_dt, h & ~3, b * L + (s_begin + s) * kQ, bar2(LB.dt_full, s));
        ++issued_dt;
      };
      load_dt(0);
      if (nsteps > 1) load_dt(1);
      load_x(0);
      for (int s = 0; s < nsteps; ++s) {
        if (s + 1 < nsteps) {
          // x(s+1) goes where the 16-bit state copy of step s sat: free once C.S_in(s) has retired
          ok = mbar_wait(bar2(LB.inter_done, s), par2(s), abort_flag);
          if (!ok) { ssd_report(status, kErrSsdProducer, 4 * s); break; }
          load_x(s + 1);
          if (s + 2 < nsteps) load_dt(s + 2);   // its buffer held dt(s), consumed before step s's first product
        }
        // the finished Y tile sits where x(s) was
        ok = mbar_wait(bar2(LB.y_staged, s), par2(s), abort_flag);
        if (!ok) { ssd_report(status, kErrSsdProducer, 4 * s + 2); break; }
        tma_store_2d(&tm_y, sU + (s & 3) * kXBytes, h * kP, b * L + (s_begin + s) * kQ);
        tma_store_commit();
        if (s + 2 < nsteps) {   // w*x(s+2) is written into this buffer: the store must have read it
          tma_store_wait_read();
          mbar_arrive(bar2(LB.y_free, s));
        }
      }
      tma_store_wait_all();
      if (!ok) {
        for (int spin = 0; spin < 100000; ++spin) {  // let the loads in flight land before smem goes away
          bool done = true;
          for (int n = 0; n < 2; ++n) {
            const int sx = issued_x - 1 - n, sd = issued_dt - 1 - n;
            if (sx >= 0) done = done && mbar_try_wait(bar2(LB.x_full, sx), par2(sx));
            if (sd >= 0) done = done && mbar_try_wait(bar2(LB.dt_full, sd), par2(sd));
          }
          if (done) break;
          __nanosleep(100);
        }
      }
    }
    __syncwarp();
  } else if (warp == 10 || warp == 11) {
    // ================================ per-head MMA issuer =================================================
    if (lane == 0 && lane_active) {
      constexpr int fmt = (DT == NB200_BF16) ? 1 : 0;
      constexpr uint32_t id_inter = umma_idesc_f16_ab(fmt, 0, 1, kQ, kP);   // A: C (K-major), B: S_in [n][p] MN-major
      constexpr uint32_t id_g = umma_idesc_f16_ab(fmt, 0, 0, kQ, kQ);       // A: C, B: B, both K-major
      constexpr uint32_t id_z = umma_idesc_f16_ab(fmt, 1, 1, kN, kP);       // A: B^T (MN-major), B: w x (MN-major)
      constexpr uint32_t id_m2 = umma_idesc_f16_ab(fmt, 0, 1, kQ, kP);      // A: TMEM, B: x (MN-major)
      // descriptors differ only in the start address field (bits 0-13, address >> 4): keep one of each kind and add
      const uint64_t dC0 = umma_desc_sw128(sC, 16, 1024), dB0 = umma_desc_sw128(sB, 16, 1024);
      const uint64_t dBt0 = umma_desc_sw128(sB, kBCBox, 1024);   // reduction over rows: 16 rows = 2 KB per MMA
      const uint64_t dU0 = umma_desc_sw128(sU, kXBytes, 1024);
      auto kmaj = [](uint64_t d0, int kk) { return d0 + static_cast<uint64_t>(((kk >> 2) * kBCBox + (kk & 3) * 32) >> 4); };
      auto rows16 = [](uint64_t d0, int buf, int kk) { return d0 + static_cast<uint64_t>((buf * kXBytes + kk * 2048) >> 4); };
      bool ok = true;
      for (int s = 0; s < nsteps && ok; ++s) {
        ok = mbar_wait(bar2(bars->c_full, s), par2(s), abort_flag) && mbar_wait(bar2(bars->b_full, s), par2(s), abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 8 * s); break; }
        if (q == 0) {
          // the shared G = C . B^T: its TMEM columns are free once both heads have masked step s - 1
          if (s > 0) {
            for (int k = 0; k < lanes && ok; ++k)
              ok = mbar_wait(bar2(bars->lane[k].m_ready, s - 1), par2(s - 1), abort_flag);
            if (!ok) { ssd_report(status, kErrSsdMma, 8 * s + 1); break; }
          }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) umma_ss(tG, kmaj(dC0, kk), kmaj(dB0, kk), id_g, kk > 0);
          umma_commit(bar2(bars->g_ready, s));
        }
        ok = mbar_wait(bar2(LB.e1a, s), par2(s), abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 8 * s + 2); break; }
        tc_fence_after();
        // Y = C . S_in      (rows are scaled by e^cum_i afterwards)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_ss(tY, kmaj(dC0, kk), rows16(dU0, (s + 1) & 3, kk), id_inter, kk > 0);
        umma_commit(bar2(LB.inter_done, s));
        // S = (e^cum_last S) + B^T . (w x)
        ok = mbar_wait(bar2(LB.e1b, s), par2(s), abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 8 * s + 3); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(tS, dBt0 + static_cast<uint64_t>((kk * 2048) >> 4), rows16(dU0, (s + 2) & 3, kk), id_z, 1u);
        umma_commit(bar2(LB.z_done, s));
        // Y += (G o decay o mask) . x
        ok = mbar_wait(bar2(LB.m_ready, s), par2(s), abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 8 * s + 4); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_ts(tY, tM + kk * 8, rows16(dU0, s & 3, kk), id_m2, 1u);
        umma_commit(bar2(LB.y_ready, s));
      }
    }
    __syncwarp();
  } else if (warp == 12 || warp == 13) {
    // ================================ per-head prefix warp ================================================
    // Lane l owns rows 4l..4l+3 of the step.  Per step sp it leaves in table sp & 1:
    //   cum[j]  inclusive prefix sum of dt*A*log2(e) inside the step (cum[127] is the step total, cum[31], cum[63],
    //           cum[95] are the references of column chunks 0..2)
    //   dt[j]
    //   lb[j]   cum_j - log2(dt_j)
    //   cf[j]   e^(r - cum_j) dt_j with r the cum at the last row of j's 32-column chunk: the column factor of the
    //           chunks left of the diagonal, where e^(cum_i - cum_j) dt_j = e^(cum_i - r) * cf[j] and both
    //           exponents are <= 0 for every row i below the chunk
    if (lane_active) {
      const float a_log2 = A[h] * kLog2e;
      bool ok = true;
      for (int sp = 0; sp < nsteps && ok; ++sp) {
        float *tab = pf_all + (sp & 1) * kPfFloats;
        float dt4[4], cum4[4];
        if (dt_by_tma) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar2(LB.dt_full, sp), par2(sp), abort_flag));
          if (!ok) { if (lane == 0) ssd_report(status, kErrSsdPrefix, 2 * sp); break; }
          const float *tile = dt_tile + (sp & 1) * (kQ * 4) + (h & 3);
#pragma unroll
          for (int e = 0; e < 4; ++e) dt4[e] = tile[(4 * lane + e) * 4];
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            dt4[e] = dt[(static_cast<size_t>(b) * L + static_cast<size_t>(s_begin + sp) * kQ + 4 * lane + e) * H + h];
        }
        cum4[0] = dt4[0] * a_log2;
#pragma unroll
        for (int e = 1; e < 4; ++e) cum4[e] = cum4[e - 1] + dt4[e] * a_log2;
        float incl = cum4[3];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const float o = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += o;
        }
        const float excl = incl - cum4[3];
#pragma unroll
        for (int e = 0; e < 4; ++e) cum4[e] += excl;
        const float4 lbv =
            make_float4(cum4[0] - lg2(dt4[0]), cum4[1] - lg2(dt4[1]), cum4[2] - lg2(dt4[2]), cum4[3] - lg2(dt4[3]));
        const float r_own = __shfl_sync(0xffffffffu, cum4[3], lane | 7);
        const float4 cfv = make_float4(ex2(r_own - lbv.x), ex2(r_own - lbv.y), ex2(r_own - lbv.z), ex2(r_own - lbv.w));
        if (sp >= 2) {  // the table still holds step sp - 2 until every row has released it
          ok = __all_sync(0xffffffffu, mbar_wait(bar2(LB.pf_free, sp - 2), par2(sp - 2), abort_flag));
          if (!ok) { if (lane == 0) ssd_report(status, kErrSsdPrefix, 2 * sp + 1); break; }
        }
        *reinterpret_cast<float4 *>(tab + 4 * lane) = make_float4(cum4[0], cum4[1], cum4[2], cum4[3]);
        *reinterpret_cast<float4 *>(tab + kQ + 4 * lane) = make_float4(dt4[0], dt4[1], dt4[2], dt4[3]);
        *reinterpret_cast<float4 *>(tab + 2 * kQ + 4 * lane) = lbv;
        *reinterpret_cast<float4 *>(tab + 3 * kQ + 4 * lane) = cfv;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar2(LB.pf_full, sp));
      }
    }
  } else if (lane_active) {
    // ================================ element-wise warps ==================================================
    const int wq = warp & 3;                                   // TMEM lane quarter of this warp
    const int i = wq * 32 + lane;                              // row of the step == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    {  // the incoming state: zero for the first segment; else the recurrence over the states Z_j that the earlier
       // segments reach from zero, S_in = sum_j 2^(T_{j+1} + ... + T_{seg-1}) Z_j (T_j: total log2 decay of segment
       // j), summed from the nearest segment backwards until the weight underflows
      float acc[kP];
#pragma unroll
      for (int k = 0; k < kP; ++k) acc[k] = 0.f;
      if (seg > 0) {
        // The kernel is launched as a programmatic dependent of the segment-state kernel: it may start before that
        // one has ended (first segments, which need nothing from it, run on the SMs it leaves idle); the states are
        // read only behind this wait, which returns once the whole segment-state grid has finished.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const size_t slot0 = (static_cast<size_t>(b) * H + h) * (nseg - 1);
        float lg = 0.f;
        for (int j = seg - 1; j >= 0; --j) {
          const float wgt = ex2(lg);
          if (wgt == 0.f) break;   // the same for every thread of the CTA's head
          const float4 *src = reinterpret_cast<const float4 *>(seg_states + (slot0 + j) * kStateFloats + static_cast<size_t>(i) * kP);
#pragma unroll
          for (int k = 0; k < kP / 4; ++k) {
            const float4 v = src[k];
            acc[4 * k] = fmaf(wgt, v.x, acc[4 * k]);
            acc[4 * k + 1] = fmaf(wgt, v.y, acc[4 * k + 1]);
            acc[4 * k + 2] = fmaf(wgt, v.z, acc[4 * k + 2]);
            acc[4 * k + 3] = fmaf(wgt, v.w, acc[4 * k + 3]);
          }
          lg += seg_totals[slot0 + j];
        }
      }
      uint32_t z[kP];
#pragma unroll
      for (int k = 0; k < kP; ++k) z[k] = __float_as_uint(acc[k]);
      tmem_st32(tS + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(z));
      tmem_st32(tS + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(z + 32));
      tmem_wait_st();
    }
    bool ok = true;
    for (int s = 0; s < nsteps && ok; ++s) {
      unsigned char *pX = pLane + (s & 3) * kXBytes;            // x(s), later the finished Y(s)
      unsigned char *pSc = pLane + ((s + 1) & 3) * kXBytes;     // 16-bit copy of the incoming state
      unsigned char *pWx = pLane + ((s + 2) & 3) * kXBytes;     // w * x(s)
      // this step's row quantities, from the prefix warp's table
      ok = __all_sync(0xffffffffu, mbar_wait(bar2(LB.pf_full, s), par2(s), abort_flag));
      if (!ok) { ssd_report(status, kErrSsdCompute, 16 * s); break; }
      const float *tab = pf_all + (s & 1) * kPfFloats;
      const float *lb = tab + 2 * kQ, *cf = tab + 3 * kQ;
      const float cum_i = tab[i], dt_i = tab[kQ + i], total = tab[kQ - 1];
      const float ref0 = tab[31], ref1 = tab[63], ref2 = tab[95];

      // ---- E1a: S_in -> 16 bit in smem; S *= e^cum_last.  (The state is final: the previous step's y_ready,
      //      waited for in E3, was committed after its state update; the copy's buffer held w*x of that step.) ----
      {
        uint32_t sv[kP];
        tmem_ld32p(tS + lane_addr, sv);
        tmem_ld32p(tS + lane_addr + 32, sv + 32);
        tmem_wait_ld();
        const float et = ex2(total);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint4 w;
          w.x = pack2<DT>(__uint_as_float(sv[8 * cc + 0]), __uint_as_float(sv[8 * cc + 1]));
          w.y = pack2<DT>(__uint_as_float(sv[8 * cc + 2]), __uint_as_float(sv[8 * cc + 3]));
          w.z = pack2<DT>(__uint_as_float(sv[8 * cc + 4]), __uint_as_float(sv[8 * cc + 5]));
          w.w = pack2<DT>(__uint_as_float(sv[8 * cc + 6]), __uint_as_float(sv[8 * cc + 7]));
          *reinterpret_cast<uint4 *>(pSc + sw128(i, cc)) = w;
        }
#pragma unroll
        for (int k = 0; k < kP; ++k) sv[k] = __float_as_uint(__uint_as_float(sv[k]) * et);
        tmem_st32(tS + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(sv));
        tmem_st32(tS + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
        tmem_wait_st();
        tc_fence_before();
        fence_proxy_async_smem();   // the tensor core reads shared memory through the async proxy
        mbar_arrive(bar2(LB.e1a, s));
      }

      // ---- E1b: w_i x_i -> smem, into the buffer from which Y(s-2) was stored ----
      {
        ok = __all_sync(0xffffffffu, mbar_wait(bar2(LB.x_full, s), par2(s), abort_flag));
        if (ok && s >= 2) ok = __all_sync(0xffffffffu, mbar_wait(bar2(LB.y_free, s - 2), par2(s - 2), abort_flag));
        if (!ok) { ssd_report(status, kErrSsdCompute, 16 * s + 1); break; }
        const float wi = ex2(total - cum_i) * dt_i;
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          const uint4 w = *reinterpret_cast<const uint4 *>(pX + sw128(i, cc));
          const float2 f0 = unpack2<DT>(w.x), f1 = unpack2<DT>(w.y), f2 = unpack2<DT>(w.z), f3 = unpack2<DT>(w.w);
          *reinterpret_cast<uint4 *>(pWx + sw128(i, cc)) =
              make_uint4(pack2<DT>(f0.x * wi, f0.y * wi), pack2<DT>(f1.x * wi, f1.y * wi),
                         pack2<DT>(f2.x * wi, f2.y * wi), pack2<DT>(f3.x * wi, f3.y * wi));
        }
        fence_proxy_async_smem();
        mbar_arrive(bar2(LB.e1b, s));
      }

      // ---- E2: G_ij e^(cum_i - cum_j) dt_j for j <= i, else 0 -> 16 bit into this head's TMEM columns ----
      ok = __all_sync(0xffffffffu, mbar_wait(bar2(bars->g_ready, s), par2(s), abort_flag));
      if (!ok) { ssd_report(status, kErrSsdCompute, 16 * s + 2); break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
        if (c < wq) {  // a chunk left of the diagonal: every column is visible to every row of this warp
          uint32_t gv[32];
          tmem_ld32(tG + lane_addr + c * 32, gv);
          const float rf = ex2(cum_i - (c == 0 ? ref0 : (c == 1 ? ref1 : ref2)));
          const uint64_t rf2 = f2_pack(rf, rf);
          tmem_wait_ld();
#pragma unroll
          for (int qq = 0; qq < 8; ++qq) {
            const ulonglong2 c4 = *reinterpret_cast<const ulonglong2 *>(cf + c * 32 + qq * 4);
            const float2 m01 = f2_unpack(f2_mul(f2_mul(f2_pack(__uint_as_float(gv[qq * 4]), __uint_as_float(gv[qq * 4 + 1])), c4.x), rf2));
            const float2 m23 = f2_unpack(f2_mul(f2_mul(f2_pack(__uint_as_float(gv[qq * 4 + 2]), __uint_as_float(gv[qq * 4 + 3])), c4.y), rf2));
            pk[qq * 2] = pack2<DT>(m01.x, m01.y);
            pk[qq * 2 + 1] = pack2<DT>(m23.x, m23.y);
          }
        } else if (c == wq) {  // the diagonal chunk: exponent and mask per element
          uint32_t gv[32];
          tmem_ld32(tG + lane_addr + c * 32, gv);
          tmem_wait_ld();
#pragma unroll
          for (int qq = 0; qq < 8; ++qq) {
            const float4 l4 = *reinterpret_cast<const float4 *>(lb + c * 32 + qq * 4);
            const float lbs[4] = {l4.x, l4.y, l4.z, l4.w};
            float m[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = c * 32 + qq * 4 + e;
              const float val = __uint_as_float(gv[qq * 4 + e]) * ex2(cum_i - lbs[e]);
              m[e] = (j <= i) ? val : 0.f;
            }
            pk[qq * 2] = pack2<DT>(m[0], m[1]);
            pk[qq * 2 + 1] = pack2<DT>(m[2], m[3]);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) pk[k] = 0u;
        }
        tmem_st16(tM + lane_addr + c * 16, pk);
      }
      {  // Y = C . S_in has retired: scale row i by e^cum_i
        ok = __all_sync(0xffffffffu, mbar_wait(bar2(LB.inter_done, s), par2(s), abort_flag));
        if (!ok) { ssd_report(status, kErrSsdCompute, 16 * s + 3); break; }
        tc_fence_after();
        const float ei = ex2(cum_i);
        uint32_t yv[kP];
        tmem_ld32p(tY + lane_addr, yv);
        tmem_ld32p(tY + lane_addr + 32, yv + 32);
        tmem_wait_ld();
#pragma unroll
        for (int k = 0; k < kP; ++k) yv[k] = __float_as_uint(__uint_as_float(yv[k]) * ei);
        tmem_st32(tY + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(yv));
        tmem_st32(tY + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(yv + 32));
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar2(LB.m_ready, s));
      mbar_arrive(bar2(LB.pf_free, s));   // nothing of step s reads the table any more

      // ---- E3: Y -> storage dtype -> the buffer x occupied (x is dead once Y is complete);
      //      the producer warp stores the tile with one TMA copy ----
      ok = __all_sync(0xffffffffu, mbar_wait(bar2(LB.y_ready, s), par2(s), abort_flag));
      if (!ok) { ssd_report(status, kErrSsdCompute, 16 * s + 4); break; }
      tc_fence_after();
      {
        uint32_t yv[kP];
        tmem_ld32p(tY + lane_addr, yv);
        tmem_ld32p(tY + lane_addr + 32, yv + 32);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint4 w;
          w.x = pack2<DT>(__uint_as_float(yv[8 * cc + 0]), __uint_as_float(yv[8 * cc + 1]));
          w.y = pack2<DT>(__uint_as_float(yv[8 * cc + 2]), __uint_as_float(yv[8 * cc + 3]));
          w.z = pack2<DT>(__uint_as_float(yv[8 * cc + 4]), __uint_as_float(yv[8 * cc + 5]));
          w.w = pack2<DT>(__uint_as_float(yv[8 * cc + 6]), __uint_as_float(yv[8 * cc + 7]));
          *reinterpret_cast<uint4 *>(pX + sw128(i, cc)) = w;
        }
        fence_proxy_async_smem();
        mbar_arrive(bar2(LB.y_staged, s));
      }
      tc_fence_before();  // orders these TMEM reads before the next step's products, via the e1a arrival
    }
  }

  // ================================ tear-down =====================================
  tc_fence_before();
  __syncthreads();
  if (warp == 10) {
    tc_fence_after();
    tmem_dealloc(tmem, kSsdTmemCols);
  }
}

// ---- the state a segment reaches from zero ------------------------------------------------------------
// Z = sum_j e^(cum_end - cum_j) dt_j x_j (outer) B_j over the rows of one segment of one (batch, head), and the
// segment's total log2 decay cum_end.  Weights are taken relative to the END of the segment, so the accumulator
// needs no rescaling between steps: one tensor-core product per 128 rows into the same TMEM columns.  The steps
// are taken from the LAST one of the segment backwards, so that the decay from the end of a step to the end of
// the segment is simply the running sum of the totals of the steps already done; the exponent of row j is
// (total of its step - cum_j inside the step) + that sum, both summed from small terms, which keeps it accurate
// where it matters: near the end of the segment.
// Like the fused kernel a CTA takes two heads that share B (one head if they do not): warps 0-3 / 4-7: thread i =
// row i of head 0 / 1: w_i x_i in place in shared memory; warp 8: TMA producer (B, x, dt; three stages, so that
// loads run two steps ahead of the arithmetic); warp 9: MMA issuer.
constexpr int kSegStages = 3;
constexpr int kSegThreads = 320;
constexpr int kSegStageBytes = kBCBytes + 2 * kXBytes + 2 * kDtBytes;   // 68 KB
constexpr int kSegSmem = kSegStages * kSegStageBytes + 1024;

struct SegBarriers {
  uint64_t full[kSegStages], ready[kSegStages], empty[kSegStages], done;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(SegBarriers) <= 1024, "segment barrier block");

template <int DT>
__global__ void __launch_bounds__(kSegThreads, 1)
ssd_segment_state_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_b,
                         const __grid_constant__ CUtensorMap tm_dt, int dt_by_tma, const float *__restrict__ dt,
                         const float *__restrict__ A, int L, int H, int G, int lanes, int nseg, int steps_per_seg,
                         float *__restrict__ seg_states, float *__restrict__ seg_totals, int *status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t base = smem_u32(smem);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) ssd_report(status, kErrSsdAlign, static_cast<int>(base));
    return;
  }
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the fused kernel may be scheduled from now on
  SegBarriers *bars = reinterpret_cast<SegBarriers *>(smem + kSegStages * kSegStageBytes);
  volatile int *abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nsm1 = nseg - 1, groups = H / lanes;
  const int seg = blockIdx.x % nsm1, hg = (blockIdx.x / nsm1) % groups, b = blockIdx.x / (nsm1 * groups);
  const int h_first = hg * lanes;
  const int g = h_first / (H / G);
  const int s_begin = seg * steps_per_seg, nsteps = steps_per_seg;   // every segment but the last is full
  const size_t row0 = static_cast<size_t>(b) * L + static_cast<size_t>(s_begin) * kQ;

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    for (int p = 0; p < kSegStages; ++p) {
      mbar_init(smem_u32(&bars->full[p]), 1);
      mbar_init(smem_u32(&bars->ready[p]), 128 * lanes);
      mbar_init(smem_u32(&bars->empty[p]), 1);
    }
    mbar_init(smem_u32(&bars->done), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == 9) {
    tmem_alloc(smem_u32(&bars->tmem_base), 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tZ = bars->tmem_base;

  if (warp == 8) {
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int s = 0; s < nsteps; ++s) {
        const int st = s % kSegStages;
        if (s >= kSegStages) {
          ok = mbar_wait(smem_u32(&bars->empty[st]), ((s / kSegStages) - 1) & 1, abort_flag);
          if (!ok) { ssd_report(status, kErrSegState, 4 * s); break; }
        }
        const uint32_t sb = base + st * kSegStageBytes, bar = smem_u32(&bars->full[st]);
        const int row = static_cast<int>(row0) + (nsteps - 1 - s) * kQ;   // last step of the segment first
        mbar_arrive_expect_tx(bar, kBCBytes + lanes * (kXBytes + (dt_by_tma ? kDtBytes : 0)));
        tma_load_2d(sb, &tm_b, g * kN, row, bar);
        tma_load_2d(sb + kBCBox, &tm_b, g * kN + 64, row, bar);
        for (int q = 0; q < lanes; ++q) {
          tma_load_2d(sb + kBCBytes + q * kXBytes, &tm_x, (h_first + q) * kP, row, bar);
          if (dt_by_tma) tma_load_2d(sb + kBCBytes + 2 * kXBytes + q * kDtBytes, &tm_dt, (h_first + q) & ~3, row, bar);
        }
        ++issued;
      }
      if (!ok) {
        for (int spin = 0; spin < 100000; ++spin) {
          bool done = true;
          for (int n = 0; n < kSegStages; ++n) {
            const int s = issued - 1 - n;
            if (s >= 0) done = done && mbar_try_wait(smem_u32(&bars->full[s % kSegStages]), (s / kSegStages) & 1);
          }
          if (done) break;
          __nanosleep(100);
        }
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    if (lane == 0) {
      constexpr int fmt = (DT == NB200_BF16) ? 1 : 0;
      constexpr uint32_t id_z = umma_idesc_f16_ab(fmt, 1, 1, kN, kP);
      bool ok = true;
      for (int s = 0; s < nsteps; ++s) {
        const int st = s % kSegStages;
        ok = mbar_wait(smem_u32(&bars->ready[st]), (s / kSegStages) & 1, abort_flag);
        if (!ok) { ssd_report(status, kErrSegState, 4 * s + 1); break; }
        tc_fence_after();
        const uint32_t sb = base + st * kSegStageBytes;
        const uint64_t dBt0 = umma_desc_sw128(sb, kBCBox, 1024);
        for (int q = 0; q < lanes; ++q) {
          const uint64_t dX0 = umma_desc_sw128(sb + kBCBytes + q * kXBytes, kXBytes, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(tZ + 64 * q, dBt0 + static_cast<uint64_t>((kk * 2048) >> 4), dX0 + static_cast<uint64_t>((kk * 2048) >> 4),
                    id_z, (s > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&bars->empty[st]));
      }
      if (ok) umma_commit(smem_u32(&bars->done));
    }
    __syncwarp();
  } else if ((warp >> 2) < lanes) {
    const int q = warp >> 2, wq = warp & 3, h = h_first + q;
    const int i = wq * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(wq * 32) << 16;
    const float a_log2 = A[h] * kLog2e;
    float after = 0.f;   // log2 decay from the end of the step in hand to the end of the segment
    bool ok = true;
    for (int s = 0; s < nsteps && ok; ++s) {
      const int st = s % kSegStages;
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->full[st]), (s / kSegStages) & 1, abort_flag));
      if (!ok) { ssd_report(status, kErrSegState, 4 * s + 2); break; }
      unsigned char *pX = smem + st * kSegStageBytes + kBCBytes + q * kXBytes;
      const float *dtt = reinterpret_cast<const float *>(smem + st * kSegStageBytes + kBCBytes + 2 * kXBytes + q * kDtBytes);
      // every warp scans the 128 dt values of the step itself (lane l: rows 4l..4l+3), then picks its own row's
      float dt4[4], cum4[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        dt4[e] = dt_by_tma ? dtt[(4 * lane + e) * 4 + (h & 3)]
                           : dt[(row0 + static_cast<size_t>(nsteps - 1 - s) * kQ + 4 * lane + e) * H + h];
      cum4[0] = dt4[0] * a_log2;
#pragma unroll
      for (int e = 1; e < 4; ++e) cum4[e] = cum4[e - 1] + dt4[e] * a_log2;
      float incl = cum4[3];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      const float excl = incl - cum4[3];
      const float step_total = __shfl_sync(0xffffffffu, incl, 31);
      const int src = 8 * wq + (lane >> 2), comp = lane & 3;
      float cum_i = 0.f, dt_i = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float cv = __shfl_sync(0xffffffffu, cum4[e] + excl, src), dv = __shfl_sync(0xffffffffu, dt4[e], src);
        if (comp == e) { cum_i = cv; dt_i = dv; }
      }
      const float wi = ex2((step_total - cum_i) + after) * dt_i;
      after += step_total;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        uint4 *p = reinterpret_cast<uint4 *>(pX + sw128(i, cc));
        const uint4 w = *p;
        const float2 f0 = unpack2<DT>(w.x), f1 = unpack2<DT>(w.y), f2 = unpack2<DT>(w.z), f3 = unpack2<DT>(w.w);
        *p = make_uint4(pack2<DT>(f0.x * wi, f0.y * wi), pack2<DT>(f1.x * wi, f1.y * wi),
                        pack2<DT>(f2.x * wi, f2.y * wi), pack2<DT>(f3.x * wi, f3.y * wi));
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&bars->ready[st]));
    }
    if (ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->done), 0, abort_flag));
      if (!ok) ssd_report(status, kErrSegState, -1);
    }
    if (ok) {
      tc_fence_after();
      uint32_t zv[kP];
      tmem_ld32p(tZ + 64 * q + lane_addr, zv);
      tmem_ld32p(tZ + 64 * q + lane_addr + 32, zv + 32);
      tmem_wait_ld();
      const size_t slot = (static_cast<size_t>(b) * H + h) * nsm1 + seg;
      float4 *dst = reinterpret_cast<float4 *>(seg_states + slot * kStateFloats + static_cast<size_t>(i) * kP);
#pragma unroll
      for (int k = 0; k < kP / 4; ++k)
        dst[k] = make_float4(__uint_as_float(zv[4 * k]), __uint_as_float(zv[4 * k + 1]), __uint_as_float(zv[4 * k + 2]),
                             __uint_as_float(zv[4 * k + 3]));
      if (i == 0) seg_totals[slot] = after;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tZ, 128);
  }
}

// How a problem is cut: heads per CTA (2 when the heads of a pair share B and C), segments per sequence.
struct SsdPlan {
  int lanes, nseg, steps_per_seg;
};

constexpr long long kSsdMaxCtas = 512;   // a cut never makes more CTAs than this (it bounds the workspace)

// Largest number of segments a plan may use for this problem, whatever the device.
int ssd_max_segments(int B, int L, int H, int G) {
  const int lanes = ((H / G) % 2 == 0) ? 2 : 1;
  const long long chains = (long long)B * (H / lanes);
  const long long k = kSsdMaxCtas / chains;
  const int nsteps = L / kQ;
  return static_cast<int>(k < 1 ? 1 : (k > nsteps ? nsteps : k));
}

SsdPlan ssd_plan(int B, int L, int H, int G, int sms) {
  SsdPlan p;
  p.lanes = ((H / G) % 2 == 0) ? 2 : 1;
  const int nsteps = L / kQ;
  const long long chains = (long long)B * (H / p.lanes);
  // Cost of a cut into k segments, in steps of the fused kernel: waves * (steps per segment + one step of fixed
  // cost), plus for k > 1 the pass that prepares the segment states (about 0.4 of a fused step per row block)
  // and two more launches.
  int best = 1;
  double best_cost = 0.0;
  for (int k = 1; k <= ssd_max_segments(B, L, H, G); ++k) {
    const int sps = (nsteps + k - 1) / k;
    if (k > 1 && ((k - 1) * sps >= nsteps || sps < 2)) continue;   // every segment but the last must be full and non-empty
    const long long ctas = chains * k;
    const double waves = static_cast<double>((ctas + sms - 1) / sms);
    double cost = waves * (sps + 1.0);
    if (k > 1) {
      const long long ctas_a = chains * (k - 1);
      cost += static_cast<double>((ctas_a + sms - 1) / sms) * (0.25 * sps + 1.0) + 1.0;
    }
    if (k == 1 || cost < best_cost * 0.97) {
      best = k;
      best_cost = cost;
    }
  }
  p.nseg = best;
  p.steps_per_seg = (nsteps + best - 1) / best;
  return p;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <int DT>
int launch_ssd(const void *x, const float *dt, const float *A, const void *Bm, const void *Cm, void *y, int B, int L,
               int H, int G, int dtype, const SsdPlan &plan, unsigned char *workspace, cudaStream_t st) {
  int *status = reinterpret_cast<int *>(workspace);
  CUtensorMap tx, tb, tc, ty, tdt;
  int rc;
  if ((rc = tma_map_2d_sw128(&tx, x, (long long)B * L, (long long)H * kP, dtype, kQ, "ssd_chunk_scan")) != NB200_OK) return rc;
  if ((rc = tma_map_2d_sw128(&tb, Bm, (long long)B * L, (long long)G * kN, dtype, kQ, "ssd_chunk_scan")) != NB200_OK) return rc;
  if ((rc = tma_map_2d_sw128(&tc, Cm, (long long)B * L, (long long)G * kN, dtype, kQ, "ssd_chunk_scan")) != NB200_OK) return rc;
  if ((rc = tma_map_2d_sw128(&ty, y, (long long)B * L, (long long)H * kP, dtype, kQ, "ssd_chunk_scan")) != NB200_OK) return rc;
  // dt through the copy engine needs rows of H floats to be a multiple of 16 bytes and a 16-byte aligned base
  const int dt_by_tma = (H % 4 == 0 && aligned16(dt)) ? 1 : 0;
  if (dt_by_tma) {
    if ((rc = tma_map_2d_f32(&tdt, dt, (long long)B * L, H, 4, kQ, "ssd_chunk_scan")) != NB200_OK) return rc;
  } else {
    tdt = tx;  // never used by the kernels
  }
  float *seg_totals = nullptr, *seg_states = nullptr;
  if (plan.nseg > 1) {
    const size_t slots = (size_t)B * H * (plan.nseg - 1);
    seg_totals = reinterpret_cast<float *>(workspace + 256);
    seg_states = reinterpret_cast<float *>(workspace + 256 + align_up(slots * sizeof(float), 256));
    NB200_CHECK_CUDA(cudaFuncSetAttribute(ssd_segment_state_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSegSmem));
    NB200_CHECK_CUDA(cudaFuncSetAttribute(ssd_segment_state_kernel<DT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
    ssd_segment_state_kernel<DT><<<dim3(B * (H / plan.lanes) * (plan.nseg - 1)), dim3(kSegThreads), kSegSmem, st>>>(
        tx, tb, tdt, dt_by_tma, dt, A, L, H, G, plan.lanes, plan.nseg, plan.steps_per_seg, seg_states, seg_totals, status);
    NB200_CHECK_CUDA(cudaGetLastError());
  }
  NB200_CHECK_CUDA(cudaFuncSetAttribute(ssd_fused_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSsdSmem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(B * (H / plan.lanes) * plan.nseg);
  cfg.blockDim = dim3(kSsdThreads);
  cfg.dynamicSmemBytes = kSsdSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = plan.nseg > 1 ? 1 : 0;   // behind the segment-state kernel only
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  NB200_CHECK_CUDA(cudaLaunchKernelEx(&cfg, ssd_fused_kernel<DT>, tx, tb, tc, ty, tdt, dt_by_tma, dt, A, L, H, G, plan.lanes,
                                      plan.nseg, plan.steps_per_seg, static_cast<const float *>(seg_states),
                                      static_cast<const float *>(seg_totals), status));
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

bool ssd_shape_ok(int B, int L, int H, int P, int N, int G, int chunk) {
  return B > 0 && L > 0 && H > 0 && G > 0 && P == kP && N == kN && H % G == 0 &&
         (chunk == 64 || chunk == 128 || chunk == 256) && L % kQ == 0 && L % chunk == 0;
}

int current_sms() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return 0;
  return sms;
}

// NB200_SSD_SEGMENTS=k forces the number of segments (tests use it to reach the segmented path on small problems)
int forced_segments() {
  const char *e = getenv("NB200_SSD_SEGMENTS");
  return e ? atoi(e) : 0;
}

SsdPlan ssd_plan_for(int B, int L, int H, int G) {
  int sms = current_sms();
  if (sms <= 0) sms = 148;   // no device visible (sizing a workspace on a build host): plan for a B200
  SsdPlan p = ssd_plan(B, L, H, G, sms);
  const int f = forced_segments();
  const int nsteps = L / kQ;
  if (f > 0) {
    const int cap = ssd_max_segments(B, L, H, G);
    int k = f > cap ? cap : f;
    while (k > 1 && (k - 1) * ((nsteps + k - 1) / k) >= nsteps) --k;
    p.nseg = k;
    p.steps_per_seg = (nsteps + k - 1) / k;
  }
  return p;
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_ssd_workspace_bytes(int B, int L, int H, int P, int N, int G, int chunk) {
  if (!ssd_shape_ok(B, L, H, P, N, G, chunk)) return 0;
  // status words; and, when the sequence is cut into segments, per (batch, head, segment but the last) the total
  // decay and the fp32 state.  Sized for the largest cut the planner may choose, so that it does not depend on the
  // device the call later runs on.
  const int max_seg = ssd_max_segments(B, L, H, G);
  const size_t slots = (size_t)B * H * (max_seg > 1 ? max_seg - 1 : 0);
  return 256 + align_up(slots * sizeof(float), 256) + slots * kStateFloats * sizeof(float);
}

extern "C" int nb200_ssd_launches(int B, int L, int H, int P, int N, int G, int chunk) {
  if (!ssd_shape_ok(B, L, H, P, N, G, chunk)) return 0;
  return ssd_plan_for(B, L, H, G).nseg > 1 ? 2 : 1;
}

extern "C" int nb200_ssd_chunk_scan_fwd(const void *x, const float *dt, const float *A, const void *Bm,
                                        const void *Cm, void *y, void *workspace, int B, int L, int H, int P,
                                        int N, int G, int chunk, int dtype, void *stream) {
  NB200_REQUIRE(x && dt && A && Bm && Cm && y && workspace, NB200_ERR_BAD_ARG, "ssd_chunk_scan: null pointer");
  NB200_REQUIRE(B > 0 && L > 0 && H > 0 && G > 0, NB200_ERR_BAD_ARG, "ssd_chunk_scan: non-positive extent");
  NB200_REQUIRE(ssd_shape_ok(B, L, H, P, N, G, chunk), NB200_ERR_UNSUPPORTED,
                "ssd_chunk_scan: need P == 64, N == 128, H %% G == 0, chunk in {64,128,256}, L a multiple of 128 and of chunk");
  NB200_REQUIRE(aligned16(x) && aligned16(Bm) && aligned16(Cm) && aligned16(y) && aligned16(workspace),
                NB200_ERR_BAD_ARG, "ssd_chunk_scan: tensors and workspace must be 16-byte aligned");
  NB200_REQUIRE((long long)B * L < (1ll << 31) && (long long)B * H * 64 < (1ll << 31), NB200_ERR_UNSUPPORTED,
                "ssd_chunk_scan: problem too large");
  auto st = static_cast<cudaStream_t>(stream);
  const SsdPlan plan = ssd_plan_for(B, L, H, G);
  NB200_CHECK_CUDA(cudaMemsetAsync(workspace, 0, NB200_STATUS_WORDS * sizeof(int), st));
  auto *ws = static_cast<unsigned char *>(workspace);
  if (dtype == NB200_BF16) return launch_ssd<NB200_BF16>(x, dt, A, Bm, Cm, y, B, L, H, G, dtype, plan, ws, st);
  if (dtype == NB200_F16) return launch_ssd<NB200_F16>(x, dt, A, Bm, Cm, y, B, L, H, G, dtype, plan, ws, st);
  return fail(NB200_ERR_UNSUPPORTED, "ssd_chunk_scan: dtype %d (f16 and bf16 only)", dtype);
}
