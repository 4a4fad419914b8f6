// Mamba-2 SSD scan forward, fused into one kernel with the state kept on chip.
//
//   S <- exp(dt*A) S + dt * x (outer) B ;   y = S . C        (S is P x N per (batch, head))
//
// One CTA owns one (batch, head) and walks the sequence in steps of 128 rows; the fp32 state
// S (N x P = 128 x 64) never leaves tensor memory, x is read once and y written once.  With
// cum_i = sum_{s<=i} dt_s*A inside a step (kept in the log2 domain) a step is four tensor-core
// products and three element-wise passes:
//
//   G  = C . B^T                             both operands TMA tiles in shared memory      (128x128x128)
//   Y  = C . S_in, then row i scaled by      B: S_in rounded to 16 bit in shared memory; the scaling is
//        e^cum_i in TMEM                     an element-wise pass over the 64 columns      (128x64x128)
//   S  = e^cum_last S + B^T . (w x)          w_j = e^(cum_last - cum_j) dt_j; both operands MN-major
//                                            shared-memory tiles, accumulator = the state  (128x64x128)
//   Y += (G o decay o mask) . x              decay_ij = e^(cum_i - cum_j) dt_j for j <= i; A is G
//                                            overwritten in place as 16-bit in TMEM        (128x64x128)
//
//   warps 0-3   thread i = row i of the step = TMEM lane i: the scaled copies of x and S, the
//               decay/mask pass over G (an exponential per element only in the 32-column chunk on
//               the diagonal; chunks left of it take one factor per row and one per column), and
//               the epilogue (Y -> 16 bit -> staging buffer)
//   warp 6      prefix sum of dt*A over the 128 rows of a step and everything derived from it alone
//               (cum_j, dt_j, cum_j - log2 dt_j, the column factors), written to a double-buffered
//               table in shared memory one to two steps ahead of the element-wise warps, which
//               used to spend a quarter of their step on it
//   warp 4      TMA producer: the C, B and x tiles of the next step, each issued as soon as the
//               product that last read its buffer has retired, and the TMA store of the finished
//               Y tile (staged by the element-wise warps in the buffer x occupied).  The two 16 KB
//               buffers for x and for the state copy / w*x swap roles every step, so that x(s+1)
//               is loaded right after the state update of step s instead of after the Y store
//   warp 5      MMA issuer, operand descriptors built once
//
// All exponents are <= 0 (A < 0), so nothing overflows.  TMEM: columns 0-127 hold G, then the masked
// product (overwriting it in place), 128-191 Y, 192-255 the state; two CTAs
// fit per SM.  Every wait is bounded and reports through the status words.
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
constexpr int kSsdThreads = 224;
constexpr int kBCBytes = kQ * kN * 2;      // 32 KB: two 64-column boxes of 16 KB
constexpr int kBCBox = kBCBytes / 2;
constexpr int kXBytes = kQ * kP * 2;       // 16 KB: one box
constexpr int kTileBytes = 2 * kBCBytes + kXBytes;
constexpr int kDtBytes = kQ * 4 * 4;      // 128 rows x 4 heads of dt (fp32): the 16-byte minimum of a TMA box row
constexpr int kPfFloats = 4 * kQ;        // one prefix table: cum[128] | dt[128] | lb[128] | cf[128]
constexpr int kPfBytes = kPfFloats * 4;
constexpr int kSsdSmem = 2 * kBCBytes + 2 * kXBytes + 2 * kPfBytes + 2 * kDtBytes + 256 /*barriers*/;
constexpr int kSsdTmemCols = 256;
constexpr float kLog2e = 1.4426950408889634f;

enum : int { kErrSsdProducer = 11, kErrSsdMma = 12, kErrSsdCompute = 13, kErrSsdPrefix = 14, kErrSsdAlign = 15 };

struct SsdBarriers {
  uint64_t c_full, b_full, x_full, z_done, y_staged, y_free, e1a, inter_done, e1b, g_ready, m_ready, y_ready, dt_full[2],
      pf_full[2], pf_free[2];
  uint32_t tmem_base;
  int abort_flag;
  int skip;
};

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

template <int DT>
__global__ void __launch_bounds__(kSsdThreads, 2)
ssd_fused_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_b,
                 const __grid_constant__ CUtensorMap tm_c, const __grid_constant__ CUtensorMap tm_y,
                 const __grid_constant__ CUtensorMap tm_dt, int dt_by_tma, const float *__restrict__ dt, const float *__restrict__ A,
                 uint16_t *__restrict__ y, int L, int H, int G, int *status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t base = smem_u32(smem);
  if ((base & 1023u) != 0) {
    if (threadIdx.x == 0) ssd_report(status, kErrSsdAlign, static_cast<int>(base));
    return;
  }
  // Two 16 KB buffers U0, U1 change roles every step: in step s, U[s&1] holds x(s) and later the finished Y(s),
  // U[(s+1)&1] holds the 16-bit copy of the incoming state, then w*x(s), then (loaded ahead) x(s+1).
  const uint32_t sB = base, sC = base + kBCBytes, sU = base + 2 * kBCBytes;
  unsigned char *pU = smem + 2 * kBCBytes;
  float *pf_all = reinterpret_cast<float *>(smem + 2 * kBCBytes + 2 * kXBytes);  // [2 steps][cum | dt | lb | cf][128]
  const float *dt_tile = reinterpret_cast<const float *>(smem + 2 * kBCBytes + 2 * kXBytes + 2 * kPfBytes);  // [2][128][4]
  const uint32_t sDt = base + 2 * kBCBytes + 2 * kXBytes + 2 * kPfBytes;
  SsdBarriers *bars = reinterpret_cast<SsdBarriers *>(smem + 2 * kBCBytes + 2 * kXBytes + 2 * kPfBytes + 2 * kDtBytes);
  volatile int *abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x % H, b = blockIdx.x / H;
  const int g = h / (H / G);
  const int nsteps = L / kQ;

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    bars->skip = (status != nullptr && *reinterpret_cast<volatile int *>(status) != 0) ? 1 : 0;
    mbar_init(smem_u32(&bars->c_full), 1);
    mbar_init(smem_u32(&bars->b_full), 1);
    mbar_init(smem_u32(&bars->x_full), 1);
    mbar_init(smem_u32(&bars->z_done), 1);
    mbar_init(smem_u32(&bars->y_staged), 128);
    mbar_init(smem_u32(&bars->y_free), 1);
    mbar_init(smem_u32(&bars->e1a), 128);
    mbar_init(smem_u32(&bars->inter_done), 1);
    mbar_init(smem_u32(&bars->e1b), 128);
    mbar_init(smem_u32(&bars->g_ready), 1);
    mbar_init(smem_u32(&bars->m_ready), 128);
    mbar_init(smem_u32(&bars->y_ready), 1);
    mbar_init(smem_u32(&bars->dt_full[0]), 1);
    mbar_init(smem_u32(&bars->dt_full[1]), 1);
    mbar_init(smem_u32(&bars->pf_full[0]), 1);
    mbar_init(smem_u32(&bars->pf_full[1]), 1);
    mbar_init(smem_u32(&bars->pf_free[0]), 128);
    mbar_init(smem_u32(&bars->pf_free[1]), 128);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (bars->skip) return;

  if (warp == 5) {
    tmem_alloc(smem_u32(&bars->tmem_base), kSsdTmemCols);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
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
  const uint32_t tR = tmem, tY = tmem + 128, tS = tmem + 192;

  const uint32_t b_c_full = smem_u32(&bars->c_full), b_b_full = smem_u32(&bars->b_full),
                 b_x_full = smem_u32(&bars->x_full), b_z_done = smem_u32(&bars->z_done),
                 b_y_staged = smem_u32(&bars->y_staged), b_y_free = smem_u32(&bars->y_free), b_e1a = smem_u32(&bars->e1a), b_inter_done = smem_u32(&bars->inter_done),
                 b_e1b = smem_u32(&bars->e1b), b_g_ready = smem_u32(&bars->g_ready),
                 b_m_ready = smem_u32(&bars->m_ready), b_y_ready = smem_u32(&bars->y_ready),
                 b_dt_full = smem_u32(&bars->dt_full[0]),  // buffer p is at + 8 * p
                 b_pf_full = smem_u32(&bars->pf_full[0]), b_pf_free = smem_u32(&bars->pf_free[0]);

  if (warp == 4) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      bool ok = true;
      int issued_c = 0, issued_b = 0, issued_x = 0, issued_dt = 0;
      auto load_c = [&](int s) {
        const int row = b * L + s * kQ;
        mbar_arrive_expect_tx(b_c_full, kBCBytes);
        tma_load_2d(sC, &tm_c, g * kN, row, b_c_full);
        tma_load_2d(sC + kBCBox, &tm_c, g * kN + 64, row, b_c_full);
        ++issued_c;
      };
      auto load_b = [&](int s) {
        const int row = b * L + s * kQ;
        mbar_arrive_expect_tx(b_b_full, kBCBytes);
        tma_load_2d(sB, &tm_b, g * kN, row, b_b_full);
        tma_load_2d(sB + kBCBox, &tm_b, g * kN + 64, row, b_b_full);
        ++issued_b;
      };
      auto load_x = [&](int s) {
        mbar_arrive_expect_tx(b_x_full, kXBytes);
        tma_load_2d(sU + (s & 1) * kXBytes, &tm_x, h * kP, b * L + s * kQ, b_x_full);
        ++issued_x;
      };
      // dt of one step for the four heads around h (a TMA box row cannot be narrower than 16 bytes): a strided
      // gather that the copy engine does well and 128 threads doing 4-byte loads 256 bytes apart do badly
      auto load_dt = [&](int s) {
        if (!dt_by_tma) return;
        mbar_arrive_expect_tx(b_dt_full + 8 * (s & 1), kDtBytes);
        tma_load_2d(sDt + (s & 1) * kDtBytes, &tm_dt, h & ~3, b * L + s * kQ, b_dt_full + 8 * (s & 1));
        ++issued_dt;
      };
      load_dt(0);
      if (nsteps > 1) load_dt(1);
      load_c(0);
      load_b(0);
      load_x(0);
      for (int s = 0; s < nsteps; ++s) {
        const uint32_t ph = s & 1;
        const bool more = s + 1 < nsteps;
        // the buffers of step s become free in this order: C (after G and C.S_in); B and the buffer of w*x
        // (after the state update), which takes x(s+1) at once so that the load has most of a step to arrive
        if (more) {
          ok = mbar_wait(b_inter_done, ph, abort_flag);
          if (!ok) { ssd_report(status, kErrSsdProducer, 4 * s); break; }
          load_c(s + 1);
          if (s + 2 < nsteps) load_dt(s + 2);   // its buffer held dt(s), consumed before this step's first product
          ok = mbar_wait(b_z_done, ph, abort_flag);
          if (!ok) { ssd_report(status, kErrSsdProducer, 4 * s + 1); break; }
          load_b(s + 1);
          load_x(s + 1);
        }
        // the finished Y tile sits where x(s) was: store it; the next step's state copy may overwrite the
        // buffer once the store has read it
        ok = mbar_wait(b_y_staged, ph, abort_flag);
        if (!ok) { ssd_report(status, kErrSsdProducer, 4 * s + 2); break; }
        tma_store_2d(&tm_y, sU + (s & 1) * kXBytes, h * kP, b * L + s * kQ);
        tma_store_commit();
        if (more) {
          tma_store_wait_read();
          mbar_arrive(b_y_free);
        }
      }
      tma_store_wait_all();
      if (!ok) {
        for (int spin = 0; spin < 100000; ++spin) {  // let the loads in flight land before smem goes away
          const bool c_ok = issued_c == 0 || mbar_try_wait(b_c_full, (issued_c - 1) & 1);
          const bool b_ok = issued_b == 0 || mbar_try_wait(b_b_full, (issued_b - 1) & 1);
          const bool x_ok = issued_x == 0 || mbar_try_wait(b_x_full, (issued_x - 1) & 1);
          bool d_ok = true;
          for (int n = 0; n < 2; ++n) {  // the last two dt loads
            const int sd = issued_dt - 1 - n;
            if (sd >= 0) d_ok = d_ok && mbar_try_wait(b_dt_full + 8 * (sd & 1), (sd >> 1) & 1);
          }
          if (c_ok && b_ok && x_ok && d_ok) break;
          __nanosleep(100);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ================================ MMA issuer ==================================
    if (lane == 0) {
      constexpr int fmt = (DT == NB200_BF16) ? 1 : 0;
      constexpr uint32_t id_inter = umma_idesc_f16_ab(fmt, 0, 1, kQ, kP);   // A: C (K-major), B: S_in [n][p] MN-major
      constexpr uint32_t id_g = umma_idesc_f16_ab(fmt, 0, 0, kQ, kQ);       // A: C, B: B, both K-major
      constexpr uint32_t id_z = umma_idesc_f16_ab(fmt, 1, 1, kN, kP);       // A: B^T (MN-major), B: w x (MN-major)
      constexpr uint32_t id_m2 = umma_idesc_f16_ab(fmt, 0, 1, kQ, kP);      // A: TMEM, B: x (MN-major)
      uint64_t dC[8], dB[8], dBt[8], dU[2][8];
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t off = (kk >> 2) * kBCBox + (kk & 3) * 32;  // 16 elements of n per MMA inside the swizzled row
        dC[kk] = umma_desc_sw128(sC + off, 16, 1024);
        dB[kk] = umma_desc_sw128(sB + off, 16, 1024);
        // reduction over rows (time steps / state rows): 16 rows = 2 KB per MMA; 64-column blocks 16 KB apart
        dBt[kk] = umma_desc_sw128(sB + kk * 2048, kBCBox, 1024);
        dU[0][kk] = umma_desc_sw128(sU + kk * 2048, kXBytes, 1024);
        dU[1][kk] = umma_desc_sw128(sU + kXBytes + kk * 2048, kXBytes, 1024);
      }
      bool ok = true;
      for (int s = 0; s < nsteps && ok; ++s) {
        const uint32_t ph = s & 1;
        ok = mbar_wait(b_c_full, ph, abort_flag) && mbar_wait(b_b_full, ph, abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 4 * s); break; }
        tc_fence_after();
        // G = C . B^T needs nothing from the element-wise warps: issue it first
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_ss(tR, dC[kk], dB[kk], id_g, kk > 0);
        umma_commit(b_g_ready);
        ok = mbar_wait(b_e1a, ph, abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 4 * s + 1); break; }
        tc_fence_after();
        // Y = C . S_in      (S_in sits in the buffer that later holds w*x; rows are scaled by e^cum_i afterwards)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_ss(tY, dC[kk], (s & 1) ? dU[0][kk] : dU[1][kk], id_inter, kk > 0);
        umma_commit(b_inter_done);   // also: the C tile is free
        // S = (e^cum_last S) + B^T . (w x)
        ok = mbar_wait(b_e1b, ph, abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 4 * s + 2); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_ss(tS, dBt[kk], (s & 1) ? dU[0][kk] : dU[1][kk], id_z, 1u);
        umma_commit(b_z_done);
        // Y += (G o decay o mask) . x
        ok = mbar_wait(b_x_full, ph, abort_flag) && mbar_wait(b_m_ready, ph, abort_flag);
        if (!ok) { ssd_report(status, kErrSsdMma, 4 * s + 3); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) umma_ts(tY, tR + kk * 8, (s & 1) ? dU[1][kk] : dU[0][kk], id_m2, 1u);
        umma_commit(b_y_ready);
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ================================ prefix warp =================================
    // Lane l owns rows 4l..4l+3 of the step.  Per step sp it leaves in table sp & 1:
    //   cum[j]  inclusive prefix sum of dt*A*log2(e) inside the step (cum[127] is the step total, cum[31], cum[63],
    //           cum[95] are the references of column chunks 0..2)
    //   dt[j]
    //   lb[j]   cum_j - log2(dt_j)
    //   cf[j]   e^(r - cum_j) dt_j with r the cum at the last row of j's 32-column chunk: the column factor of the
    //           chunks left of the diagonal, where e^(cum_i - cum_j) dt_j = e^(cum_i - r) * cf[j] and both
    //           exponents are <= 0 for every row i below the chunk
    // It runs up to two steps ahead of the element-wise warps (a table is rewritten once all 128 rows have
    // released it), so the scan never sits on their critical path.
    const float a_log2 = A[h] * kLog2e;
    bool ok = true;
    for (int sp = 0; sp < nsteps && ok; ++sp) {
      float *tab = pf_all + (sp & 1) * kPfFloats;
      float dt4[4], cum4[4];
      if (dt_by_tma) {
        ok = __all_sync(0xffffffffu, mbar_wait(b_dt_full + 8 * (sp & 1), (sp >> 1) & 1, abort_flag));
        if (!ok) { if (lane == 0) ssd_report(status, kErrSsdPrefix, 2 * sp); break; }
        const float *tile = dt_tile + (sp & 1) * (kQ * 4) + (h & 3);
#pragma unroll
        for (int e = 0; e < 4; ++e) dt4[e] = tile[(4 * lane + e) * 4];
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          dt4[e] = dt[(static_cast<size_t>(b) * L + static_cast<size_t>(sp) * kQ + 4 * lane + e) * H + h];
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
        ok = __all_sync(0xffffffffu, mbar_wait(b_pf_free + 8 * (sp & 1), ((sp >> 1) - 1) & 1, abort_flag));
        if (!ok) { if (lane == 0) ssd_report(status, kErrSsdPrefix, 2 * sp + 1); break; }
      }
      *reinterpret_cast<float4 *>(tab + 4 * lane) = make_float4(cum4[0], cum4[1], cum4[2], cum4[3]);
      *reinterpret_cast<float4 *>(tab + kQ + 4 * lane) = make_float4(dt4[0], dt4[1], dt4[2], dt4[3]);
      *reinterpret_cast<float4 *>(tab + 2 * kQ + 4 * lane) = lbv;
      *reinterpret_cast<float4 *>(tab + 3 * kQ + 4 * lane) = cfv;
      __syncwarp();
      if (lane == 0) mbar_arrive(b_pf_full + 8 * (sp & 1));
    }
  } else {
    // ================================ element-wise warps ==========================
    const int i = warp * 32 + lane;                           // row of the step == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    {  // the state starts at zero
      uint32_t z[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) z[k] = 0u;
      tmem_st32(tS + lane_addr, z);
      tmem_st32(tS + lane_addr + 32, z);
      tmem_wait_st();
    }
    bool ok = true;
    for (int s = 0; s < nsteps && ok; ++s) {
      const uint32_t ph = s & 1;
      unsigned char *pX = pU + (s & 1) * kXBytes, *pXs = pU + ((s & 1) ^ 1) * kXBytes;
      // this step's row quantities, from the prefix warp's table
      ok = __all_sync(0xffffffffu, mbar_wait(b_pf_full + 8 * (s & 1), (s >> 1) & 1, abort_flag));
      if (!ok) { ssd_report(status, kErrSsdCompute, 8 * s + 7); break; }
      const float *tab = pf_all + (s & 1) * kPfFloats;
      const float *lb = tab + 2 * kQ, *cf = tab + 3 * kQ;
      const float cum_i = tab[i], dt_i = tab[kQ + i], total = tab[kQ - 1];
      const float ref0 = tab[31], ref1 = tab[63], ref2 = tab[95];

      // ---- E1a: S_in -> 16 bit in smem; S *= e^cum_last.  (The state is final: the previous step's
      //      y_ready, waited for in E3, was committed after its state update.) ----
      {
        uint32_t sv[kP];
        tmem_ld32p(tS + lane_addr, sv);
        tmem_ld32p(tS + lane_addr + 32, sv + 32);
        tmem_wait_ld();
        const float et = ex2(total);
        uint4 cp[8];  // the 16-bit copy, held back until its buffer is free
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          cp[cc].x = pack2<DT>(__uint_as_float(sv[8 * cc + 0]), __uint_as_float(sv[8 * cc + 1]));
          cp[cc].y = pack2<DT>(__uint_as_float(sv[8 * cc + 2]), __uint_as_float(sv[8 * cc + 3]));
          cp[cc].z = pack2<DT>(__uint_as_float(sv[8 * cc + 4]), __uint_as_float(sv[8 * cc + 5]));
          cp[cc].w = pack2<DT>(__uint_as_float(sv[8 * cc + 6]), __uint_as_float(sv[8 * cc + 7]));
        }
#pragma unroll
        for (int k = 0; k < kP; ++k) sv[k] = __float_as_uint(__uint_as_float(sv[k]) * et);
        tmem_st32(tS + lane_addr, *reinterpret_cast<uint32_t(*)[32]>(sv));
        tmem_st32(tS + lane_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
        if (s > 0) {  // the copy goes where Y(s-1) was staged: its store must have read the buffer
          ok = __all_sync(0xffffffffu, mbar_wait(b_y_free, (s - 1) & 1, abort_flag));
        }
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) *reinterpret_cast<uint4 *>(pXs + sw128(i, cc)) = cp[cc];
        tmem_wait_st();
        if (!ok) { ssd_report(status, kErrSsdCompute, 8 * s + 5); break; }
        tc_fence_before();
        fence_proxy_async_smem();   // the tensor core reads shared memory through the async proxy
        mbar_arrive(b_e1a);
      }

      // ---- E1b: w_i x_i -> smem (the buffer S_in occupied, free once the first product has retired);
      //      the scaled row is prepared in registers while that product runs ----
      {
        ok = __all_sync(0xffffffffu, mbar_wait(b_x_full, ph, abort_flag));
        if (!ok) { ssd_report(status, kErrSsdCompute, 8 * s + 4); break; }
        const float wi = ex2(total - cum_i) * dt_i;
        uint4 xs[8];
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          const uint4 w = *reinterpret_cast<const uint4 *>(pX + sw128(i, cc));
          const float2 f0 = unpack2<DT>(w.x), f1 = unpack2<DT>(w.y), f2 = unpack2<DT>(w.z), f3 = unpack2<DT>(w.w);
          xs[cc] = make_uint4(pack2<DT>(f0.x * wi, f0.y * wi), pack2<DT>(f1.x * wi, f1.y * wi),
                              pack2<DT>(f2.x * wi, f2.y * wi), pack2<DT>(f3.x * wi, f3.y * wi));
        }
        ok = __all_sync(0xffffffffu, mbar_wait(b_inter_done, ph, abort_flag));
        if (!ok) { ssd_report(status, kErrSsdCompute, 8 * s + 1); break; }
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) *reinterpret_cast<uint4 *>(pXs + sw128(i, cc)) = xs[cc];
        fence_proxy_async_smem();
        mbar_arrive(b_e1b);
      }

      // ---- E2: G_ij e^(cum_i - cum_j) dt_j for j <= i, else 0 -> 16 bit over G in place ----
      ok = __all_sync(0xffffffffu, mbar_wait(b_g_ready, ph, abort_flag));
      if (!ok) { ssd_report(status, kErrSsdCompute, 8 * s + 2); break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
        if (c < warp) {  // a chunk left of the diagonal: every column is visible to every row of this warp
          uint32_t gv[32];
          tmem_ld32(tR + lane_addr + c * 32, gv);
          const float rf = ex2(cum_i - (c == 0 ? ref0 : (c == 1 ? ref1 : ref2)));
          const uint64_t rf2 = f2_pack(rf, rf);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const ulonglong2 c4 = *reinterpret_cast<const ulonglong2 *>(cf + c * 32 + q * 4);
            const float2 m01 = f2_unpack(f2_mul(f2_mul(f2_pack(__uint_as_float(gv[q * 4]), __uint_as_float(gv[q * 4 + 1])), c4.x), rf2));
            const float2 m23 = f2_unpack(f2_mul(f2_mul(f2_pack(__uint_as_float(gv[q * 4 + 2]), __uint_as_float(gv[q * 4 + 3])), c4.y), rf2));
            pk[q * 2] = pack2<DT>(m01.x, m01.y);
            pk[q * 2 + 1] = pack2<DT>(m23.x, m23.y);
          }
        } else if (c == warp) {  // the diagonal chunk: exponent and mask per element
          uint32_t gv[32];
          tmem_ld32(tR + lane_addr + c * 32, gv);
          tmem_wait_ld();
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 l4 = *reinterpret_cast<const float4 *>(lb + c * 32 + q * 4);
            const float lbs[4] = {l4.x, l4.y, l4.z, l4.w};
            float m[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = c * 32 + q * 4 + e;
              const float val = __uint_as_float(gv[q * 4 + e]) * ex2(cum_i - lbs[e]);
              m[e] = (j <= i) ? val : 0.f;
            }
            pk[q * 2] = pack2<DT>(m[0], m[1]);
            pk[q * 2 + 1] = pack2<DT>(m[2], m[3]);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 16; ++k) pk[k] = 0u;
        }
        tmem_st16(tR + lane_addr + c * 16, pk);
      }
      {  // Y = C . S_in has retired (inter_done was waited for above): scale row i by e^cum_i
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
      mbar_arrive(b_m_ready);
      mbar_arrive(b_pf_free + 8 * (s & 1));   // nothing of step s reads the table any more

      // ---- E3: Y -> storage dtype -> the buffer x occupied (x is dead once Y is complete);
      //      the producer warp stores the tile with one TMA copy ----
      ok = __all_sync(0xffffffffu, mbar_wait(b_y_ready, ph, abort_flag));
      if (!ok) { ssd_report(status, kErrSsdCompute, 8 * s + 3); break; }
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
        mbar_arrive(b_y_staged);
      }
      tc_fence_before();  // orders these TMEM reads before the next step's products, via the e1a arrival
    }
  }

  // ================================ tear-down =====================================
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, kSsdTmemCols);
  }
}

template <int DT>
int launch_ssd(const void *x, const float *dt, const float *A, const void *Bm, const void *Cm, void *y, int B, int L,
               int H, int G, int dtype, int *status, cudaStream_t st) {
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
    tdt = tx;  // never used by the kernel
  }
  NB200_CHECK_CUDA(cudaFuncSetAttribute(ssd_fused_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSsdSmem));
  NB200_CHECK_CUDA(cudaFuncSetAttribute(ssd_fused_kernel<DT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
  ssd_fused_kernel<DT><<<dim3(B * H), dim3(kSsdThreads), kSsdSmem, st>>>(tx, tb, tc, ty, tdt, dt_by_tma, dt, A, static_cast<uint16_t *>(y),
                                                                         L, H, G, status);
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

bool ssd_shape_ok(int B, int L, int H, int P, int N, int G, int chunk) {
  return B > 0 && L > 0 && H > 0 && G > 0 && P == kP && N == kN && H % G == 0 &&
         (chunk == 64 || chunk == 128 || chunk == 256) && L % kQ == 0 && L % chunk == 0;
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_ssd_workspace_bytes(int B, int L, int H, int P, int N, int G, int chunk) {
  if (!ssd_shape_ok(B, L, H, P, N, G, chunk)) return 0;
  return NB200_STATUS_WORDS * sizeof(int);  // the state stays on chip; only the status words live here
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
  NB200_REQUIRE((long long)B * L < (1ll << 31) && (long long)B * H < (1ll << 31), NB200_ERR_UNSUPPORTED,
                "ssd_chunk_scan: problem too large");
  auto st = static_cast<cudaStream_t>(stream);
  int *status = static_cast<int *>(workspace);
  NB200_CHECK_CUDA(cudaMemsetAsync(status, 0, NB200_STATUS_WORDS * sizeof(int), st));
  if (dtype == NB200_BF16) return launch_ssd<NB200_BF16>(x, dt, A, Bm, Cm, y, B, L, H, G, dtype, status, st);
  if (dtype == NB200_F16) return launch_ssd<NB200_F16>(x, dt, A, Bm, Cm, y, B, L, H, G, dtype, status, st);
  return fail(NB200_ERR_UNSUPPORTED, "ssd_chunk_scan: dtype %d (f16 and bf16 only)", dtype);
}
