// Fused attention forward on Blackwell tensor cores: persistent CTAs, KV blocks of 128 rows, two softmax
// warpgroups taking alternate blocks (f16 / bf16 storage, D = 128).
//
// A CTA (one per SM) works through tiles of 128 query rows, taken one at a time from a global counter in launch
// order (heads in groups, longest causal tiles first), so that all CTAs end within one short tile of each other.
// The KV sequence of a tile is walked in blocks
// of 128 rows; the blocks of all the CTA's tiles form one stream, numbered g = 0, 1, 2, ...:
//
//   S(g) = Q K(g)^T      8 x tcgen05.mma 128x128x16, both operands in shared memory, into TMEM buffer g % 3
//   softmax(g)           warpgroup g & 1 (thread = row = TMEM lane): scores to registers, row maximum, p = 2^(s - m),
//                        P(g) as packed 16-bit over the first 64 columns of the same TMEM buffer
//   O += P(g) V(g)       8 x tcgen05.mma 128x128x16 with P read from TMEM, O in TMEM columns 384..511
//
// The score products run up to three blocks ahead of the PV products (three S/P buffers): S(g+3) may start as
// soon as PV(g) has retired, so between the end of QK(g) and the start of PV(g) the tensor pipe has other products
// to do for about as long as the softmax of one block takes, and the two warpgroups together deliver a block per
// two products.  Nothing of one block waits for anything but its own inputs, and the stream does not stop at tile
// boundaries: while the last blocks of a tile are in the softmax, the score products of the next tile are already
// running, and a fourth warpgroup writes the finished tile out.  Each product has an issuing thread of its own:
// a tcgen05.mma costs its issuing thread 45-60 cycles and a commit or a barrier test 50-150, so a single thread
// issuing both could not keep the pipe fed (measured: ~2000 cycles per block for sixteen 64-cycle products).
//
// Against blocks of 64 KV rows with two CTAs per SM, a 128x128x16 score product costs 64 cycles where two 128x64x16
// cost 96: they are bound by operand reads from shared memory (128 B/clk), and Q is read half as often per FLOP.
//
// The running maximum of a row passes between the two warpgroups through shared memory (block g needs the value
// block g-1 decided on); each keeps a partial row sum under the maximum it last used, and the epilogue combines
// the two.  O is rescaled only when a maximum grows by more than 2^8.
//
//   warps 0-3 / 4-7  softmax of even / odd blocks           warps 8-11   epilogue (O / l -> global)
//   warp 12, 15      TMA producers: Q and K; V (warp 15 also allocates the 512 TMEM columns)
//   warp 13, 14      issuers of the score products and of the PV products (one lane each)
//
// Registers are moved from the producer / issuer / epilogue warps to the softmax warps with setmaxnreg (a softmax
// thread holds the 128 scores of its row).  One CTA per SM: 192 KB of shared memory (two buffers of 32 KB each for
// Q, K and V), all 512 TMEM columns.  No multicast anywhere.
//
// Every wait is bounded; on expiry the CTA records a code in the status words and unwinds.
#include <cuda.h>

#include <atomic>

#include "nb200_common.cuh"
#include "sm100_primitives.cuh"

namespace nb200 {
namespace {

using namespace sm100;

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kD = 128;
constexpr int kHeadGroup = 16;
constexpr int kThreads = 512;
constexpr int kTileBytes = 128 * kD * 2;        // 32 KB: two 64-column boxes of 16 KB
constexpr int kBox = kTileBytes / 2;
constexpr int kSBufs = 3;
constexpr int kTmemCols = 512;                  // S/P 0 | S/P 1 | S/P 2 | O, 128 columns each
constexpr int kTmemO = 384;
constexpr float kRescaleThreshold = 8.0f;
constexpr int kSched = 16;                      // ring of tile indices handed from the scheduling thread to the other roles

enum : int { kErrProducer = 1, kErrMma = 2, kErrSoftmax = 3, kErrEpilogue = 4 };

struct Shared {
  uint64_t q_full[2], q_empty[2], k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[kSBufs], p_full[kSBufs], pv_done[kSBufs];
  uint64_t o_full, o_free, m_ready[2], lm_ready, lm_free;
  uint64_t sched_full[kSched];
  int tile_slot[kSched];
  uint32_t tmem_base;
  int abort_flag;
  int skip;
  int pad;
  float mslot[2][128];      // running maximum decided by block g, slot g & 1
  float lm[2][128][2];      // per warpgroup: (maximum last used, partial row sum) of the finished tile
};
constexpr int kSmemBytes = 6 * kTileBytes + 1024 + static_cast<int>(sizeof(Shared));

__device__ __forceinline__ void report(int *status, int code, int detail) {
  if (status && atomicCAS(status, 0, code) == 0) {
    status[1] = static_cast<int>(blockIdx.x);
    status[2] = detail;
    status[3] = static_cast<int>(threadIdx.x);
  }
}

// Polling wait (mbarrier.test_wait never suspends the thread): the waiter continues a few cycles after the phase
// completes instead of the 200-300 a suspended thread takes to come back.  For the single issuing thread only.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_test_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      *abort_flag = 1;
      return false;
    }
  }
}

// tcgen05.mma with the shared-memory descriptors given as low word + common high word.
__device__ __forceinline__ void umma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

struct Problem {
  int Sq, Skv, n_qtiles, n_units, group, causal, total;
};
struct Tile {
  int bh, qt, nblk;
};
// Launch order: heads in groups, tile-major inside a group, longest causal tiles first.
__device__ __forceinline__ Tile tile_of(const Problem &p, int i) {
  const int per_group = p.group * p.n_qtiles;
  const int grp = i / per_group, rem = i % per_group;
  const int heads_here = min(p.group, p.n_units - grp * p.group);
  const int qi = rem / heads_here;
  Tile t;
  t.bh = grp * p.group + rem % heads_here;
  t.qt = p.causal ? (p.n_qtiles - 1 - qi) : qi;
  const int last_col = p.causal ? min(p.Skv - 1, t.qt * kBM + (p.Skv - p.Sq) + kBM - 1) : p.Skv - 1;
  t.nblk = last_col / kBN + 1;
  return t;
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, uint16_t *__restrict__ out, const Problem prob,
                   float scale_log2, unsigned int *tile_counter, int *status
                   ) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char *smem = smem_raw + (base - raw);
  const uint32_t sQ = base;                                   // buffer n & 1 of tile n
  const uint32_t sK = base + 2 * kTileBytes;                  // stage g & 1
  const uint32_t sV = base + 4 * kTileBytes;
  Shared *sh = reinterpret_cast<Shared *>(smem + 6 * kTileBytes);
  volatile int *abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;

  if (threadIdx.x == 0) {
    sh->abort_flag = 0;
    sh->skip = (status != nullptr && *reinterpret_cast<volatile int *>(status) != 0) ? 1 : 0;
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->q_full[b]), 1);
      mbar_init(smem_u32(&sh->q_empty[b]), 1);
      mbar_init(smem_u32(&sh->k_full[b]), 1);
      mbar_init(smem_u32(&sh->k_empty[b]), 1);
      mbar_init(smem_u32(&sh->v_full[b]), 1);
      mbar_init(smem_u32(&sh->v_empty[b]), 1);
      mbar_init(smem_u32(&sh->m_ready[b]), 128);
    }
    for (int b = 0; b < kSBufs; ++b) {
      mbar_init(smem_u32(&sh->s_full[b]), 1);
      mbar_init(smem_u32(&sh->p_full[b]), 128);
      mbar_init(smem_u32(&sh->pv_done[b]), 1);
    }
    mbar_init(smem_u32(&sh->o_full), 1);
    mbar_init(smem_u32(&sh->o_free), 128);
    mbar_init(smem_u32(&sh->lm_ready), 256);
    mbar_init(smem_u32(&sh->lm_free), 128);
    for (int b = 0; b < kSched; ++b) mbar_init(smem_u32(&sh->sched_full[b]), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (sh->skip) return;

  if (warp == 15) {
    tmem_alloc(smem_u32(&sh->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 12 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;

  const uint32_t b_q_full = smem_u32(&sh->q_full[0]), b_q_empty = smem_u32(&sh->q_empty[0]),
                 b_k_full = smem_u32(&sh->k_full[0]), b_k_empty = smem_u32(&sh->k_empty[0]),
                 b_v_full = smem_u32(&sh->v_full[0]), b_v_empty = smem_u32(&sh->v_empty[0]),
                 b_s_full = smem_u32(&sh->s_full[0]), b_p_full = smem_u32(&sh->p_full[0]),
                 b_pv_done = smem_u32(&sh->pv_done[0]), b_o_full = smem_u32(&sh->o_full),
                 b_o_free = smem_u32(&sh->o_free), b_m_ready = smem_u32(&sh->m_ready[0]),
                 b_lm_ready = smem_u32(&sh->lm_ready), b_lm_free = smem_u32(&sh->lm_free),
                 b_sched = smem_u32(&sh->sched_full[0]);  // element i at + 8 * i

  // Tiles are dealt dynamically: the K producer takes the CTA's n-th tile from a global counter (the first one is
  // the CTA's own index, so nothing waits at the start) and posts it in a ring; every other role reads it there.
  // With the longest tiles first this keeps the CTAs within one short tile of each other at the end, where a fixed
  // round-robin deal left 4 % (256 heads) to 15 % (32 heads) of imbalance.  The roles are never more than 7 tiles
  // apart (2 Q buffers, 3 score buffers, one O), so 16 slots need no "empty" barrier.  A value >= total ends the list;
  // -1 is an expired wait.
  auto tile_at = [&](int n) -> int {
    if (!mbar_wait(b_sched + 8 * (n % kSched), (n / kSched) & 1, abort_flag)) return -1;
    return *reinterpret_cast<volatile int *>(&sh->tile_slot[n % kSched]);
  };

  if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    if (warp == 12 || warp == 15) {
      // ================================ TMA producers ================================
      // warp 12: Q of every tile and the K blocks, in the order the score products want them; warp 15: the V blocks.
      if (lane == 0) {
        const bool is_k = warp == 12;
        const CUtensorMap *tm = is_k ? &tm_k : &tm_v;
        const uint32_t s_dst = is_k ? sK : sV, b_full = is_k ? b_k_full : b_v_full, b_empty = is_k ? b_k_empty : b_v_empty;
        bool ok = true;
        int g = 0, issued = 0, q_issued = 0;
        for (int n = 0; ok; ++n) {
          int i;
          if (is_k) {   // this thread is the scheduler
            i = n == 0 ? static_cast<int>(blockIdx.x) : G + static_cast<int>(atomicAdd(tile_counter, 1u));
            sh->tile_slot[n % kSched] = i;
            mbar_arrive(b_sched + 8 * (n % kSched));
          } else {
            i = tile_at(n);
            if (i < 0) { report(status, kErrProducer, -1000 - n); ok = false; break; }
          }
          if (i >= prob.total) break;
          const Tile t = tile_of(prob, i);
          if (is_k) {
            ok = mbar_wait(b_q_empty + 8 * (n & 1), ((n >> 1) & 1) ^ 1, abort_flag);
            if (!ok) { report(status, kErrProducer, -1 - n); break; }
            mbar_arrive_expect_tx(b_q_full + 8 * (n & 1), kTileBytes);
            tma_load_3d(sQ + (n & 1) * kTileBytes, &tm_q, 0, t.qt * kBM, t.bh, b_q_full + 8 * (n & 1));
            tma_load_3d(sQ + (n & 1) * kTileBytes + kBox, &tm_q, 64, t.qt * kBM, t.bh, b_q_full + 8 * (n & 1));
            ++q_issued;
          }
          for (int j = 0; j < t.nblk && ok; ++j, ++g) {
            const int b = g & 1;
            ok = mbar_wait(b_empty + 8 * b, ((g >> 1) & 1) ^ 1, abort_flag);
            if (!ok) { report(status, kErrProducer, 2 * g + (is_k ? 0 : 1)); break; }
            mbar_arrive_expect_tx(b_full + 8 * b, kTileBytes);
            tma_load_3d(s_dst + b * kTileBytes, tm, 0, j * kBN, t.bh, b_full + 8 * b);
            tma_load_3d(s_dst + b * kTileBytes + kBox, tm, 64, j * kBN, t.bh, b_full + 8 * b);
            ++issued;
          }
        }
        if (!ok) {
          // Unwinding: let the copies already in flight land before the CTA's shared memory goes away.
          for (int spin = 0; spin < 100000; ++spin) {
            bool done = true;
            for (int n = 0; n < 2; ++n) {
              const int jg = issued - 1 - n, jq = q_issued - 1 - n;
              if (jg >= 0) done = done && mbar_try_wait(b_full + 8 * (jg & 1), (jg >> 1) & 1);
              if (jq >= 0) done = done && mbar_try_wait(b_q_full + 8 * (jq & 1), (jq >> 1) & 1);
            }
            if (done) break;
            __nanosleep(100);
          }
        }
      }
      __syncwarp();
    } else if (warp == 13) {
      // ================================ score-product issuer ==================================
      // A thread of its own for each of the two products: a tcgen05.mma costs its issuing thread 45-60 cycles and a
      // commit or barrier test 50-150, so one thread for both could not feed the pipe (measured: ~2000 cycles per
      // block for 16 products).  S(g) goes into the buffer P(g-3) was read from: wait for that PV product first.
      if (lane == 0) {
        constexpr int fmt = (DT == NB200_BF16) ? 1 : 0;
        constexpr uint32_t idesc_qk = umma_idesc_f16(fmt, 0, kBM, kBN);
        // Descriptors are built once (low words; the high word is common).  K-major operands: 16 elements of the
        // reduction = 32 bytes inside the 128-byte swizzled row, the two 64-column boxes kBox apart.
        const uint32_t d_hi = static_cast<uint32_t>(umma_desc_sw128(0, 16, 1024) >> 32);
        uint32_t dq_lo[kD / 16], dk_lo[kD / 16];   // buffer / stage 1 is kStageStep further
        constexpr uint32_t kStageStep = kTileBytes >> 4;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kBox + (kk & 3) * 32;
          dq_lo[kk] = static_cast<uint32_t>(umma_desc_sw128(sQ + off, 16, 1024));
          dk_lo[kk] = static_cast<uint32_t>(umma_desc_sw128(sK + off, 16, 1024));
        }
        bool ok = true;
        int g = 0;
        for (int n = 0; ok; ++n) {
          const int i = tile_at(n);
          if (i < 0) { report(status, kErrMma, -1000 - n); break; }
          if (i >= prob.total) break;
          const int nblk = tile_of(prob, i).nblk;
          ok = mbar_wait(b_q_full + 8 * (n & 1), (n >> 1) & 1, abort_flag);
          if (!ok) { report(status, kErrMma, -1 - n); break; }
          const uint32_t q_step = (n & 1) * kStageStep;
          for (int j = 0; j < nblk && ok; ++j, ++g) {
            const int sb = g % kSBufs;
            ok = mbar_wait(b_k_full + 8 * (g & 1), (g >> 1) & 1, abort_flag);
            if (!ok) { report(status, kErrMma, 4 * g); break; }
            if (g >= kSBufs) {
              ok = mbar_wait_poll(b_pv_done + 8 * sb, ((g - kSBufs) / kSBufs) & 1, abort_flag);
              if (!ok) { report(status, kErrMma, 4 * g + 1); break; }
            }
            tc_fence_after();
            const uint32_t d_tmem = tmem + sb * 128, k_step = (g & 1) * kStageStep;
#pragma unroll
            for (int kk = 0; kk < kD / 16; ++kk) umma_ss_lo(d_tmem, dq_lo[kk] + q_step, dk_lo[kk] + k_step, d_hi, idesc_qk, kk > 0);
            umma_commit(b_s_full + 8 * sb);
            umma_commit(b_k_empty + 8 * (g & 1));
          }
          if (ok) umma_commit(b_q_empty + 8 * (n & 1));
        }
      }
      __syncwarp();
    } else if (warp == 14) {
      // ================================ PV-product issuer ==================================
      if (lane == 0) {
        constexpr int fmt = (DT == NB200_BF16) ? 1 : 0;
        constexpr uint32_t idesc_pv = umma_idesc_f16(fmt, 1, kBM, kD);
        // V is MN-major: 16 kv rows = 2 KB, the two 64-column blocks kBox apart
        const uint32_t d_hi = static_cast<uint32_t>(umma_desc_sw128(0, 16, 1024) >> 32);
        uint32_t dv_lo[kBN / 16];
        constexpr uint32_t kStageStep = kTileBytes >> 4;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk) dv_lo[kk] = static_cast<uint32_t>(umma_desc_sw128(sV + kk * 2048, kBox, 1024));
        bool ok = true;
        int g = 0;
        for (int n = 0; ok; ++n) {
          const int i = tile_at(n);
          if (i < 0) { report(status, kErrMma, -1000 - n); break; }
          if (i >= prob.total) break;
          const int nblk = tile_of(prob, i).nblk;
          for (int j = 0; j < nblk && ok; ++j, ++g) {
            const int sb = g % kSBufs;
            ok = mbar_wait(b_v_full + 8 * (g & 1), (g >> 1) & 1, abort_flag);
            if (!ok) { report(status, kErrMma, 4 * g + 2); break; }
            if (j == 0 && n > 0) {   // the epilogue of the previous tile has read O
              ok = mbar_wait(b_o_free, (n - 1) & 1, abort_flag);
              if (!ok) { report(status, kErrMma, 4 * g + 3); break; }
            }
            ok = mbar_wait_poll(b_p_full + 8 * sb, (g / kSBufs) & 1, abort_flag);
            if (!ok) { report(status, kErrMma, 4 * g + 3); break; }
            tc_fence_after();
            const uint32_t p_tmem = tmem + sb * 128, v_step = (g & 1) * kStageStep;
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk)   // P: 16 packed 16-bit values = 8 TMEM columns per product
              umma_ts_lo(tmem + kTmemO, p_tmem + kk * 8, dv_lo[kk] + v_step, d_hi, idesc_pv, (kk > 0 || j > 0) ? 1u : 0u);
            umma_commit(b_pv_done + 8 * sb);
            umma_commit(b_v_empty + 8 * (g & 1));
            if (j + 1 == nblk) umma_commit(b_o_full);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp >= 8) {
    // ================================ epilogue: O / l -> storage dtype -> global ==========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    const int r = (warp & 3) * 32 + lane;
    const uint32_t tO = tmem + kTmemO + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    bool ok = true;
    for (int n = 0;; ++n) {
      const int i = __shfl_sync(0xffffffffu, tile_at(n), 0);
      if (i < 0) { report(status, kErrEpilogue, -1000 - n); break; }
      if (i >= prob.total) break;
      const Tile t = tile_of(prob, i);
      ok = __all_sync(0xffffffffu, mbar_wait(b_lm_ready, n & 1, abort_flag));
      if (!ok) { report(status, kErrEpilogue, 2 * n); break; }
      const float m0 = sh->lm[0][r][0], l0 = sh->lm[0][r][1], m1 = sh->lm[1][r][0], l1 = sh->lm[1][r][1];
      mbar_arrive(b_lm_free);
      const float mf = fmaxf(m0, m1);   // the running maximum never decreases: the later one is the larger
      const float l = (l0 > 0.f ? l0 * ex2(m0 - mf) : 0.f) + (l1 > 0.f ? l1 * ex2(m1 - mf) : 0.f);
      const float inv = 1.f / l;
      ok = __all_sync(0xffffffffu, mbar_wait(b_o_full, n & 1, abort_flag));
      if (!ok) { report(status, kErrEpilogue, 2 * n + 1); break; }
      tc_fence_after();
      const int q_row = t.qt * kBM + r;
      uint16_t *dst = out + (static_cast<size_t>(t.bh) * prob.Sq + q_row) * kD;
      const bool row_exists = q_row < prob.Sq;
#pragma unroll 1
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + c * 32, o);
        tmem_wait_ld();
        if (c == kD / 32 - 1) {   // O is in registers: the next tile may overwrite it
          tc_fence_before();
          mbar_arrive(b_o_free);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint4 w;
          w.x = pack2<DT>(__uint_as_float(o[8 * k + 0]) * inv, __uint_as_float(o[8 * k + 1]) * inv);
          w.y = pack2<DT>(__uint_as_float(o[8 * k + 2]) * inv, __uint_as_float(o[8 * k + 3]) * inv);
          w.z = pack2<DT>(__uint_as_float(o[8 * k + 4]) * inv, __uint_as_float(o[8 * k + 5]) * inv);
          w.w = pack2<DT>(__uint_as_float(o[8 * k + 6]) * inv, __uint_as_float(o[8 * k + 7]) * inv);
          if (row_exists) *reinterpret_cast<uint4 *>(dst + c * 32 + k * 8) = w;
        }
      }
    }
  } else {
    // ================================ softmax: warpgroup w takes the blocks g with g & 1 == w ================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
    const int w = warp >> 2;
    const int r = (warp & 3) * 32 + lane;                     // row in the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tO = tmem + kTmemO + lane_addr;
    const int kv_off = prob.Skv - prob.Sq;
    int n = 0, g0 = 0;
    int i = __shfl_sync(0xffffffffu, tile_at(0), 0);
    bool ok = i >= 0;
    if (!ok) report(status, kErrSoftmax, -1000);
    Tile t = (ok && i < prob.total) ? tile_of(prob, i) : Tile{0, 0, 0};
    float m_mine = -INFINITY, l = 0.f;
    for (int g = w; ok; g += 2) {
      // tiles that end before block g: hand (maximum, partial sum) to the epilogue and move on
      while (i < prob.total && g >= g0 + t.nblk) {
        if (n > 0) {   // the epilogue has read the previous tile's values
          ok = __all_sync(0xffffffffu, mbar_wait(b_lm_free, (n - 1) & 1, abort_flag));
          if (!ok) { report(status, kErrSoftmax, -1 - n); break; }
        }
        sh->lm[w][r][0] = m_mine;
        sh->lm[w][r][1] = l;
        mbar_arrive(b_lm_ready);
        m_mine = -INFINITY;
        l = 0.f;
        g0 += t.nblk;
        ++n;
        i = __shfl_sync(0xffffffffu, tile_at(n), 0);
        if (i < 0) { report(status, kErrSoftmax, -1000 - n); ok = false; break; }
        if (i < prob.total) t = tile_of(prob, i);
      }
      if (!ok || i >= prob.total) break;
      const int j = g - g0;
      const int sb = g % kSBufs;
      const uint32_t tS = tmem + sb * 128 + lane_addr;
      ok = __all_sync(0xffffffffu, mbar_wait(b_s_full + 8 * sb, (g / kSBufs) & 1, abort_flag));
      if (!ok) { report(status, kErrSoftmax, g); break; }
      tc_fence_after();
      float m_prev = 0.f;
      if (g > 0) {
        // block g-1 has decided on its maximum (and, before that, has read the slot this block will overwrite)
        ok = __all_sync(0xffffffffu, mbar_wait(b_m_ready + 8 * ((g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag));
        if (!ok) { report(status, kErrSoftmax, 1000 + g); break; }
        if (j > 0) m_prev = sh->mslot[(g - 1) & 1][r];
      }
      uint32_t v[kBN];
      tmem_ld32p(tS, v);
      tmem_ld32p(tS + 32, v + 32);
      tmem_ld32p(tS + 64, v + 64);
      tmem_ld32p(tS + 96, v + 96);
      tmem_wait_ld();
      // column c of block j exists iff j*128 + c < Skv and, if causal, row r sees it iff j*128 + c <= qt*128 + kv_off + r
      const int vis = min(prob.causal ? (t.qt * kBM + kv_off + r - j * kBN) : kBN, prob.Skv - 1 - j * kBN);
      if (vis < kBN - 1) {
#pragma unroll
        for (int c = 0; c < kBN; ++c) v[c] = (c > vis) ? 0xff800000u : v[c];
      }
      // ---- row maximum: eight chains of three-input maxima ----
      float mc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        mc[c] = max3(__uint_as_float(v[c * 16]), __uint_as_float(v[c * 16 + 1]), __uint_as_float(v[c * 16 + 2]));
#pragma unroll
      for (int k = 3; k + 1 < 16; k += 2) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          mc[c] = max3(mc[c], __uint_as_float(v[c * 16 + k]), __uint_as_float(v[c * 16 + k + 1]));
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) mc[c] = fmaxf(mc[c], __uint_as_float(v[c * 16 + 15]));
      const float mx = fmaxf(max3(mc[0], mc[1], mc[2]), fmaxf(max3(mc[3], mc[4], mc[5]), fmaxf(mc[6], mc[7])));
      const float m_blk = mx * scale_log2;                     // -inf if the whole row is masked in this block
      // ---- the maximum to use: the one block g-1 decided on, unless this block exceeds it by more than 2^8 ----
      float m_new = m_blk;                                     // block 0 of a tile always has a visible column
      bool need = false;
      if (j > 0) {
        need = m_blk > m_prev + kRescaleThreshold;
        m_new = need ? m_blk : m_prev;
      }
      sh->mslot[g & 1][r] = m_new;
      mbar_arrive(b_m_ready + 8 * (g & 1));
      if (__any_sync(0xffffffffu, need)) {
        // O must hold every product up to block g-1 and none may be in flight
        ok = __all_sync(0xffffffffu, mbar_wait(b_pv_done + 8 * ((g - 1) % kSBufs), ((g - 1) / kSBufs) & 1, abort_flag));
        if (!ok) { report(status, kErrSoftmax, 2000 + g); break; }
        tc_fence_after();
        const float f = need ? ex2(m_prev - m_blk) : 1.f;
#pragma unroll 1
        for (int c = 0; c < kD / 16; ++c) {
          uint32_t o[16];
          tmem_ld16(tO + c * 16, o);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 16; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * f);
          tmem_st16(tO + c * 16, o);
        }
        tmem_wait_st();
      }
      if (m_mine != m_new) {   // bring the partial sum to the new maximum (2^(-inf) = 0 on the first block)
        l *= ex2(m_mine - m_new);
        m_mine = m_new;
      }
      // ---- p = 2^(s*scale - m), row sum, pack to 16 bit; P overwrites columns 0..63 of S ----
      const uint64_t c2 = f2_pack(scale_log2, scale_log2), nm2 = f2_pack(-m_new, -m_new);
      uint64_t lsum2 = f2_pack(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const uint64_t x2 = f2_fma(
              f2_pack(__uint_as_float(v[c * 32 + 2 * k]), __uint_as_float(v[c * 32 + 2 * k + 1])), c2, nm2);
          const float2 x = f2_unpack(x2);
          const float p0 = ex2(x.x), p1 = ex2(x.y);
          lsum2 = f2_add(lsum2, f2_pack(p0, p1));
          pk[k] = pack2<DT>(p0, p1);
        }
        tmem_st16(tS + c * 16, pk);
      }
      {
        const float2 ls = f2_unpack(lsum2);
        l += ls.x + ls.y;
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(b_p_full + 8 * sb);
    }
  }

  // ================================ tear-down =====================================
  tc_fence_before();
  __syncthreads();
  if (warp == 15) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_tile_map(CUtensorMap *tm, const void *ptr, long long slices, long long rows, int dtype, int box_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  NB200_REQUIRE(enc, NB200_ERR_LAUNCH, "attn_fwd: cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(slices)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kD) * 2, static_cast<cuuint64_t>(rows) * kD * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(tm, dtype == NB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         3, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  NB200_REQUIRE(r == CUDA_SUCCESS, NB200_ERR_LAUNCH, "attn_fwd: cuTensorMapEncodeTiled failed with code %d", (int)r);
  return NB200_OK;
}

// Tile counters of the launches in flight: a launch takes the next slot and zeroes it on its stream before the kernel.
__device__ unsigned int g_tile_counters[64];

template <int DT>
int launch_tc(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, void *out, int BH, int Sq,
              int Skv, float scale_log2, int causal, int *status, cudaStream_t st) {
  NB200_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_tcgen05_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  int dev = 0, sms = 0;
  NB200_CHECK_CUDA(cudaGetDevice(&dev));
  NB200_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  Problem p;
  p.Sq = Sq;
  p.Skv = Skv;
  p.n_qtiles = (Sq + kBM - 1) / kBM;
  p.n_units = BH;
  p.group = min(BH, kHeadGroup);
  p.causal = causal;
  p.total = BH * p.n_qtiles;
  const int grid = min(p.total, sms);
  static std::atomic<unsigned> next_slot{0};
  unsigned int *counters = nullptr;
  NB200_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&counters), g_tile_counters));
  unsigned int *counter = counters + (next_slot.fetch_add(1) & 63u);
  NB200_CHECK_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned int), st));
  attn_fwd_tcgen05_kernel<DT><<<dim3(grid), dim3(kThreads), kSmemBytes, st>>>(tq, tk, tv, static_cast<uint16_t *>(out), p,
                                                                        scale_log2, counter, status
  );
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

}  // namespace

int attn_simt_launch(const void *q, const void *k, const void *v, void *out, int B, int H, int Sq, int Skv,
                     int D, int dtype, float scale_log2, int causal, cudaStream_t st);

}  // namespace nb200

using namespace nb200;

extern "C" int nb200_attn_fwd(const void *q, const void *k, const void *v, void *out, int B, int H, int Sq,
                              int Skv, int D, int dtype, float scale_log2, int causal, int *status,
                              void *stream) {
  NB200_REQUIRE(q && k && v && out, NB200_ERR_BAD_ARG, "attn_fwd: null pointer");
  NB200_REQUIRE(B > 0 && H > 0 && Sq > 0 && Skv > 0 && D > 0, NB200_ERR_BAD_ARG, "attn_fwd: non-positive extent");
  NB200_REQUIRE(scale_log2 > 0.f, NB200_ERR_BAD_ARG, "attn_fwd: scale_log2 must be positive");
  NB200_REQUIRE(!causal || Skv >= Sq, NB200_ERR_UNSUPPORTED, "attn_fwd: causal needs Skv >= Sq");
  NB200_REQUIRE(dtype == NB200_F16 || dtype == NB200_BF16 || dtype == NB200_F32, NB200_ERR_UNSUPPORTED,
                "attn_fwd: dtype %d", dtype);
  auto st = static_cast<cudaStream_t>(stream);
  const bool tensor_path = (dtype == NB200_F16 || dtype == NB200_BF16) && D == kD &&
                           (long long)B * H * ((Sq + kBM - 1) / kBM) < (1ll << 31) &&
                           (long long)B * H * (long long)(Sq > Skv ? Sq : Skv) < (1ll << 31);
  if (!tensor_path) return attn_simt_launch(q, k, v, out, B, H, Sq, Skv, D, dtype, scale_log2, causal, st);

  NB200_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), NB200_ERR_BAD_ARG,
                "attn_fwd: tensors must be 16-byte aligned");
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tile_map(&tq, q, (long long)B * H, Sq, dtype, kBM)) != NB200_OK) return rc;
  if ((rc = make_tile_map(&tk, k, (long long)B * H, Skv, dtype, kBN)) != NB200_OK) return rc;
  if ((rc = make_tile_map(&tv, v, (long long)B * H, Skv, dtype, kBN)) != NB200_OK) return rc;
  if (dtype == NB200_BF16)
    return launch_tc<NB200_BF16>(tq, tk, tv, out, B * H, Sq, Skv, scale_log2, causal, status, st);
  return launch_tc<NB200_F16>(tq, tk, tv, out, B * H, Sq, Skv, scale_log2, causal, status, st);
}
