// Fused attention forward on Blackwell tensor cores (f16 / bf16 storage, D = 128).
//
// One CTA computes a tile of 128 query rows of one (batch, head) against the KV sequence in blocks
// of 64 rows, with the online softmax of the HTile program
// (tests/data/flash_attention_htile.mlir:40-143 of the reference) kept in the exp2 domain.  The
// three stages of a block -- S = Q K^T, softmax, O += P V -- run as a software pipeline, each stage on
// warps of its own that meet only at mbarriers:
//
//   warp 4, warp 7      TMA producers (one lane each): Q once and K(j); V(j).  Two 16 KB buffers per
//   (one lane each)     operand (128-byte swizzled), re-armed when the MMA that read a buffer has
//                       retired.  Separate threads because K(j+1) is wanted a whole block before
//                       V(j+1): one thread waiting for the V buffer would hold the K load back
//   warp 5 (one lane)   QK issuer, operand descriptors built once: S = Q K(j)^T (8 x tcgen05.mma
//                       128x64x16, both operands in smem) into TMEM columns 0..63.  The softmax warps
//                       copy S(j-1) into registers first thing and release the buffer, so S(j) is
//                       computed while they work on block j-1
//   warp 6 (one lane)   PV issuer: O += P_b V(j) (4 x tcgen05.mma 128x128x16) with P read from TMEM
//                       (two buffers of 32 columns, packed 16-bit) and V as an MN-major smem operand;
//                       the accumulator O lives in TMEM columns 128..255.  A thread of its own, so
//                       that a product is issued the moment P arrives instead of queueing behind
//                       the score products of a later block
//   warps 0-3           softmax: thread r owns row r (TMEM lane r), so row max and row sum need no
//                       cross-thread traffic; the 64 scores are read from TMEM once into registers
//                       (three-input maxima, packed f32x2 scale/sum, exp2, pack to 16 bit).
//                       O is rescaled in TMEM only when a row maximum grows by more than 2^8,
//                       which leaves the result unchanged (the same stale maximum scales P and
//                       the running sum) but makes the rescale rare
//
// Two CTAs are resident per SM (96 KB smem, 256 TMEM columns each).  Tiles are numbered so that
// CTAs running at the same time work on the same few heads (K/V stay in L2) and, for causal
// problems, the long tiles of a head are issued first.  Every wait is bounded; on expiry the CTA
// records a code in the status words and unwinds.
#include <cuda.h>

#include "nb200_common.cuh"
#include "sm100_primitives.cuh"

namespace nb200 {
namespace {

using namespace sm100;

constexpr int kBM = 128;            // query rows per CTA
constexpr int kBN = 64;             // kv rows per pipeline step
constexpr int kHeadGroup = 16;      // heads whose tiles are interleaved (tile-major) in the launch order
constexpr int kD = 128;             // head dimension
constexpr int kThreads = 256;       // 4 softmax warps, K producer, QK issuer, PV issuer, V producer
constexpr int kQBytes = kBM * kD * 2;           // 32 KB: two 64-column boxes of 16 KB
constexpr int kQBox = kQBytes / 2;
constexpr int kKVBytes = kBN * kD * 2;          // 16 KB: two 64-column boxes of 8 KB
constexpr int kKVBox = kKVBytes / 2;
constexpr int kTmemCols = 256;                  // S (64) | P0 (32) | P1 (32) | O (128)
constexpr int kSmemBytes = kQBytes + 4 * kKVBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr float kRescaleThreshold = 8.0f;       // log2 units

enum : int { kErrProducer = 1, kErrMma = 2, kErrSoftmax = 3, kErrEpilogue = 4 };

struct Barriers {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, s_free, p_full[2], pv_done[2], o_full;
  uint32_t tmem_base;
  int abort_flag;
  int skip;
};

__device__ __forceinline__ void report(int *status, int code, int detail) {
  if (status && atomicCAS(status, 0, code) == 0) {
    status[1] = static_cast<int>(blockIdx.x);
    status[2] = detail;
    status[3] = static_cast<int>(threadIdx.x);
  }
}

template <int DT>
__global__ void __launch_bounds__(kThreads, 2)
attn_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, uint16_t *__restrict__ out, int Sq, int Skv,
                        int n_qtiles, int n_units, int group, float scale_log2, int causal, int *status) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char *smem = smem_raw + (base - raw);
  const uint32_t sQ = base;
  const uint32_t sK0 = base + kQBytes, sV0 = base + kQBytes + 2 * kKVBytes;  // buffer b is at + b * kKVBytes
  Barriers *bars = reinterpret_cast<Barriers *>(smem + kQBytes + 4 * kKVBytes);
  volatile int *abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // tile -> (head, query tile).  Heads are taken in groups of `group`; inside a group the order is tile-major
  // with the longest causal tiles first, so that the CTAs in flight at any moment belong to few heads (their
  // K/V stay in L2) while the last CTAs of a group, and of the launch, are the shortest ones.
  const int per_group = group * n_qtiles;
  const int grp = blockIdx.x / per_group, rem = blockIdx.x % per_group;
  const int heads_here = min(group, n_units - grp * group);
  const int qi = rem / heads_here;
  const int bh = grp * group + rem % heads_here;
  const int qt = causal ? (n_qtiles - 1 - qi) : qi;
  const int kv_off = Skv - Sq;                                    // causal diagonal offset (>= 0)
  // last kv column any row of the tile sees; Sq and Skv need not be multiples of the tile sizes: rows and
  // columns past the end of a (batch, head) slice load as zeros (3-D tensor maps), the columns are masked in
  // the softmax and the rows are not stored
  const int last_col = causal ? min(Skv - 1, qt * kBM + kv_off + kBM - 1) : Skv - 1;
  const int nblk = last_col / kBN + 1;
  const int q_row0 = qt * kBM;                                    // row inside the (batch, head) slice

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    bars->skip = (status != nullptr && *reinterpret_cast<volatile int *>(status) != 0) ? 1 : 0;
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars->k_full[b]), 1);
      mbar_init(smem_u32(&bars->k_empty[b]), 1);
      mbar_init(smem_u32(&bars->v_full[b]), 1);
      mbar_init(smem_u32(&bars->v_empty[b]), 1);
      mbar_init(smem_u32(&bars->p_full[b]), 128);
      mbar_init(smem_u32(&bars->pv_done[b]), 1);
    }
    mbar_init(smem_u32(&bars->o_full), 1);
    mbar_init(smem_u32(&bars->s_full), 1);
    mbar_init(smem_u32(&bars->s_free), 128);
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (bars->skip) return;  // an earlier CTA of this launch already reported a failure

  if (warp == 5) {
    tmem_alloc(smem_u32(&bars->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  const uint32_t tS = tmem, tP0 = tmem + kBN, tO = tmem + 2 * kBN;  // P buffer b is at tP0 + b * kBN / 2 columns

  const uint32_t b_q_full = smem_u32(&bars->q_full), b_k_full = smem_u32(&bars->k_full[0]),
                 b_k_empty = smem_u32(&bars->k_empty[0]), b_v_full = smem_u32(&bars->v_full[0]),
                 b_v_empty = smem_u32(&bars->v_empty[0]), b_s_full = smem_u32(&bars->s_full), b_s_free = smem_u32(&bars->s_free),
                 b_p_full = smem_u32(&bars->p_full[0]), b_pv_done = smem_u32(&bars->pv_done[0]),
                 b_o_full = smem_u32(&bars->o_full);  // buffer b of a pair is at +8*b

  if (warp == 4) {
    // ================================ TMA producer: Q and K ================================
    // K and V have a producer thread each: K(j+1) is wanted a whole block before V(j+1), and a single
    // thread that waits for the V buffer first would hold the K load back.
    if (lane == 0) {
      mbar_arrive_expect_tx(b_q_full, kQBytes);
      tma_load_3d(sQ, &tm_q, 0, q_row0, bh, b_q_full);
      tma_load_3d(sQ + kQBox, &tm_q, 64, q_row0, bh, b_q_full);
      int issued = 0;
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int b = j & 1;
        ok = mbar_wait(b_k_empty + 8 * b, ((j >> 1) & 1) ^ 1, abort_flag);
        if (!ok) { report(status, kErrProducer, 2 * j); break; }
        mbar_arrive_expect_tx(b_k_full + 8 * b, kKVBytes);
        tma_load_3d(sK0 + b * kKVBytes, &tm_k, 0, j * kBN, bh, b_k_full + 8 * b);
        tma_load_3d(sK0 + b * kKVBytes + kKVBox, &tm_k, 64, j * kBN, bh, b_k_full + 8 * b);
        ++issued;
      }
      if (!ok) {
        // Unwinding: let the copies already in flight land before the CTA's shared memory goes away.
        mbar_wait(b_q_full, 0, abort_flag);
        for (int spin = 0; spin < 100000; ++spin) {
          bool done = true;
          for (int n = 0; n < 2; ++n) {  // the last two loads
            const int jk = issued - 1 - n;
            if (jk >= 0) done = done && mbar_try_wait(b_k_full + 8 * (jk & 1), (jk >> 1) & 1);
          }
          if (done) break;
          __nanosleep(100);
        }
      }
    }
    __syncwarp();
  } else if (warp == 7) {
    // ================================ TMA producer: V ======================================
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int b = j & 1;
        ok = mbar_wait(b_v_empty + 8 * b, ((j >> 1) & 1) ^ 1, abort_flag);
        if (!ok) { report(status, kErrProducer, 2 * j + 1); break; }
        mbar_arrive_expect_tx(b_v_full + 8 * b, kKVBytes);
        tma_load_3d(sV0 + b * kKVBytes, &tm_v, 0, j * kBN, bh, b_v_full + 8 * b);
        tma_load_3d(sV0 + b * kKVBytes + kKVBox, &tm_v, 64, j * kBN, bh, b_v_full + 8 * b);
        ++issued;
      }
      if (!ok) {
        for (int spin = 0; spin < 100000; ++spin) {
          bool done = true;
          for (int n = 0; n < 2; ++n) {
            const int jv = issued - 1 - n;
            if (jv >= 0) done = done && mbar_try_wait(b_v_full + 8 * (jv & 1), (jv >> 1) & 1);
          }
          if (done) break;
          __nanosleep(100);
        }
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ================================ QK issuer ===================================
    // S = Q K(j)^T.  The softmax warps copy S(j-1) into registers first thing and release the buffer,
    // so S(j) is computed while they work on block j-1.  A thread of its own, so that the score
    // products keep flowing while the other issuer waits for the softmax warps.
    if (lane == 0) {
      constexpr int fmt = (DT == NB200_BF16) ? 1 : 0;
      constexpr uint32_t idesc_qk = umma_idesc_f16(fmt, 0, kBM, kBN);
      // Operand descriptors never change: build them once, so that issuing an MMA is a couple of
      // instructions (building one per MMA costs ~90 cycles of scalar work and starves the pipe).
      uint64_t dq[kD / 16], dk[2][kD / 16];
#pragma unroll
      for (int kk = 0; kk < kD / 16; ++kk) {
        // 16 elements of the reduction per MMA = 32 bytes inside the 128-byte swizzled row
        dq[kk] = umma_desc_sw128(sQ + (kk >> 2) * kQBox + (kk & 3) * 32, 16, 1024);
#pragma unroll
        for (int b = 0; b < 2; ++b) dk[b][kk] = umma_desc_sw128(sK0 + b * kKVBytes + (kk >> 2) * kKVBox + (kk & 3) * 32, 16, 1024);
      }
      bool ok = mbar_wait(b_q_full, 0, abort_flag);
      if (!ok) report(status, kErrMma, -1);
      for (int j = 0; j < nblk && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(b_k_full + 8 * b, ph, abort_flag);
        if (!ok) { report(status, kErrMma, 3 * j); break; }
        if (j >= 1) {
          ok = mbar_wait(b_s_free, (j - 1) & 1, abort_flag);   // the softmax warps hold S(j-1) in registers
          if (!ok) { report(status, kErrMma, 3 * j + 1); break; }
        }
        tc_fence_after();
        if (b == 0) {
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) umma_ss(tS, dq[kk], dk[0][kk], idesc_qk, kk > 0);
        } else {
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) umma_ss(tS, dq[kk], dk[1][kk], idesc_qk, kk > 0);
        }
        umma_commit(b_k_empty + 8 * b);
        umma_commit(b_s_full);
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ================================ PV issuer ===================================
    if (lane == 0) {
      constexpr int fmt = (DT == NB200_BF16) ? 1 : 0;
      constexpr uint32_t idesc_pv = umma_idesc_f16(fmt, 1, kBM, kD);
      uint64_t dv[2][kBN / 16];
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk)  // V: 16 kv rows = 2 KB; the two 64-column blocks are 8 KB apart
          dv[b][kk] = umma_desc_sw128(sV0 + b * kKVBytes + kk * 2048, kKVBox, 1024);
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        ok = mbar_wait(b_v_full + 8 * b, ph, abort_flag);
        if (!ok) { report(status, kErrMma, 3 * j + 2); break; }
        ok = mbar_wait(b_p_full + 8 * b, ph, abort_flag);
        if (!ok) { report(status, kErrMma, 3 * j + 1); break; }
        tc_fence_after();
        // P: 16 packed 16-bit values = 8 TMEM columns per MMA
        const uint32_t acc0 = j > 0 ? 1u : 0u;
        if (b == 0) {
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) umma_ts(tO, tP0 + kk * 8, dv[0][kk], idesc_pv, kk > 0 ? 1u : acc0);
        } else {
#pragma unroll
          for (int kk = 0; kk < kBN / 16; ++kk) umma_ts(tO, tP0 + kBN / 2 + kk * 8, dv[1][kk], idesc_pv, kk > 0 ? 1u : acc0);
        }
        umma_commit(b_v_empty + 8 * b);
        umma_commit(b_pv_done + 8 * b);   // P_b is free again, and O holds every product up to block j
      }
      if (ok) umma_commit(b_o_full);
    }
    __syncwarp();
  } else {
    // ================================ softmax + epilogue ==========================
    const int r = warp * 32 + lane;                         // row in the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      const int b = j & 1;
      // warp-uniform outcome: the TMEM accesses below are warp-collective
      ok = __all_sync(0xffffffffu, mbar_wait(b_s_full, j & 1, abort_flag));
      if (!ok) { report(status, kErrSoftmax, j); break; }
      tc_fence_after();
      const uint32_t tPb = tP0 + b * (kBN / 2) + lane_addr;

      // ---- the 64 scores of this row into registers (one TMEM read); S is then free for block j+1 ----
      uint32_t v[kBN];
      tmem_ld32p(tS + lane_addr, v);
      tmem_ld32p(tS + lane_addr + 32, v + 32);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(b_s_free);
      // column c of block j exists iff j*64 + c < Skv and, if causal, is visible to row r iff j*64 + c <= qt*128 + kv_off + r
      const int vis = min(causal ? (qt * kBM + kv_off + r - j * kBN) : kBN, Skv - 1 - j * kBN);  // columns 0..vis are visible
      if (vis < kBN - 1) {
#pragma unroll
        for (int i = 0; i < kBN; ++i) v[i] = (i > vis) ? 0xff800000u : v[i];  // -inf: 2^(-inf) = 0
      }

      // ---- row maximum (four chains of three-input maxima) ----
      float mc[4];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        mc[c] = max3(__uint_as_float(v[c * 16]), __uint_as_float(v[c * 16 + 1]), __uint_as_float(v[c * 16 + 2]));
#pragma unroll
      for (int i = 3; i + 1 < 16; i += 2) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          mc[c] = max3(mc[c], __uint_as_float(v[c * 16 + i]), __uint_as_float(v[c * 16 + i + 1]));
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) mc[c] = fmaxf(mc[c], __uint_as_float(v[c * 16 + 15]));
      const float mx = fmaxf(max3(mc[0], mc[1], mc[2]), mc[3]);
      const float m_blk = mx * scale_log2;                   // scale_log2 > 0; -inf if the whole row is masked
      if (j == 0) {
        m_used = m_blk;                                      // block 0 always has a visible column
      } else {
        const bool need = m_blk > m_used + kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          // O must hold every product up to block j-1 and none may be in flight: wait for PV(j-1)
          // (the products before it were issued earlier by the same thread and complete in order).
          ok = __all_sync(0xffffffffu, mbar_wait(b_pv_done + 8 * ((j - 1) & 1), ((j - 1) >> 1) & 1, abort_flag));
          if (!ok) { report(status, kErrSoftmax, 1000 + j); break; }
          tc_fence_after();
          const float f = need ? ex2(m_used - m_blk) : 1.f;
          if (need) m_used = m_blk;
          l *= f;
#pragma unroll 1
          for (int c = 0; c < kD / 16; ++c) {  // 16 columns at a time: the scores stay live in registers
            uint32_t o[16];
            tmem_ld16(tO + lane_addr + c * 16, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
            tmem_st16(tO + lane_addr + c * 16, o);
          }
          tmem_wait_st();
        }
      }

      // ---- p = 2^(s*scale - m) on packed pairs, row sum, pack to 16 bit, write P_b ----
      if (j >= 2) {  // PV(j-2) read P_b; it completed long ago, this only makes the order formal
        ok = __all_sync(0xffffffffu, mbar_wait(b_pv_done + 8 * b, ((j - 2) >> 1) & 1, abort_flag));
        if (!ok) { report(status, kErrSoftmax, 2000 + j); break; }
        tc_fence_after();
      }
      const uint64_t c2 = f2_pack(scale_log2, scale_log2), nm2 = f2_pack(-m_used, -m_used);
      uint64_t lsum2 = f2_pack(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint64_t x2 = f2_fma(
              f2_pack(__uint_as_float(v[c * 32 + 2 * i]), __uint_as_float(v[c * 32 + 2 * i + 1])), c2, nm2);
          const float2 x = f2_unpack(x2);
          const float p0 = ex2(x.x), p1 = ex2(x.y);
          lsum2 = f2_add(lsum2, f2_pack(p0, p1));
          pk[i] = pack2<DT>(p0, p1);
        }
        tmem_st16(tPb + c * 16, pk);
      }
      {
        const float2 ls = f2_unpack(lsum2);
        l += ls.x + ls.y;
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(b_p_full + 8 * b);
    }

    // ---- epilogue: O / l -> storage dtype -> global ----
    if (ok) {
      ok = __all_sync(0xffffffffu, mbar_wait(b_o_full, 0, abort_flag));
      if (!ok) report(status, kErrEpilogue, 0);
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      uint16_t *dst = out + (static_cast<size_t>(bh) * Sq + q_row0 + r) * kD;
      const bool row_exists = q_row0 + r < Sq;   // the last tile of a slice may be partial
#pragma unroll 1
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tO + lane_addr + c * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 w;
          w.x = pack2<DT>(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
          w.y = pack2<DT>(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
          w.z = pack2<DT>(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
          w.w = pack2<DT>(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
          if (row_exists) *reinterpret_cast<uint4 *>(dst + c * 32 + i * 8) = w;
        }
      }
    }
  }

  // ================================ tear-down =====================================
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// cuTensorMapEncodeTiled, resolved through the runtime so that the library does not link libcuda.
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

// [slices, rows, 128] 16-bit row-major tensor, boxes of 1 slice x box_rows rows x 64 columns, 128-byte swizzle.
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

template <int DT>
int launch_tc(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, void *out, int BH, int Sq,
              int Skv, float scale_log2, int causal, int *status, cudaStream_t st) {
  // per-device attribute: set on every call so that any current device is covered
  NB200_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_tcgen05_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        kSmemBytes));
  // two CTAs of ~97 KB must fit: ask for the largest shared-memory carve-out
  NB200_CHECK_CUDA(cudaFuncSetAttribute(attn_fwd_tcgen05_kernel<DT>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                        cudaSharedmemCarveoutMaxShared));
  const int n_qtiles = (Sq + kBM - 1) / kBM;
  const int group = min(BH, kHeadGroup);
  attn_fwd_tcgen05_kernel<DT><<<dim3(BH * n_qtiles), dim3(kThreads), kSmemBytes, st>>>(
      tq, tk, tv, static_cast<uint16_t *>(out), Sq, Skv, n_qtiles, BH, group, scale_log2, causal, status);
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
