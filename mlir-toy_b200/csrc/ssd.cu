// Mamba-2 SSD chunked scan forward.
//
//   S <- exp(dt*A) S + dt * x (outer) B ;   y = S . C        (S is P x N per (batch, head))
//
// evaluated chunk by chunk (chunk length Q), with cum_i = sum_{s<=i} dt_s*A inside a chunk:
//   kernel 1  per (b, chunk, head): cum -> workspace; chunk state
//             Z = sum_j e^(cum_Q - cum_j) dt_j x_j (outer) B_j            (tensor cores, fp32 accumulate)
//   kernel 2  per (b, head): the fp32 recurrence S_in(c) = e^(cum_Q(c-1)) S_in(c-1) + Z(c-1), in place
//   kernel 3  per (b, chunk, head, 64-row block): y = e^(cum_i) C_i . S_in
//             + sum_{j<=i} (C_i . B_j) e^(cum_i - cum_j) dt_j x_j         (tensor cores, fp32 accumulate)
// All exponents are <= 0 (A < 0), so nothing overflows.  Matrix products run on warp-level bf16/f16
// MMA (16x16x16 fragments) with fp32 accumulation; decay factors are applied in fp32 between the
// two products of kernel 3 and the masked product is rounded to the storage dtype before it
// multiplies x, exactly as the CPU oracle's chunked form does.
#include <mma.h>

#include "nb200_common.cuh"

namespace nb200 {
namespace {

using namespace nvcuda;

constexpr int kP = 64;     // head dimension
constexpr int kN = 128;    // state dimension
constexpr int kJB = 64;    // rows per staged block
constexpr int kLdN = kN + 8;   // padded leading dimensions (elements)
constexpr int kLdP = kP + 8;
constexpr int kLdG = kJB + 4;  // fp32 scratch
constexpr float kLog2e = 1.4426950408889634f;

template <int DT> struct WmmaElem;
template <> struct WmmaElem<NB200_F16> { using type = __half; };
template <> struct WmmaElem<NB200_BF16> { using type = __nv_bfloat16; };

template <int DT> __device__ __forceinline__ typename WmmaElem<DT>::type to_elem(float x);
template <> __device__ __forceinline__ __half to_elem<NB200_F16>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 to_elem<NB200_BF16>(float x) { return __float2bfloat16_rn(x); }

// ---- kernel 1: cumulative decay and chunk state -------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(128)
ssd_chunk_state_kernel(const uint16_t *__restrict__ x, const float *__restrict__ dt, const float *__restrict__ A,
                       const uint16_t *__restrict__ Bm, float *__restrict__ cum_ws, float *__restrict__ state_ws,
                       int L, int H, int G, int Q) {
  using T = typename WmmaElem<DT>::type;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *sXs = reinterpret_cast<T *>(smem_raw);                        // [kJB][kLdP]  w_j * x_j
  T *sB = sXs + kJB * kLdP;                                        // [kJB][kLdN]
  float *sCum = reinterpret_cast<float *>(sB + kJB * kLdN);        // [Q]
  float *sW = sCum + Q;                                            // [Q]  e^(cum_Q - cum_j) dt_j

  const int h = blockIdx.x, c = blockIdx.y, b = blockIdx.z;
  const int nc = L / Q;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = h / (H / G);
  const size_t t0 = (size_t)b * L + (size_t)c * Q;                 // first time step of the chunk (row index)
  const float a = A[h];

  // inclusive prefix sum of dt*A over the chunk: warp 0, Q/32 consecutive values per lane
  if (warp == 0) {
    const int per = Q / 32;
    float run = 0.f;
    for (int i = 0; i < per; ++i) {
      run += dt[(t0 + lane * per + i) * H + h] * a;
      sCum[lane * per + i] = run;
    }
    float offs = run;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, offs, d);
      if (lane >= d) offs += o;
    }
    offs -= run;  // exclusive prefix of the lane totals
    for (int i = 0; i < per; ++i) sCum[lane * per + i] += offs;
  }
  __syncthreads();
  const float cum_last = sCum[Q - 1];
  float *cum_out = cum_ws + (((size_t)b * H + h) * nc + c) * Q;
  for (int i = tid; i < Q; i += 128) {
    const float ci = sCum[i];
    cum_out[i] = ci;
    sW[i] = ex2((cum_last - ci) * kLog2e) * dt[(t0 + i) * H + h];
  }
  __syncthreads();

  // Z[p][n] = sum_j Xs[j][p] * B[j][n]; warp w owns p in [16w, 16w+16)
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[kN / 16];
#pragma unroll
  for (int n = 0; n < kN / 16; ++n) wmma::fill_fragment(acc[n], 0.f);

  for (int j0 = 0; j0 < Q; j0 += kJB) {
    // stage: x rows are 64 elements (128 B) = 8 x 16 B; B rows are 128 elements = 16 x 16 B
    for (int idx = tid; idx < kJB * 8; idx += 128) {
      const int r = idx >> 3, seg = idx & 7;
      const uint4 w = *reinterpret_cast<const uint4 *>(x + ((t0 + j0 + r) * H + h) * kP + seg * 8);
      const float wj = sW[j0 + r];
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
      uint4 o;
      uint32_t *os = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack2<DT>(ws[e]);
        os[e] = pack2<DT>(f.x * wj, f.y * wj);
      }
      *reinterpret_cast<uint4 *>(sXs + r * kLdP + seg * 8) = o;
    }
    for (int idx = tid; idx < kJB * 16; idx += 128) {
      const int r = idx >> 4, seg = idx & 15;
      *reinterpret_cast<uint4 *>(sB + r * kLdN + seg * 8) =
          *reinterpret_cast<const uint4 *>(Bm + ((t0 + j0 + r) * G + g) * kN + seg * 8);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kJB / 16; ++k) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::col_major> fa;   // A[p][j] = Xs[j][p]
      wmma::load_matrix_sync(fa, sXs + (k * 16) * kLdP + warp * 16, kLdP);
#pragma unroll
      for (int n = 0; n < kN / 16; ++n) {
        wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::row_major> fb;  // B[j][n]
        wmma::load_matrix_sync(fb, sB + (k * 16) * kLdN + n * 16, kLdN);
        wmma::mma_sync(acc[n], fa, fb, acc[n]);
      }
    }
    __syncthreads();
  }
  float *z = state_ws + ((((size_t)b * H + h) * nc + c) * kP + warp * 16) * kN;
#pragma unroll
  for (int n = 0; n < kN / 16; ++n) wmma::store_matrix_sync(z + n * 16, acc[n], kN, wmma::mem_row_major);
}

// ---- kernel 2: fp32 state recurrence across chunks, in place ------------------------------------
__global__ void __launch_bounds__(256)
ssd_state_pass_kernel(const float *__restrict__ cum_ws, float *__restrict__ state_ws, int nc, int Q) {
  const size_t bh = blockIdx.y;
  const int e = blockIdx.x * 256 + threadIdx.x;  // element of the P x N state
  float s = 0.f;
  for (int c = 0; c < nc; ++c) {
    float *p = state_ws + (bh * nc + c) * (size_t)(kP * kN) + e;
    const float z = *p;
    *p = s;  // state entering chunk c
    const float decay = ex2(cum_ws[(bh * nc + c) * Q + (Q - 1)] * kLog2e);
    s = fmaf(decay, s, z);
  }
}

// ---- kernel 3: outputs ---------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(128)
ssd_chunk_scan_kernel(const uint16_t *__restrict__ x, const float *__restrict__ dt, const uint16_t *__restrict__ Bm,
                      const uint16_t *__restrict__ Cm, const float *__restrict__ cum_ws,
                      const float *__restrict__ state_ws, uint16_t *__restrict__ y, int L, int H, int G, int Q) {
  using T = typename WmmaElem<DT>::type;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *sC = reinterpret_cast<T *>(smem_raw);          // [64][kLdN]  C rows of this block
  T *sB = sC + kJB * kLdN;                          // [64][kLdN]  B rows of block j
  T *sS = sB + kJB * kLdN;                          // [64 p][kLdN] entering state, rounded
  T *sX = sS + kP * kLdN;                           // [64][kLdP]  x rows of block j
  T *sM = sX + kJB * kLdP;                          // [64][kLdP]  masked, decayed C.B^T
  float *sG = reinterpret_cast<float *>(sM + kJB * kLdP);  // [64][kLdG] fp32 scratch
  float *sCumI = sG + kJB * kLdG;                   // [64]
  float *sCumJ = sCumI + kJB;                       // [64]
  float *sDtJ = sCumJ + kJB;                        // [64]

  const int nib = Q / kJB;
  const int ib = blockIdx.x % nib, h = blockIdx.x / nib, c = blockIdx.y, b = blockIdx.z;
  const int nc = L / Q;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = h / (H / G);
  const size_t t0 = (size_t)b * L + (size_t)c * Q;
  const size_t bhc = ((size_t)b * H + h) * nc + c;
  const float *cum = cum_ws + bhc * Q;
  const int i0 = ib * kJB;

  for (int idx = tid; idx < kJB * 16; idx += 128) {
    const int r = idx >> 4, seg = idx & 15;
    *reinterpret_cast<uint4 *>(sC + r * kLdN + seg * 8) =
        *reinterpret_cast<const uint4 *>(Cm + ((t0 + i0 + r) * G + g) * kN + seg * 8);
  }
  {
    const float *st = state_ws + bhc * (size_t)(kP * kN);
    for (int idx = tid; idx < kP * kN / 4; idx += 128) {
      const int p = idx / (kN / 4), q = idx % (kN / 4);
      const float4 f = *reinterpret_cast<const float4 *>(st + p * kN + q * 4);
      uint2 w;
      w.x = pack2<DT>(f.x, f.y);
      w.y = pack2<DT>(f.z, f.w);
      *reinterpret_cast<uint2 *>(sS + p * kLdN + q * 4) = w;
    }
  }
  if (tid < kJB) sCumI[tid] = cum[i0 + tid];
  __syncthreads();

  // inter-chunk term: Y = e^(cum_i) * (C_i . S_in^T); warp w owns rows [16w, 16w+16)
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> yacc[kP / 16];
#pragma unroll
  for (int n = 0; n < kP / 16; ++n) wmma::fill_fragment(yacc[n], 0.f);
#pragma unroll
  for (int k = 0; k < kN / 16; ++k) {
    wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::row_major> fa;
    wmma::load_matrix_sync(fa, sC + (warp * 16) * kLdN + k * 16, kLdN);
#pragma unroll
    for (int n = 0; n < kP / 16; ++n) {
      wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::col_major> fb;  // B[k=n_state][p] = S[p][n_state]
      wmma::load_matrix_sync(fb, sS + (n * 16) * kLdN + k * 16, kLdN);
      wmma::mma_sync(yacc[n], fa, fb, yacc[n]);
    }
  }
  float *gw = sG + (warp * 16) * kLdG;  // this warp's 16 rows of scratch
#pragma unroll
  for (int n = 0; n < kP / 16; ++n) wmma::store_matrix_sync(gw + n * 16, yacc[n], kLdG, wmma::mem_row_major);
  __syncwarp();
  for (int e = lane; e < 16 * kP; e += 32) {
    const int r = e / kP, col = e % kP;
    gw[r * kLdG + col] *= ex2(sCumI[warp * 16 + r] * kLog2e);
  }
  __syncwarp();
#pragma unroll
  for (int n = 0; n < kP / 16; ++n) wmma::load_matrix_sync(yacc[n], gw + n * 16, kLdG, wmma::mem_row_major);

  // intra-chunk term over the blocks j <= i
  for (int jb = 0; jb <= ib; ++jb) {
    const int j0 = jb * kJB;
    __syncthreads();  // previous block's sB / sX fully consumed
    for (int idx = tid; idx < kJB * 16; idx += 128) {
      const int r = idx >> 4, seg = idx & 15;
      *reinterpret_cast<uint4 *>(sB + r * kLdN + seg * 8) =
          *reinterpret_cast<const uint4 *>(Bm + ((t0 + j0 + r) * G + g) * kN + seg * 8);
    }
    for (int idx = tid; idx < kJB * 8; idx += 128) {
      const int r = idx >> 3, seg = idx & 7;
      *reinterpret_cast<uint4 *>(sX + r * kLdP + seg * 8) =
          *reinterpret_cast<const uint4 *>(x + ((t0 + j0 + r) * H + h) * kP + seg * 8);
    }
    if (tid < kJB) {
      sCumJ[tid] = cum[j0 + tid];
      sDtJ[tid] = dt[(t0 + j0 + tid) * H + h];
    }
    __syncthreads();

    // G = C_i . B_j^T  (16 rows of this warp x 64 columns)
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> gacc[kJB / 16];
#pragma unroll
    for (int n = 0; n < kJB / 16; ++n) wmma::fill_fragment(gacc[n], 0.f);
#pragma unroll
    for (int k = 0; k < kN / 16; ++k) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::row_major> fa;
      wmma::load_matrix_sync(fa, sC + (warp * 16) * kLdN + k * 16, kLdN);
#pragma unroll
      for (int n = 0; n < kJB / 16; ++n) {
        wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::col_major> fb;  // B[k][j] = Bm[j][k]
        wmma::load_matrix_sync(fb, sB + (n * 16) * kLdN + k * 16, kLdN);
        wmma::mma_sync(gacc[n], fa, fb, gacc[n]);
      }
    }
#pragma unroll
    for (int n = 0; n < kJB / 16; ++n) wmma::store_matrix_sync(gw + n * 16, gacc[n], kLdG, wmma::mem_row_major);
    __syncwarp();
    // M = G * e^(cum_i - cum_j) * dt_j for j <= i, else 0; rounded to the storage dtype
    T *mw = sM + (warp * 16) * kLdP;
    for (int e = lane; e < 16 * kJB; e += 32) {
      const int r = e / kJB, col = e % kJB;
      const int gi = i0 + warp * 16 + r, gj = j0 + col;
      float m = 0.f;
      if (gj <= gi) m = gw[r * kLdG + col] * ex2((sCumI[warp * 16 + r] - sCumJ[col]) * kLog2e) * sDtJ[col];
      mw[r * kLdP + col] = to_elem<DT>(m);
    }
    __syncwarp();
    // Y += M . X_j
#pragma unroll
    for (int k = 0; k < kJB / 16; ++k) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, T, wmma::row_major> fa;
      wmma::load_matrix_sync(fa, mw + k * 16, kLdP);
#pragma unroll
      for (int n = 0; n < kP / 16; ++n) {
        wmma::fragment<wmma::matrix_b, 16, 16, 16, T, wmma::row_major> fb;  // X[j][p]
        wmma::load_matrix_sync(fb, sX + (k * 16) * kLdP + n * 16, kLdP);
        wmma::mma_sync(yacc[n], fa, fb, yacc[n]);
      }
    }
  }

  // y rows -> storage dtype -> global (rows are 64 elements = 128 bytes)
#pragma unroll
  for (int n = 0; n < kP / 16; ++n) wmma::store_matrix_sync(gw + n * 16, yacc[n], kLdG, wmma::mem_row_major);
  __syncwarp();
  for (int e = lane; e < 16 * (kP / 8); e += 32) {
    const int r = e / (kP / 8), seg = e % (kP / 8);
    const float *src = gw + r * kLdG + seg * 8;
    uint4 w;
    w.x = pack2<DT>(src[0], src[1]);
    w.y = pack2<DT>(src[2], src[3]);
    w.z = pack2<DT>(src[4], src[5]);
    w.w = pack2<DT>(src[6], src[7]);
    *reinterpret_cast<uint4 *>(y + ((t0 + i0 + warp * 16 + r) * H + h) * kP + seg * 8) = w;
  }
}

size_t k1_smem(int Q) { return (size_t)(kJB * kLdP + kJB * kLdN) * 2 + (size_t)2 * Q * sizeof(float); }
size_t k3_smem() {
  return (size_t)(2 * kJB * kLdN + kP * kLdN + 2 * kJB * kLdP) * 2 + (size_t)(kJB * kLdG + 3 * kJB) * sizeof(float);
}

template <int DT>
int launch_ssd(const void *x, const float *dt, const float *A, const void *Bm, const void *Cm, void *y,
               void *workspace, int B, int L, int H, int G, int Q, cudaStream_t st) {
  const int nc = L / Q;
  float *cum_ws = static_cast<float *>(workspace);
  float *state_ws = cum_ws + (size_t)B * H * nc * Q;
  const auto *xp = static_cast<const uint16_t *>(x);
  const auto *bp = static_cast<const uint16_t *>(Bm);
  const auto *cp = static_cast<const uint16_t *>(Cm);
  NB200_CHECK_CUDA(cudaFuncSetAttribute(ssd_chunk_scan_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)k3_smem()));
  ssd_chunk_state_kernel<DT><<<dim3(H, nc, B), 128, k1_smem(Q), st>>>(xp, dt, A, bp, cum_ws, state_ws, L, H, G, Q);
  NB200_CHECK_CUDA(cudaGetLastError());
  ssd_state_pass_kernel<<<dim3(kP * kN / 256, B * H), 256, 0, st>>>(cum_ws, state_ws, nc, Q);
  NB200_CHECK_CUDA(cudaGetLastError());
  ssd_chunk_scan_kernel<DT><<<dim3(H * (Q / kJB), nc, B), 128, k3_smem(), st>>>(
      xp, dt, bp, cp, cum_ws, state_ws, static_cast<uint16_t *>(y), L, H, G, Q);
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

bool ssd_shape_ok(int B, int L, int H, int P, int N, int G, int chunk) {
  return B > 0 && L > 0 && H > 0 && G > 0 && P == kP && N == kN && H % G == 0 &&
         (chunk == 64 || chunk == 128 || chunk == 256) && L % chunk == 0;
}

}  // namespace
}  // namespace nb200

using namespace nb200;

extern "C" size_t nb200_ssd_workspace_bytes(int B, int L, int H, int P, int N, int G, int chunk) {
  if (!ssd_shape_ok(B, L, H, P, N, G, chunk)) return 0;
  const size_t nc = L / chunk;
  return (size_t)B * H * nc * ((size_t)chunk + (size_t)P * N) * sizeof(float);
}

extern "C" int nb200_ssd_chunk_scan_fwd(const void *x, const float *dt, const float *A, const void *Bm,
                                        const void *Cm, void *y, void *workspace, int B, int L, int H, int P,
                                        int N, int G, int chunk, int dtype, void *stream) {
  NB200_REQUIRE(x && dt && A && Bm && Cm && y && workspace, NB200_ERR_BAD_ARG, "ssd_chunk_scan: null pointer");
  NB200_REQUIRE(B > 0 && L > 0 && H > 0 && G > 0, NB200_ERR_BAD_ARG, "ssd_chunk_scan: non-positive extent");
  NB200_REQUIRE(ssd_shape_ok(B, L, H, P, N, G, chunk), NB200_ERR_UNSUPPORTED,
                "ssd_chunk_scan: need P == 64, N == 128, H %% G == 0, chunk in {64,128,256}, L %% chunk == 0");
  NB200_REQUIRE(aligned16(x) && aligned16(Bm) && aligned16(Cm) && aligned16(y) &&
                    (reinterpret_cast<uintptr_t>(workspace) & 31u) == 0,
                NB200_ERR_BAD_ARG, "ssd_chunk_scan: tensors must be 16-byte and the workspace 32-byte aligned");
  NB200_REQUIRE(B <= 65535 && L / chunk <= 65535, NB200_ERR_UNSUPPORTED, "ssd_chunk_scan: grid too large");
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == NB200_BF16) return launch_ssd<NB200_BF16>(x, dt, A, Bm, Cm, y, workspace, B, L, H, G, chunk, st);
  if (dtype == NB200_F16) return launch_ssd<NB200_F16>(x, dt, A, Bm, Cm, y, workspace, B, L, H, G, chunk, st);
  return fail(NB200_ERR_UNSUPPORTED, "ssd_chunk_scan: dtype %d (f16 and bf16 only)", dtype);
}
