// Exact-fp32 attention forward on CUDA cores.
//
// Serves the shapes the tensor-core kernel does not: fp32 storage (whose 1e-4 tolerance rules out
// reduced-precision MMA inputs), head dimensions other than 128 and sequence lengths that are not
// multiples of 128.  These are correctness-class problems (tens of MFLOP), so the kernel favours a
// simple mapping: one warp per query row, 32 keys per step (one key per lane for the scores, one
// slice of the head dimension per lane for the PV product), online softmax in the exp2 domain as
// in the HTile program (tests/data/flash_attention_htile.mlir:40-128 of the reference).
#include "nb200_common.cuh"

namespace nb200 {
namespace {

constexpr int kSimtWarps = 4;
constexpr int kMaxD = 256;

template <int DT>
__global__ void __launch_bounds__(kSimtWarps * 32)
attn_simt_kernel(const void *__restrict__ q, const void *__restrict__ k, const void *__restrict__ v,
                 void *__restrict__ out, int Sq, int Skv, int D, float scale_log2, int causal) {
  __shared__ float sq[kSimtWarps][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kSimtWarps + warp;
  const size_t bh = blockIdx.y;
  if (row >= Sq) return;  // whole warp leaves together; no block-wide barrier follows

  const size_t qoff = (bh * Sq + row) * (size_t)D;
  for (int d = lane; d < D; d += 32) sq[warp][d] = load1<DT>(q, qoff + d) * scale_log2;
  __syncwarp();

  const int nd = D / 32;  // output elements per lane (D is a multiple of 32)
  float o[kMaxD / 32];
#pragma unroll
  for (int i = 0; i < kMaxD / 32; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int last = causal ? min(Skv - 1, row + (Skv - Sq)) : Skv - 1;  // last visible key

  for (int j0 = 0; j0 <= last; j0 += 32) {
    const int j = j0 + lane;
    float s = -INFINITY;
    if (j <= last) {
      const size_t koff = (bh * Skv + j) * (size_t)D;
      float acc = 0.f;
      for (int d = 0; d < D; ++d) acc = fmaf(sq[warp][d], load1<DT>(k, koff + d), acc);
      s = acc;
    }
    float mb = s;
#pragma unroll
    for (int x = 16; x > 0; x >>= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, x));
    const float m_new = fmaxf(m, mb);  // finite: key j0 is always visible
    const float alpha = exp2f(m - m_new);
    const float p = exp2f(s - m_new);
    float ps = p;
#pragma unroll
    for (int x = 16; x > 0; x >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, x);
    l = l * alpha + ps;
    m = m_new;
#pragma unroll
    for (int i = 0; i < kMaxD / 32; ++i) o[i] *= alpha;
    const int nj = min(32, last - j0 + 1);
    for (int jj = 0; jj < nj; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const size_t voff = (bh * Skv + j0 + jj) * (size_t)D;
#pragma unroll
      for (int i = 0; i < kMaxD / 32; ++i)
        if (i < nd) o[i] = fmaf(pj, load1<DT>(v, voff + lane + 32 * i), o[i]);
    }
  }
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < kMaxD / 32; ++i)
    if (i < nd) store1<DT>(out, qoff + lane + 32 * i, o[i] * inv);
}

}  // namespace

int attn_simt_launch(const void *q, const void *k, const void *v, void *out, int B, int H, int Sq, int Skv,
                     int D, int dtype, float scale_log2, int causal, cudaStream_t st) {
  NB200_REQUIRE(D % 32 == 0 && D <= kMaxD, NB200_ERR_UNSUPPORTED,
                "attn_fwd: head dimension %d (need a multiple of 32, at most %d)", D, kMaxD);
  NB200_REQUIRE((long long)B * H <= 65535, NB200_ERR_UNSUPPORTED, "attn_fwd: B*H too large for the SIMT kernel");
  const dim3 grid((Sq + kSimtWarps - 1) / kSimtWarps, B * H), block(kSimtWarps * 32);
  switch (dtype) {
    case NB200_F32: attn_simt_kernel<NB200_F32><<<grid, block, 0, st>>>(q, k, v, out, Sq, Skv, D, scale_log2, causal); break;
    case NB200_F16: attn_simt_kernel<NB200_F16><<<grid, block, 0, st>>>(q, k, v, out, Sq, Skv, D, scale_log2, causal); break;
    case NB200_BF16: attn_simt_kernel<NB200_BF16><<<grid, block, 0, st>>>(q, k, v, out, Sq, Skv, D, scale_log2, causal); break;
    default: return fail(NB200_ERR_UNSUPPORTED, "attn_fwd: dtype %d", dtype);
  }
  NB200_CHECK_CUDA(cudaGetLastError());
  return NB200_OK;
}

}  // namespace nb200
