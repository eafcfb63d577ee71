// Stage 1a: per-key importance = mean over the last query block of softmax(q . k / sqrt(D)).
//
// Follows pbs_attn/src/permute_states.py:44-50 of the reference: the logits are produced in the
// input dtype (fp32 accumulate, rounded once after the dot product and once after the division by
// sqrt(D)), the softmax runs in fp32 over all keys of the complete segments, and the mean over the
// block's query rows is an fp32 sum in the reference's summation order.
//
// Three kernels:
//   logits_kernel     (L/64 x B*Hq CTAs)  logits tile -> scratch, per-tile row max / sum(exp)
//   rowstats_kernel   (B*Hq CTAs)         merges the per-tile statistics into one (max, sum) per row
//   importance_kernel (L/256 x B*Hq CTAs) mean_r exp(logit - max_r) / sum_r
// HBM traffic per (b, h): K read once (L*D*e), logits written once and read once (2*bs*L*e),
// importance written once (4*L).
#include "pbs_common.cuh"

namespace pbs {
namespace {

constexpr int TM = 64;   // query rows per pass
constexpr int TN = 64;   // keys per CTA
constexpr int KC = 32;   // head-dim chunk staged in shared memory
constexpr int LDT = TM + 4;

template <int DT>
__global__ void __launch_bounds__(256)
logits_kernel(const typename Elem<DT>::T* __restrict__ q, Strides qs,
              const typename Elem<DT>::T* __restrict__ k, Strides ks,
              typename Elem<DT>::T* __restrict__ logits, float2* __restrict__ partials,
              int Hq, int group, int S, int D, int bs, int L, float sqrt_d) {
  using E = Elem<DT>;
  using T = typename E::T;
  __shared__ __align__(16) float Qs[KC][LDT];
  __shared__ __align__(16) float Ks[KC][LDT];

  const int jt = blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / Hq, h = bh % Hq;
  const int ntile = gridDim.x;
  const T* qbase = q + (int64_t)b * qs.b + (int64_t)h * qs.h + (int64_t)(S - bs) * qs.s;
  const T* kbase = k + (int64_t)b * ks.b + (int64_t)(h / group) * ks.h + (int64_t)jt * TN * ks.s;
  const int nkeys = min(TN, L - jt * TN);

  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int lrow = threadIdx.x >> 2;          // row / key this thread stages
  const int lcol = (threadIdx.x & 3) * 8;     // first of its 8 head-dim elements

  for (int r0 = 0; r0 < bs; r0 += TM) {
    const int nrows = min(TM, bs - r0);
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int d0 = 0; d0 < D; d0 += KC) {
      __syncthreads();
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int d = d0 + lcol + e;
        float qv = 0.f, kv = 0.f;
        if (d < D) {
          if (lrow < nrows) qv = E::ld(qbase + (int64_t)(r0 + lrow) * qs.s + d);
          if (lrow < nkeys) kv = E::ld(kbase + (int64_t)lrow * ks.s + d);
        }
        Qs[lcol + e][lrow] = qv;
        Ks[lcol + e][lrow] = kv;
      }
      __syncthreads();
#pragma unroll
      for (int d = 0; d < KC; ++d) {
        const float4 a = *reinterpret_cast<const float4*>(&Qs[d][ty * 4]);
        const float4 c = *reinterpret_cast<const float4*>(&Ks[d][tx * 4]);
        const float av[4] = {a.x, a.y, a.z, a.w};
        const float cv[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], cv[j], acc[i][j]);
      }
    }

    // round like the reference, store, and reduce the tile's row statistics
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + ty * 4 + i;
      float y[4];
      float m = -CUDART_INF_F;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        y[j] = E::rnd(E::rnd(acc[i][j]) / sqrt_d);
        if (tx * 4 + j < nkeys) m = fmaxf(m, y[j]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      float z = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (tx * 4 + j < nkeys) z += expf(y[j] - m);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
      if (r < bs) {
        T* dst = logits + ((int64_t)bh * bs + r) * L + (int64_t)jt * TN + tx * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (tx * 4 + j < nkeys) dst[j] = E::cvt(y[j]);
        if (tx == 0) partials[((int64_t)bh * ntile + jt) * bs + r] = make_float2(m, z);
      }
    }
  }
}

__global__ void rowstats_kernel(const float2* __restrict__ partials, float2* __restrict__ rowstats,
                                int ntile, int bs) {
  const int bh = blockIdx.x;
  const int r = threadIdx.x;
  if (r >= bs) return;
  const float2* p = partials + (int64_t)bh * ntile * bs + r;
  float m = -CUDART_INF_F;
  for (int t = 0; t < ntile; ++t) m = fmaxf(m, p[(int64_t)t * bs].x);
  float z = 0.f;
  for (int t = 0; t < ntile; ++t) {
    const float2 v = p[(int64_t)t * bs];
    z += v.y * expf(v.x - m);
  }
  rowstats[(int64_t)bh * bs + r] = make_float2(m, z);
}

template <int DT>
__global__ void __launch_bounds__(256)
importance_kernel(const typename Elem<DT>::T* __restrict__ logits, const float2* __restrict__ rowstats,
                  float* __restrict__ importance, int bs, int L) {
  using E = Elem<DT>;
  extern __shared__ float2 stats[];
  const int bh = blockIdx.y;
  for (int r = threadIdx.x; r < bs; r += blockDim.x) stats[r] = rowstats[(int64_t)bh * bs + r];
  __syncthreads();
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= L) return;
  const typename E::T* col = logits + (int64_t)bh * bs * L + j;
  CascadeSum sum;
  for (int r = 0; r < bs; ++r) {
    const float2 st = stats[r];
    sum.add(expf(E::ld(col + (int64_t)r * L) - st.x) / st.y);
  }
  importance[(int64_t)bh * L + j] = sum.total() / (float)bs;
}

template <int DT>
int run(const Dims& d, const void* q, Strides qs, const void* k, Strides ks, void* logits, void* partials,
        void* rowstats, float* importance, cudaStream_t st) {
  using T = typename Elem<DT>::T;
  const int BH = d.B * d.Hq;
  const int ntile = (d.L + TN - 1) / TN;
  logits_kernel<DT><<<dim3(ntile, BH), 256, 0, st>>>(
      (const T*)q, qs, (const T*)k, ks, (T*)logits, (float2*)partials, d.Hq, d.group, d.S, d.D, d.bs, d.L,
      (float)sqrt((double)d.D));
  PBS_CUDA_CHECK_LAUNCH("logits_kernel");
  rowstats_kernel<<<BH, ((d.bs + 31) / 32) * 32, 0, st>>>((const float2*)partials, (float2*)rowstats, ntile, d.bs);
  PBS_CUDA_CHECK_LAUNCH("rowstats_kernel");
  importance_kernel<DT><<<dim3((d.L + 255) / 256, BH), 256, d.bs * sizeof(float2), st>>>(
      (const T*)logits, (const float2*)rowstats, importance, d.bs, d.L);
  PBS_CUDA_CHECK_LAUNCH("importance_kernel");
  return PBS_OK;
}

}  // namespace

int launch_key_importance(const Dims& d, int dt, const void* q, Strides qs, const void* k, Strides ks,
                          void* logits, void* partials, void* rowstats, float* importance, cudaStream_t st) {
  if (d.L == 0) return PBS_OK;
  switch (dt) {
    case PBS_BF16: return run<PBS_BF16>(d, q, qs, k, ks, logits, partials, rowstats, importance, st);
    case PBS_FP16: return run<PBS_FP16>(d, q, qs, k, ks, logits, partials, rowstats, importance, st);
    default: return run<PBS_FP32>(d, q, qs, k, ks, logits, partials, rowstats, importance, st);
  }
}

}  // namespace pbs
