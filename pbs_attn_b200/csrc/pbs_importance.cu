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
constexpr int kMmaTilesPerCta = 4;   // 64-key tiles per CTA of the tensor-core logits kernel
constexpr int kStageLd = TN + 8;     // elements per row of the per-warp output staging tile

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

// Tensor-core variant of logits_kernel for 16-bit inputs (mma.sync m16n8k16, fp32 accumulate: the
// products of 16-bit values are exact and the sum is rounded like any fp32 GEMM).  One CTA = 64 keys x
// all query rows of the last block (128 per pass); warp w owns rows 16w..16w+15 of the pass.  Q and K
// tiles sit in shared memory with 16 bytes of padding per row so ldmatrix is conflict free.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <int DT>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (DT == PBS_BF16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int DT>
__global__ void __launch_bounds__(256)
logits_mma_kernel(const typename Elem<DT>::T* __restrict__ q, Strides qs,
                  const typename Elem<DT>::T* __restrict__ k, Strides ks,
                  typename Elem<DT>::T* __restrict__ logits, float2* __restrict__ partials,
                  int Hq, int group, int S, int D, int bs, int L, int ntile, float sqrt_d) {
  using E = Elem<DT>;
  using T = typename E::T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int ld = D + 8;                                    // padded row length in elements
  T* Qs = reinterpret_cast<T*>(smem_raw);                  // [128][ld]
  T* Ks = Qs + 128 * ld;                                   // [64][ld]
  T* stage = Ks + TN * ld;                                 // [8 warps][16 rows][kStageLd]

  const int bh = blockIdx.y;
  const int b = bh / Hq, h = bh % Hq;
  const T* qbase = q + (int64_t)b * qs.b + (int64_t)h * qs.h + (int64_t)(S - bs) * qs.s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cpr = D / 8;                                   // 16-byte chunks per row

  // The query rows are staged once per pass and reused for kMmaTilesPerCta key tiles.
  for (int r0 = 0; r0 < bs; r0 += 128) {
    const int nrows = min(128, bs - r0);
    __syncthreads();
    for (int i = threadIdx.x; i < 128 * cpr; i += blockDim.x) {
      const int r = i / cpr, c = i % cpr;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < nrows) val = *reinterpret_cast<const uint4*>(qbase + (int64_t)(r0 + r) * qs.s + c * 8);
      *reinterpret_cast<uint4*>(Qs + r * ld + c * 8) = val;
    }
   for (int it = 0; it < kMmaTilesPerCta; ++it) {
    const int jt = blockIdx.x * kMmaTilesPerCta + it;
    if (jt >= ntile) break;
    const T* kbase = k + (int64_t)b * ks.b + (int64_t)(h / group) * ks.h + (int64_t)jt * TN * ks.s;
    const int nkeys = min(TN, L - jt * TN);
    __syncthreads();                                       // previous tile's K fully consumed
    for (int i = threadIdx.x; i < TN * cpr; i += blockDim.x) {
      const int r = i / cpr, c = i % cpr;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (r < nkeys) val = *reinterpret_cast<const uint4*>(kbase + (int64_t)r * ks.s + c * 8);
      *reinterpret_cast<uint4*>(Ks + r * ld + c * 8) = val;
    }
    __syncthreads();
    if (warp * 16 < nrows) {
      float acc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int t = 0; t < 4; ++t) acc[j][t] = 0.f;
      const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs + (warp * 16 + (lane & 15)) * ld + (lane >> 4) * 8);
      const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(Ks + ((lane >> 4) * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
      for (int d0 = 0; d0 < D; d0 += 16) {
        uint32_t a[4];
        ldmatrix_x4(a, q_addr + d0 * 2);
#pragma unroll
        for (int jp = 0; jp < 4; ++jp) {                   // two 8-key tiles per ldmatrix
          uint32_t bq[4];
          ldmatrix_x4(bq, k_addr + (jp * 16 * ld + d0) * 2);
          mma_16816<DT>(acc[2 * jp], a, bq[0], bq[1]);
          mma_16816<DT>(acc[2 * jp + 1], a, bq[2], bq[3]);
        }
      }
      // this thread: rows lane/4 and lane/4 + 8 of the warp's 16, keys 8j + 2(lane%4), +1
      const bool full = nkeys == TN;
      const float rinv = 1.f / sqrt_d;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = r0 + warp * 16 + (lane >> 2) + 8 * half;
        float y[16];
        float m = -CUDART_INF_F;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            // a / sqrt_d in fp32: reciprocal product corrected by one exact-remainder step, which
            // gives the correctly rounded quotient; then the second rounding to the input type
            const float a = E::rnd(acc[j][2 * half + t]);
            float qv = a * rinv;
            qv = fmaf(fmaf(-qv, sqrt_d, a), rinv, qv);
            y[2 * j + t] = E::rnd(qv);
            if (full || 8 * j + 2 * (lane & 3) + t < nkeys) m = fmaxf(m, y[2 * j + t]);
          }
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        float z = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (full || 8 * j + 2 * (lane & 3) + t < nkeys) z += __expf(y[2 * j + t] - m);
        z += __shfl_xor_sync(0xffffffffu, z, 1);
        z += __shfl_xor_sync(0xffffffffu, z, 2);
        // the rounded logits go through a per-warp staging tile (rows padded by 8 elements, which
        // spreads the eight rows of a store over all banks) and leave as 16-byte pieces
        T* srow = stage + (warp * 16 + (lane >> 2) + 8 * half) * kStageLd;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          T pair[2] = {E::cvt(y[2 * j]), E::cvt(y[2 * j + 1])};
          *reinterpret_cast<uint32_t*>(srow + 8 * j + 2 * (lane & 3)) = *reinterpret_cast<const uint32_t*>(pair);
        }
        if (r < bs && (lane & 3) == 0) partials[((int64_t)bh * ntile + jt) * bs + r] = make_float2(m, z);
      }
      __syncwarp();
      if (full) {
        // four rows per store instruction: 8 lanes x 16 bytes cover the 64 keys of a row
#pragma unroll
        for (int rr = 0; rr < 16; rr += 4) {
          const int lr = rr + (lane >> 3);
          const int r = r0 + warp * 16 + lr;
          if (r < bs) {
            T* dst = logits + ((int64_t)bh * bs + r) * L + (int64_t)jt * TN + (lane & 7) * 8;
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(stage + (warp * 16 + lr) * kStageLd + (lane & 7) * 8);
          }
        }
      } else {
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const int r = r0 + warp * 16 + rr;
          if (r < bs && 2 * lane < nkeys) {
            T* dst = logits + ((int64_t)bh * bs + r) * L + (int64_t)jt * TN;
            *reinterpret_cast<uint32_t*>(dst + 2 * lane) = *reinterpret_cast<const uint32_t*>(stage + (warp * 16 + rr) * kStageLd + 2 * lane);
          }
        }
      }
      __syncwarp();
    }
   }
  }
}

// One warp per (b, h, row): lanes stride the key tiles, each merging its (max, sum) pairs online,
// then the 32 partial pairs are merged by shuffles.
__global__ void __launch_bounds__(256)
rowstats_kernel(const float2* __restrict__ partials, float2* __restrict__ rowstats, int ntile, int bs) {
  const int bh = blockIdx.y;
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= bs) return;
  const float2* p = partials + (int64_t)bh * ntile * bs + r;
  float m = -CUDART_INF_F, z = 0.f;
  for (int t = lane; t < ntile; t += 32) {
    const float2 v = p[(int64_t)t * bs];
    const float mn = fmaxf(m, v.x);
    z = z * expf(m - mn) + v.y * expf(v.x - mn);
    m = mn;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float mo = __shfl_xor_sync(0xffffffffu, m, o);
    const float zo = __shfl_xor_sync(0xffffffffu, z, o);
    const float mn = fmaxf(m, mo);
    const float a = (m == -CUDART_INF_F) ? 0.f : z * expf(m - mn);
    const float c = (mo == -CUDART_INF_F) ? 0.f : zo * expf(mo - mn);
    z = a + c;
    m = mn;
  }
  if (lane == 0) rowstats[(int64_t)bh * bs + r] = make_float2(m, z);
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
  int r = 0;
  for (; r + 8 <= bs; r += 8) {                      // eight loads in flight per thread
    float y[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) y[u] = E::ld(col + (int64_t)(r + u) * L);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float2 st = stats[r + u];
      sum.add(expf(y[u] - st.x) / st.y);
    }
  }
  for (; r < bs; ++r) {
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
  const float sq = (float)sqrt((double)d.D);
  if (DT != PBS_FP32 && d.D % 16 == 0 && qs.s % 8 == 0 && ks.s % 8 == 0) {
    // 16-bit inputs: tensor cores
    auto kern = logits_mma_kernel<DT>;
    const size_t smem = ((size_t)(128 + TN) * (d.D + 8) + 8 * 16 * kStageLd) * sizeof(T);
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cuda_fail(e, "logits_mma_kernel smem attribute");
    }
    kern<<<dim3((ntile + kMmaTilesPerCta - 1) / kMmaTilesPerCta, BH), 256, smem, st>>>(
        (const T*)q, qs, (const T*)k, ks, (T*)logits, (float2*)partials, d.Hq, d.group, d.S, d.D, d.bs, d.L, ntile, sq);
    PBS_CUDA_CHECK_LAUNCH("logits_mma_kernel");
  } else {
    logits_kernel<DT><<<dim3(ntile, BH), 256, 0, st>>>(
        (const T*)q, qs, (const T*)k, ks, (T*)logits, (float2*)partials, d.Hq, d.group, d.S, d.D, d.bs, d.L, sq);
    PBS_CUDA_CHECK_LAUNCH("logits_kernel");
  }
  rowstats_kernel<<<dim3((d.bs + 7) / 8, BH), 256, 0, st>>>((const float2*)partials, (float2*)rowstats, ntile, d.bs);
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
