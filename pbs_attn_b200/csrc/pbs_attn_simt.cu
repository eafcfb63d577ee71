// Stage 3b, generic kernel: block-sparse causal flash-attention forward on CUDA cores.
//
// Same math as the reference's Triton kernel (pbs_attn/src/kernels/permuted_block_sparse_attention.py
// :7-90,241-311): fp32 scores scaled by 1/sqrt(D), key visible iff its original position <= the
// query's, online softmax in base 2, probabilities rounded to the input dtype before P.V, fp32
// accumulators, output = acc / row sum.  It takes any dtype / block size / head dim the library
// accepts and is the path for shapes the tcgen05 kernel does not cover (fp32 inputs, head dims other
// than 64/128, block sizes other than 64/128); it also serves as an on-device cross-check of the
// tcgen05 kernel in the tests.  One CTA per (32-row query tile, b, h); the block mask row of the
// tile's query block decides which 32-key tiles are visited.
#include "pbs_common.cuh"

namespace pbs {
namespace {

constexpr int BM = 32;        // query rows per CTA
constexpr int BN = 32;        // keys per step
constexpr int NT = 128;       // threads: 4 per query row

template <int DT>
__global__ void __launch_bounds__(NT)
attn_simt_kernel(const typename Elem<DT>::T* __restrict__ q, Strides qs,
                 const typename Elem<DT>::T* __restrict__ pk, const typename Elem<DT>::T* __restrict__ pv,
                 const int32_t* __restrict__ idx, const uint8_t* __restrict__ mask,
                 typename Elem<DT>::T* __restrict__ out, Strides os,
                 int Hq, int S, int D, int bs, int nb, int tile, float scale_log2e) {
  using E = Elem<DT>;
  using T = typename E::T;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                       // [BM][D]
  float* Ks = Qs + BM * D;              // [BN][D + 1]
  float* Vs = Ks + BN * (D + 1);        // [BN][D]
  float* Ps = Vs + BN * D;              // [BM][BN + 1]
  __shared__ int kidx[BN];

  const int r0 = blockIdx.x * tile;     // `tile` <= BM rows are live (tile divides the block size)
  const int bh = blockIdx.y;
  const int b = bh / Hq, h = bh % Hq;
  const int qb = r0 / bs;
  const uint8_t* mrow = mask + ((int64_t)bh * nb + qb) * nb;
  const T* qbase = q + (int64_t)b * qs.b + (int64_t)h * qs.h;
  const T* kbase = pk + (int64_t)bh * S * D;
  const T* vbase = pv + (int64_t)bh * S * D;
  const int32_t* ibase = idx + (int64_t)bh * S;

  const int row = threadIdx.x >> 2;     // 0..31
  const int sub = threadIdx.x & 3;      // 4 threads per row
  const int qpos = r0 + row;
  const bool row_live = row < tile && qpos < S;

  for (int i = threadIdx.x; i < BM * D; i += NT) {
    const int r = i / D, d = i % D;
    Qs[i] = (r < tile && r0 + r < S) ? E::ld(qbase + (int64_t)(r0 + r) * qs.s + d) : 0.f;
  }

  const int nacc = D / 4;               // output columns sub, sub+4, ... of this thread's row
  float acc[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) acc[i] = 0.f;
  float m_run = -CUDART_INF_F, l_run = 0.f;

  const int kv_tiles_per_block = bs / tile;
  for (int kb = 0; kb < nb; ++kb) {
    if (!mrow[kb]) continue;
    for (int sub_t = 0; sub_t < kv_tiles_per_block; ++sub_t) {
      const int k0 = kb * bs + sub_t * tile;
      if (k0 >= S) break;
      __syncthreads();
      for (int i = threadIdx.x; i < BN * D; i += NT) {
        const int r = i / D, d = i % D;
        const bool live = r < tile && k0 + r < S;
        Ks[r * (D + 1) + d] = live ? E::ld(kbase + (int64_t)(k0 + r) * D + d) : 0.f;
        Vs[r * D + d] = live ? E::ld(vbase + (int64_t)(k0 + r) * D + d) : 0.f;
      }
      if (threadIdx.x < BN) {
        const int r = threadIdx.x;
        kidx[r] = (r < tile && k0 + r < S) ? ibase[k0 + r] : 0x7fffffff;
      }
      __syncthreads();
      // scores of this thread: keys sub*8 .. sub*8+7 of its row
      float s[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] = 0.f;
      const float* qr = Qs + row * D;
      for (int d = 0; d < D; ++d) {
        const float qv = qr[d];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] = fmaf(qv, Ks[(sub * 8 + j) * (D + 1) + d], s[j]);
      }
      float m_tile = -CUDART_INF_F;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool vis = row_live && kidx[sub * 8 + j] <= qpos;
        s[j] = vis ? s[j] * scale_log2e : -CUDART_INF_F;
        m_tile = fmaxf(m_tile, s[j]);
      }
      m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
      m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
      const float m_new = fmaxf(m_run, m_tile);
      const float alpha = (m_new == -CUDART_INF_F) ? 1.f : exp2f(m_run - m_new);
      float l_tile = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float p = (m_new == -CUDART_INF_F) ? 0.f : exp2f(s[j] - m_new);
        l_tile += p;
        Ps[row * (BN + 1) + sub * 8 + j] = E::rnd(p);
      }
      l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 1);
      l_tile += __shfl_xor_sync(0xffffffffu, l_tile, 2);
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      __syncwarp();                     // the 4 threads of a row share a warp
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (i < nacc) acc[i] *= alpha;
      for (int kk = 0; kk < BN; ++kk) {
        const float p = Ps[row * (BN + 1) + kk];
        const float* vr = Vs + kk * D + sub;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i < nacc) acc[i] = fmaf(p, vr[4 * i], acc[i]);
      }
    }
  }
  if (row_live) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    T* orow = out + (int64_t)b * os.b + (int64_t)h * os.h + (int64_t)qpos * os.s;
#pragma unroll
    for (int i = 0; i < 64; ++i)
      if (i < nacc) orow[sub + 4 * i] = E::cvt(acc[i] * inv);
  }
}

}  // namespace

int launch_attn_simt(const Dims& d, int dt, const void* q, Strides qs, const void* pk, const void* pv,
                     const int32_t* idx, const uint8_t* mask, void* out, Strides os, cudaStream_t st) {
  const int tile = (d.bs % 32 == 0) ? 32 : 16;
  const size_t smem = sizeof(float) * ((size_t)BM * d.D + (size_t)BN * (d.D + 1) + (size_t)BN * d.D + (size_t)BM * (BN + 1));
  const float scale = (float)(1.4426950408889634 / sqrt((double)d.D));
  dim3 grid((d.S + tile - 1) / tile, d.B * d.Hq);
#define PBS_SIMT(DT, TT)                                                                                  \
  {                                                                                                       \
    auto kern = attn_simt_kernel<DT>;                                                                     \
    if (smem > 48 * 1024) {                                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return cuda_fail(e, "attn_simt_kernel smem attribute");                       \
    }                                                                                                     \
    kern<<<grid, NT, smem, st>>>((const TT*)q, qs, (const TT*)pk, (const TT*)pv, idx, mask, (TT*)out, os, \
                                 d.Hq, d.S, d.D, d.bs, d.nb, tile, scale);                                \
  }
  switch (dt) {
    case PBS_BF16: PBS_SIMT(PBS_BF16, __nv_bfloat16) break;
    case PBS_FP16: PBS_SIMT(PBS_FP16, __half) break;
    default: PBS_SIMT(PBS_FP32, float)
  }
#undef PBS_SIMT
  PBS_CUDA_CHECK_LAUNCH("attn_simt_kernel");
  return PBS_OK;
}

}  // namespace pbs
