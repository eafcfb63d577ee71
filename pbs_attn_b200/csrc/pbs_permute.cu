// Stage 1b: per-segment stable descending sort of the key importance, gather of K and V rows into
// permuted order, pooling of the permuted K per block, and the block that holds original token 0.
//
// Follows pbs_attn/src/permute_states.py:52-83 (argsort per segment, gather, tail left in place),
// pbs_attn/src/pbs.py:213-215 (V gathered with the K permutation), pbs_attn/src/utils.py:24-27 with
// the zero padding of pbs_attn/src/pbs.py:78-80 (key pooling) and pbs_attn/src/pbs.py:10-25.
// Ties are broken towards the lower original position (a stable sort).
//
// One CTA per (segment, b, h); the heads of a KV group are adjacent in the grid.  HBM traffic per (b, h):
// importance read (4*L), K and V rows read (from L2 for all but one of the Hq/Hkv heads that share a KV
// head) and written once each (2*S*D*e), indices written (4*S), pooled K written (nb*D*e).
#include "pbs_common.cuh"

namespace pbs {
namespace {

template <int DT>
__global__ void __launch_bounds__(256)
segment_permute_kernel(const float* __restrict__ importance,
                       const typename Elem<DT>::T* __restrict__ k, Strides ks,
                       const typename Elem<DT>::T* __restrict__ v, Strides vs,
                       int32_t* __restrict__ idx_out,
                       typename Elem<DT>::T* __restrict__ perm_k, typename Elem<DT>::T* __restrict__ perm_v,
                       typename Elem<DT>::T* __restrict__ pooled_k, int pool_mode,
                       int32_t* __restrict__ first_block,
                       int Hq, int group, int S, int D, int bs, int seg, int nseg, int nb, int npow2) {
  using E = Elem<DT>;
  using T = typename E::T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem_raw);
  int32_t* order = reinterpret_cast<int32_t*>(keys + npow2);   // original position of each slot

  // the query heads of a KV group sit next to each other in the grid: they gather the same K/V rows,
  // which then come from HBM once and from L2 for the others
  const int sg = blockIdx.x / group, hin = blockIdx.x % group;
  const int Hkv = Hq / group;
  const int b = blockIdx.y / Hkv, h = (blockIdx.y % Hkv) * group + hin;
  const int bh = b * Hq + h;
  const int seg0 = sg * seg;
  const int n = min(seg, S - seg0);        // rows of this segment (the tail segment is shorter)
  const int L = nseg * seg;

  if (sg < nseg) {
    const float* imp = importance + (int64_t)bh * L + seg0;
    for (int i = threadIdx.x; i < npow2; i += blockDim.x) {
      unsigned long long key = 0ull;       // padding sorts last
      if (i < seg) key = ((unsigned long long)float_order_key(imp[i]) << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i);
      keys[i] = key;
    }
    __syncthreads();
    // 256 threads: up to 4 keys per thread sort in registers and shuffles, larger segments in shared memory
    if (npow2 <= 256) bitonic_sort_desc_regs<1>(keys, npow2);
    else if (npow2 == 512) bitonic_sort_desc_regs<2>(keys, npow2);
    else if (npow2 == 1024) bitonic_sort_desc_regs<4>(keys, npow2);
    else bitonic_sort_desc(keys, npow2);
    for (int i = threadIdx.x; i < seg; i += blockDim.x)
      order[i] = seg0 + (int32_t)(0xFFFFFFFFu - (uint32_t)(keys[i] & 0xFFFFFFFFull));
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) order[i] = seg0 + i;
  }
  __syncthreads();

  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int src = order[i];
    idx_out[(int64_t)bh * S + seg0 + i] = src;
    if (src == 0) first_block[bh] = (seg0 + i) / bs;
  }

  // gather rows: 16-byte chunks, one row per group of `cpr` threads
  const int cpr = D * (int)sizeof(T) / 16;
  const int rows_per_pass = blockDim.x / cpr;
  const int c = threadIdx.x % cpr;
  const T* kb = k + (int64_t)b * ks.b + (int64_t)(h / group) * ks.h;
  const T* vb = v + (int64_t)b * vs.b + (int64_t)(h / group) * vs.h;
  T* pk = perm_k + ((int64_t)bh * S + seg0) * D;
  T* pv = perm_v + ((int64_t)bh * S + seg0) * D;
  if (threadIdx.x < rows_per_pass * cpr) {
    for (int i = threadIdx.x / cpr; i < n; i += rows_per_pass) {
      const int src = order[i];
      const uint4 kq = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(kb + (int64_t)src * ks.s) + c * 16);
      const uint4 vq = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(vb + (int64_t)src * vs.s) + c * 16);
      *reinterpret_cast<uint4*>(reinterpret_cast<char*>(pk + (int64_t)i * D) + c * 16) = kq;
      *reinterpret_cast<uint4*>(reinterpret_cast<char*>(pv + (int64_t)i * D) + c * 16) = vq;
    }
  }

  // pooled K of each block of the segment, rows taken in permuted order
  const int nblk = (n + bs - 1) / bs;
  for (int t = threadIdx.x; t < nblk * D; t += blockDim.x) {
    const int blk = t / D, d = t % D;
    const int r0 = blk * bs, r1 = min(r0 + bs, n);
    float res;
    if (pool_mode == PBS_POOL_MEAN) {
      CascadeSum sum;
      for (int r = r0; r < r1; ++r) sum.add(E::ld(kb + (int64_t)order[r] * ks.s + d));
      res = sum.total() / (float)bs;
    } else {
      float m = (r1 - r0 < bs) ? 0.f : -CUDART_INF_F;    // zero padding takes part in the max
      for (int r = r0; r < r1; ++r) m = fmaxf(m, E::ld(kb + (int64_t)order[r] * ks.s + d));
      res = m;
    }
    pooled_k[((int64_t)bh * nb + seg0 / bs + blk) * D + d] = E::cvt(res);
  }
}

// One CTA per (q block, b, h).  A thread owns one 16-row group x one 16-byte piece of the row: its 16
// loads are independent (all in flight at once), its sums follow the reference's reduction order (rows
// one after the other inside a group of 16); a second step adds the group sums in order.
template <int DT>
__global__ void __launch_bounds__(256)
pool_queries_kernel(const typename Elem<DT>::T* __restrict__ q, Strides qs,
                    typename Elem<DT>::T* __restrict__ pooled_q, int pool_mode,
                    int Hq, int S, int D, int bs, int nb) {
  using E = Elem<DT>;
  using T = typename E::T;
  constexpr int EPV = 16 / (int)sizeof(T);
  __shared__ float part[16 * 256];                         // [16-row group][dim]
  const int blk = blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / Hq, h = bh % Hq;
  const T* qb = q + (int64_t)b * qs.b + (int64_t)h * qs.h;
  const int r0 = blk * bs, r1 = min(r0 + bs, S);
  const int groups = bs / 16, cpr = D / EPV;
  const bool mean = pool_mode == PBS_POOL_MEAN;
  for (int i = threadIdx.x; i < groups * cpr; i += blockDim.x) {
    const int g = i / cpr, c = i % cpr;
    const int g0 = r0 + 16 * g, n = max(0, min(16, r1 - g0));
    uint4 raw[16];
#pragma unroll
    for (int rr = 0; rr < 16; ++rr)
      if (rr < n) raw[rr] = *reinterpret_cast<const uint4*>(qb + (int64_t)(g0 + rr) * qs.s + c * EPV);
    float acc[EPV];
#pragma unroll
    for (int t = 0; t < EPV; ++t) acc[t] = mean ? 0.f : -CUDART_INF_F;
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) {
      if (rr < n) {
        const T* e = reinterpret_cast<const T*>(&raw[rr]);
#pragma unroll
        for (int t = 0; t < EPV; ++t) acc[t] = mean ? acc[t] + E::ld(e + t) : fmaxf(acc[t], E::ld(e + t));
      }
    }
#pragma unroll
    for (int t = 0; t < EPV; ++t) part[g * D + c * EPV + t] = acc[t];
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float res;
    if (mean) {
      float a1 = 0.f;
      for (int g = 0; g < groups; ++g) a1 += part[g * D + d];
      res = a1 / (float)bs;
    } else {
      float m = (r1 - r0 < bs) ? 0.f : -CUDART_INF_F;     // zero padding takes part in the max
      for (int g = 0; g < groups; ++g) m = fmaxf(m, part[g * D + d]);
      res = m;
    }
    pooled_q[((int64_t)bh * nb + blk) * D + d] = E::cvt(res);
  }
}

template <int DT>
int run_permute(const Dims& d, const float* importance, const void* k, Strides ks, const void* v, Strides vs,
                int32_t* idx, void* perm_k, void* perm_v, void* pooled_k, int pool_mode, int32_t* first_block,
                cudaStream_t st) {
  using T = typename Elem<DT>::T;
  const int nsegs_all = (d.S + d.seg - 1) / d.seg;
  const int npow2 = next_pow2(d.seg);
  const size_t smem = (size_t)npow2 * 8 + (size_t)d.seg * 4;
  auto kern = segment_permute_kernel<DT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "segment_permute_kernel smem attribute");
  }
  kern<<<dim3(nsegs_all * d.group, d.B * d.Hkv), 256, smem, st>>>(
      importance, (const T*)k, ks, (const T*)v, vs, idx, (T*)perm_k, (T*)perm_v, (T*)pooled_k, pool_mode,
      first_block, d.Hq, d.group, d.S, d.D, d.bs, d.seg, d.nseg, d.nb, npow2);
  PBS_CUDA_CHECK_LAUNCH("segment_permute_kernel");
  return PBS_OK;
}

}  // namespace

int launch_segment_permute(const Dims& d, int dt, const float* importance, const void* k, Strides ks,
                           const void* v, Strides vs, int32_t* idx, void* perm_k, void* perm_v,
                           void* pooled_k, int pool_mode, int32_t* first_block, cudaStream_t st) {
  switch (dt) {
    case PBS_BF16: return run_permute<PBS_BF16>(d, importance, k, ks, v, vs, idx, perm_k, perm_v, pooled_k, pool_mode, first_block, st);
    case PBS_FP16: return run_permute<PBS_FP16>(d, importance, k, ks, v, vs, idx, perm_k, perm_v, pooled_k, pool_mode, first_block, st);
    default: return run_permute<PBS_FP32>(d, importance, k, ks, v, vs, idx, perm_k, perm_v, pooled_k, pool_mode, first_block, st);
  }
}

int launch_pool_queries(const Dims& d, int dt, const void* q, Strides qs, void* pooled_q, int pool_mode,
                        cudaStream_t st) {
  dim3 grid(d.nb, d.B * d.Hq);
  const int threads = d.D <= 128 ? 128 : 256;
  switch (dt) {
    case PBS_BF16:
      pool_queries_kernel<PBS_BF16><<<grid, threads, 0, st>>>((const __nv_bfloat16*)q, qs, (__nv_bfloat16*)pooled_q, pool_mode, d.Hq, d.S, d.D, d.bs, d.nb);
      break;
    case PBS_FP16:
      pool_queries_kernel<PBS_FP16><<<grid, threads, 0, st>>>((const __half*)q, qs, (__half*)pooled_q, pool_mode, d.Hq, d.S, d.D, d.bs, d.nb);
      break;
    default:
      pool_queries_kernel<PBS_FP32><<<grid, threads, 0, st>>>((const float*)q, qs, (float*)pooled_q, pool_mode, d.Hq, d.S, d.D, d.bs, d.nb);
  }
  PBS_CUDA_CHECK_LAUNCH("pool_queries_kernel");
  return PBS_OK;
}

}  // namespace pbs
