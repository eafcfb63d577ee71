// Stage 2b and 3a: pooled block scores, cumulative-threshold block selection, tile lists.
//
// select_kernel follows pbs_attn/src/utils.py:30-34 (pooled logits in the input dtype: fp32
// accumulate, rounded after the dot product and after the division by sqrt(D); -inf outside the
// candidates; fp32 softmax), pbs_attn/src/utils.py:38-86 (descending sort, running sum accumulated
// in double and rounded to fp32 per element as CPU torch does, first rank whose sum >= threshold,
// keep the ranks up to it, nothing if never reached), pbs_attn/src/pbs.py:95-107 (candidates = kv
// blocks of earlier segments), :120-127 (select-all mode, first-token block) and :209 (the q block's
// own segment is always on).  Ties are broken towards the lower kv-block id (a stable sort).
//
// One CTA per (q block, b, h).  Scores never reach HBM: a row of up to 4096 blocks lives in shared
// memory.  HBM traffic per (b, h): pooled Q and K read (2*nb*D*e, K re-read from L2 per row), the
// mask written once (nb*nb bytes).
#include "pbs_common.cuh"

namespace pbs {
namespace {

constexpr int SEL_THREADS = 256;

// KPT: sort keys per thread held in registers (0: sort in shared memory, any size)
template <int DT, int KPT>
__global__ void __launch_bounds__(SEL_THREADS)
select_kernel(const typename Elem<DT>::T* __restrict__ pooled_q, const typename Elem<DT>::T* __restrict__ pooled_k,
              const int32_t* __restrict__ first_block, const float* __restrict__ thr_per_head, float thr_scalar,
              int select_all, int force_first, int diag_candidates, uint8_t* __restrict__ mask,
              float* __restrict__ scores, int Hq, int D, int nb, int bps, float sqrt_d, int npow2_max) {
  using E = Elem<DT>;
  using T = typename E::T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem_raw);      // npow2_max
  float* pq = reinterpret_cast<float*>(keys + npow2_max);                          // D
  float* vals = pq + D;                                                            // logits, then probabilities
  __shared__ float red[SEL_THREADS / 32];
  __shared__ double dred[SEL_THREADS / 32];
  __shared__ int first_rank;

  const int qb = blockIdx.x;
  const int bh = blockIdx.y;
  const int h = bh % Hq;
  // candidates: kv blocks of earlier segments, or (MeanPooling variant) every block up to the diagonal
  const int ncand = diag_candidates ? qb + 1 : (qb / bps) * bps;
  uint8_t* row = mask + ((int64_t)bh * nb + qb) * nb;
  float* srow = scores ? scores + ((int64_t)bh * nb + qb) * nb : nullptr;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float thr = thr_per_head ? thr_per_head[h] : thr_scalar;

  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    row[i] = 0;
    if (srow) srow[i] = 0.f;
  }
  if (threadIdx.x == 0) first_rank = 0x7fffffff;
  __syncthreads();

  int n_keep = 0;                                      // ranks kept, in sorted order
  int npow2 = 1;
  if (select_all) {
    for (int i = threadIdx.x; i < ncand; i += blockDim.x) row[i] = 1;
  } else if (ncand > 0) {
    while (npow2 < ncand) npow2 <<= 1;
    if (KPT > 1 && npow2 < KPT) npow2 = KPT;
    for (int d = threadIdx.x; d < D; d += blockDim.x) pq[d] = E::ld(pooled_q + ((int64_t)bh * nb + qb) * D + d);
    __syncthreads();
    constexpr int EPV = 16 / (int)sizeof(T);             // elements per 16-byte vector
    const int cpr = D / EPV;                             // 16-byte chunks per pooled row
    if (cpr <= 32 && (cpr & (cpr - 1)) == 0) {
      // pooled logits, rows shared by the lanes of a warp: lane = (row in group, chunk), so one load
      // instruction fetches 32 / cpr whole rows as consecutive 16-byte pieces; each lane multiplies
      // its piece with the matching piece of pooled q (kept in registers) and the partial sums are
      // folded over the cpr lanes of a row.
      const int chunk = lane % cpr, rpp = 32 / cpr;      // rows per warp-wide load
      float pqr[EPV];
#pragma unroll
      for (int t = 0; t < EPV; ++t) pqr[t] = pq[chunk * EPV + t];
      constexpr int U = 4;                               // independent loads in flight per lane
      for (int kb0 = warp * rpp; kb0 < ncand; kb0 += U * (SEL_THREADS / 32) * rpp) {
        uint4 buf[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int kb = kb0 + u * (SEL_THREADS / 32) * rpp + lane / cpr;
          buf[u] = make_uint4(0u, 0u, 0u, 0u);
          if (kb < ncand) buf[u] = reinterpret_cast<const uint4*>(pooled_k + ((int64_t)bh * nb + kb) * D)[chunk];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int kb = kb0 + u * (SEL_THREADS / 32) * rpp + lane / cpr;
          const T* e = reinterpret_cast<const T*>(&buf[u]);
          float acc = 0.f;
#pragma unroll
          for (int t = 0; t < EPV; ++t) acc = fmaf(pqr[t], E::ld(e + t), acc);
          for (int o = cpr >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
          if (chunk == 0 && kb < ncand) vals[kb] = E::rnd(E::rnd(acc) / sqrt_d);
        }
      }
    } else {
      // generic head sizes: one thread per kv block, its pooled-K row fetched with independent loads
      for (int kb = threadIdx.x; kb < ncand; kb += SEL_THREADS) {
        const uint4* pk4 = reinterpret_cast<const uint4*>(pooled_k + ((int64_t)bh * nb + kb) * D);
        float acc = 0.f;
        for (int c0 = 0; c0 < cpr; c0 += 8) {
          uint4 buf[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c0 + j < cpr) buf[j] = pk4[c0 + j];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (c0 + j < cpr) {
              const T* e = reinterpret_cast<const T*>(&buf[j]);
#pragma unroll
              for (int t = 0; t < EPV; ++t) acc = fmaf(pq[(c0 + j) * EPV + t], E::ld(e + t), acc);
            }
          }
        }
        vals[kb] = E::rnd(E::rnd(acc) / sqrt_d);
      }
    }
    __syncthreads();
    // fp32 softmax over the candidates
    float m = -CUDART_INF_F;
    for (int i = threadIdx.x; i < ncand; i += blockDim.x) m = fmaxf(m, vals[i]);
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < SEL_THREADS / 32; ++w) m = fmaxf(m, red[w]);
    __syncthreads();
    float z = 0.f;
    for (int i = threadIdx.x; i < ncand; i += blockDim.x) {
      const float e = expf(vals[i] - m);
      vals[i] = e;
      z += e;
    }
    z = warp_sum(z);
    if (lane == 0) red[warp] = z;
    __syncthreads();
    z = 0.f;
#pragma unroll
    for (int w = 0; w < SEL_THREADS / 32; ++w) z += red[w];
    // sort keys: (probability, lower block id first)
    for (int i = threadIdx.x; i < npow2; i += blockDim.x) {
      unsigned long long key = 0ull;
      if (i < ncand) {
        float p = vals[i] / z;
        if (p != p) p = 0.f;                           // nan_to_num
        if (srow) srow[i] = p;
        key = ((unsigned long long)float_order_key(p) << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)i);
      }
      keys[i] = key;
    }
    __syncthreads();
    if constexpr (KPT > 0) bitonic_sort_desc_regs<KPT>(keys, npow2);
    else bitonic_sort_desc(keys, npow2);
    // running sum in double over the sorted probabilities; each thread owns a contiguous chunk
    const int chunk = (ncand + SEL_THREADS - 1) / SEL_THREADS;
    const int c0 = min(threadIdx.x * chunk, ncand), c1 = min(c0 + chunk, ncand);
    auto prob_at = [&](int i) -> float {
      const uint32_t u = (uint32_t)(keys[i] >> 32);
      return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u);
    };
    double local = 0.0;
    for (int i = c0; i < c1; ++i) local += (double)prob_at(i);
    // exclusive scan of the chunk totals across the block
    double incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) dred[warp] = incl;
    __syncthreads();
    double offset = 0.0;
    for (int w = 0; w < warp; ++w) offset += dred[w];
    double run = offset + (incl - local);
    int mine = 0x7fffffff;
    for (int i = c0; i < c1; ++i) {
      run += (double)prob_at(i);
      if ((float)run >= thr) { mine = i; break; }
    }
    if (mine != 0x7fffffff) atomicMin(&first_rank, mine);
    __syncthreads();
    n_keep = (first_rank == 0x7fffffff) ? 0 : first_rank + 1;
    for (int i = threadIdx.x; i < n_keep; i += blockDim.x)
      row[0xFFFFFFFFu - (uint32_t)(keys[i] & 0xFFFFFFFFull)] = 1;
  } else if (thr <= 0.f) {
    // no candidate: every score is 0 and a non-positive threshold is met at rank 0 (kv block 0)
    if (threadIdx.x == 0) row[0] = 1;
  }
  __syncthreads();
  if (force_first && threadIdx.x == 0) row[first_block[bh]] = 1;
  const int s0 = (qb / bps) * bps, s1 = min(s0 + bps, nb);
  for (int i = s0 + threadIdx.x; i < s1; i += blockDim.x) row[i] = 1;
}

__global__ void fill_ones_kernel(uint8_t* p, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = 1;
}

// Tile-list entry: bits 0-15 tile id (128 keys each); bits 16/17: used by query tile 0/1 of the
// group (128 rows each); bits 18/19: that query tile must mask this tile element-wise (the tile
// lies in the query tile's own segment); bits 20-23 / 24-27: which (q block, kv block) sub-blocks
// of the 128x128 tile are selected for query tile 0 / 1, bit = 2*qi + ki (only bit 0 when
// block_size is 128).
__global__ void __launch_bounds__(128)
tile_list_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ list, int32_t* __restrict__ count,
                 int S, int bs, int seg, int nb, int ngroups, int ntiles) {
  const int g = blockIdx.x;
  const int bh = blockIdx.y;
  uint32_t* out = list + ((int64_t)bh * ngroups + g) * ntiles;
  __shared__ int wbase;
  __shared__ int wcnt[4];
  if (threadIdx.x == 0) wbase = 0;
  __syncthreads();
  const int sub = 128 / bs;                              // blocks per 128-row / 128-key tile (1 or 2)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int t0 = 0; t0 < ntiles; t0 += blockDim.x) {
    const int t = t0 + threadIdx.x;
    uint32_t e = 0;
    if (t < ntiles) {
      for (int m = 0; m < 2; ++m) {
        const int r0 = g * 256 + m * 128;
        if (r0 >= S) continue;
        uint32_t bits = 0;
        for (int qi = 0; qi < sub; ++qi) {
          const int qb = r0 / bs + qi;
          if (qb >= nb) continue;
          for (int ki = 0; ki < sub; ++ki) {
            const int kb = t * sub + ki;
            if (kb < nb && mask[((int64_t)bh * nb + qb) * nb + kb]) bits |= 1u << (2 * qi + ki);
          }
        }
        if (bits) {
          e |= (1u << (16 + m)) | (bits << (20 + 4 * m));
          const int q_seg_first = r0 / seg, q_seg_last = (min(r0 + 128, S) - 1) / seg;
          const int k_seg_last = (min(t * 128 + 128, S) - 1) / seg;
          (void)q_seg_last;
          if (k_seg_last >= q_seg_first) e |= 1u << (18 + m);
        }
      }
      if (e) e |= (uint32_t)t;
    }
    const unsigned ball = __ballot_sync(0xffffffffu, e != 0);
    if (lane == 0) wcnt[warp] = __popc(ball);
    __syncthreads();
    int base = wbase;
    for (int w = 0; w < warp; ++w) base += wcnt[w];
    if (e) out[base + __popc(ball & ((1u << lane) - 1))] = e;
    __syncthreads();
    if (threadIdx.x == 0) wbase += wcnt[0] + wcnt[1] + wcnt[2] + wcnt[3];
    __syncthreads();
  }
  if (threadIdx.x == 0) count[(int64_t)bh * ngroups + g] = wbase;
}

}  // namespace

int launch_select_blocks(const Dims& d, int dt, const void* pooled_q, const void* pooled_k,
                         const int32_t* first_block, const pbs_options_t& opt, uint8_t* mask, float* scores,
                         cudaStream_t st) {
  const int npow2 = next_pow2(d.nb);
  const size_t smem = (size_t)npow2 * 8 + (size_t)d.D * 4 + (size_t)d.nb * 4;
  dim3 grid(d.nb, d.B * d.Hq);
  const float sq = (float)sqrt((double)d.D);
#define PBS_SEL_E(DT, TT, EE)                                                                                 \
  {                                                                                                           \
    auto kern = select_kernel<DT, EE>;                                                                        \
    if (smem > 48 * 1024) {                                                                                   \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
      if (e != cudaSuccess) return cuda_fail(e, "select_kernel smem attribute");                              \
    }                                                                                                         \
    kern<<<grid, SEL_THREADS, smem, st>>>((const TT*)pooled_q, (const TT*)pooled_k, first_block,              \
                                          opt.threshold_per_head, opt.threshold, opt.select_all,             \
                                          opt.force_select_first_block, opt.diagonal_candidates, mask,       \
                                          scores, d.Hq, d.D, d.nb, d.bps, sq, npow2);                         \
  }
  // keys per thread of the register sort; beyond 16 the sort runs in shared memory
#define PBS_SEL(DT, TT)                                                                                       \
  {                                                                                                           \
    const int per_thread = (npow2 + SEL_THREADS - 1) / SEL_THREADS;                                           \
    if (per_thread <= 1) PBS_SEL_E(DT, TT, 1)                                                                 \
    else if (per_thread == 2) PBS_SEL_E(DT, TT, 2)                                                            \
    else if (per_thread == 4) PBS_SEL_E(DT, TT, 4)                                                            \
    else if (per_thread == 8) PBS_SEL_E(DT, TT, 8)                                                            \
    else if (per_thread == 16) PBS_SEL_E(DT, TT, 16)                                                          \
    else PBS_SEL_E(DT, TT, 0)                                                                                 \
  }
  switch (dt) {
    case PBS_BF16: PBS_SEL(PBS_BF16, __nv_bfloat16) break;
    case PBS_FP16: PBS_SEL(PBS_FP16, __half) break;
    default: PBS_SEL(PBS_FP32, float)
  }
#undef PBS_SEL
#undef PBS_SEL_E
  PBS_CUDA_CHECK_LAUNCH("select_kernel");
  return PBS_OK;
}

int launch_fill_mask_ones(const Dims& d, uint8_t* mask, cudaStream_t st) {
  const int64_t n = (int64_t)d.B * d.Hq * d.nb * d.nb;
  fill_ones_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(mask, n);
  PBS_CUDA_CHECK_LAUNCH("fill_ones_kernel");
  return PBS_OK;
}

int launch_build_tile_lists(const Dims& d, const uint8_t* mask, uint32_t* list, int32_t* count, cudaStream_t st) {
  const int ngroups = (d.S + 255) / 256, ntiles = (d.S + 127) / 128;
  tile_list_kernel<<<dim3(ngroups, d.B * d.Hq), 128, 0, st>>>(mask, list, count, d.S, d.bs, d.seg, d.nb, ngroups, ntiles);
  PBS_CUDA_CHECK_LAUNCH("tile_list_kernel");
  return PBS_OK;
}

}  // namespace pbs
