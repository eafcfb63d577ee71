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
#include <atomic>

#include "pbs_common.cuh"

namespace pbs {
namespace {

constexpr int SEL_THREADS = 256;

// KPT: sort keys per thread held in registers (0: sort in shared memory, any size)
template <int DT, int KPT>
__global__ void __launch_bounds__(SEL_THREADS)
select_kernel(const typename Elem<DT>::T* __restrict__ pooled_q, const typename Elem<DT>::T* __restrict__ pooled_k,
              const int32_t* __restrict__ first_block, const float* __restrict__ thr_per_head, float thr_scalar,
              int select_all, int force_first, int diag_candidates, int own_segment, uint8_t* __restrict__ mask,
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
  if (own_segment) {
    const int s0 = (qb / bps) * bps, s1 = min(s0 + bps, nb);
    for (int i = s0 + threadIdx.x; i < s1; i += blockDim.x) row[i] = 1;
  }
}


// ---------------------------------------------------------------------------------------------
// Tiled variant: one CTA = 16 consecutive q blocks of one (b, h).
//
// Phase A computes the pooled logits of the 16 rows against 64-kv-block chunks of pooled K that
// arrive in shared memory by cp.async (each pooled-K row is then read once per 16 rows instead of
// once per row).  The dot product keeps the summation order of select_kernel: 16-byte pieces are
// summed front to back, the piece sums are combined in the order of a butterfly over the pieces.
// Phases B-D run one warp per row: fp32 softmax (the exponent sum is taken in the same order as the
// 256-thread reduction of select_kernel), then the cut of the cumulative-threshold selection is
// found WITHOUT sorting: the bits of the cut probability are fixed one at a time, each step summing
// (in double) the probabilities at or above the trial value; blocks above the cut are kept, blocks
// equal to it are added in kv-block order until the running sum reaches the threshold -- the set a
// stable descending sort followed by a running sum selects.
// ---------------------------------------------------------------------------------------------
constexpr int TS_ROWS = 16;       // q blocks per CTA
constexpr int TS_CHUNK = 64;      // kv blocks per staged chunk

template <int N>
__device__ __forceinline__ float butterfly_sum(float (&p)[N]) {
  // the value lane 0 of an N-lane xor-butterfly (offsets N/2 .. 1) ends up with
#pragma unroll
  for (int o = N / 2; o > 0; o >>= 1)
#pragma unroll
    for (int c = 0; c < o; ++c) p[c] = p[c] + p[c ^ o];
  return p[0];
}

__device__ __forceinline__ double warp_sum_double(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// CPR: 16-byte pieces per pooled row; KPT: kv blocks per lane held in registers (32 * KPT >= nb)
template <int DT, int CPR, int KPT>
__global__ void __launch_bounds__(256)
select_tiled_kernel(const typename Elem<DT>::T* __restrict__ pooled_q, const typename Elem<DT>::T* __restrict__ pooled_k,
                    const int32_t* __restrict__ first_block, const float* __restrict__ thr_per_head, float thr_scalar,
                    int select_all, int force_first, int diag_candidates, int own_segment, uint8_t* __restrict__ mask,
                    float* __restrict__ scores, int Hq, int nb, int bps, float sqrt_d, int ncpad) {
  using E = Elem<DT>;
  using T = typename E::T;
  constexpr int EPV = 16 / (int)sizeof(T);
  constexpr int D = CPR * EPV;
  constexpr int LDK = D + EPV;                             // padded pooled-K row in shared memory
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* Qs = reinterpret_cast<float*>(smem_raw);          // [16][D] fp32
  T* Kc = reinterpret_cast<T*>(Qs + TS_ROWS * D);          // [2][64][LDK]
  T* lg = Kc + 2 * TS_CHUNK * LDK;                         // [16][ncpad] rounded logits

  const int qb0 = blockIdx.x * TS_ROWS;
  const int bh = blockIdx.y;
  const int h = bh % Hq;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qb_last = min(qb0 + TS_ROWS, nb) - 1;
  const int ncmax = diag_candidates ? qb_last + 1 : (qb_last / bps) * bps;   // candidates of the tile's last row
  const T* kbase = pooled_k + (int64_t)bh * nb * D;
  const int nchunks = select_all ? 0 : (ncmax + TS_CHUNK - 1) / TS_CHUNK;

  auto load_chunk = [&](int buf, int c) {
    for (int i = threadIdx.x; i < TS_CHUNK * CPR; i += blockDim.x) {
      const int r = i / CPR, pc = i % CPR;
      const int kb = c * TS_CHUNK + r;
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(Kc + (buf * TS_CHUNK + r) * LDK + pc * EPV);
      const T* src = kbase + (int64_t)min(kb, nb - 1) * D + pc * EPV;
      const int bytes = kb < nb ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  if (nchunks > 0) load_chunk(0, 0);
  for (int i = threadIdx.x; i < TS_ROWS * D; i += blockDim.x) {
    const int r = i / D, d = i % D;
    Qs[i] = qb0 + r < nb ? E::ld(pooled_q + ((int64_t)bh * nb + qb0 + r) * D + d) : 0.f;
  }

  // ---- phase A: logits.  Thread = (row, kv lane): row t / 16, kv blocks t % 16 + 16 a of the chunk.
  const int arow = threadIdx.x >> 4, aj0 = threadIdx.x & 15;
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) {
      load_chunk((c + 1) & 1, c + 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const T* Kt = Kc + (c & 1) * TS_CHUNK * LDK;
    const float* qr = Qs + arow * D;
#pragma unroll
    for (int a = 0; a < TS_CHUNK / 16; ++a) {
      const int j = aj0 + 16 * a;
      const int kb = c * TS_CHUNK + j;
      if (kb >= ncmax) continue;
      float piece[CPR];
#pragma unroll
      for (int pc = 0; pc < CPR; ++pc) {
        const uint4 raw = *reinterpret_cast<const uint4*>(Kt + j * LDK + pc * EPV);
        const T* e = reinterpret_cast<const T*>(&raw);
        float acc = 0.f;
#pragma unroll
        for (int t = 0; t < EPV; ++t) acc = fmaf(qr[pc * EPV + t], E::ld(e + t), acc);
        piece[pc] = acc;
      }
      const float dot = butterfly_sum<CPR>(piece);
      lg[arow * ncpad + kb] = E::cvt(E::rnd(E::rnd(dot) / sqrt_d));
    }
    __syncthreads();
  }
  if (nchunks == 0) __syncthreads();

  // ---- phases B-D: one warp per row (rows 2 * warp and 2 * warp + 1)
  const float thr = thr_per_head ? thr_per_head[h] : thr_scalar;
  for (int rr = 0; rr < TS_ROWS / 8; ++rr) {
    const int r = warp * (TS_ROWS / 8) + rr;
    const int qb = qb0 + r;
    if (qb >= nb) break;
    const int ncand = diag_candidates ? qb + 1 : (qb / bps) * bps;
    const int kmax = (ncand + 31) >> 5;                    // register slots in use
    uint8_t* row = mask + ((int64_t)bh * nb + qb) * nb;
    float* srow = scores ? scores + ((int64_t)bh * nb + qb) * nb : nullptr;
    unsigned long long sel = 0ull;                         // bit k: candidate 32 k + lane is kept

    if (select_all) {
#pragma unroll
      for (int k = 0; k < KPT; ++k)
        if (32 * k + lane < ncand) sel |= 1ull << k;
    } else if (ncand > 0) {
      // fp32 softmax over the candidates
      float pv[KPT];
      float m = -CUDART_INF_F;
#pragma unroll
      for (int k = 0; k < KPT; ++k) {
        pv[k] = -CUDART_INF_F;
        if (k < kmax && 32 * k + lane < ncand) pv[k] = E::ld(lg + r * ncpad + 32 * k + lane);
        m = fmaxf(m, pv[k]);
      }
      m = warp_max(m);
      // exponent sum in the order of a 256-thread strided reduction: 8 interleaved accumulators,
      // each reduced over the lanes, then added up one after the other
      float zacc[8];
#pragma unroll
      for (int w = 0; w < 8; ++w) zacc[w] = 0.f;
#pragma unroll
      for (int k = 0; k < KPT; ++k) {
        const bool valid = k < kmax && 32 * k + lane < ncand;
        const float e = valid ? expf(pv[k] - m) : 0.f;
        pv[k] = e;
        if (valid) zacc[k & 7] += e;
      }
      float z = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) z += warp_sum(zacc[w]);
      float pmax = 0.f;
#pragma unroll
      for (int k = 0; k < KPT; ++k) {
        const bool valid = k < kmax && 32 * k + lane < ncand;
        float p = pv[k] / z;
        if (p != p) p = 0.f;                               // nan_to_num
        if (!valid) p = 0.f;
        pv[k] = p;
        pmax = fmaxf(pmax, p);
        if (srow && valid) srow[32 * k + lane] = p;
      }
      pmax = warp_max(pmax);

      // total mass: if even that stays below the threshold nothing is selected
      double tot = 0.0;
#pragma unroll
      for (int k = 0; k < KPT; ++k)
        if (k < kmax) tot += (double)pv[k];
      tot = warp_sum_double(tot);
      if ((float)tot >= thr) {
        // cut = largest probability value v with (float) sum{p >= v} >= thr (bit pattern order)
        const uint32_t umax = __float_as_uint(pmax);
        uint32_t cut = umax;
        if (thr > 0.f && umax != 0u) {
          cut = 0u;
          for (int b = 31 - __clz(umax); b >= 0; --b) {
            const uint32_t cand = cut | (1u << b);
            if (cand > umax) continue;
            double g = 0.0;
#pragma unroll
            for (int k = 0; k < KPT; ++k)
              if (k < kmax && __float_as_uint(pv[k]) >= cand) g += (double)pv[k];
            g = warp_sum_double(g);
            if ((float)g >= thr) cut = cand;
          }
        }
        // everything above the cut; then the blocks equal to it, in kv-block order, until reached
        double run = 0.0;
#pragma unroll
        for (int k = 0; k < KPT; ++k) {
          const bool valid = k < kmax && 32 * k + lane < ncand;
          if (valid && __float_as_uint(pv[k]) > cut) { run += (double)pv[k]; sel |= 1ull << k; }
        }
        run = warp_sum_double(run);
        const double pcut = (double)__uint_as_float(cut);
        bool done = false;
#pragma unroll
        for (int k = 0; k < KPT; ++k) {
          if (k >= kmax) break;
          const bool valid = 32 * k + lane < ncand;
          unsigned ties = __ballot_sync(0xffffffffu, valid && __float_as_uint(pv[k]) == cut);
          while (ties && !done) {
            const int l = __ffs(ties) - 1;
            ties &= ties - 1;
            run += pcut;
            if (lane == l) sel |= 1ull << k;
            if ((float)run >= thr) done = true;
          }
          if (done) break;
        }
      }
    } else if (thr <= 0.f) {
      // no candidate: every score is 0 and a non-positive threshold is met at rank 0 (kv block 0)
      if (lane == 0) sel |= 1ull;
    }

    // ---- write the row: selection, first-token block, own segment
    const int fb = force_first ? first_block[bh] : -1;
    const int s0 = own_segment ? (qb / bps) * bps : 0, s1 = own_segment ? min(s0 + bps, nb) : 0;
    const bool no_cand_rule = !select_all && ncand == 0;   // the kept block is kv block 0 even with no candidate
    for (int k = 0; 32 * k < nb; ++k) {
      const int i = 32 * k + lane;
      if (i >= nb) break;
      bool on = (k < KPT) && ((sel >> k) & 1ull) && (i < ncand || no_cand_rule);
      on = on || i == fb || (i >= s0 && i < s1);
      row[i] = on ? 1 : 0;
      if (srow && (select_all || i >= ncand)) srow[i] = 0.f;
    }
  }
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

template <int DT, int CPR, int KPT>
int run_select_tiled(const Dims& d, const void* pooled_q, const void* pooled_k, const int32_t* first_block,
                     const pbs_options_t& opt, uint8_t* mask, float* scores, cudaStream_t st) {
  using T = typename Elem<DT>::T;
  constexpr int EPV = 16 / (int)sizeof(T);
  const int ncpad = ((d.nb + TS_CHUNK - 1) / TS_CHUNK) * TS_CHUNK;
  const size_t smem = (size_t)TS_ROWS * d.D * sizeof(float) + (size_t)2 * TS_CHUNK * (d.D + EPV) * sizeof(T) +
                      (size_t)TS_ROWS * ncpad * sizeof(T);
  auto kern = select_tiled_kernel<DT, CPR, KPT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "select_tiled_kernel smem attribute");
  }
  kern<<<dim3((d.nb + TS_ROWS - 1) / TS_ROWS, d.B * d.Hq), 256, smem, st>>>(
      (const T*)pooled_q, (const T*)pooled_k, first_block, opt.threshold_per_head, opt.threshold, opt.select_all,
      opt.force_select_first_block, opt.diagonal_candidates, opt.no_own_segment ? 0 : 1, mask, scores, d.Hq, d.nb, d.bps,
      (float)sqrt((double)d.D), ncpad);
  PBS_CUDA_CHECK_LAUNCH("select_tiled_kernel");
  return PBS_OK;
}

template <int DT, int CPR>
int run_select_tiled_k(const Dims& d, const void* pooled_q, const void* pooled_k, const int32_t* first_block,
                       const pbs_options_t& opt, uint8_t* mask, float* scores, cudaStream_t st) {
  if (d.nb <= 256) return run_select_tiled<DT, CPR, 8>(d, pooled_q, pooled_k, first_block, opt, mask, scores, st);
  if (d.nb <= 512) return run_select_tiled<DT, CPR, 16>(d, pooled_q, pooled_k, first_block, opt, mask, scores, st);
  if (d.nb <= 1024) return run_select_tiled<DT, CPR, 32>(d, pooled_q, pooled_k, first_block, opt, mask, scores, st);
  return run_select_tiled<DT, CPR, 64>(d, pooled_q, pooled_k, first_block, opt, mask, scores, st);
}

// The tiled kernel covers pooled rows of 8, 16 or 32 16-byte pieces and up to 2048 blocks per row.
bool select_tiled_supported(const Dims& d, int dt) {
  const int cpr = d.D * elem_bytes(dt) / 16;
  return d.nb <= 2048 && (d.D * elem_bytes(dt)) % 16 == 0 && (cpr == 8 || cpr == 16 || cpr == 32);
}

int launch_select_tiled(const Dims& d, int dt, const void* pooled_q, const void* pooled_k, const int32_t* first_block,
                        const pbs_options_t& opt, uint8_t* mask, float* scores, cudaStream_t st) {
  const int cpr = d.D * elem_bytes(dt) / 16;
#define PBS_TS(DT)                                                                                                \
  (cpr == 8 ? run_select_tiled_k<DT, 8>(d, pooled_q, pooled_k, first_block, opt, mask, scores, st)                 \
   : cpr == 16 ? run_select_tiled_k<DT, 16>(d, pooled_q, pooled_k, first_block, opt, mask, scores, st)             \
               : run_select_tiled_k<DT, 32>(d, pooled_q, pooled_k, first_block, opt, mask, scores, st))
  switch (dt) {
    case PBS_BF16: return PBS_TS(PBS_BF16);
    case PBS_FP16: return PBS_TS(PBS_FP16);
    default: return PBS_TS(PBS_FP32);
  }
#undef PBS_TS
}

}  // namespace

namespace {
std::atomic<int> g_select_impl{0};     // 0: tiled where supported; 1: always the one-row-per-CTA kernel
}
void set_select_impl(int impl) { g_select_impl.store(impl, std::memory_order_relaxed); }

int launch_select_blocks(const Dims& d, int dt, const void* pooled_q, const void* pooled_k,
                         const int32_t* first_block, const pbs_options_t& opt, uint8_t* mask, float* scores,
                         cudaStream_t st) {
  if (g_select_impl.load(std::memory_order_relaxed) == 0 && select_tiled_supported(d, dt))
    return launch_select_tiled(d, dt, pooled_q, pooled_k, first_block, opt, mask, scores, st);
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
                                          opt.force_select_first_block, opt.diagonal_candidates,             \
                                          opt.no_own_segment ? 0 : 1, mask,                                  \
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
