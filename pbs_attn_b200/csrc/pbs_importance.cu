// Stage 1a: per-key importance = mean over the last query block of softmax(q . k / sqrt(D)).
//
// Follows pbs_attn/src/permute_states.py:44-50 of the reference: the logits are produced in the
// input dtype (fp32 accumulate, rounded once after the dot product and once after the division by
// sqrt(D)), the softmax runs in fp32 over all keys of the complete segments, and the mean over the
// block's query rows is an fp32 sum in the reference's summation order.
//
// The logits never reach HBM: the softmax is taken in two passes that each RECOMPUTE the last
// block's logits from K (same instructions, same order, hence the same bits):
//   pass 1  score kernel<1>   per 64-key tile and query row: max and sum(exp) of the tile -> partials
//           rowstats_kernel   merges the per-tile pairs into one (max, sum) per row
//   pass 2  score kernel<2>   p = exp(logit - max_r) / sum_r, summed over the rows r in the order of
//                             the reference's reduction (16-row groups, then the groups) -> importance
// HBM traffic per (b, h): K read once per pass (the query heads of a KV group run next to each other
// and share its tiles in L2), the last query block, the per-tile statistics (16 bytes per row and
// 64 keys) and the importance written once (4*L).
#include <cmath>
#include <type_traits>
#include <cstring>
#include <map>
#include <mutex>

#include "pbs_common.cuh"

namespace pbs {
namespace {

constexpr int TM = 64;   // query rows per pass of the CUDA-core kernel
constexpr int TN = 64;   // keys per tile
constexpr int KC = 32;   // head-dim chunk staged in shared memory (CUDA-core kernel)
constexpr int LDT = TM + 4;
constexpr int kStageLd = TN + 8;     // elements per row of the per-warp logits staging tile
constexpr int kPLd = TN + 8;         // floats per row of the probability tile: 8-byte stores of the MMA layout
                                     // (8 rows x 4 pairs per instruction) and column reads are both conflict free
constexpr int kMaxGroups = 16;       // 16-row groups of a block of up to 256 rows

// Column sums of a tile of probabilities in the order of the reference's CPU reduction: rows are
// added one after the other inside groups of 16; the caller adds the group sums one after the other.
// 256 threads: thread t owns key t % 64 and the 16-row groups (t / 64) * gpt .. + gpt - 1 of this pass.
__device__ __forceinline__ void group_sums(const float* P, float* gs, int rows_in_pass, int first_group, int gpt) {
  const int key = threadIdx.x & (TN - 1), part = threadIdx.x >> 6;
  for (int gg = 0; gg < gpt; ++gg) {
    const int g = part * gpt + gg;
    if (g * 16 >= rows_in_pass) break;
    float a0 = 0.f;
#pragma unroll
    for (int rr = 0; rr < 16; ++rr) a0 += P[(g * 16 + rr) * kPLd + key];
    gs[(first_group + g) * TN + key] = a0;
  }
}

// importance of the tile's keys from the group sums (level 1 of the cascade, then the mean)
__device__ __forceinline__ void finish_tile(const float* gs, float* __restrict__ importance, int64_t out0, int nkeys, int bs) {
  if (threadIdx.x < TN && (int)threadIdx.x < nkeys) {
    float a1 = 0.f;
    for (int g = 0; g < bs / 16; ++g) a1 += gs[g * TN + threadIdx.x];
    importance[out0 + threadIdx.x] = a1 / (float)bs;
  }
}

// CUDA-core kernel (fp32 inputs, or 16-bit inputs whose layout the tensor-core kernel cannot read).
// One CTA = one 64-key tile x all rows of the last block, 64 rows per pass.
template <int DT, int PASS>
__global__ void __launch_bounds__(256)
score_kernel(const typename Elem<DT>::T* __restrict__ q, Strides qs,
             const typename Elem<DT>::T* __restrict__ k, Strides ks,
             float2* __restrict__ partials, const float2* __restrict__ rowstats, float* __restrict__ importance,
             typename Elem<DT>::T* __restrict__ logits_out,
             int Hq, int group, int S, int D, int bs, int L, float sqrt_d) {
  using E = Elem<DT>;
  using T = typename E::T;
  __shared__ __align__(16) float Qs[KC][LDT];
  __shared__ __align__(16) float Ks[KC][LDT];
  __shared__ __align__(16) float P[PASS == 2 ? TM * kPLd : 4];
  __shared__ float gs[PASS == 2 ? kMaxGroups * TN : 1];
  __shared__ float2 stats[PASS == 2 ? 256 : 1];

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
  if (PASS == 2)
    for (int r = threadIdx.x; r < bs; r += blockDim.x) stats[r] = rowstats[(int64_t)bh * bs + r];

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

    // round like the reference; pass 1: the tile's row statistics, pass 2: probabilities
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + ty * 4 + i;
      float y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = E::rnd(E::rnd(acc[i][j]) / sqrt_d);
      if (PASS == 1) {
        float m = -CUDART_INF_F;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (tx * 4 + j < nkeys) m = fmaxf(m, y[j]);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float z = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (tx * 4 + j < nkeys) z += expf(y[j] - m);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
        if (r < bs) {
          if (logits_out) {
            T* dst = logits_out + ((int64_t)bh * bs + r) * L + (int64_t)jt * TN + tx * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (tx * 4 + j < nkeys) dst[j] = E::cvt(y[j]);
          }
          if (tx == 0) partials[((int64_t)bh * ntile + jt) * bs + r] = make_float2(m, z);
        }
      } else {
        const float2 st = stats[min(r, bs - 1)];
        *reinterpret_cast<float4*>(&P[(ty * 4 + i) * kPLd + tx * 4]) =
            make_float4(expf(y[0] - st.x) / st.y, expf(y[1] - st.x) / st.y, expf(y[2] - st.x) / st.y, expf(y[3] - st.x) / st.y);
      }
    }
    if (PASS == 2) {
      __syncthreads();
      group_sums(P, gs, nrows, r0 >> 4, 1);
    }
  }
  if (PASS == 2) {
    __syncthreads();
    finish_tile(gs, importance, (int64_t)bh * L + (int64_t)jt * TN, nkeys, bs);
  }
}

// Tensor-core kernel for 16-bit inputs (mma.sync m16n8k16, fp32 accumulate: the products of 16-bit
// values are exact and the sum is rounded like any fp32 GEMM).  A CTA keeps the whole last query
// block in shared memory and walks `tiles_per_cta` consecutive 64-key tiles, the next tile arriving
// by cp.async while the current one is multiplied; warp w owns rows 16w..16w+15 of a 128-row pass.
// Rows are padded by 16 bytes so ldmatrix is conflict free.
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

// x / z for a divisor used many times: reciprocal product corrected by one exact-remainder step (the
// correctly rounded quotient for all but a few divisors with an all-ones significand, where the result
// may differ from it in the last bit).
__device__ __forceinline__ float div_by(float x, float z, float rz) {
  const float qv = x * rz;
  return fmaf(fmaf(-qv, z, x), rz, qv);
}

// FASTDIV: rounding a * (1 / sqrt(D)) to the input type gives the same bits as rounding a / sqrt(D)
// for EVERY value a of that type (established on the host by trying all 65536 of them)
// DH: head_dim when it is 64 or 128 (loops unroll, index arithmetic folds), 0 = any multiple of 16
template <int DT, int PASS, bool FASTDIV, int DH>
__global__ void __launch_bounds__(256, PASS == 1 ? 3 : 2)
score_mma_kernel(const typename Elem<DT>::T* __restrict__ q, Strides qs,
                 const typename Elem<DT>::T* __restrict__ k, Strides ks,
                 float2* __restrict__ partials, const float2* __restrict__ rowstats, float* __restrict__ importance,
                 typename Elem<DT>::T* __restrict__ logits_out,
                 int Hq, int group, int S, int D_rt, int bs, int L, int ntile, int tiles_per_cta, float sqrt_d) {
  using E = Elem<DT>;
  using T = typename E::T;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = DH ? DH : D_rt;
  const int ld = D + 8;                                    // padded row length in elements
  const int qrows = (bs + 127) & ~127;                     // staged query rows (whole 128-row passes)
  T* Qs = reinterpret_cast<T*>(smem_raw);                  // [qrows][ld]
  T* Ks = Qs + qrows * ld;                                 // [2][64][ld]
  unsigned char* extra = reinterpret_cast<unsigned char*>(Ks + 2 * TN * ld);
  T* stage = reinterpret_cast<T*>(extra);                  // pass 1 with logits_out: [8 warps][16 rows][kStageLd]
  float* P = reinterpret_cast<float*>(extra);              // pass 2: [8 warps][8 rows][kPLd], private to each warp
  float* gs = P + 64 * kPLd;                               //         [2][kMaxGroups][64] group sums, double buffered
  float3* stats = reinterpret_cast<float3*>(gs + 2 * kMaxGroups * TN);   // [bs] (max, sum, 1 / sum)

  // the query heads of a KV group sit next to each other in the grid: they read the same K tiles
  const int hin = blockIdx.x % group, chunk = blockIdx.x / group;
  const int Hkv = Hq / group;
  const int b = blockIdx.y / Hkv, hkv = blockIdx.y % Hkv;
  const int h = hkv * group + hin;
  const int bh = b * Hq + h;
  const T* qbase = q + (int64_t)b * qs.b + (int64_t)h * qs.h + (int64_t)(S - bs) * qs.s;
  const T* khead = k + (int64_t)b * ks.b + (int64_t)hkv * ks.h;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cpr = D / 8;                                   // 16-byte chunks per row
  const int jt0 = chunk * tiles_per_cta;
  const int ntiles_here = min(tiles_per_cta, ntile - jt0);
  if (ntiles_here <= 0) return;

  auto load_k = [&](int buf, int jt) {
    const int nkeys = min(TN, L - jt * TN);
    const T* kbase = khead + (int64_t)jt * TN * ks.s;
#pragma unroll 4
    for (int i = threadIdx.x; i < TN * cpr; i += blockDim.x) {
      const int r = i / cpr, c = i % cpr;                  // shifts when head_dim is a compile-time constant
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(Ks + (buf * TN + r) * ld + c * 8);
      const T* src = kbase + (int64_t)min(r, nkeys - 1) * ks.s + c * 8;
      const int bytes = r < nkeys ? 16 : 0;                // rows past the end are filled with zeros
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // importance of a finished tile from its group sums: the groups added one after the other, then the mean
  auto finish_tile = [&](int it) {
    if (threadIdx.x < TN) {
      const int jt = jt0 + it;
      const float* g0 = gs + (it & 1) * kMaxGroups * TN + threadIdx.x;
      float a1 = 0.f;
      for (int g = 0; g < bs / 16; ++g) a1 += g0[g * TN];
      if ((int)threadIdx.x < min(TN, L - jt * TN)) importance[(int64_t)bh * L + (int64_t)jt * TN + threadIdx.x] = a1 / (float)bs;
    }
  };

  load_k(0, jt0);
  for (int i = threadIdx.x; i < qrows * cpr; i += blockDim.x) {
    const int r = i / cpr, c = i % cpr;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (r < bs) val = *reinterpret_cast<const uint4*>(qbase + (int64_t)r * qs.s + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * ld + c * 8) = val;
  }
  if (PASS == 2)
    for (int r = threadIdx.x; r < bs; r += blockDim.x) {
      const float2 st = rowstats[(int64_t)bh * bs + r];
      stats[r] = make_float3(st.x, st.y, 1.f / st.y);
    }

  const float rinv = 1.f / sqrt_d;
  // One block-wide barrier per tile: it publishes tile `it` (copied during the previous iteration) and
  // the previous tile's group sums, and it tells that every warp is done with the other K buffer, which
  // the copy of tile it + 1 then overwrites while this tile is multiplied.
  for (int it = 0; it < ntiles_here; ++it) {
    const int jt = jt0 + it;
    const int buf = it & 1;
    const int nkeys = min(TN, L - jt * TN);
    const bool full = nkeys == TN;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (it + 1 < ntiles_here) load_k(buf ^ 1, jt + 1);
    if (PASS == 2 && it > 0) finish_tile(it - 1);
    const T* Kt = Ks + buf * TN * ld;
    float* gcur = gs + buf * kMaxGroups * TN;
    for (int r0 = 0; r0 < bs; r0 += 128) {
      const int nrows = min(128, bs - r0);
      if (warp * 16 >= nrows) continue;
      float acc[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int t = 0; t < 4; ++t) acc[j][t] = 0.f;
      const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(Qs + (r0 + warp * 16 + (lane & 15)) * ld + (lane >> 4) * 8);
      const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(Kt + ((lane >> 4) * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
#pragma unroll
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
      float* Pw = P + warp * 8 * kPLd;
      float colsum[2] = {0.f, 0.f};                        // keys lane and lane + 32 of the tile, rows added in order
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int lr = (lane >> 2) + 8 * half;             // row inside the warp's 16
        const int r = r0 + warp * 16 + lr;
        float y[16];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            // a / sqrt_d in fp32 (the correctly rounded quotient), then the second rounding to the input type
            const float a = E::rnd(acc[j][2 * half + t]);
            y[2 * j + t] = E::rnd(FASTDIV ? a * rinv : div_by(a, sqrt_d, rinv));
          }
        if (PASS == 1) {
          float m = -CUDART_INF_F;
          float z = 0.f;
          if (full) {                                      // the common case: no per-key bound checks
#pragma unroll
            for (int c = 0; c < 16; ++c) m = fmaxf(m, y[c]);
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
#pragma unroll
            for (int c = 0; c < 16; ++c) z += __expf(y[c] - m);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
              for (int t = 0; t < 2; ++t)
                if (8 * j + 2 * (lane & 3) + t < nkeys) m = fmaxf(m, y[2 * j + t]);
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
              for (int t = 0; t < 2; ++t)
                if (8 * j + 2 * (lane & 3) + t < nkeys) z += __expf(y[2 * j + t] - m);
          }
          z += __shfl_xor_sync(0xffffffffu, z, 1);
          z += __shfl_xor_sync(0xffffffffu, z, 2);
          if (r < bs && (lane & 3) == 0) partials[((int64_t)bh * ntile + jt) * bs + r] = make_float2(m, z);
          if (logits_out) {
            // inspection output: the rounded logits leave through a per-warp staging tile
            T* srow = stage + (warp * 16 + lr) * kStageLd;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              T pair[2] = {E::cvt(y[2 * j]), E::cvt(y[2 * j + 1])};
              *reinterpret_cast<uint32_t*>(srow + 8 * j + 2 * (lane & 3)) = *reinterpret_cast<const uint32_t*>(pair);
            }
          }
        } else {
          // The warp's 16 rows are exactly one 16-row group of the reduction.  Its probabilities pass
          // through the warp's own tile, 8 rows at a time, so that each lane can add up two key
          // columns row after row.
          const float3 st = stats[min(r, bs - 1)];
          float* prow = Pw + (lane >> 2) * kPLd + 2 * (lane & 3);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float2*>(prow + 8 * j) =
                make_float2(div_by(expf(y[2 * j] - st.x), st.y, st.z), div_by(expf(y[2 * j + 1] - st.x), st.y, st.z));
          __syncwarp();
#pragma unroll
          for (int kk = 0; kk < 2; ++kk)
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) colsum[kk] += Pw[rr * kPLd + lane + 32 * kk];
          __syncwarp();
        }
      }
      __syncwarp();
      if (PASS == 1 && logits_out) {
#pragma unroll 4
        for (int rr = 0; rr < 16; ++rr) {
          const int r = r0 + warp * 16 + rr;
          if (r < bs && 2 * lane < nkeys) {
            T* dst = logits_out + ((int64_t)bh * bs + r) * L + (int64_t)jt * TN;
            *reinterpret_cast<uint32_t*>(dst + 2 * lane) = *reinterpret_cast<const uint32_t*>(stage + (warp * 16 + rr) * kStageLd + 2 * lane);
          }
        }
      }
      if (PASS == 2) {
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) gcur[((r0 >> 4) + warp) * TN + lane + 32 * kk] = colsum[kk];
      }
      __syncwarp();                                        // the warp's staging / probability tile is free again
    }
  }
  if (PASS == 2) {
    __syncthreads();
    finish_tile(ntiles_here - 1);
  }
}

// Merges the per-tile (max, sum) pairs into one pair per (b, h, row).  Per row there are 32 running
// pairs, pair l taking the tiles l, l + 32, ... one after the other, and the 32 pairs are then merged by a
// butterfly.  One CTA = 32 rows: warp l owns the running pairs number l of all 32 rows, so that its loads
// are 32 consecutive pairs (the statistics are stored tile-major, row-minor); the pairs then change hands
// through shared memory, warp j taking the 32 pairs of row j for the butterfly.
__global__ void __launch_bounds__(1024)
rowstats_kernel(const float2* __restrict__ partials, float2* __restrict__ rowstats, int ntile, int bs) {
  __shared__ float2 run[32][33];
  const int bh = blockIdx.y;
  const int r0 = blockIdx.x * 32;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    const int r = r0 + lane;
    const float2* p = partials + (int64_t)bh * ntile * bs + r;
    float m = -CUDART_INF_F, z = 0.f;
    if (r < bs) {
      int t = w;
      for (; t + 32 * 3 < ntile; t += 32 * 4) {           // four loads in flight
        float2 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = p[(int64_t)(t + 32 * u) * bs];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float mn = fmaxf(m, v[u].x);
          z = z * expf(m - mn) + v[u].y * expf(v[u].x - mn);
          m = mn;
        }
      }
      for (; t < ntile; t += 32) {
        const float2 v = p[(int64_t)t * bs];
        const float mn = fmaxf(m, v.x);
        z = z * expf(m - mn) + v.y * expf(v.x - mn);
        m = mn;
      }
    }
    run[w][lane] = make_float2(m, z);
  }
  __syncthreads();
  const int r = r0 + w;
  if (r >= bs) return;
  float m = run[lane][w].x, z = run[lane][w].y;
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

// Does rounding a * (1 / sqrt_d) to the 16-bit type T give the bits of rounding a / sqrt_d for every a?
// Tried once per (type, head_dim) over all 65536 bit patterns, on the host, with the device's arithmetic
// (IEEE fp32 product and quotient, round-to-nearest-even conversions).
template <int DT>
bool mul_equals_div(int D) {
  static std::mutex mu;
  static std::map<int, bool> known;
  std::lock_guard<std::mutex> lock(mu);
  auto it = known.find(D);
  if (it != known.end()) return it->second;
  const float sq = (float)sqrt((double)D);
  const volatile float rinv = 1.f / sq;
  bool same = true;
  for (uint32_t bits = 0; bits < 65536u && same; ++bits) {
    float a;
    uint16_t want, got;
    if (DT == PBS_BF16) {
      const uint32_t w = bits << 16;
      memcpy(&a, &w, 4);
      if (!std::isfinite(a)) continue;
      const volatile float quot = a / sq, prod = a * rinv;
      const __nv_bfloat16 x = __float2bfloat16_rn(quot), y = __float2bfloat16_rn(prod);
      memcpy(&want, &x, 2); memcpy(&got, &y, 2);
    } else {
      __half hv;
      const uint16_t hb = (uint16_t)bits;
      memcpy(&hv, &hb, 2);
      a = __half2float(hv);
      if (!std::isfinite(a)) continue;
      const volatile float quot = a / sq, prod = a * rinv;
      const __half x = __float2half_rn(quot), y = __float2half_rn(prod);
      memcpy(&want, &x, 2); memcpy(&got, &y, 2);
    }
    same = want == got;
  }
  known[D] = same;
  return same;
}

template <int DT>
int run(const Dims& d, const void* q, Strides qs, const void* k, Strides ks, void* logits, void* partials,
        void* rowstats, float* importance, cudaStream_t st) {
  using T = typename Elem<DT>::T;
  const int BH = d.B * d.Hq;
  const int ntile = (d.L + TN - 1) / TN;
  const float sq = (float)sqrt((double)d.D);
  const bool mma = DT != PBS_FP32 && d.D % 16 == 0 && qs.s % 8 == 0 && ks.s % 8 == 0 && d.bs % 16 == 0;
  // enough CTAs to fill the GPU a few times over, long enough runs of tiles to amortise the query block
  int tiles_per_cta = 16;
  while (tiles_per_cta > 1 && (int64_t)((ntile + tiles_per_cta - 1) / tiles_per_cta) * BH < 592) tiles_per_cta >>= 1;
  const int chunks = (ntile + tiles_per_cta - 1) / tiles_per_cta;
  const int qrows = (d.bs + 127) & ~127;
  const size_t smem_base = (size_t)(qrows + 2 * TN) * (d.D + 8) * sizeof(T);
  const size_t smem1 = smem_base + (logits ? (size_t)8 * 16 * kStageLd * sizeof(T) : 0);
  const size_t smem2 = smem_base + (size_t)(64 * kPLd + 2 * kMaxGroups * TN) * sizeof(float) + (size_t)d.bs * sizeof(float3);
  bool fastdiv = false;
  if constexpr (DT != PBS_FP32) fastdiv = mma && mul_equals_div<DT>(d.D);

  for (int pass = 1; pass <= 2; ++pass) {
    if constexpr (DT != PBS_FP32) {
      if (mma) {
        using Kern = void (*)(const T*, Strides, const T*, Strides, float2*, const float2*, float*, T*, int, int, int, int,
                              int, int, int, int, float);
        auto pick = [&](auto dh) -> Kern {
          constexpr int DH = decltype(dh)::value;
          return pass == 1 ? (fastdiv ? (Kern)score_mma_kernel<DT, 1, true, DH> : (Kern)score_mma_kernel<DT, 1, false, DH>)
                           : (fastdiv ? (Kern)score_mma_kernel<DT, 2, true, DH> : (Kern)score_mma_kernel<DT, 2, false, DH>);
        };
        Kern kern = d.D == 128 ? pick(std::integral_constant<int, 128>{})
                    : d.D == 64 ? pick(std::integral_constant<int, 64>{}) : pick(std::integral_constant<int, 0>{});
        const size_t smem = pass == 1 ? smem1 : smem2;
        if (smem > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
          if (e != cudaSuccess) return cuda_fail(e, "score_mma_kernel smem attribute");
        }
        kern<<<dim3(chunks * d.group, d.B * d.Hkv), 256, smem, st>>>(
            (const T*)q, qs, (const T*)k, ks, (float2*)partials, (const float2*)rowstats, importance,
            pass == 1 ? (T*)logits : nullptr, d.Hq, d.group, d.S, d.D, d.bs, d.L, ntile, tiles_per_cta, sq);
        PBS_CUDA_CHECK_LAUNCH("score_mma_kernel");
      }
    }
    if (!mma) {
      auto kern = pass == 1 ? score_kernel<DT, 1> : score_kernel<DT, 2>;
      kern<<<dim3(ntile, BH), 256, 0, st>>>(
          (const T*)q, qs, (const T*)k, ks, (float2*)partials, (const float2*)rowstats, importance,
          pass == 1 ? (T*)logits : nullptr, d.Hq, d.group, d.S, d.D, d.bs, d.L, sq);
      PBS_CUDA_CHECK_LAUNCH("score_kernel");
    }
    if (pass == 1) {
      rowstats_kernel<<<dim3((d.bs + 31) / 32, BH), 1024, 0, st>>>((const float2*)partials, (float2*)rowstats, ntile, d.bs);
      PBS_CUDA_CHECK_LAUNCH("rowstats_kernel");
    }
  }
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
