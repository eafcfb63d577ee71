// Shared device/host helpers of the PBS prefill kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/pbs_b200.h"

namespace pbs {

// ---------------------------------------------------------------------------------------------
// Element types.  `rnd` rounds an fp32 value to the storage type and back: the reference runs its
// scoring GEMMs and divisions in the input dtype, so bf16/fp16 calls round at those points.
// ---------------------------------------------------------------------------------------------
template <int DT> struct Elem;
template <> struct Elem<PBS_BF16> {
  using T = __nv_bfloat16;
  static __device__ __forceinline__ float ld(const T* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ T cvt(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Elem<PBS_FP16> {
  using T = __half;
  static __device__ __forceinline__ float ld(const T* p) { return __half2float(*p); }
  static __device__ __forceinline__ T cvt(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float rnd(float x) { return __half2float(__float2half_rn(x)); }
};
template <> struct Elem<PBS_FP32> {
  using T = float;
  static __device__ __forceinline__ float ld(const T* p) { return *p; }
  static __device__ __forceinline__ T cvt(float x) { return x; }
  static __device__ __forceinline__ float rnd(float x) { return x; }
};

static inline __host__ __device__ int elem_bytes(int dt) { return dt == PBS_FP32 ? 4 : 2; }

// Strides of one (B, H, S, D) operand, in elements (d stride is 1).
struct Strides {
  int64_t b, h, s;
};

struct Dims {
  int B, Hq, Hkv, S, D, bs, seg;
  int nseg;   // complete segments
  int L;      // nseg * seg
  int nb;     // ceil(S / bs)
  int bps;    // blocks per segment
  int group;  // Hq / Hkv
};

static inline Dims make_dims(const pbs_shape_t& s) {
  Dims d;
  d.B = s.batch; d.Hq = s.q_heads; d.Hkv = s.kv_heads; d.S = s.seq_len; d.D = s.head_dim;
  d.bs = s.block_size; d.seg = s.segment_size;
  d.nseg = d.S / d.seg; d.L = d.nseg * d.seg; d.nb = (d.S + d.bs - 1) / d.bs; d.bps = d.seg / d.bs;
  d.group = d.Hq / d.Hkv;
  return d;
}

// Sum in the order of the CPU reduction the reference's means go through: items are added
// sequentially into a level-0 accumulator that is flushed into level 1 every 16 items, level 1
// into level 2 every 256, and the levels are added up at the end.  Keeping the same order keeps
// pooled means bit-identical to the reference's.
struct CascadeSum {
  float a0 = 0.f, a1 = 0.f, a2 = 0.f;
  int n = 0;
  __device__ __forceinline__ void add(float x) {
    a0 += x;
    ++n;
    if ((n & 15) == 0) {
      a1 += a0; a0 = 0.f;
      if ((n & 255) == 0) { a2 += a1; a1 = 0.f; }
    }
  }
  __device__ __forceinline__ float total() const { return (a0 + a1) + a2; }
};

// Monotone map float -> uint32 (larger float = larger key); NaN sorts above +inf like torch.sort.
__device__ __forceinline__ uint32_t float_order_key(float x) {
  if (x != x) return 0xFFFFFFFFu;
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// In-place bitonic sort of n (power of two) 64-bit keys in shared memory, descending.
__device__ __forceinline__ void bitonic_sort_desc(unsigned long long* keys, int n) {
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = threadIdx.x; i < n; i += blockDim.x) {
        int p = i ^ j;
        if (p > i) {
          unsigned long long a = keys[i], b = keys[p];
          bool desc = (i & k) == 0;
          if (desc ? (a < b) : (a > b)) { keys[i] = b; keys[p] = a; }
        }
      }
      __syncthreads();
    }
  }
}

// The same result with E keys per thread held in registers (thread t owns keys t*E .. t*E+E-1):
// compare-exchange distances below E stay inside a thread, distances below 32*E go through warp
// shuffles, and only the few larger ones through shared memory.  n is a power of two with
// E <= n <= E * blockDim.x; every thread of the block must call it.
template <int E>
__device__ __forceinline__ void bitonic_sort_desc_regs(unsigned long long* keys, int n) {
  const int base = (int)threadIdx.x * E;
  const bool active = base < n;
  unsigned long long x[E];
#pragma unroll
  for (int r = 0; r < E; ++r) x[r] = active ? keys[base + r] : 0ull;
  for (int k = 2; k <= n; k <<= 1) {
    for (int j = k >> 1; j >= E; j >>= 1) {
      const int tj = j / E;                                // distance of the partner thread
      const bool take_max = ((base & j) == 0) == ((base & k) == 0);
      if (tj >= 32) {
        __syncthreads();
        if (active) {
#pragma unroll
          for (int r = 0; r < E; ++r) keys[base + r] = x[r];
        }
        __syncthreads();
        if (active) {
#pragma unroll
          for (int r = 0; r < E; ++r) {
            const unsigned long long y = keys[(base + r) ^ j];
            x[r] = take_max ? (x[r] > y ? x[r] : y) : (x[r] < y ? x[r] : y);
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < E; ++r) {
          const unsigned long long y = __shfl_xor_sync(0xffffffffu, x[r], tj);
          x[r] = take_max ? (x[r] > y ? x[r] : y) : (x[r] < y ? x[r] : y);
        }
      }
    }
#pragma unroll
    for (int jj = E / 2; jj >= 1; jj >>= 1) {
      if (jj <= (k >> 1)) {
#pragma unroll
        for (int r = 0; r < E; ++r) {
          if ((r & jj) == 0) {
            const bool desc = ((base + r) & k) == 0;
            const unsigned long long a = x[r], b = x[r | jj];
            if (desc ? (a < b) : (a > b)) { x[r] = b; x[r | jj] = a; }
          }
        }
      }
    }
  }
  __syncthreads();
  if (active) {
#pragma unroll
    for (int r = 0; r < E; ++r) keys[base + r] = x[r];
  }
  __syncthreads();
}

static inline int next_pow2(int x) { int p = 1; while (p < x) p <<= 1; return p; }

// Error reporting of the C ABI (thread local message).
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

void count_launch();

#define PBS_CUDA_CHECK_LAUNCH(what)                                   \
  do {                                                                \
    cudaError_t e__ = cudaGetLastError();                             \
    if (e__ != cudaSuccess) return ::pbs::cuda_fail(e__, what);       \
    ::pbs::count_launch();                                            \
  } while (0)

// Stage launchers (defined one per .cu file).
int launch_key_importance(const Dims& d, int dt, const void* q, Strides qs, const void* k, Strides ks,
                          void* logits, void* partials, void* rowstats, float* importance, cudaStream_t st);
int launch_segment_permute(const Dims& d, int dt, const float* importance, const void* k, Strides ks,
                           const void* v, Strides vs, int32_t* idx, void* perm_k, void* perm_v,
                           void* pooled_k, int pool_mode, int32_t* first_block, cudaStream_t st);
int launch_pool_queries(const Dims& d, int dt, const void* q, Strides qs, void* pooled_q, int pool_mode,
                        cudaStream_t st);
int launch_rope(int dt, int B, int H, int S, int D, void* x, Strides xs, const void* cosp, const void* sinp,
                int64_t cs_b, int64_t cs_s, cudaStream_t st);
int launch_select_blocks(const Dims& d, int dt, const void* pooled_q, const void* pooled_k,
                         const int32_t* first_block, const pbs_options_t& opt, uint8_t* mask, float* scores,
                         cudaStream_t st);
void set_select_impl(int impl);
int launch_fill_mask_ones(const Dims& d, uint8_t* mask, cudaStream_t st);
int launch_build_tile_lists(const Dims& d, const uint8_t* mask, uint32_t* list, int32_t* count, cudaStream_t st);
int launch_attn_simt(const Dims& d, int dt, const void* q, Strides qs, const void* pk, const void* pv,
                     const int32_t* idx, const uint8_t* mask, void* out, Strides os, cudaStream_t st);
bool attn_tc_supported(const Dims& d, int dt);
void set_attn_wait(unsigned long long wait_ns, int drop_arrive);
int launch_attn_tc(const Dims& d, int dt, const void* q, Strides qs, const void* pk, const void* pv,
                   const int32_t* idx, const uint32_t* list, const int32_t* count, void* out, Strides os,
                   int32_t* status, const pbs_out_replicas_t* replicas, cudaStream_t st);

}  // namespace pbs
