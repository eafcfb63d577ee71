// Rotary position embedding of the projected queries / keys, in place, one pass over the tensor.
//
// The caller of the prefill path applies x * cos + rotate_half(x) * sin to Q and K with five
// element-wise tensor operations (reference: pbs_attn/patch/huggingface.py:14-26, called at :203).
// This kernel reads and writes every element once and reproduces the arithmetic of those operations
// exactly: each product and the sum are rounded to the tensor's type, as separate tensor ops do.
#include "pbs_common.cuh"

namespace pbs {
namespace {

template <int DT>
__global__ void __launch_bounds__(256)
rope_kernel(typename Elem<DT>::T* __restrict__ x, Strides xs, const typename Elem<DT>::T* __restrict__ cosp,
            const typename Elem<DT>::T* __restrict__ sinp, int64_t cs_b, int64_t cs_s, int H, int S, int D,
            int64_t n_chunks) {
  using E = Elem<DT>;
  using T = typename E::T;
  constexpr int EPV = 16 / (int)sizeof(T);                 // elements per 16-byte vector
  const int half = D / 2, cph = half / EPV;                // 16-byte chunks per half row
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_chunks; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % cph);
    int64_t r = i / cph;
    const int s = (int)(r % S);
    r /= S;
    const int h = (int)(r % H);
    const int b = (int)(r / H);
    T* row = x + (int64_t)b * xs.b + (int64_t)h * xs.h + (int64_t)s * xs.s;
    const T* crow = cosp + (int64_t)b * cs_b + (int64_t)s * cs_s;
    const T* srow = sinp + (int64_t)b * cs_b + (int64_t)s * cs_s;
    const uint4 x1v = *reinterpret_cast<const uint4*>(row + c * EPV);
    const uint4 x2v = *reinterpret_cast<const uint4*>(row + half + c * EPV);
    const uint4 c1v = *reinterpret_cast<const uint4*>(crow + c * EPV);
    const uint4 c2v = *reinterpret_cast<const uint4*>(crow + half + c * EPV);
    const uint4 s1v = *reinterpret_cast<const uint4*>(srow + c * EPV);
    const uint4 s2v = *reinterpret_cast<const uint4*>(srow + half + c * EPV);
    const T* x1 = reinterpret_cast<const T*>(&x1v);
    const T* x2 = reinterpret_cast<const T*>(&x2v);
    const T* c1 = reinterpret_cast<const T*>(&c1v);
    const T* c2 = reinterpret_cast<const T*>(&c2v);
    const T* s1 = reinterpret_cast<const T*>(&s1v);
    const T* s2 = reinterpret_cast<const T*>(&s2v);
    uint4 o1v, o2v;
    T* o1 = reinterpret_cast<T*>(&o1v);
    T* o2 = reinterpret_cast<T*>(&o2v);
#pragma unroll
    for (int t = 0; t < EPV; ++t) {
      const float a = E::ld(x1 + t), bb = E::ld(x2 + t);
      // first half: x1 * cos + (-x2) * sin; second half: x2 * cos + x1 * sin
      // (explicit single-rounding intrinsics: the compiler must not contract these into FMAs)
      o1[t] = E::cvt(__fadd_rn(E::rnd(__fmul_rn(a, E::ld(c1 + t))), E::rnd(__fmul_rn(-bb, E::ld(s1 + t)))));
      o2[t] = E::cvt(__fadd_rn(E::rnd(__fmul_rn(bb, E::ld(c2 + t))), E::rnd(__fmul_rn(a, E::ld(s2 + t)))));
    }
    *reinterpret_cast<uint4*>(row + c * EPV) = o1v;
    *reinterpret_cast<uint4*>(row + half + c * EPV) = o2v;
  }
}

}  // namespace

int launch_rope(int dt, int B, int H, int S, int D, void* x, Strides xs, const void* cosp, const void* sinp,
                int64_t cs_b, int64_t cs_s, cudaStream_t st) {
  const int esize = dt == PBS_FP32 ? 4 : 2;
  const int epv = 16 / esize;
  const int64_t n_chunks = (int64_t)B * H * S * (D / 2 / epv);
  if (n_chunks == 0) return PBS_OK;
  const int64_t want = (n_chunks + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 32 ? want : 148 * 32);
  switch (dt) {
    case PBS_BF16:
      rope_kernel<PBS_BF16><<<grid, 256, 0, st>>>((__nv_bfloat16*)x, xs, (const __nv_bfloat16*)cosp, (const __nv_bfloat16*)sinp, cs_b, cs_s, H, S, D, n_chunks);
      break;
    case PBS_FP16:
      rope_kernel<PBS_FP16><<<grid, 256, 0, st>>>((__half*)x, xs, (const __half*)cosp, (const __half*)sinp, cs_b, cs_s, H, S, D, n_chunks);
      break;
    default:
      rope_kernel<PBS_FP32><<<grid, 256, 0, st>>>((float*)x, xs, (const float*)cosp, (const float*)sinp, cs_b, cs_s, H, S, D, n_chunks);
  }
  PBS_CUDA_CHECK_LAUNCH("rope_kernel");
  return PBS_OK;
}

}  // namespace pbs
