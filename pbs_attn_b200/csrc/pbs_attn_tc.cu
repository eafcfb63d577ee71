// Stage 3b, Blackwell kernel: block-sparse causal flash-attention forward on tcgen05 tensor cores.
//
// Math follows the reference's Triton kernel (pbs_attn/src/kernels/permuted_block_sparse_attention.py
// :7-90,241-311): S = Q K^T accumulated in fp32, keys of the query tile's own segment are visible iff
// their original position <= the query's, online softmax in base 2, P rounded to the input dtype
// before P V, fp32 output accumulator, O / row-sum stored in the input dtype.
//
// Work item = 256 consecutive queries of one (b, h): two 128-row query tiles that share every K/V
// tile staged in shared memory.  The item's tile list (built by tile_list_kernel) names the 128-key
// tiles that either query tile selected.  A persistent CTA (one per SM) walks its items with
// twelve warps in four roles:
//   warp 0      TMA producer: Q tiles, then K and V tiles of the list into two 2-deep rings
//   warps 1, 3  MMA issuers, one per query tile.  A 128-key tile is two half-steps of 64 keys with
//               their own 64 TMEM columns: S_h = Q K_h^T (SS, both operands K-major, 128B swizzle,
//               M=128 N=64) and O += P_h V_h (TS: P_h read from TMEM, V MN-major from shared memory)
//   warp 2      owns the TMEM allocation (all 512 columns: per query tile S_0 S_1 (64 each) and O (128))
//   warps 4-7   softmax of query tile 0: per half-step tcgen05.ld S_h, mask, exp2 relative to the row
//   warps 8-11  softmax of query tile 1  maximum in use (the new maximum is computed beside it and only a
//               row that outgrew the lazy-rescale threshold makes the warp rescale O in TMEM and start
//               over), row sum, P_h written back over the first 32 columns of S_h as packed 16-bit
//               pairs; final O / l epilogue to global through a per-warp transposition tile
// An issuer runs, per list entry and half h: O += P_h V_h, then S_h of the next entry into the
// columns P_h vacated.  So while a softmax warpgroup works on one half, the MMAs of the other half
// (and of the other query tile) run, and the next S is ready when the warpgroup comes back for it.
// One issuer's barrier bookkeeping overlaps the other issuer's MMAs.
// Every wait on an mbarrier is bounded (2 s unless pbs_debug_set_attn_wait says otherwise); when one
// runs out the CTA raises a flag, all roles leave their loops, in-flight copies and MMAs are waited
// out (bounded), TMEM is freed and status[0] tells the host which wait it was.
#include <cuda.h>

#include <atomic>

#include "pbs_common.cuh"

namespace pbs {
namespace {

constexpr int kThreads = 384;
constexpr int NK = 2;                     // K ring depth
constexpr int NV = 2;                     // V ring depth
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.f;  // log2 units: O is rescaled only when the max grows by more

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// One lane of a fully converged warp; the surrounding code stays warp-uniform, which lets the
// compiler keep descriptors and addresses in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, %1;\n\t"
      "@px mov.s32 %0, 1;\n\t}"
      : "+r"(pred)
      : "r"(0xFFFFFFFFu));
  return pred != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// L2 eviction policies for the TMA loads: K/V tiles are re-read by every query group of the head
// (keep them), Q tiles are read once (let them go first).
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Executed by a converged warp; one elected lane commits.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  if (elect_one())
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem], accumulate flag known at compile time (no predicate set-up).
template <bool ACC>
__device__ __forceinline__ void mma_ss_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  if (elect_one())
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC ? 1 : 0)
      : "memory");
}
template <bool ACC>
__device__ __forceinline__ void mma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  if (elect_one())
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "n"(ACC ? 1 : 0)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (elect_one())
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100).
// lbo / sbo are byte offsets (multiples of 16).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float ex2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

template <int DT> struct PackP;
template <> struct PackP<PBS_BF16> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct PackP<PBS_FP16> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// ---------------------------------------------------------------------------------------------
// Shared-memory plan
// ---------------------------------------------------------------------------------------------
struct Bars {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[NK], k_empty[NK];
  uint64_t v_full[NV], v_empty[NV];
  uint64_t s_full[2][2], p_full[2][2], o_full[2][2];   // [query tile][key half]
  uint64_t drain;                                       // teardown after an abort: both issuers' MMAs retired
};

struct Params {
  const int32_t* idx;         // (B*Hq, S)
  const uint32_t* list;       // (B*Hq, G, T)
  const int32_t* count;       // (B*Hq, G)
  void* out;
  Strides os;
  int Hq, S, G, T, n_items;
  int bs;
  float scale_log2e;
  int32_t* status;
  void* extra_out[PBS_MAX_OUT_REPLICAS];   // further destinations of the output (same strides), e.g. on peer GPUs
  int n_extra;
  unsigned long long wait_ns;   // limit of every device-side wait
  int drop_arrive;              // diagnostic: CTA 0's first softmax warpgroup skips one arrive (a wait then runs out)
};

struct Ctl {
  uint32_t tmem_base;
  volatile int abort_flag;
  unsigned long long wait_ns;
};

// Work order.  Within a head the query groups are taken in the order G-1, 0, G-2, 1, ... and a CTA
// takes two consecutive positions at a time, i.e. a long group followed by the short group that
// complements it: every such pair has the same number of key tiles (2G + 2 in the dense case), so
// (a) the CTAs stay balanced without a dynamic queue and (b) all CTAs start their long group at the
// same time and walk up the head's key range together -- a K/V tile is then fetched from HBM once
// and served to the other CTAs from L2, instead of every CTA sweeping at its own position.
// n-th item of this CTA -> position in that order, or -1 past the end.
__device__ __forceinline__ int item_position(int n, int n_items) {
  const int pos = 2 * ((int)blockIdx.x + (n >> 1) * (int)gridDim.x) + (n & 1);
  return pos < n_items ? pos : -1;
}
__device__ __forceinline__ void item_decode(int pos, int G, int& bh, int& g) {
  bh = pos / G;
  const int r = pos % G;
  g = (r & 1) ? (r >> 1) : (G - 1 - (r >> 1));
}

// Bounded wait: false when the CTA is aborting (this wait or another one ran out of time).
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, Ctl* ctl, int32_t* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (ctl->abort_flag) return false;
      if (global_timer_ns() - t0 > ctl->wait_ns) {
        ctl->abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// The same for a whole converged warp: every lane polls, the verdict is made warp-uniform.
__device__ __forceinline__ bool wait_bar_warp(uint32_t bar, uint32_t parity, Ctl* ctl, int32_t* status, int code) {
  return __all_sync(0xffffffffu, wait_bar(bar, parity, ctl, status, code));
}

template <int D>
struct Smem {
  static constexpr int kTileBytes = 128 * D * 2;          // one 128-row tile
  static constexpr int kQ = 0;                            // 2 tiles
  static constexpr int kK = kQ + 2 * kTileBytes;          // NK tiles
  static constexpr int kV = kK + NK * kTileBytes;         // NV tiles
  static constexpr int kIdx = kV + NV * kTileBytes;       // 8 warps x 128 int32
  static constexpr int kStage = kIdx + 8 * 128 * 4;       // 8 warps x 32 rows x (64 + 16) bytes: epilogue transposition
  static constexpr int kStageRow = 80;                    // bytes per staged row piece (64 of data + 16 of padding)
  static constexpr int kBars = kStage + 8 * 32 * kStageRow;
  static constexpr int kCtl = kBars + (int)sizeof(Bars);
  static constexpr int kTotal = kCtl + (int)sizeof(Ctl) + 1024;   // + slack for 1024-byte alignment
};

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int DT, int D>
__global__ void __launch_bounds__(kThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, Params p) {
  using E = Elem<DT>;
  using T = typename E::T;
  using SM = Smem<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  Bars* bars = reinterpret_cast<Bars*>(smem + SM::kBars);
  Ctl* ctl = reinterpret_cast<Ctl*>(smem + SM::kCtl);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->q_full[i]), 1);
      mbar_init(smem_u32(&bars->q_empty[i]), 1);
      for (int h = 0; h < 2; ++h) {
        mbar_init(smem_u32(&bars->s_full[i][h]), 1);
        mbar_init(smem_u32(&bars->p_full[i][h]), 128);
        mbar_init(smem_u32(&bars->o_full[i][h]), 1);
      }
    }
    for (int i = 0; i < NK; ++i) { mbar_init(smem_u32(&bars->k_full[i]), 1); mbar_init(smem_u32(&bars->k_empty[i]), 2); }
    for (int i = 0; i < NV; ++i) { mbar_init(smem_u32(&bars->v_full[i]), 1); mbar_init(smem_u32(&bars->v_empty[i]), 2); }
    mbar_init(smem_u32(&bars->drain), 2);
    ctl->abort_flag = 0;
    ctl->wait_ns = p.wait_ns;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  const uint32_t tmem_S[2] = {tmem + 0u, tmem + 128u};
  const uint32_t tmem_O[2] = {tmem + 256u, tmem + 384u};

  constexpr int KH = D / 64;                              // 64-column (128-byte) slabs per tile row
  constexpr uint32_t kSlab = 128 * 128;                   // bytes of one 128-row slab
  constexpr uint32_t kTile = SM::kTileBytes;
  // instruction descriptors: fp32 accumulate, A/B = bf16 or fp16, M = 128
  constexpr uint32_t kFmt = (DT == PBS_BF16) ? 1u : 0u;
  constexpr uint32_t kIdescQK = (1u << 4) | (kFmt << 7) | (kFmt << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);   // N = 64
  constexpr uint32_t kIdescPV = (1u << 4) | (kFmt << 7) | (kFmt << 10) | (1u << 16) | (((uint32_t)D >> 3) << 17) | ((128u >> 4) << 24);


#if PBS_SETMAXNREG
  // The softmax warps hold a half-step of S in registers; the four warps of the other roles need few.
  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PBS_SETMAXNREG));
  else asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(((64512 - 128 * PBS_SETMAXNREG) / 256) & ~7));
#endif

  if (warp == 0) {
    // =========================================================================== TMA producer
    // The whole warp walks the lists (uniform control flow); one elected lane issues the copies.
    {
      uint32_t kc = 0, vc = 0, qc[2] = {0, 0};
      bool ok = true;
      const uint64_t pol_kv = l2_policy_evict_last(), pol_q = l2_policy_evict_first();
      for (int it = 0, pos; (pos = item_position(it, p.n_items)) >= 0 && ok; ++it) {
        int bh, g;
        item_decode(pos, p.G, bh, g);
        const int b = bh / p.Hq, h = bh % p.Hq;
        for (int i = 0; i < 2 && ok; ++i) {
          const int r0 = g * 256 + i * 128;
          if (r0 >= p.S) continue;
          ok = wait_bar_warp(smem_u32(&bars->q_empty[i]), (qc[i] & 1u) ^ 1u, ctl, p.status, 1);
          if (!ok) break;
          const uint32_t bar = smem_u32(&bars->q_full[i]);
          if (elect_one()) {
            mbar_expect_tx(bar, kTile);
            for (int kh = 0; kh < KH; ++kh)
              tma_load_4d(sbase + SM::kQ + i * kTile + kh * kSlab, &map_q, bar, kh * 64, r0, h, b, pol_q);
          }
          ++qc[i];
        }
        const int n = p.count[(int64_t)bh * p.G + g];
        const uint32_t* lst = p.list + ((int64_t)bh * p.G + g) * p.T;
        uint32_t ent = n > 0 ? lst[0] : 0u;
        for (int e = 0; e < n && ok; ++e) {
          const int t = (int)(ent & 0xFFFFu);
          if (e + 1 < n) ent = lst[e + 1];                 // fetched one entry ahead of its use
          {
            const uint32_t s = kc % NK;
            ok = wait_bar_warp(smem_u32(&bars->k_empty[s]), ((kc / NK) & 1u) ^ 1u, ctl, p.status, 2);
            if (!ok) break;
            const uint32_t bar = smem_u32(&bars->k_full[s]);
            if (elect_one()) {
              mbar_expect_tx(bar, kTile);
              for (int kh = 0; kh < KH; ++kh)
                tma_load_3d(sbase + SM::kK + s * kTile + kh * kSlab, &map_k, bar, kh * 64, t * 128, bh, pol_kv);
            }
            ++kc;
          }
          {
            const uint32_t s = vc % NV;
            ok = wait_bar_warp(smem_u32(&bars->v_empty[s]), ((vc / NV) & 1u) ^ 1u, ctl, p.status, 3);
            if (!ok) break;
            const uint32_t bar = smem_u32(&bars->v_full[s]);
            if (elect_one()) {
              mbar_expect_tx(bar, kTile);
              for (int kh = 0; kh < KH; ++kh)
                tma_load_3d(sbase + SM::kV + s * kTile + kh * kSlab, &map_v, bar, kh * 64, t * 128, bh, pol_kv);
            }
            ++vc;
          }
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // =========================================================================== MMA issuers
    // Warp 1 issues for query tile 0, warp 3 for query tile 1.  Control flow is uniform for the
    // whole warp; each tcgen05.mma / commit is issued by one elected lane.  Both warps walk the
    // whole list (the K/V ring is indexed by list position) and act on the entries their tile uses;
    // a ring stage is free again once BOTH have committed on its `empty` barrier.  The bookkeeping
    // of one warp (barrier waits, list reads) overlaps the other warp's MMAs on the tensor pipe.
    {
      const int i = warp >> 1;                              // query tile of this issuer
      uint32_t kc = 0, vc = 0, qc = 0, pc = 0;
      bool ok = true;
      const uint32_t use_bit = 1u << (16 + i);

      // Descriptors are built once; per instruction only a compile-time constant is added to the
      // start-address field.
      const uint64_t dq = smem_desc(sbase + SM::kQ + i * kTile, 16, 1024);
      const uint32_t bar_sfull[2] = {smem_u32(&bars->s_full[i][0]), smem_u32(&bars->s_full[i][1])};
      const uint32_t bar_ofull[2] = {smem_u32(&bars->o_full[i][0]), smem_u32(&bars->o_full[i][1])};
      const uint32_t tS = tmem_S[i], tO = tmem_O[i];

      // A 128-key tile is processed as two half-steps of 64 keys (h = 0, 1), each with its own 64
      // columns of S, so that the softmax of one half overlaps the MMAs of the other.
      // S_h = Q K_h^T: M = 128, N = 64; K_h = rows 64h .. 64h+63 of the staged K tile.
      auto issue_qk = [&](uint32_t kstage, int h) {
        const uint64_t b0 = smem_desc(sbase + SM::kK + kstage * kTile + h * 64 * 128, 16, 1024);
        const uint32_t d = tS + 64 * h;
        mma_ss_c<false>(d, dq, b0, kIdescQK);
#pragma unroll
        for (int ks = 1; ks < D / 16; ++ks) {
          const uint64_t off = (uint64_t)(((ks >> 2) * kSlab + (ks & 3) * 32) >> 4);
          mma_ss_c<true>(d, dq + off, b0 + off, kIdescQK);
        }
        tc_commit(bar_sfull[h]);
      };
      // O += P_h V_h: P_h (64 keys as 32 columns of 16-bit pairs) sits in the first half of S_h.
      auto issue_pv = [&](uint32_t vstage, bool accumulate, int h) {
        const uint64_t b0 = smem_desc(sbase + SM::kV + vstage * kTile, kSlab, 1024) + (uint64_t)h * ((4 * 2048) >> 4);
        const uint32_t a0 = tS + 64 * h;
        mma_ts(tO, a0, b0, kIdescPV, accumulate);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) mma_ts_c<true>(tO, a0 + ks * 8, b0 + (uint64_t)((ks * 2048) >> 4), kIdescPV);
        tc_commit(bar_ofull[h]);
      };

      for (int it = 0, pos; (pos = item_position(it, p.n_items)) >= 0 && ok; ++it) {
        int bh, g;
        item_decode(pos, p.G, bh, g);
        const int n = p.count[(int64_t)bh * p.G + g];
        const uint32_t* lst = p.list + ((int64_t)bh * p.G + g) * p.T;
        const bool have = g * 256 + i * 128 < p.S;
        if (have) {
          ok = wait_bar_warp(smem_u32(&bars->q_full[i]), qc & 1u, ctl, p.status, 4);
          ++qc;
          if (!ok) break;
        }
        bool started = false;                               // O_i holds a partial sum of this item
        uint32_t cur = n > 0 ? lst[0] : 0u;
        uint32_t nxt = n > 1 ? lst[1] : 0u;
        if (n > 0) {
          // A stage's `full` barrier is awaited even when this tile skips the entry: an issuer must
          // not arrive on `empty` for a later round of the stage before the other issuer has arrived
          // for this one.
          const uint32_t s = kc % NK;
          ok = wait_bar_warp(smem_u32(&bars->k_full[s]), (kc / NK) & 1u, ctl, p.status, 5);
          if (!ok) break;
          if (cur & use_bit) {
            tc_fence_after();
            issue_qk(s, 0);
            issue_qk(s, 1);
          }
          tc_commit(smem_u32(&bars->k_empty[s]));
          ++kc;
        }
        for (int e = 0; e < n && ok; ++e) {
          const uint32_t nn = (e + 2 < n) ? lst[e + 2] : 0u;    // read two entries ahead of its use
          const uint32_t vs = vc % NV, ks = kc % NK;
          ok = wait_bar_warp(smem_u32(&bars->v_full[vs]), (vc / NV) & 1u, ctl, p.status, 6);
          if (!ok) break;
          if (nxt) {
            ok = wait_bar_warp(smem_u32(&bars->k_full[ks]), (kc / NK) & 1u, ctl, p.status, 8);
            if (!ok) break;
          }
          // per half: O += P_h V_h of this entry, then S_h of the next entry into the columns that
          // P_h just vacated
#pragma unroll
          for (int h = 0; h < 2 && ok; ++h) {
            if (cur & use_bit) {
              ok = wait_bar_warp(smem_u32(&bars->p_full[i][h]), pc & 1u, ctl, p.status, 7);
              if (!ok) break;
              tc_fence_after();
              issue_pv(vs, started || h == 1, h);
            }
            if (nxt & use_bit) {
              tc_fence_after();
              issue_qk(ks, h);
            }
          }
          if (!ok) break;
          if (cur & use_bit) {
            ++pc;
            started = true;
          }
          tc_commit(smem_u32(&bars->v_empty[vs]));
          ++vc;
          if (nxt) {
            tc_commit(smem_u32(&bars->k_empty[ks]));
            ++kc;
          }
          cur = nxt;
          nxt = nn;
        }
        if (!ok) break;
        if (have) tc_commit(smem_u32(&bars->q_empty[i]));
      }
      // Abort path: this commit arrives once every MMA this warp issued has retired.
      if (ctl->abort_flag) tc_commit(smem_u32(&bars->drain));
    }
  } else if (warp >= 4) {
    // =========================================================================== softmax + epilogue
    const int i = (warp - 4) >> 2;                         // query tile of this warpgroup
    const int wq = warp & 3;                               // TMEM lane quarter of this warp
    const int row = wq * 32 + lane;
    const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
    int32_t* kidx = reinterpret_cast<int32_t*>(smem + SM::kIdx) + (warp - 4) * 128;
    const uint32_t bar_s[2] = {smem_u32(&bars->s_full[i][0]), smem_u32(&bars->s_full[i][1])};
    const uint32_t bar_p[2] = {smem_u32(&bars->p_full[i][0]), smem_u32(&bars->p_full[i][1])};
    const uint32_t bar_o[2] = {smem_u32(&bars->o_full[i][0]), smem_u32(&bars->o_full[i][1])};
    uint32_t sc = 0;                                       // list entries done by this warpgroup
    bool ok = true;

    for (int it = 0, pos; (pos = item_position(it, p.n_items)) >= 0 && ok; ++it) {
      int bh, g;
      item_decode(pos, p.G, bh, g);
      const int r0 = g * 256 + i * 128;
      if (r0 >= p.S) continue;
      const int b = bh / p.Hq, h = bh % p.Hq;
      const int qpos = r0 + row;
      const int n = p.count[(int64_t)bh * p.G + g];
      const uint32_t* lst = p.list + ((int64_t)bh * p.G + g) * p.T;
      const int32_t* ibase = p.idx + (int64_t)bh * p.S;
      float m_used = -CUDART_INF_F;                        // scaled (log2) max the exponents refer to
      float l = 0.f;
      uint32_t steps = 0;                                  // entries of this item done

      uint32_t ent_next = n > 0 ? lst[0] : 0u;
      for (int e = 0; e < n && ok; ++e) {
        const uint32_t ent = ent_next;
        if (e + 1 < n) ent_next = lst[e + 1];              // fetched one entry ahead of its use
        if (!(ent & (1u << (16 + i)))) continue;
        const int t = (int)(ent & 0xFFFFu);
        const bool elem_mask = ent & (1u << (18 + i));
        const uint32_t bits = (ent >> (20 + 4 * i)) & 0xFu;
        if (elem_mask) {
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int kp = t * 128 + c * 32 + lane;
            kidx[c * 32 + lane] = kp < p.S ? ibase[kp] : 0x7fffffff;
          }
          __syncwarp();
        }

        // Two half-steps of 64 keys, each an ordinary online-softmax step on its own 64 columns of S.
#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
          ok = __all_sync(0xffffffffu, wait_bar(bar_s[hs], sc & 1u, ctl, p.status, 9));
          if (!ok) break;
          tc_fence_after();
          const uint32_t s_addr = tmem_S[i] + lane_off + 64 * hs;

          // S_h is read from TMEM once and stays in registers for the maximum and the exponentiation.
          uint32_t sr[2][32];
          tmem_ld32(s_addr, sr[0]);
          tmem_ld32(s_addr + 32, sr[1]);
          tmem_wait_ld();
          float (&v)[64] = *reinterpret_cast<float (*)[64]>(&sr[0][0]);
          // masks: keys of the own segment that lie after the query; with block_size 64 the 64x64
          // sub-block (query half, key half) may not be selected
          if (elem_mask) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (kidx[64 * hs + c] > qpos) v[c] = -CUDART_INF_F;
          }
          if (p.bs == 64 && !((bits >> (2 * (row >> 6) + hs)) & 1u)) {
#pragma unroll
            for (int c = 0; c < 64; ++c) v[c] = -CUDART_INF_F;
          }
          // Row maximum (four independent chains) and, without waiting for it, the exponentials relative to
          // the maximum in use: the lazy rescale keeps that maximum for almost every half-step, so the chain
          // of maxima leaves the critical path.  When a row's maximum did grow past the threshold (always in
          // a row's first half-step) the warp rescales and exponentiates again.
          float mx4[4];
#pragma unroll
          for (int a = 0; a < 4; ++a) {
            float m = max3(v[16 * a], v[16 * a + 1], v[16 * a + 2]);
#pragma unroll
            for (int c = 3; c + 1 < 16; c += 2) m = max3(m, v[16 * a + c], v[16 * a + c + 1]);
            mx4[a] = fmaxf(m, v[16 * a + 15]);
          }
          const float2 sc2 = make_float2(p.scale_log2e, p.scale_log2e);
          float2 acc2[2];
          // P_h goes back over the first 32 columns of S_h in two stores of 32 keys
          auto exp_pass = [&](float m_ref) {
            const float2 nm2 = make_float2(-m_ref, -m_ref);
            acc2[0] = make_float2(0.f, 0.f);
            acc2[1] = make_float2(0.f, 0.f);
            uint32_t pk[16];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                const int col = 32 * q + 2 * c;
                const float2 x = __ffma2_rn(make_float2(v[col], v[col + 1]), sc2, nm2);
                const float2 ex = make_float2(ex2(x.x), ex2(x.y));
                acc2[c & 1] = __fadd2_rn(acc2[c & 1], ex);
                pk[c] = PackP<DT>::pack(ex.x, ex.y);
              }
              tmem_st16(s_addr + 16 * q, pk);
            }
          };
          exp_pass(m_used == -CUDART_INF_F ? 0.f : m_used);
          const float mt = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2e;
          const bool grew = mt > m_used + kRescaleThreshold;   // also the first finite maximum
          if (__any_sync(0xffffffffu, grew)) {
            float alpha = 1.f;
            if (grew) {
              alpha = ex2(m_used - mt);                      // 0 when m_used is -inf
              m_used = mt;
              l *= alpha;
            }
            if (steps > 0 || hs == 1) {
              // O_i holds the sum up to the previous half-step: wait for that P V, then scale in place.
              // Half 0 follows the second half of the previous entry, half 1 the first half of this one.
              const uint32_t par = hs == 0 ? ((sc - 1u) & 1u) : (sc & 1u);
              ok = __all_sync(0xffffffffu, wait_bar(bar_o[hs ^ 1], par, ctl, p.status, 10));
              if (!ok) break;
              tc_fence_after();
#pragma unroll
              for (int c = 0; c < D / 16; ++c) {
                uint32_t o[16];
                tmem_ld16(tmem_O[i] + lane_off + c * 16, o);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                tmem_st16(tmem_O[i] + lane_off + c * 16, o);
              }
            }
            exp_pass(m_used == -CUDART_INF_F ? 0.f : m_used);
          }
          tmem_wait_st();
          tc_fence_before();
          // diagnostic hook of the failure-path test: the very first hand-over of CTA 0 is withheld,
          // so the issuer's wait for it runs out and the CTA takes the abort path
          if (!(p.drop_arrive && blockIdx.x == 0 && i == 0 && sc == 0 && hs == 0)) mbar_arrive(bar_p[hs]);
          l += (acc2[0].x + acc2[0].y) + (acc2[1].x + acc2[1].y);
        }
        if (!ok) break;
        ++sc;
        ++steps;
      }
      if (!ok) break;

      // epilogue: O / l in the input dtype, original token order (queries are not permuted)
      if (steps > 0) {
        ok = __all_sync(0xffffffffu, wait_bar(bar_o[1], (sc - 1u) & 1u, ctl, p.status, 11));
        if (!ok) break;
        tc_fence_after();
      }
      // Rows leave through a per-warp transposition tile: a thread owns one row of O in TMEM, but four
      // lanes then store one row's 64-byte piece together, so a store instruction writes 8 rows x 64
      // contiguous bytes instead of 32 rows x 16 -- this matters for the replicas, which travel over NVLink.
      const float inv = l > 0.f ? 1.f / l : 0.f;
      unsigned char* stage = smem + SM::kStage + (warp - 4) * 32 * SM::kStageRow;
      const int64_t obase = (int64_t)b * p.os.b + (int64_t)h * p.os.h;
      const int wrow0 = r0 + wq * 32;                      // first query row of this warp
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (steps > 0) {
          tmem_ld32(tmem_O[i] + lane_off + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 w;
          w.x = PackP<DT>::pack(__uint_as_float(o[8 * j + 0]) * inv, __uint_as_float(o[8 * j + 1]) * inv);
          w.y = PackP<DT>::pack(__uint_as_float(o[8 * j + 2]) * inv, __uint_as_float(o[8 * j + 3]) * inv);
          w.z = PackP<DT>::pack(__uint_as_float(o[8 * j + 4]) * inv, __uint_as_float(o[8 * j + 5]) * inv);
          w.w = PackP<DT>::pack(__uint_as_float(o[8 * j + 6]) * inv, __uint_as_float(o[8 * j + 7]) * inv);
          *reinterpret_cast<uint4*>(stage + lane * SM::kStageRow + j * 16) = w;
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int rr = (lane >> 2) + 8 * j, piece = lane & 3;
          const int grow = wrow0 + rr;
          if (grow < p.S) {
            const uint4 w = *reinterpret_cast<const uint4*>(stage + rr * SM::kStageRow + piece * 16);
            const int64_t off = obase + (int64_t)grow * p.os.s + c * 32 + piece * 8;
            __stcs(reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.out) + off), w);   // written once, not re-read here
            // replicas (peer GPUs of a head-sharded call): plain stores, they travel over NVLink
            for (int x = 0; x < p.n_extra; ++x)
              *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.extra_out[x]) + off) = w;
          }
        }
        __syncwarp();
      }
      // the next item's first P V overwrites O_i: order our TMEM reads before the arrive that lets it go
      tc_fence_before();
    }
  }

  // =============================================================================== teardown
  // After an abort, work may still be in flight when the roles leave their loops: TMA copies into
  // this CTA's shared memory and MMAs into its TMEM.  Neither may outlive the CTA, so everybody
  // first lets the copies land (a copy takes a few microseconds; 100 us, bounded) and the TMEM owner
  // waits (bounded again) until both issuers' MMAs have retired before it frees the columns.
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (ctl->abort_flag) {
    for (int n = 0; n < 100; ++n) __nanosleep(1000);
    if (warp == 2) {
      const uint64_t t0 = global_timer_ns();
      while (!mbar_try_wait(smem_u32(&bars->drain), 0) && global_timer_ns() - t0 < 2000000ull) { }
      tc_fence_after();
    }
    __syncthreads();
  }
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
// Limit of every device-side wait and the diagnostic hook, process wide (pbs_debug_set_attn_wait).
std::atomic<unsigned long long> g_wait_ns{2000000000ull};
std::atomic<int> g_drop_arrive{0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int make_map(CUtensorMap* map, int dt, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return PBS_ERR_CUDA; }
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, dt == PBS_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank,
                  const_cast<void*>(base), dims, strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r); return PBS_ERR_CUDA; }
  return PBS_OK;
}

template <int DT, int D>
int run_tc(const Dims& d, const void* q, Strides qs, const void* pk, const void* pv, const int32_t* idx,
           const uint32_t* list, const int32_t* count, void* out, Strides os, int32_t* status,
           const pbs_out_replicas_t* replicas, cudaStream_t st) {
  CUtensorMap mq, mk, mv;
  const cuuint64_t e = 2;
  {
    // q: (D, S, Hq, B) with the caller's strides; size-1 dims get a harmless stride
    cuuint64_t dims[4] = {(cuuint64_t)d.D, (cuuint64_t)d.S, (cuuint64_t)d.Hq, (cuuint64_t)d.B};
    cuuint64_t row = (cuuint64_t)qs.s * e;
    cuuint64_t sh = d.Hq > 1 ? (cuuint64_t)qs.h * e : row * d.S;
    cuuint64_t sb = d.B > 1 ? (cuuint64_t)qs.b * e : (d.Hq > 1 ? sh * d.Hq : row * d.S);
    if (sh == 0 || sb == 0) { set_error("q: zero head/batch stride is not supported by the tcgen05 kernel"); return PBS_ERR_LAYOUT; }
    cuuint64_t strides[3] = {row, sh, sb};
    int rc = make_map(&mq, DT, q, 4, dims, strides);
    if (rc) return rc;
  }
  {
    cuuint64_t dims[3] = {(cuuint64_t)d.D, (cuuint64_t)d.S, (cuuint64_t)d.B * d.Hq};
    cuuint64_t strides[2] = {(cuuint64_t)d.D * e, (cuuint64_t)d.S * d.D * e};
    int rc = make_map(&mk, DT, pk, 3, dims, strides);
    if (rc) return rc;
    rc = make_map(&mv, DT, pv, 3, dims, strides);
    if (rc) return rc;
  }
  Params p;
  p.idx = idx; p.list = list; p.count = count; p.out = out; p.os = os;
  p.Hq = d.Hq; p.S = d.S; p.G = (d.S + 255) / 256; p.T = (d.S + 127) / 128;
  p.n_items = d.B * d.Hq * p.G;
  p.bs = d.bs;
  p.scale_log2e = (float)(1.4426950408889634 / sqrt((double)d.D));
  p.status = status;

  p.n_extra = replicas ? replicas->count : 0;
  for (int x = 0; x < PBS_MAX_OUT_REPLICAS; ++x) p.extra_out[x] = x < p.n_extra ? replicas->out[x] : nullptr;
  p.wait_ns = g_wait_ns.load(std::memory_order_relaxed);
  p.drop_arrive = g_drop_arrive.load(std::memory_order_relaxed);
  int dev = 0, sm_count = 0;                               // of the device this launch goes to
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      sm_count <= 0)
    sm_count = 148;
  auto kern = attn_tc_kernel<DT, D>;
  const int smem = Smem<D>::kTotal;
  cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (ce != cudaSuccess) return cuda_fail(ce, "attn_tc_kernel smem attribute");
  const int pairs = (p.n_items + 1) / 2;
  const int grid = pairs < sm_count ? pairs : sm_count;
  kern<<<grid, kThreads, smem, st>>>(mq, mk, mv, p);
  PBS_CUDA_CHECK_LAUNCH("attn_tc_kernel");
  return PBS_OK;
}

}  // namespace

void set_attn_wait(unsigned long long wait_ns, int drop_arrive) {
  g_wait_ns.store(wait_ns ? wait_ns : 2000000000ull, std::memory_order_relaxed);
  g_drop_arrive.store(drop_arrive ? 1 : 0, std::memory_order_relaxed);
}

bool attn_tc_supported(const Dims& d, int dt) {
  return (dt == PBS_BF16 || dt == PBS_FP16) && (d.D == 64 || d.D == 128) && (d.bs == 64 || d.bs == 128) &&
         (d.seg % 128 == 0 || (d.seg == 64 && d.bs == 64)) && (d.S + 127) / 128 <= 0xFFFF;
}

int launch_attn_tc(const Dims& d, int dt, const void* q, Strides qs, const void* pk, const void* pv,
                   const int32_t* idx, const uint32_t* list, const int32_t* count, void* out, Strides os,
                   int32_t* status, const pbs_out_replicas_t* replicas, cudaStream_t st) {
  if (dt == PBS_BF16) {
    if (d.D == 128) return run_tc<PBS_BF16, 128>(d, q, qs, pk, pv, idx, list, count, out, os, status, replicas, st);
    return run_tc<PBS_BF16, 64>(d, q, qs, pk, pv, idx, list, count, out, os, status, replicas, st);
  }
  if (d.D == 128) return run_tc<PBS_FP16, 128>(d, q, qs, pk, pv, idx, list, count, out, os, status, replicas, st);
  return run_tc<PBS_FP16, 64>(d, q, qs, pk, pv, idx, list, count, out, os, status, replicas, st);
}

}  // namespace pbs
