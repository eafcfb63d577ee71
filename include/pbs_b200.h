/*
 * pbs_b200.h -- C ABI of the B200 (sm_100a) PBS-Attn prefill library, libpbs_b200.so.
 *
 * Every entry point takes raw DEVICE pointers, sizes and element strides, launches
 * its kernels on the given CUDA stream (of the CURRENT device: make the tensors' device
 * current before calling) and returns without synchronising.  Nothing here allocates:
 * scratch memory is passed in by the caller (sizes come from pbs_scratch_sizes), except
 * for pbs_key_importance_static, whose scratch is an array built into the library.
 * Return value: 0 on success, a negative pbs_status_t on a rejected call;
 * pbs_last_error_string() describes the last rejection on the calling thread.  Arguments
 * are validated before the first kernel is enqueued, so a call rejected with PBS_ERR_SHAPE,
 * _LAYOUT, _ARG or _UNSUPPORTED has launched nothing; PBS_ERR_CUDA reports a failing CUDA
 * call, after which earlier stages of the same call may already be on the stream.
 *
 * "Replaces" lines cite the reference project's Python interface that each entry
 * point stands in for (paths relative to the reference root, xinghaow99/pbs-attn).
 *
 * Tensors: q is (B, Hq, S, D), k and v are (B, Hkv, S, D) with Hkv dividing Hq; query
 * head h reads KV head h / (Hq / Hkv) (the reference repeats K/V to Hq heads before
 * its call, pbs_attn/patch/huggingface.py:209-211; passing the repeated tensors with
 * Hkv == Hq is equally valid).  Strides are in ELEMENTS, order (b, h, s, d); the d
 * stride must be 1, rows must start on 16-byte boundaries, head strides may be 0.
 */
#ifndef PBS_B200_H_
#define PBS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { PBS_BF16 = 0, PBS_FP16 = 1, PBS_FP32 = 2 } pbs_dtype_t;
typedef enum { PBS_POOL_MEAN = 0, PBS_POOL_MAX = 1 } pbs_pool_t;
typedef enum { PBS_ATTN_AUTO = 0, PBS_ATTN_SIMT = 1, PBS_ATTN_TCGEN05 = 2 } pbs_attn_impl_t;

typedef enum {
  PBS_OK = 0,
  PBS_ERR_SHAPE = -1,     /* unsupported or inconsistent sizes                         */
  PBS_ERR_LAYOUT = -2,    /* stride / alignment the kernels cannot read                */
  PBS_ERR_ARG = -3,       /* null pointer, bad enum                                    */
  PBS_ERR_CUDA = -4,      /* a CUDA runtime / driver call failed                       */
  PBS_ERR_UNSUPPORTED = -5 /* requested kernel cannot run this shape (e.g. tcgen05 path) */
} pbs_status_t;

/* Problem sizes shared by all entry points. */
typedef struct {
  int32_t batch;         /* B                                              */
  int32_t q_heads;       /* Hq                                             */
  int32_t kv_heads;      /* Hkv, divides Hq                                */
  int32_t seq_len;       /* S (q_len == kv_len: prefill)                   */
  int32_t head_dim;      /* D, multiple of 8, <= 256                       */
  int32_t block_size;    /* selection granularity, multiple of 16, <= 256  */
  int32_t segment_size;  /* permutation granularity, multiple of block_size */
  int32_t dtype;         /* pbs_dtype_t of q, k, v and the output          */
} pbs_shape_t;

/* Element counts (NOT bytes) of every scratch buffer for a shape. */
typedef struct {
  int64_t logits;        /* dtype   : (B, Hq, block_size, L), L = (S / seg) * seg.  OPTIONAL inspection
                                       output of stage 1a (the rounded scoring logits); the path itself never
                                       stores them, pass NULL                                              */
  int64_t partials;      /* float2  : (B, Hq, ceil(L / 64), block_size) per-tile row max / sum      */
  int64_t rowstats;      /* float2  : (B, Hq, block_size) row max and 1 / row sum                   */
  int64_t importance;    /* float   : (B, Hq, L)                                                    */
  int64_t key_indices;   /* int32   : (B, Hq, S)                                                    */
  int64_t perm_kv;       /* dtype   : (B, Hq, S, D), once for K and once for V                      */
  int64_t pooled;        /* dtype   : (B, Hq, nb, D), once for Q and once for K, nb = ceil(S / bs)  */
  int64_t first_block;   /* int32   : (B, Hq)                                                       */
  int64_t block_mask;    /* uint8   : (B, Hq, nb, nb)                                               */
  int64_t tile_list;     /* uint32  : (B, Hq, ceil(S / 256), ceil(S / 128))                         */
  int64_t tile_count;    /* int32   : (B, Hq, ceil(S / 256))                                        */
  int64_t status;        /* int32   : 8 words, device-side error flags                              */
} pbs_scratch_sizes_t;

/* Device pointers of the scratch buffers, sized by pbs_scratch_sizes. */
typedef struct {
  void* logits;          /* may be NULL (optional inspection output) */
  void* partials;
  void* rowstats;
  float* importance;
  int32_t* key_indices;
  void* perm_k;
  void* perm_v;
  void* pooled_q;
  void* pooled_k;
  int32_t* first_block;
  uint8_t* block_mask;
  uint32_t* tile_list;
  int32_t* tile_count;
  int32_t* status;
} pbs_scratch_t;

/* Extra destinations of the attention output.  The tcgen05 attention kernel writes every output row
 * to `out` and, with the same strides, to each of these pointers.  They may be buffers on PEER GPUs
 * of the node (mapped into this process, peer access enabled: pbs_enable_peer_access): a rank of a
 * head-sharded call then stores its heads straight into every rank's full (B, Hq, S, D) tensor from
 * the kernel's epilogue, plain stores over NVLink, and no all-gather follows.  Replaces the gather
 * after the call in a head-parallel deployment (the reference leaves it to Hugging Face tensor
 * parallelism, pbs_attn/patch/huggingface.py:194-199).  A peer's copy is complete once this rank's
 * kernel has finished AND the ranks have synchronised (e.g. a one-element all-reduce on the stream). */
#define PBS_MAX_OUT_REPLICAS 15
typedef struct {
  int32_t count;                          /* 0 .. PBS_MAX_OUT_REPLICAS */
  int32_t reserved;
  void* out[PBS_MAX_OUT_REPLICAS];        /* device pointers, 16-byte aligned rows like `out` */
} pbs_out_replicas_t;

/* Options of the whole-path call; mirrors the keyword arguments of
 * permuted_block_sparse_attn_fwd (pbs_attn/src/pbs.py:132-146). */
typedef struct {
  const float* threshold_per_head; /* device, (Hq) floats, or NULL to use `threshold`        */
  float threshold;                 /* cumulative-score threshold, compared in fp32           */
  int32_t select_all;              /* 1: threshold was the Python int 1 -> every candidate   */
  int32_t force_select_first_block;
  int32_t query_pool_mode;         /* pbs_pool_t                                             */
  int32_t key_pool_mode;           /* pbs_pool_t                                             */
  int32_t attn_impl;               /* pbs_attn_impl_t                                        */
  int32_t no_permutation;          /* 1: keys stay in place (identity order); with segment_size ==
                                      block_size and diagonal_candidates this is the reference's
                                      MeanPooling baseline (pbs_attn/baselines/MeanPooling.py:43-58)   */
  int32_t diagonal_candidates;     /* 1: the q block's own kv block is a selection candidate too
                                      (block-level causal mask incl. the diagonal, MeanPooling.py:43-48) */
  int32_t no_own_segment;          /* 1: the q block's own segment is NOT forced on (MeanPooling with
                                      force_select_current_block=False, MeanPooling.py:55-58 skipped)  */
  const pbs_out_replicas_t* out_replicas; /* NULL, or extra destinations of the output (tcgen05 kernel only) */
} pbs_options_t;

const char* pbs_last_error_string(void);
int pbs_version(void);
/* Number of kernels this library has launched in the calling process so far. */
int64_t pbs_launch_count(void);

/* Diagnostic.  Every device-side wait of the tcgen05 attention kernel is bounded; wait_ns sets the
 * bound for later launches of this process (0 restores the default of 2 s).  drop_arrive = 1 makes
 * the first softmax warpgroup of CTA 0 withhold one barrier arrive, so that exactly one wait runs
 * out: the kernel then returns with status[0] != 0 instead of a result.  The failure-path test uses
 * this (with a bound of a few milliseconds) to exercise the abort path without faulting or hanging
 * the GPU.  No counterpart in the reference. */
int pbs_debug_set_attn_wait(int64_t wait_ns, int32_t drop_arrive);

/* Diagnostic.  Stage 2b has two kernels that must give identical masks: a tiled one (16 q blocks per
 * CTA, cut found by bisection; used wherever it applies: up to 2048 blocks per row, pooled rows of 8,
 * 16 or 32 16-byte pieces) and the general one (one q block per CTA, full sort).  impl = 1 forces the
 * general kernel for later calls of this process, 0 restores the default.  The tests compare the two. */
int pbs_debug_set_select_impl(int32_t impl);

/* Validates the shape and fills the scratch element counts. */
int pbs_scratch_sizes(const pbs_shape_t* shape, pbs_scratch_sizes_t* sizes);

/* Stage 1a.  importance[b,h,j] = mean over the last block's queries of
 * softmax_j(q . k_j / sqrt(D)) over the keys of the complete segments.  Two passes that each
 * recompute the logits from K; only the per-tile statistics (partials, rowstats) are scratch.
 * logits: NULL, or a (B, Hq, block_size, L) buffer that receives the rounded scoring logits
 * (for inspection and tests; 16-byte aligned).
 * Replaces pbs_attn/src/permute_states.py:44-50 (inside last_block_attn_sorting). */
int pbs_key_importance(const pbs_shape_t* shape,
                       const void* q, const int64_t q_strides[4],
                       const void* k, const int64_t k_strides[4],
                       void* logits, void* partials, void* rowstats,
                       float* importance, void* stream);

/* Stage 1a without caller scratch.  No counterpart in the reference: it exists for hosts that can
 * pass only inputs and outputs and may not allocate device memory themselves (a plugin boundary
 * that owns all memory, a running serving loop where cudaMalloc could stall the device).  Same
 * result as pbs_key_importance; the per-tile and per-row softmax statistics live in an array built
 * into the library (PBS_STATIC_SCRATCH_BYTES on every GPU that loads it, until the process exits).  Shapes
 * whose scratch exceeds that size are rejected with PBS_ERR_SHAPE.  Never calls cudaMalloc/cudaFree.
 * The first call on a device looks up the array's address (cudaGetSymbolAddress, that device must be
 * current); make that first call before starting any stream capture.  All calls on a device share
 * the one array, which keeps the previous call's contents (the stage overwrites all it reads, so
 * nothing needs clearing): two calls that overlap on the GPU race -- serialise them on one stream. */
#define PBS_STATIC_SCRATCH_BYTES (64u << 20)
int pbs_key_importance_static(const pbs_shape_t* shape,
                              const void* q, const int64_t q_strides[4],
                              const void* k, const int64_t k_strides[4],
                              float* importance, void* stream);

/* Stage 1b.  Stable descending sort of the importance inside each segment, gather of
 * K and V rows into permuted order, block pooling of the permuted K, and the index of
 * the permuted block that holds original token 0.
 * Replaces pbs_attn/src/permute_states.py:52-83 (argsort + gather), pbs_attn/src/pbs.py:213-215
 * (V gather), pbs_attn/src/utils.py:24-27 (key pooling), pbs_attn/src/pbs.py:10-25 (first token). */
int pbs_segment_permute(const pbs_shape_t* shape, const float* importance,
                        const void* k, const int64_t k_strides[4],
                        const void* v, const int64_t v_strides[4],
                        int32_t* key_indices, void* perm_k, void* perm_v,
                        void* pooled_k, int32_t key_pool_mode, int32_t* first_block,
                        void* stream);

/* Caller side of the path (the step before it).  Rotary position embedding applied IN PLACE to a
 * (B, H, S, D) tensor of projected queries or keys: x <- x * cos + rotate_half(x) * sin, with each
 * product and the sum rounded to the tensor's type exactly as the separate tensor operations of
 * pbs_attn/patch/huggingface.py:14-26 (called at :203) round them.  cos and sin are (B or 1, S, D)
 * tables of the same type; cs_strides = {batch stride (0 to broadcast), position stride, 1}.
 * Each half row (head_dim / 2 elements) must be a whole number of 16-byte pieces. */
int pbs_apply_rope(int32_t dtype, int32_t batch, int32_t heads, int32_t seq_len, int32_t head_dim,
                   void* x, const int64_t x_strides[4], const void* cos_table, const void* sin_table,
                   const int64_t cs_strides[3], void* stream);

/* Stage 2a.  Block pooling of the queries.  Replaces pbs_attn/src/utils.py:18-21. */
int pbs_pool_queries(const pbs_shape_t* shape, const void* q, const int64_t q_strides[4],
                     void* pooled_q, int32_t query_pool_mode, void* stream);

/* Stage 2b.  Pooled logits, fp32 softmax over the kv blocks of earlier segments,
 * cumulative-threshold selection, then OR of the first-token block and of the q block's
 * own segment.  block_mask is (B, Hq, nb, nb) bytes of 0/1.  block_scores may be NULL; if given,
 * (B, Hq, nb, nb) floats receive the pooled softmax scores the reference's
 * permuted_block_selection also returns (0 outside the candidates; for inspection and tests).
 * Replaces pbs_attn/src/utils.py:30-34 (block_pooled_attn), :38-86 (select_blocks),
 * pbs_attn/src/pbs.py:95-127 (permuted_block_selection) and :209. */
int pbs_select_blocks(const pbs_shape_t* shape, const void* pooled_q, const void* pooled_k,
                      const int32_t* first_block, const pbs_options_t* options,
                      uint8_t* block_mask, float* block_scores, void* stream);

/* Stage 3a.  Per 256-query group, the compact list of 128-key tiles that any of its
 * query blocks selected (consumed by the tcgen05 attention kernel). */
int pbs_build_tile_lists(const pbs_shape_t* shape, const uint8_t* block_mask,
                         uint32_t* tile_list, int32_t* tile_count, void* stream);

/* Stage 3b.  Block-sparse causal flash-attention forward over permuted K/V; the output is
 * written in original token order with the given strides (queries are never permuted,
 * pbs_attn/src/pbs.py:191-193, so the inverse permutation is the identity and is folded
 * into the store).  Replaces the launch at pbs_attn/src/pbs.py:220-246 of the kernel
 * pbs_attn/src/kernels/permuted_block_sparse_attention.py:134-311.
 * status: 8 int32 words, zero on entry; word 0 becomes non-zero if a bounded device-side
 * wait ran out (the output is then invalid).  out_replicas: NULL or extra destinations. */
int pbs_attn_fwd(const pbs_shape_t* shape,
                 const void* q, const int64_t q_strides[4],
                 const void* perm_k, const void* perm_v, const int32_t* key_indices,
                 const uint8_t* block_mask, const uint32_t* tile_list, const int32_t* tile_count,
                 void* out, const int64_t out_strides[4],
                 int32_t attn_impl, int32_t* status, const pbs_out_replicas_t* out_replicas, void* stream);

/* CUDA IPC plumbing for output replicas on peer GPUs, one process per GPU on one node.  No
 * counterpart in the reference.
 *   pbs_ipc_export   handle (64 bytes, cudaIpcMemHandle_t) of the device allocation that contains
 *                    device_ptr, and device_ptr's byte offset inside it; the allocation must come
 *                    from cudaMalloc (PyTorch's default caching allocator qualifies).
 *   pbs_ipc_import   in ANOTHER process: maps that allocation into the current device's address
 *                    space (peer access is enabled as needed) and returns its base; open a given
 *                    handle once per process.
 *   pbs_ipc_release  unmaps it again. */
int pbs_ipc_export(const void* device_ptr, unsigned char handle[64], int64_t* offset);
int pbs_ipc_import(const unsigned char handle[64], void** base_ptr);
int pbs_ipc_release(void* base_ptr);

/* Enables access from the current device to memory of `peer_device` (cudaDeviceEnablePeerAccess; a
 * no-op when it is already enabled).  Needed once per process and peer before a pointer into that
 * peer's memory is used as an output replica.  No counterpart in the reference. */
int pbs_enable_peer_access(int32_t peer_device);

/* Whole path: stages 1a..3b in order on one stream.  For S <= segment_size it runs dense
 * causal attention like the reference (pbs_attn/src/pbs.py:175-182).
 * Replaces permuted_block_sparse_attn_fwd, pbs_attn/src/pbs.py:132-257. */
int pbs_prefill_fwd(const pbs_shape_t* shape,
                    const void* q, const int64_t q_strides[4],
                    const void* k, const int64_t k_strides[4],
                    const void* v, const int64_t v_strides[4],
                    void* out, const int64_t out_strides[4],
                    const pbs_options_t* options, const pbs_scratch_t* scratch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PBS_B200_H_ */
