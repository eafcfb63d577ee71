// extern "C" entry points of libpbs_b200.so: argument validation, error strings, stage dispatch.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>

#include "pbs_common.cuh"

namespace pbs {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return PBS_ERR_CUDA;
}

namespace {

int check_shape(const pbs_shape_t* s) {
  if (!s) { set_error("shape is null"); return PBS_ERR_ARG; }
  if (s->dtype < PBS_BF16 || s->dtype > PBS_FP32) { set_error("dtype %d is not bf16/fp16/fp32", s->dtype); return PBS_ERR_ARG; }
  if (s->batch < 1 || s->q_heads < 1 || s->kv_heads < 1 || s->seq_len < 1) {
    set_error("batch, heads and seq_len must be positive (got B=%d Hq=%d Hkv=%d S=%d)", s->batch, s->q_heads, s->kv_heads, s->seq_len);
    return PBS_ERR_SHAPE;
  }
  if (s->q_heads % s->kv_heads) { set_error("kv_heads %d does not divide q_heads %d", s->kv_heads, s->q_heads); return PBS_ERR_SHAPE; }
  if (s->head_dim < 8 || s->head_dim > 256 || s->head_dim % 8) { set_error("head_dim %d: need a multiple of 8 in [8, 256]", s->head_dim); return PBS_ERR_SHAPE; }
  if (s->block_size < 16 || s->block_size > 256 || s->block_size % 16) { set_error("block_size %d: need a multiple of 16 in [16, 256]", s->block_size); return PBS_ERR_SHAPE; }
  if (s->segment_size < s->block_size || s->segment_size % s->block_size) {
    set_error("segment_size %d must be a multiple of block_size %d", s->segment_size, s->block_size);
    return PBS_ERR_SHAPE;
  }
  if (s->segment_size > 4096) { set_error("segment_size %d > 4096 is not supported", s->segment_size); return PBS_ERR_SHAPE; }
  if ((s->seq_len + s->block_size - 1) / s->block_size > 4096) {
    set_error("seq_len %d with block_size %d gives more than 4096 blocks per row", s->seq_len, s->block_size);
    return PBS_ERR_SHAPE;
  }
  return PBS_OK;
}

int check_tensor(const char* name, const void* p, const int64_t* st, int dt, Strides* out) {
  if (!p || !st) { set_error("%s: null pointer or strides", name); return PBS_ERR_ARG; }
  const int e = elem_bytes(dt);
  if (st[3] != 1) { set_error("%s: innermost (head_dim) stride is %lld, must be 1", name, (long long)st[3]); return PBS_ERR_LAYOUT; }
  if (((uintptr_t)p & 15) || ((st[0] * e) & 15) || ((st[1] * e) & 15) || ((st[2] * e) & 15)) {
    set_error("%s: base pointer and every row must be 16-byte aligned", name);
    return PBS_ERR_LAYOUT;
  }
  if (st[0] < 0 || st[1] < 0 || st[2] <= 0) { set_error("%s: negative or zero-length row stride", name); return PBS_ERR_LAYOUT; }
  out->b = st[0]; out->h = st[1]; out->s = st[2];
  return PBS_OK;
}

#define PBS_TRY(x) do { int rc__ = (x); if (rc__ != PBS_OK) return rc__; } while (0)
#define PBS_NONNULL(p) do { if (!(p)) { set_error(#p " is null"); return PBS_ERR_ARG; } } while (0)

int check_pool(int mode) {
  if (mode != PBS_POOL_MEAN && mode != PBS_POOL_MAX) { set_error("Invalid pool mode: %d", mode); return PBS_ERR_ARG; }
  return PBS_OK;
}

}  // namespace
}  // namespace pbs

using namespace pbs;

extern "C" {

const char* pbs_last_error_string(void) { return g_err; }
int pbs_version(void) { return 100; }
int64_t pbs_launch_count(void) { return (int64_t)g_launches.load(); }

int pbs_scratch_sizes(const pbs_shape_t* shape, pbs_scratch_sizes_t* z) {
  PBS_TRY(check_shape(shape));
  PBS_NONNULL(z);
  const Dims d = make_dims(*shape);
  const int64_t BH = (int64_t)d.B * d.Hq;
  z->logits = BH * d.bs * d.L;
  z->partials = BH * ((d.L + 63) / 64) * d.bs;
  z->rowstats = BH * d.bs;
  z->importance = BH * d.L;
  z->key_indices = BH * d.S;
  z->perm_kv = BH * d.S * d.D;
  z->pooled = BH * d.nb * d.D;
  z->first_block = BH;
  z->block_mask = BH * d.nb * d.nb;
  z->tile_list = BH * ((d.S + 255) / 256) * ((d.S + 127) / 128);
  z->tile_count = BH * ((d.S + 255) / 256);
  z->status = 8;
  return PBS_OK;
}

int pbs_key_importance(const pbs_shape_t* shape, const void* q, const int64_t q_strides[4],
                       const void* k, const int64_t k_strides[4], void* logits, void* partials,
                       void* rowstats, float* importance, void* stream) {
  PBS_TRY(check_shape(shape));
  Strides qs, ks;
  PBS_TRY(check_tensor("q", q, q_strides, shape->dtype, &qs));
  PBS_TRY(check_tensor("k", k, k_strides, shape->dtype, &ks));
  PBS_NONNULL(logits); PBS_NONNULL(partials); PBS_NONNULL(rowstats); PBS_NONNULL(importance);
  const Dims d = make_dims(*shape);
  if (d.S < d.bs) { set_error("seq_len %d shorter than block_size %d", d.S, d.bs); return PBS_ERR_SHAPE; }
  return launch_key_importance(d, shape->dtype, q, qs, k, ks, logits, partials, rowstats, importance, (cudaStream_t)stream);
}

int pbs_segment_permute(const pbs_shape_t* shape, const float* importance, const void* k,
                        const int64_t k_strides[4], const void* v, const int64_t v_strides[4],
                        int32_t* key_indices, void* perm_k, void* perm_v, void* pooled_k,
                        int32_t key_pool_mode, int32_t* first_block, void* stream) {
  PBS_TRY(check_shape(shape));
  PBS_TRY(check_pool(key_pool_mode));
  Strides ks, vs;
  PBS_TRY(check_tensor("k", k, k_strides, shape->dtype, &ks));
  PBS_TRY(check_tensor("v", v, v_strides, shape->dtype, &vs));
  PBS_NONNULL(key_indices); PBS_NONNULL(perm_k); PBS_NONNULL(perm_v); PBS_NONNULL(pooled_k); PBS_NONNULL(first_block);
  Dims d = make_dims(*shape);
  if (!importance) { d.nseg = 0; d.L = 0; }          // identity order (dense fallback)
  return launch_segment_permute(d, shape->dtype, importance, k, ks, v, vs, key_indices, perm_k, perm_v,
                                pooled_k, key_pool_mode, first_block, (cudaStream_t)stream);
}

int pbs_pool_queries(const pbs_shape_t* shape, const void* q, const int64_t q_strides[4], void* pooled_q,
                     int32_t query_pool_mode, void* stream) {
  PBS_TRY(check_shape(shape));
  PBS_TRY(check_pool(query_pool_mode));
  Strides qs;
  PBS_TRY(check_tensor("q", q, q_strides, shape->dtype, &qs));
  PBS_NONNULL(pooled_q);
  return launch_pool_queries(make_dims(*shape), shape->dtype, q, qs, pooled_q, query_pool_mode, (cudaStream_t)stream);
}

int pbs_apply_rope(int32_t dtype, int32_t batch, int32_t heads, int32_t seq_len, int32_t head_dim,
                   void* x, const int64_t x_strides[4], const void* cos_table, const void* sin_table,
                   const int64_t cs_strides[3], void* stream) {
  if (dtype < PBS_BF16 || dtype > PBS_FP32) { set_error("dtype %d is not bf16/fp16/fp32", dtype); return PBS_ERR_ARG; }
  if (batch < 1 || heads < 1 || seq_len < 1) { set_error("batch, heads and seq_len must be positive"); return PBS_ERR_SHAPE; }
  const int e = elem_bytes(dtype);
  if (head_dim < 2 || head_dim % 2 || (head_dim / 2 * e) % 16) {
    set_error("head_dim %d: half a row must be a whole number of 16-byte pieces", head_dim);
    return PBS_ERR_SHAPE;
  }
  Strides xs;
  PBS_TRY(check_tensor("x", x, x_strides, dtype, &xs));
  PBS_NONNULL(cos_table); PBS_NONNULL(sin_table); PBS_NONNULL(cs_strides);
  if (cs_strides[2] != 1 || cs_strides[0] < 0 || cs_strides[1] <= 0 || ((cs_strides[0] * e) & 15) || ((cs_strides[1] * e) & 15) ||
      ((uintptr_t)cos_table & 15) || ((uintptr_t)sin_table & 15)) {
    set_error("cos/sin tables: need unit innermost stride and 16-byte aligned rows");
    return PBS_ERR_LAYOUT;
  }
  return launch_rope(dtype, batch, heads, seq_len, head_dim, x, xs, cos_table, sin_table, cs_strides[0], cs_strides[1],
                     (cudaStream_t)stream);
}

int pbs_select_blocks(const pbs_shape_t* shape, const void* pooled_q, const void* pooled_k,
                      const int32_t* first_block, const pbs_options_t* options, uint8_t* block_mask,
                      float* block_scores, void* stream) {
  PBS_TRY(check_shape(shape));
  PBS_NONNULL(pooled_q); PBS_NONNULL(pooled_k); PBS_NONNULL(first_block); PBS_NONNULL(options); PBS_NONNULL(block_mask);
  return launch_select_blocks(make_dims(*shape), shape->dtype, pooled_q, pooled_k, first_block, *options, block_mask,
                              block_scores, (cudaStream_t)stream);
}

int pbs_build_tile_lists(const pbs_shape_t* shape, const uint8_t* block_mask, uint32_t* tile_list,
                         int32_t* tile_count, void* stream) {
  PBS_TRY(check_shape(shape));
  PBS_NONNULL(block_mask); PBS_NONNULL(tile_list); PBS_NONNULL(tile_count);
  const Dims d = make_dims(*shape);
  if (d.bs != 64 && d.bs != 128) { set_error("tile lists need block_size 64 or 128 (got %d)", d.bs); return PBS_ERR_UNSUPPORTED; }
  if (d.seg % 128 && !(d.seg == 64 && d.bs == 64)) { set_error("tile lists need segment_size %% 128 == 0, or 64 with block_size 64 (got %d)", d.seg); return PBS_ERR_UNSUPPORTED; }
  return launch_build_tile_lists(d, block_mask, tile_list, tile_count, (cudaStream_t)stream);
}

int pbs_attn_fwd(const pbs_shape_t* shape, const void* q, const int64_t q_strides[4], const void* perm_k,
                 const void* perm_v, const int32_t* key_indices, const uint8_t* block_mask,
                 const uint32_t* tile_list, const int32_t* tile_count, void* out,
                 const int64_t out_strides[4], int32_t attn_impl, int32_t* status, void* stream) {
  PBS_TRY(check_shape(shape));
  Strides qs, os;
  PBS_TRY(check_tensor("q", q, q_strides, shape->dtype, &qs));
  PBS_TRY(check_tensor("out", out, out_strides, shape->dtype, &os));
  PBS_NONNULL(perm_k); PBS_NONNULL(perm_v); PBS_NONNULL(key_indices);
  const Dims d = make_dims(*shape);
  const bool tc_ok = attn_tc_supported(d, shape->dtype);
  if (attn_impl == PBS_ATTN_TCGEN05 && !tc_ok) {
    set_error("tcgen05 attention needs bf16/fp16, head_dim 64/128, block_size 64/128, segment_size %% 128 == 0");
    return PBS_ERR_UNSUPPORTED;
  }
  if (attn_impl == PBS_ATTN_TCGEN05 || (attn_impl == PBS_ATTN_AUTO && tc_ok)) {
    PBS_NONNULL(tile_list); PBS_NONNULL(tile_count); PBS_NONNULL(status);
    return launch_attn_tc(d, shape->dtype, q, qs, perm_k, perm_v, key_indices, tile_list, tile_count, out, os,
                          status, (cudaStream_t)stream);
  }
  if (attn_impl != PBS_ATTN_SIMT && attn_impl != PBS_ATTN_AUTO) { set_error("attn_impl %d unknown", attn_impl); return PBS_ERR_ARG; }
  PBS_NONNULL(block_mask);
  return launch_attn_simt(d, shape->dtype, q, qs, perm_k, perm_v, key_indices, block_mask, out, os, (cudaStream_t)stream);
}

int pbs_prefill_fwd(const pbs_shape_t* shape, const void* q, const int64_t q_strides[4], const void* k,
                    const int64_t k_strides[4], const void* v, const int64_t v_strides[4], void* out,
                    const int64_t out_strides[4], const pbs_options_t* options, const pbs_scratch_t* sc,
                    void* stream) {
  PBS_TRY(check_shape(shape));
  PBS_NONNULL(options); PBS_NONNULL(sc);
  PBS_NONNULL(sc->status);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(sc->status, 0, 8 * sizeof(int32_t), st);
  if (e != cudaSuccess) return cuda_fail(e, "clear status");

  pbs_shape_t attn_shape = *shape;
  if (shape->seq_len <= shape->segment_size) {
    // Dense causal attention (pbs_attn/src/pbs.py:175-182): identity order, one segment covering
    // the whole sequence, every block on; the element-wise position test supplies causality.
    const int bs = shape->block_size;
    attn_shape.segment_size = ((shape->seq_len + 127) / 128) * 128;
    if (attn_shape.segment_size % bs) attn_shape.segment_size = ((shape->seq_len + bs - 1) / bs) * bs;
    PBS_TRY(pbs_segment_permute(&attn_shape, nullptr, k, k_strides, v, v_strides, sc->key_indices, sc->perm_k,
                                sc->perm_v, sc->pooled_k, PBS_POOL_MEAN, sc->first_block, stream));
    PBS_NONNULL(sc->block_mask);
    PBS_TRY(launch_fill_mask_ones(make_dims(attn_shape), sc->block_mask, st));
  } else {
    if (!options->no_permutation)
      PBS_TRY(pbs_key_importance(shape, q, q_strides, k, k_strides, sc->logits, sc->partials, sc->rowstats,
                                 sc->importance, stream));
    PBS_TRY(pbs_segment_permute(shape, options->no_permutation ? nullptr : sc->importance, k, k_strides, v, v_strides, sc->key_indices, sc->perm_k,
                                sc->perm_v, sc->pooled_k, options->key_pool_mode, sc->first_block, stream));
    PBS_TRY(pbs_pool_queries(shape, q, q_strides, sc->pooled_q, options->query_pool_mode, stream));
    PBS_TRY(pbs_select_blocks(shape, sc->pooled_q, sc->pooled_k, sc->first_block, options, sc->block_mask, nullptr, stream));
  }
  const Dims d = make_dims(attn_shape);
  int impl = options->attn_impl;
  const bool tc_ok = attn_tc_supported(d, shape->dtype);
  if (impl == PBS_ATTN_AUTO) impl = tc_ok ? PBS_ATTN_TCGEN05 : PBS_ATTN_SIMT;
  if (impl == PBS_ATTN_TCGEN05 && tc_ok)
    PBS_TRY(pbs_build_tile_lists(&attn_shape, sc->block_mask, sc->tile_list, sc->tile_count, stream));
  return pbs_attn_fwd(&attn_shape, q, q_strides, sc->perm_k, sc->perm_v, sc->key_indices, sc->block_mask,
                      sc->tile_list, sc->tile_count, out, out_strides, impl, sc->status, stream);
}

}  // extern "C"
