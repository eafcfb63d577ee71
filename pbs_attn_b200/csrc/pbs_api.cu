// extern "C" entry points of libpbs_b200.so: argument validation, error strings, stage dispatch.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>

#include <cuda.h>

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

// The TMA descriptor of the query tensor cannot describe a broadcast (zero-stride) batch or head dimension.
bool q_layout_fits_tc(const Dims& d, const Strides& qs) {
  return (d.Hq == 1 || qs.h > 0) && (d.B == 1 || qs.b > 0);
}

int check_replicas(const pbs_out_replicas_t* r, int dt, const int64_t* out_strides) {
  if (!r) return PBS_OK;
  if (r->count < 0 || r->count > PBS_MAX_OUT_REPLICAS) { set_error("out_replicas: count %d outside 0..%d", r->count, PBS_MAX_OUT_REPLICAS); return PBS_ERR_ARG; }
  (void)dt; (void)out_strides;
  for (int i = 0; i < r->count; ++i) {
    if (!r->out[i]) { set_error("out_replicas: pointer %d is null", i); return PBS_ERR_ARG; }
    if ((uintptr_t)r->out[i] & 15) { set_error("out_replicas: pointer %d is not 16-byte aligned", i); return PBS_ERR_LAYOUT; }
  }
  return PBS_OK;
}

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

int pbs_debug_set_attn_wait(int64_t wait_ns, int32_t drop_arrive) {
  if (wait_ns < 0) { set_error("wait_ns must be >= 0 (0 restores the default)"); return PBS_ERR_ARG; }
  set_attn_wait((unsigned long long)wait_ns, drop_arrive);
  return PBS_OK;
}

int pbs_debug_set_select_impl(int32_t impl) {
  if (impl != 0 && impl != 1) { set_error("select impl %d: 0 (tiled where supported) or 1 (one row per CTA)", impl); return PBS_ERR_ARG; }
  set_select_impl(impl);
  return PBS_OK;
}

// ---- CUDA IPC plumbing for output replicas on peer GPUs (one process per GPU) ----
namespace {
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
GetAddressRangeFn address_range_fn() {
  static GetAddressRangeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (GetAddressRangeFn)p;
  }
  return fn;
}
}  // namespace

int pbs_ipc_export(const void* device_ptr, unsigned char handle[64], int64_t* offset) {
  PBS_NONNULL(device_ptr); PBS_NONNULL(handle); PBS_NONNULL(offset);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is 64 bytes");
  GetAddressRangeFn range = address_range_fn();
  if (!range) { set_error("cuMemGetAddressRange is not available from the driver"); return PBS_ERR_CUDA; }
  CUdeviceptr base = 0;
  size_t size = 0;
  CUresult r = range(&base, &size, (CUdeviceptr)(uintptr_t)device_ptr);
  if (r != CUDA_SUCCESS) { set_error("cuMemGetAddressRange failed with CUresult %d", (int)r); return PBS_ERR_CUDA; }
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base);
  if (e != cudaSuccess) return cuda_fail(e, "cudaIpcGetMemHandle");
  memcpy(handle, &h, 64);
  *offset = (int64_t)((uintptr_t)device_ptr - (uintptr_t)base);
  return PBS_OK;
}

int pbs_ipc_import(const unsigned char handle[64], void** base_ptr) {
  PBS_NONNULL(handle); PBS_NONNULL(base_ptr);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle");
  *base_ptr = p;
  return PBS_OK;
}

int pbs_ipc_release(void* base_ptr) {
  PBS_NONNULL(base_ptr);
  cudaError_t e = cudaIpcCloseMemHandle(base_ptr);
  if (e != cudaSuccess) return cuda_fail(e, "cudaIpcCloseMemHandle");
  return PBS_OK;
}

int pbs_enable_peer_access(int32_t peer_device) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (peer_device == dev) return PBS_OK;
  int can = 0;
  e = cudaDeviceCanAccessPeer(&can, dev, peer_device);
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceCanAccessPeer");
  if (!can) { set_error("device %d cannot access memory of device %d", dev, peer_device); return PBS_ERR_UNSUPPORTED; }
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); return PBS_OK; }
  if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceEnablePeerAccess");
  return PBS_OK;
}

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
  PBS_NONNULL(partials); PBS_NONNULL(rowstats); PBS_NONNULL(importance);
  if (((uintptr_t)partials & 7) || ((uintptr_t)rowstats & 7) || ((uintptr_t)importance & 3) || ((uintptr_t)logits & 15)) {
    set_error("key importance scratch: partials / rowstats need 8-byte, importance 4-byte, logits 16-byte alignment");
    return PBS_ERR_LAYOUT;
  }
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
                 const int64_t out_strides[4], int32_t attn_impl, int32_t* status,
                 const pbs_out_replicas_t* out_replicas, void* stream) {
  PBS_TRY(check_shape(shape));
  Strides qs, os;
  PBS_TRY(check_tensor("q", q, q_strides, shape->dtype, &qs));
  PBS_TRY(check_tensor("out", out, out_strides, shape->dtype, &os));
  PBS_TRY(check_replicas(out_replicas, shape->dtype, out_strides));
  const bool replicated = out_replicas && out_replicas->count > 0;
  PBS_NONNULL(perm_k); PBS_NONNULL(perm_v); PBS_NONNULL(key_indices);
  const Dims d = make_dims(*shape);
  const bool tc_ok = attn_tc_supported(d, shape->dtype) && q_layout_fits_tc(d, qs);
  if (attn_impl == PBS_ATTN_TCGEN05 && !tc_ok) {
    set_error("tcgen05 attention needs bf16/fp16, head_dim 64/128, block_size 64/128, segment_size %% 128 == 0 "
              "and non-zero batch / head strides of q");
    return PBS_ERR_UNSUPPORTED;
  }
  if (attn_impl == PBS_ATTN_TCGEN05 || (attn_impl == PBS_ATTN_AUTO && tc_ok)) {
    PBS_NONNULL(tile_list); PBS_NONNULL(tile_count); PBS_NONNULL(status);
    return launch_attn_tc(d, shape->dtype, q, qs, perm_k, perm_v, key_indices, tile_list, tile_count, out, os,
                          status, out_replicas, (cudaStream_t)stream);
  }
  if (attn_impl != PBS_ATTN_SIMT && attn_impl != PBS_ATTN_AUTO) { set_error("attn_impl %d unknown", attn_impl); return PBS_ERR_ARG; }
  if (replicated) { set_error("output replicas are written by the tcgen05 attention kernel only; this call runs the generic kernel"); return PBS_ERR_UNSUPPORTED; }
  PBS_NONNULL(block_mask);
  return launch_attn_simt(d, shape->dtype, q, qs, perm_k, perm_v, key_indices, block_mask, out, os, (cudaStream_t)stream);
}

int pbs_prefill_fwd(const pbs_shape_t* shape, const void* q, const int64_t q_strides[4], const void* k,
                    const int64_t k_strides[4], const void* v, const int64_t v_strides[4], void* out,
                    const int64_t out_strides[4], const pbs_options_t* options, const pbs_scratch_t* sc,
                    void* stream) {
  // ---- everything is validated before the first enqueue: a rejected call launches nothing
  PBS_TRY(check_shape(shape));
  PBS_NONNULL(options); PBS_NONNULL(sc);
  Strides qs, ks, vs, os;
  PBS_TRY(check_tensor("q", q, q_strides, shape->dtype, &qs));
  PBS_TRY(check_tensor("k", k, k_strides, shape->dtype, &ks));
  PBS_TRY(check_tensor("v", v, v_strides, shape->dtype, &vs));
  PBS_TRY(check_tensor("out", out, out_strides, shape->dtype, &os));
  PBS_TRY(check_pool(options->query_pool_mode));
  PBS_TRY(check_pool(options->key_pool_mode));
  PBS_NONNULL(sc->status); PBS_NONNULL(sc->key_indices); PBS_NONNULL(sc->perm_k); PBS_NONNULL(sc->perm_v);
  PBS_NONNULL(sc->pooled_k); PBS_NONNULL(sc->first_block); PBS_NONNULL(sc->block_mask);
  const bool dense = shape->seq_len <= shape->segment_size;
  pbs_shape_t attn_shape = *shape;
  if (dense) {
    // Dense causal attention (pbs_attn/src/pbs.py:175-182): identity order, one segment covering
    // the whole sequence, every block on; the element-wise position test supplies causality.
    const int bs = shape->block_size;
    attn_shape.segment_size = ((shape->seq_len + 127) / 128) * 128;
    if (attn_shape.segment_size % bs) attn_shape.segment_size = ((shape->seq_len + bs - 1) / bs) * bs;
  } else {
    PBS_NONNULL(sc->pooled_q);
    if (!options->no_permutation) { PBS_NONNULL(sc->partials); PBS_NONNULL(sc->rowstats); PBS_NONNULL(sc->importance); }
  }
  const Dims d = make_dims(attn_shape);
  int impl = options->attn_impl;
  if (impl != PBS_ATTN_AUTO && impl != PBS_ATTN_SIMT && impl != PBS_ATTN_TCGEN05) { set_error("attn_impl %d unknown", impl); return PBS_ERR_ARG; }
  const bool tc_ok = attn_tc_supported(d, shape->dtype) && q_layout_fits_tc(d, qs);
  if (impl == PBS_ATTN_TCGEN05 && !tc_ok) {
    set_error("tcgen05 attention needs bf16/fp16, head_dim 64/128, block_size 64/128, segment_size %% 128 == 0 "
              "and non-zero batch / head strides of q");
    return PBS_ERR_UNSUPPORTED;
  }
  if (impl == PBS_ATTN_AUTO) impl = tc_ok ? PBS_ATTN_TCGEN05 : PBS_ATTN_SIMT;
  if (impl == PBS_ATTN_TCGEN05) { PBS_NONNULL(sc->tile_list); PBS_NONNULL(sc->tile_count); }
  PBS_TRY(check_replicas(options->out_replicas, shape->dtype, out_strides));
  if (impl != PBS_ATTN_TCGEN05 && options->out_replicas && options->out_replicas->count > 0) {
    set_error("output replicas are written by the tcgen05 attention kernel only; this call runs the generic kernel");
    return PBS_ERR_UNSUPPORTED;
  }

  // ---- enqueue
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(sc->status, 0, 8 * sizeof(int32_t), st);
  if (e != cudaSuccess) return cuda_fail(e, "clear status");
  if (dense) {
    PBS_TRY(pbs_segment_permute(&attn_shape, nullptr, k, k_strides, v, v_strides, sc->key_indices, sc->perm_k,
                                sc->perm_v, sc->pooled_k, PBS_POOL_MEAN, sc->first_block, stream));
    PBS_TRY(launch_fill_mask_ones(d, sc->block_mask, st));
  } else {
    if (!options->no_permutation)
      PBS_TRY(pbs_key_importance(shape, q, q_strides, k, k_strides, sc->logits, sc->partials, sc->rowstats,
                                 sc->importance, stream));
    PBS_TRY(pbs_segment_permute(shape, options->no_permutation ? nullptr : sc->importance, k, k_strides, v, v_strides, sc->key_indices, sc->perm_k,
                                sc->perm_v, sc->pooled_k, options->key_pool_mode, sc->first_block, stream));
    PBS_TRY(pbs_pool_queries(shape, q, q_strides, sc->pooled_q, options->query_pool_mode, stream));
    PBS_TRY(pbs_select_blocks(shape, sc->pooled_q, sc->pooled_k, sc->first_block, options, sc->block_mask, nullptr, stream));
  }
  if (impl == PBS_ATTN_TCGEN05)
    PBS_TRY(pbs_build_tile_lists(&attn_shape, sc->block_mask, sc->tile_list, sc->tile_count, stream));
  return pbs_attn_fwd(&attn_shape, q, q_strides, sc->perm_k, sc->perm_v, sc->key_indices, sc->block_mask,
                      sc->tile_list, sc->tile_count, out, out_strides, impl, sc->status, options->out_replicas, stream);
}

}  // extern "C"
