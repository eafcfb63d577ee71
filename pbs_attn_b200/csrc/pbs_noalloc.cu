// pbs_key_importance_static: the key-importance stage for callers that cannot provide scratch memory.
//
// Some hosts of this library can hand it only their input and output buffers: a plugin boundary
// that owns all device memory itself, or a serving loop that is forbidden to call cudaMalloc once it
// is running because an allocation may synchronise the whole device and stall other streams.  For
// them this entry point keeps the stage's scratch (the per-tile and per-row softmax statistics of
// the last query block) in a fixed array that is part of the library image.
//
// The array costs PBS_STATIC_SCRATCH_BYTES (64 MiB) of device memory on every GPU that loads the
// library, for the life of the process.  Calls whose scratch would not fit are rejected.
#include <mutex>

#include "pbs_common.cuh"

namespace {

// In host code this name is only a handle for the runtime, not a device address: a kernel must be
// given the pointer that cudaGetSymbolAddress returns for it on the current device.
static __device__ __align__(256) unsigned char g_static_scratch[PBS_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_ptr[kMaxDevices] = {};

inline size_t round256(size_t x) { return (x + 255) & ~(size_t)255; }

}  // namespace

extern "C" int pbs_key_importance_static(const pbs_shape_t* shape, const void* q, const int64_t q_strides[4],
                                         const void* k, const int64_t k_strides[4], float* importance,
                                         void* stream) {
  pbs_scratch_sizes_t z;
  int rc = pbs_scratch_sizes(shape, &z);               // validates the shape
  if (rc != PBS_OK) return rc;
  const size_t partials_bytes = round256((size_t)z.partials * sizeof(float2));
  const size_t rowstats_bytes = round256((size_t)z.rowstats * sizeof(float2));
  const size_t need = partials_bytes + rowstats_bytes;
  if (need > (size_t)PBS_STATIC_SCRATCH_BYTES) {
    pbs::set_error("pbs_key_importance_static: this shape needs %zu bytes of scratch, the built-in array holds %zu; "
                   "use pbs_key_importance with caller-provided scratch",
                   need, (size_t)PBS_STATIC_SCRATCH_BYTES);
    return PBS_ERR_SHAPE;
  }
  // First call on a device: look the array's device address up (with that device current) and keep it.
  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return pbs::cuda_fail(ce, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) { pbs::set_error("device ordinal %d out of range", dev); return PBS_ERR_ARG; }
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
      void* ptr = nullptr;
      ce = cudaGetSymbolAddress(&ptr, g_static_scratch);
      if (ce != cudaSuccess) return pbs::cuda_fail(ce, "cudaGetSymbolAddress(static scratch)");
      g_scratch_ptr[dev] = static_cast<unsigned char*>(ptr);
    }
    base = g_scratch_ptr[dev];
  }
  // Every byte the stage reads from its scratch is written earlier in the same call (tile
  // statistics, row statistics), so nothing has to be cleared between calls.
  return pbs_key_importance(shape, q, q_strides, k, k_strides, nullptr, base, base + partials_bytes, importance, stream);
}
