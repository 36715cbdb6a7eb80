// Forward entry point for callers that must not allocate device memory.
//
// The ordinary forward needs two intermediate tensors between its launches: the chunk-local
// cumulative log gate g_cum [rows, Hv] fp32 and the inverse A [rows, Hv, 64] bf16, which the
// Python wrappers allocate with torch.  Some hosts cannot do that at the point where they call
// this library: a serving engine that carved the whole device into its own arena at start-up and
// treats any later cudaMalloc as a bug (it synchronises the device and can fail once the arena
// owns the memory), or a plugin that is handed a stream and raw pointers by its framework and
// has no allocator of its own.  For them this file keeps the two intermediates in a file-scope
// device array of fixed size, so the call only needs the caller's inputs and outputs.
//
// The array is part of the loaded library image: every GPU that loads the library holds
// SCRATCH_BYTES of it until the process exits, whether or not this entry point is ever called.
#include <cuda_runtime.h>

#include <mutex>

#include "fqla_internal.h"

namespace {

// (token, value head) pairs one call may cover: e.g. 2048 tokens x 16 heads or 4096 x 8.
constexpr long long MAX_PAIRS = 32768;
constexpr size_t A_BYTES = (size_t)MAX_PAIRS * 64 * 2;  // A: 64 bf16 per pair
constexpr size_t G_BYTES = (size_t)MAX_PAIRS * 4;       // g_cum: one float per pair
constexpr size_t SCRATCH_BYTES = A_BYTES + G_BYTES;     // 4.125 MiB

static __device__ __align__(256) unsigned char g_noalloc_scratch[SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a handle for the runtime's symbol table, not a device
// address; the address on each device is looked up once, with that device current.
constexpr int MAX_DEVICES = 64;
std::mutex g_setup_lock;
unsigned char* g_scratch_on_device[MAX_DEVICES] = {};

int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return FQLA_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> hold(g_setup_lock);
  if (!g_scratch_on_device[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!ptr) return FQLA_ERR_INVALID_ARG;
    g_scratch_on_device[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = g_scratch_on_device[dev];
  return FQLA_OK;
}

}  // namespace

extern "C" long long fqla_fwd_noalloc_max_pairs(void) { return MAX_PAIRS; }

extern "C" int fqla_fwd_noalloc(const void* q, const void* k, const void* v, const float* g,
                                const void* beta, int beta_is_f32, const float* h0, float* ht,
                                void* o, int B, int T, int Hq, int Hv, int D, float scale,
                                const void* cu_seqlens, const void* chunk_offsets,
                                const void* chunk_indices, int idx_is64, int N,
                                long long num_chunks, void* stream) {
  if (!q || !k || !v || !g || !beta || !o || B <= 0 || T <= 0 || Hq <= 0 || Hv <= 0 || Hv % Hq)
    return FQLA_ERR_INVALID_ARG;
  if (D != 128 && D != 64) return FQLA_ERR_UNSUPPORTED_DIM;
  const long long pairs = (long long)B * T * Hv;
  if (pairs > MAX_PAIRS) return FQLA_ERR_TOO_LARGE;
  unsigned char* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != FQLA_OK) return rc;
  void* A = scratch;
  float* g_cum = reinterpret_cast<float*>(scratch + A_BYTES);
  cudaStream_t st = (cudaStream_t)stream;
  // The array still holds what the call before left there.  Every row of A and g_cum that belongs
  // to a sequence is rewritten below before it is read; rows of g_cum past the last packed
  // sequence are cleared so that no launch ever sees stale bits there.
  cudaError_t e = cudaMemsetAsync(g_cum, 0, (size_t)pairs * 4, st);
  if (e != cudaSuccess) return (int)e;
  rc = fqla_kkt_solve(k, beta, beta_is_f32, g, g_cum, A, B, T, Hq, Hv, D, cu_seqlens, idx_is64,
                      chunk_indices, num_chunks, stream);
  if (rc != FQLA_OK) return rc;
  return fqla_fwd_seq(q, k, v, A, g_cum, beta, beta_is_f32, h0, ht, o, nullptr, nullptr, nullptr,
                      nullptr, nullptr, nullptr, nullptr, nullptr, 0, B, T, Hq, Hv, D, scale,
                      cu_seqlens, chunk_offsets, idx_is64, N, 0, stream);
}
