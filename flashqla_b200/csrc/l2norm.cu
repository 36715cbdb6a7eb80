// Row-wise L2 normalisation of q / k (the optional pre-op `use_qk_l2norm_in_kernel`) and its
// gradient.  Replaces the torch.compile'd expressions of the reference's
// flash_qla/utils/math.py:9-20 (y = x * rsqrt(sum x^2 + eps), rstd returned in fp32) and :38-51
// (dx = (dy - <dy, y> y) * rstd, fp32).  One warp per row, the row held in registers between the
// reduction and the write: every element is read once and written once (HBM-bound; for D = 128
// bf16 the forward moves 516 bytes per row).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "fqla_internal.h"

namespace fqla {

namespace {

constexpr int MAX_PER_LANE = 16;  // D <= 32 * MAX_PER_LANE = 512

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

// two consecutive elements, element index even
template <typename T>
__device__ __forceinline__ float2 load2(const T* p);
template <>
__device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <>
__device__ __forceinline__ float2 load2<__half>(const __half* p) {
  return __half22float2(*reinterpret_cast<const __half2*>(p));
}
template <>
__device__ __forceinline__ float2 load2<float>(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
template <typename T>
__device__ __forceinline__ void store2(T* p, float a, float b);
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
template <>
__device__ __forceinline__ void store2<__half>(__half* p, float a, float b) {
  *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
}
template <>
__device__ __forceinline__ void store2<float>(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
  return x;
}

// lane l owns the element pairs l, l + 32, ... of its row (PAIRS = D / 64 of them, rounded up)
template <typename T, int PAIRS>
__global__ void __launch_bounds__(256) l2norm_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                         float* __restrict__ rstd, long long rows,
                                                         int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * D;
  float2 v[PAIRS];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const int c = 2 * (lane + 32 * i);
    v[i] = c < D ? load2<T>(xr + c) : make_float2(0.f, 0.f);
    ss += v[i].x * v[i].x + v[i].y * v[i].y;
  }
  const float r = rsqrtf(warp_sum(ss) + eps);
  T* yr = y + row * D;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const int c = 2 * (lane + 32 * i);
    if (c < D) store2<T>(yr + c, v[i].x * r, v[i].y * r);
  }
  if (lane == 0) rstd[row] = r;
}

template <typename TY, typename TD, int PAIRS>
__global__ void __launch_bounds__(256) l2norm_bwd_kernel(const TY* __restrict__ y,
                                                         const float* __restrict__ rstd,
                                                         const TD* __restrict__ dy,
                                                         float* __restrict__ dx, long long rows,
                                                         int D) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const TY* yr = y + row * D;
  const TD* gr = dy + row * D;
  float2 a[PAIRS], g[PAIRS];
  float dot = 0.f;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const int c = 2 * (lane + 32 * i);
    a[i] = c < D ? load2<TY>(yr + c) : make_float2(0.f, 0.f);
    g[i] = c < D ? load2<TD>(gr + c) : make_float2(0.f, 0.f);
    dot += a[i].x * g[i].x + a[i].y * g[i].y;
  }
  dot = warp_sum(dot);
  const float r = rstd[row];
  float* out = dx + row * D;
#pragma unroll
  for (int i = 0; i < PAIRS; ++i) {
    const int c = 2 * (lane + 32 * i);
    if (c < D) store2<float>(out + c, (g[i].x - dot * a[i].x) * r, (g[i].y - dot * a[i].y) * r);
  }
}

template <typename T>
int launch_fwd(const void* x, void* y, float* rstd, long long rows, int D, float eps,
               cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + 7) / 8);
  const int pairs = (D + 63) / 64;
  auto go = [&](auto tag) {
    constexpr int P = decltype(tag)::value;
    l2norm_fwd_kernel<T, P><<<grid, 256, 0, st>>>((const T*)x, (T*)y, rstd, rows, D, eps);
  };
  if (pairs <= 1) go(std::integral_constant<int, 1>{});
  else if (pairs <= 2) go(std::integral_constant<int, 2>{});
  else if (pairs <= 4) go(std::integral_constant<int, 4>{});
  else go(std::integral_constant<int, MAX_PER_LANE / 2>{});
  return (int)cudaGetLastError();
}

template <typename TY, typename TD>
int launch_bwd(const void* y, const float* rstd, const void* dy, float* dx, long long rows, int D,
               cudaStream_t st) {
  const unsigned grid = (unsigned)((rows + 7) / 8);
  const int pairs = (D + 63) / 64;
  auto go = [&](auto tag) {
    constexpr int P = decltype(tag)::value;
    l2norm_bwd_kernel<TY, TD, P><<<grid, 256, 0, st>>>((const TY*)y, rstd, (const TD*)dy, dx, rows,
                                                       D);
  };
  if (pairs <= 1) go(std::integral_constant<int, 1>{});
  else if (pairs <= 2) go(std::integral_constant<int, 2>{});
  else if (pairs <= 4) go(std::integral_constant<int, 4>{});
  else go(std::integral_constant<int, MAX_PER_LANE / 2>{});
  return (int)cudaGetLastError();
}

}  // namespace

}  // namespace fqla

using namespace fqla;

extern "C" int fqla_l2norm_fwd(const void* x, void* y, float* rstd, long long rows, int D,
                               int dtype, float eps, void* stream) {
  if (!x || !y || !rstd || rows < 0 || D <= 0 || D % 2 || D > 32 * MAX_PER_LANE)
    return FQLA_ERR_INVALID_ARG;
  if (rows == 0) return FQLA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case DT_BF16: return launch_fwd<__nv_bfloat16>(x, y, rstd, rows, D, eps, st);
    case DT_F16: return launch_fwd<__half>(x, y, rstd, rows, D, eps, st);
    case DT_F32: return launch_fwd<float>(x, y, rstd, rows, D, eps, st);
    default: return FQLA_ERR_INVALID_ARG;
  }
}

extern "C" int fqla_l2norm_bwd(const void* y, const float* rstd, const void* dy, float* dx,
                               long long rows, int D, int y_dtype, int dy_dtype, void* stream) {
  if (!y || !rstd || !dy || !dx || rows < 0 || D <= 0 || D % 2 || D > 32 * MAX_PER_LANE)
    return FQLA_ERR_INVALID_ARG;
  if (rows == 0) return FQLA_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define FQLA_L2_BWD(TY)                                                                     \
  switch (dy_dtype) {                                                                       \
    case DT_BF16: return launch_bwd<TY, __nv_bfloat16>(y, rstd, dy, dx, rows, D, st);       \
    case DT_F16: return launch_bwd<TY, __half>(y, rstd, dy, dx, rows, D, st);               \
    case DT_F32: return launch_bwd<TY, float>(y, rstd, dy, dx, rows, D, st);                \
    default: return FQLA_ERR_INVALID_ARG;                                                   \
  }
  switch (y_dtype) {
    case DT_BF16: FQLA_L2_BWD(__nv_bfloat16)
    case DT_F16: FQLA_L2_BWD(__half)
    case DT_F32: FQLA_L2_BWD(float)
    default: return FQLA_ERR_INVALID_ARG;
  }
#undef FQLA_L2_BWD
}
