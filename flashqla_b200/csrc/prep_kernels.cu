// Chunk-parallel preparation kernels of the gated-delta-rule path:
//   * chunk-local cumulative sum of the log gates (forward, and reversed for the gate gradient)
//   * A = (I + strict_lower(diag(beta) K K^T * exp(g_s - g_t)))^-1 per (chunk, value head)
//   * sum of per-value-head dq/dk over each grouped-value-attention group
// These replace the reference's ops/utils/cumsum.py:14-134, blackwell/kkt_solve.py:19-281 and
// ops/utils/group_reduce.py:12-57.
#include <type_traits>
#include "common.cuh"
#include "fqla_internal.h"

namespace fqla {

// ------------------------------------------------------------------------------------------
// Chunk-local cumsum.  One CTA per chunk, one warp per head (looping), two rows per lane.
// HBM-bound: 8 bytes per (token, head).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) cumsum_kernel(const float* __restrict__ g,
                                                     float* __restrict__ out, int H, int T_rows,
                                                     SeqLayout lay, IndexTable chunk_indices,
                                                     int N, int reverse) {
  int seq, ci;
  if (lay.cu.ptr) {
    seq = (int)chunk_indices[2 * blockIdx.x];
    ci = (int)chunk_indices[2 * blockIdx.x + 1];
  } else {
    int per = (lay.T + CHUNK - 1) / CHUNK;
    seq = blockIdx.x / per;
    ci = blockIdx.x % per;
  }
  SeqSpan sp = lay.span(seq);
  long long row0 = sp.bos + (long long)ci * CHUNK;
  int valid = min(CHUNK, sp.len - ci * CHUNK);
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int h = warp; h < H; h += 4) {
    // lane owns rows 2*lane, 2*lane+1 (forward) or their mirror images (reverse)
    int r0 = 2 * lane, r1 = 2 * lane + 1;
    if (reverse) { r0 = valid - 1 - r0; r1 = valid - 1 - r1; }
    bool ok0 = reverse ? r0 >= 0 : r0 < valid;
    bool ok1 = reverse ? r1 >= 0 : r1 < valid;
    float a = ok0 ? g[(row0 + r0) * H + h] : 0.f;
    float b = ok1 ? g[(row0 + r1) * H + h] : 0.f;
    float pair = a + b, incl = pair;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      float t = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += t;
    }
    float excl = incl - pair;
    if (ok0) out[(row0 + r0) * H + h] = excl + a;
    if (ok1) out[(row0 + r1) * H + h] = excl + a + b;
  }
  // Rows past the last sequence's end (packed input shorter than the buffer) come out zero.
  if (lay.cu.ptr && seq == N - 1 && ci == sp.n_chunks - 1) {
    long long end = sp.bos + sp.len;
    for (long long i = end * H + threadIdx.x; i < (long long)T_rows * H; i += blockDim.x)
      out[i] = 0.f;
  }
}

// C[16 x 8*NT] = A[16 x 8*KT] * B[8*KT x 8*NT], both row-major fp32 in shared memory, as
// mma.m16n8k8 with tf32 inputs.  Fragment element (g = lane/4, t = lane%4): c[nt][0..3] =
// C[g][8nt+2t], C[g][8nt+2t+1], C[g+8][8nt+2t], C[g+8][8nt+2t+1].
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
template <int NT, int KT>
__device__ __forceinline__ void tf32_gemm(float (&c)[NT][4], const float* A, int lda, const float* B,
                                          int ldb, int lane) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
#pragma unroll
  for (int kt = 0; kt < KT; ++kt) {
    const uint32_t a0 = to_tf32(A[g * lda + 8 * kt + t]), a1 = to_tf32(A[(g + 8) * lda + 8 * kt + t]);
    const uint32_t a2 = to_tf32(A[g * lda + 8 * kt + t + 4]), a3 = to_tf32(A[(g + 8) * lda + 8 * kt + t + 4]);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint32_t b0 = to_tf32(B[(8 * kt + t) * ldb + 8 * nt + g]);
      const uint32_t b1 = to_tf32(B[(8 * kt + t + 4) * ldb + 8 * nt + g]);
      asm volatile(
          "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
          "{%0,%1,%2,%3};"
          : "+f"(c[nt][0]), "+f"(c[nt][1]), "+f"(c[nt][2]), "+f"(c[nt][3])
          : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
  }
}
template <int NT>
__device__ __forceinline__ void store_frag(float* C, int ldc, const float (&c)[NT][4], float sign,
                                           int lane) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    *reinterpret_cast<float2*>(C + g * ldc + 8 * nt + 2 * t) = make_float2(sign * c[nt][0], sign * c[nt][1]);
    *reinterpret_cast<float2*>(C + (g + 8) * ldc + 8 * nt + 2 * t) = make_float2(sign * c[nt][2], sign * c[nt][3]);
  }
}

// ------------------------------------------------------------------------------------------
// kkt + solve.  One CTA (128 threads) per (chunk, q head): K K^T is computed once and kept in
// registers, then scaled and inverted for each of the Hv / Hq value heads of the group in turn.
//   1. K K^T (64x64xD) on tensor cores, 2. L = strict_lower(beta_s * KK^T * exp(g_s-g_t)) in fp32,
//   3. X = (I+L)^-1 by blocked forward substitution in fp32, 4. bf16 rows out.
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(128, 6) kkt_solve_kernel(
    const bf16* __restrict__ k, const void* __restrict__ beta, int beta_is_f32,
    const float* __restrict__ g, float* __restrict__ g_cum_out, bf16* __restrict__ A, int Hq,
    int Hv, SeqLayout lay, IndexTable chunk_indices) {
  constexpr int LDK = D + 8;
  constexpr int LDL = CHUNK + 4;  // floats; rows stay 16-byte aligned
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sK = reinterpret_cast<bf16*>(smem_raw);
  // the inverse X [64][LDL] is built over the K tile, dead once K K^T is in sL (5 CTAs per SM)
  constexpr int REGION0 = CHUNK * LDK * 2 > CHUNK * LDL * 4 ? CHUNK * LDK * 2 : CHUNK * LDL * 4;
  float* sX = reinterpret_cast<float*>(smem_raw);
  float* sL = reinterpret_cast<float*>(smem_raw + REGION0);
  float* sG = sL + CHUNK * LDL;
  float* sB = sG + CHUNK;
  // partial products [32][32]: they live in the rows 0-31, columns 32-63 of L, a part of its
  // upper triangle that is neither written nor read (six CTAs per SM fit with that)
  constexpr int LDY = LDL;
  float* sY = sL + 32;

  int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hq = blockIdx.y, G = Hv / Hq;
  int seq, ci;
  if (lay.cu.ptr) {
    seq = (int)chunk_indices[2 * blockIdx.x];
    ci = (int)chunk_indices[2 * blockIdx.x + 1];
  } else {
    int per = (lay.T + CHUNK - 1) / CHUNK;
    seq = blockIdx.x / per;
    ci = blockIdx.x % per;
  }
  SeqSpan sp = lay.span(seq);
  long long row0 = sp.bos + (long long)ci * CHUNK;
  int valid = min(CHUNK, sp.len - ci * CHUNK);

  load_tile_async<D, LDK, 128>(sK, k + (row0 * Hq + hq) * D, (long long)Hq * D, valid, tid);
  cp_async_commit();
  float kkt[24];  // this thread's part of the lower blocks of K K^T
#pragma unroll 1
  for (int gi = 0; gi < G; ++gi) {
  const int hv = hq * G + gi;
  if (gi > 0) __syncthreads();  // the inverse of the head before has been written out
  if (tid < CHUNK) {
    sB[tid] = tid < valid ? load_beta(beta, beta_is_f32, (row0 + tid) * Hv + hv) : 0.f;
    if (g_cum_out) {
      // g is the raw log gate: chunk-local inclusive prefix sum over the valid rows (rows past
      // the end repeat the last value, as the clamped read below does), done by the first two warps
      float x = tid < valid ? g[(row0 + tid) * Hv + hv] : 0.f;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      if (tid == 31) sL[0] = x;
      asm volatile("bar.sync 1, 64;" ::: "memory");
      if (tid >= 32) x += sL[0];
      sG[tid] = x;
      if (tid < valid) g_cum_out[(row0 + tid) * Hv + hv] = x;
    } else {
      int r = min(tid, valid - 1);
      sG[tid] = g[(row0 + r) * Hv + hv];
    }
  }
  if (gi == 0) cp_async_wait<0>();
  __syncthreads();

  // Only the 16 x 16 blocks on and below the diagonal of K K^T are needed (10 of 16); they are
  // dealt to the four warps 3, 3, 2, 2.  rb = row block, [u0, u0 + NU) = 16-column blocks.
  auto kkt_blocks = [&](auto nu_tag, auto off_tag, int rb, int u0) {
    constexpr int NU = decltype(nu_tag)::value;
    float (&acc)[1][2 * NU][4] = *reinterpret_cast<float (*)[1][2 * NU][4]>(kkt + decltype(off_tag)::value);
    if (gi == 0) {  // the K tile is gone (the inverse is built over it) once the first head is done
      zero_acc(acc);
      warp_gemm<1, 2 * NU, D / 16, false, false>(acc, sK + rb * 16 * LDK, LDK, sK + u0 * 16 * LDK, LDK, lane);
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = rb * 16 + (lane >> 2) + hh * 8;
      const float br = sB[r], gr = sG[r];
#pragma unroll
      for (int nt = 0; nt < 2 * NU; ++nt) {
        const int c = u0 * 16 + nt * 8 + (lane & 3) * 2;  // columns c, c + 1: one 8-byte store
        const float2 gc = *reinterpret_cast<const float2*>(sG + c);
        float2 v;
        v.x = r > c ? br * acc[0][nt][2 * hh] * fast_exp(gr - gc.x) : 0.f;
        v.y = r > c + 1 ? br * acc[0][nt][2 * hh + 1] * fast_exp(gr - gc.y) : 0.f;
        *reinterpret_cast<float2*>(sL + r * LDL + c) = v;
      }
    }
  };
  if (warp == 0) {
    kkt_blocks(std::integral_constant<int, 3>{}, std::integral_constant<int, 0>{}, 3, 0);
  } else if (warp == 1) {
    kkt_blocks(std::integral_constant<int, 3>{}, std::integral_constant<int, 0>{}, 2, 0);
  } else if (warp == 2) {
    kkt_blocks(std::integral_constant<int, 1>{}, std::integral_constant<int, 0>{}, 3, 3);
    kkt_blocks(std::integral_constant<int, 1>{}, std::integral_constant<int, 8>{}, 0, 0);
  } else {
    kkt_blocks(std::integral_constant<int, 2>{}, std::integral_constant<int, 0>{}, 1, 0);
  }
  __syncthreads();

  // Inverse of the unit lower-triangular (I + L) by recursive halving:
  //   [[P, 0], [C, Q]]^-1 = [[P^-1, 0], [-Q^-1 C P^-1, Q^-1]].
  // The four 16 x 16 diagonal blocks come from forward substitution in fp32 (thread = one column
  // of one block); the two 16 x 16 and then the one 32 x 32 off-diagonal blocks are two small
  // products each, on tensor cores with tf32 inputs (round to nearest) and fp32 accumulation.
  if (tid < CHUNK) {
    const int b0 = (tid >> 4) * 16, c = tid & 15;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s = (i == c) ? 1.f : 0.f;
#pragma unroll
      for (int jj = 0; jj < i; ++jj) s -= sL[(b0 + i) * LDL + b0 + jj] * x[jj];
      x[i] = s;
      sX[(b0 + i) * LDL + b0 + c] = s;
    }
  } else {
    // the 16 x 16 blocks above the diagonal inside each 32 x 32 diagonal block are operands of
    // the last two products: they must read as zero
    const int t = tid - CHUNK, blk = t >> 5, r = (t >> 1) & 15, c0 = (t & 1) * 8;
    float* z = sX + (32 * blk + r) * LDL + 32 * blk + 16 + c0;
    *reinterpret_cast<float4*>(z) = make_float4(0.f, 0.f, 0.f, 0.f);
    *reinterpret_cast<float4*>(z + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  {
    // 32 x 32 diagonal blocks: pair p covers rows/cols [32p, 32p+32); warp = (pair, 8-column tile pair)
    const int pr = warp >> 1, bi = 32 * pr + 16, bj = 32 * pr, n0 = 8 * (warp & 1);
    float* y = sY + pr * 16 * LDY;
    float c[1][4];
    tf32_gemm<1, 2>(c, sL + bi * LDL + bj, LDL, sX + bj * LDL + bj + n0, LDL, lane);
    store_frag<1>(y + n0, LDY, c, 1.f, lane);
    __syncthreads();
    tf32_gemm<1, 2>(c, sX + bi * LDL + bi, LDL, y + n0, LDY, lane);
    store_frag<1>(sX + bi * LDL + bj + n0, LDL, c, -1.f, lane);
    __syncthreads();
  }
  {
    // the 32 x 32 block below the diagonal: warp = (16-row tile, 16-column half)
    const int m0 = 16 * (warp >> 1), n0 = 16 * (warp & 1);
    float c[2][4];
    tf32_gemm<2, 4>(c, sL + (32 + m0) * LDL, LDL, sX + n0, LDL, lane);
    store_frag<2>(sY + m0 * LDY + n0, LDY, c, 1.f, lane);
    __syncthreads();
    tf32_gemm<2, 4>(c, sX + (32 + m0) * LDL + 32, LDL, sY + n0, LDY, lane);
    store_frag<2>(sX + (32 + m0) * LDL + n0, LDL, c, -1.f, lane);
    __syncthreads();
  }
  // bf16 rows out, 16 bytes per store; blocks above the diagonal are zero
  for (int i = tid; i < CHUNK * 8; i += 128) {
    const int r = i >> 3, c0 = (i & 7) * 8;
    if (r < valid) {
      uint4 pk = make_uint4(0, 0, 0, 0);
      if ((c0 >> 4) <= (r >> 4)) {
        const float* xr = sX + r * LDL + c0;
        pk = make_uint4(pack_bf16(xr[0], xr[1]), pack_bf16(xr[2], xr[3]), pack_bf16(xr[4], xr[5]),
                        pack_bf16(xr[6], xr[7]));
      }
      *reinterpret_cast<uint4*>(A + ((row0 + r) * Hv + hv) * CHUNK + c0) = pk;
    }
  }
  }  // value heads of the group
}

// ------------------------------------------------------------------------------------------
// Grouped-value-attention reduce: out[row, hq, :] = sum_{i<G} in[row, hq*G+i, :], fp32 adds.
// HBM-bound: reads 2*D*G bytes and writes 2*D bytes per (token, q head).
// ------------------------------------------------------------------------------------------
__global__ void group_reduce_kernel(const bf16* __restrict__ in, bf16* __restrict__ out,
                                    long long n_vec, int G, int D8) {
  // one thread per 8-element (16-byte) segment of an output row
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  long long row_hq = i / D8;
  int seg = (int)(i % D8);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int j = 0; j < G; ++j) {
    uint4 raw = *reinterpret_cast<const uint4*>(in + ((row_hq * G + j) * D8 + seg) * 8);
    const bf162* p = reinterpret_cast<const bf162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = __bfloat1622float2(p[e]);
      acc[2 * e] += f.x;
      acc[2 * e + 1] += f.y;
    }
  }
  uint4 res;
  uint32_t* pr = reinterpret_cast<uint32_t*>(&res);
#pragma unroll
  for (int e = 0; e < 4; ++e) pr[e] = pack_bf16(acc[2 * e], acc[2 * e + 1]);
  *reinterpret_cast<uint4*>(out + i * 8) = res;
}

}  // namespace fqla

using namespace fqla;

extern "C" int fqla_chunk_local_cumsum(const float* g, float* out, int B, int T, int H,
                                       const void* cu_seqlens, int idx_is64, int N,
                                       const void* chunk_indices, long long num_chunks,
                                       int reverse, void* stream) {
  if (!g || !out || B <= 0 || T < 0 || H <= 0) return FQLA_ERR_INVALID_ARG;
  if (cu_seqlens && (!chunk_indices || B != 1)) return FQLA_ERR_INVALID_ARG;
  SeqLayout lay{{cu_seqlens, idx_is64}, {nullptr, idx_is64}, T};
  long long n = cu_seqlens ? num_chunks : (long long)B * ((T + CHUNK - 1) / CHUNK);
  if (n <= 0) return FQLA_OK;
  cumsum_kernel<<<(unsigned)n, 128, 0, (cudaStream_t)stream>>>(
      g, out, H, B * T, lay, IndexTable{chunk_indices, idx_is64}, cu_seqlens ? N : B, reverse);
  return (int)cudaGetLastError();
}

template <int D>
static int launch_kkt(const void* k, const void* beta, int beta_is_f32, const float* g,
                      float* g_cum_out, void* A, int Hq, int Hv, SeqLayout lay, IndexTable ci,
                      long long n, cudaStream_t st) {
  constexpr int k_tile = CHUNK * (D + 8) * 2, x_tile = CHUNK * (CHUNK + 4) * 4;
  constexpr int smem = (k_tile > x_tile ? k_tile : x_tile) + x_tile + 2 * CHUNK * 4;
  int rc = configure_smem((const void*)kkt_solve_kernel<D>, smem);
  if (rc != 0) return rc;
  kkt_solve_kernel<D><<<dim3((unsigned)n, Hq), 128, smem, st>>>(
      (const bf16*)k, beta, beta_is_f32, g, g_cum_out, (bf16*)A, Hq, Hv, lay, ci);
  return (int)cudaGetLastError();
}

extern "C" int fqla_kkt_solve(const void* k, const void* beta, int beta_is_f32,
                              const float* g_cum, float* g_cum_out, void* A, int B, int T, int Hq,
                              int Hv, int D,
                              const void* cu_seqlens, int idx_is64, const void* chunk_indices,
                              long long num_chunks, void* stream) {
  if (!k || !beta || !g_cum || !A || Hq <= 0 || Hv % Hq) return FQLA_ERR_INVALID_ARG;
  if (cu_seqlens && (!chunk_indices || B != 1)) return FQLA_ERR_INVALID_ARG;
  SeqLayout lay{{cu_seqlens, idx_is64}, {nullptr, idx_is64}, T};
  IndexTable ci{chunk_indices, idx_is64};
  long long n = cu_seqlens ? num_chunks : (long long)B * ((T + CHUNK - 1) / CHUNK);
  if (n <= 0) return FQLA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 128) return launch_kkt<128>(k, beta, beta_is_f32, g_cum, g_cum_out, A, Hq, Hv, lay, ci, n, st);
  if (D == 64) return launch_kkt<64>(k, beta, beta_is_f32, g_cum, g_cum_out, A, Hq, Hv, lay, ci, n, st);
  return FQLA_ERR_UNSUPPORTED_DIM;
}

extern "C" int fqla_group_reduce(const void* in, void* out, long long rows, int Hq, int G, int D,
                                 void* stream) {
  if (!in || !out || G <= 0 || D % 8) return FQLA_ERR_INVALID_ARG;
  long long n_vec = rows * Hq * (D / 8);
  if (n_vec <= 0) return FQLA_OK;
  group_reduce_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)in, (bf16*)out, n_vec, G, D / 8);
  return (int)cudaGetLastError();
}
