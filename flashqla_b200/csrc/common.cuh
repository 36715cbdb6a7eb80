// Shared device helpers for the gated-delta-rule kernels (sm_100a).
//
// Index conventions used by every kernel in this directory:
//   * tokens are addressed as one flat axis of B*T rows; with cu_seqlens the batch is 1 and
//     sequence n owns rows [cu[n], cu[n+1]); without it sequence n owns [n*T, (n+1)*T).
//   * chunks of 64 rows are aligned to each sequence start; sequence n's first chunk has the
//     global chunk index chunk_offsets[n] (varlen) or n*ceil(T/64) (fixed length).
//   * q, k are [rows, Hq, D]; v, o are [rows, Hv, D]; g, beta are [rows, Hv]; the A matrix is
//     [rows, Hv, 64]; states are [N, Hv, D(k), D(v)] fp32; per-chunk states [chunks, Hv, D, D] bf16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fqla {

constexpr int CHUNK = 64;

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// ---- index tables may be int32 or int64 (the dtype of the caller's cu_seqlens) -------------
struct IndexTable {
  const void* ptr;
  int is64;
  __device__ __forceinline__ long long operator[](int i) const {
    return is64 ? reinterpret_cast<const long long*>(ptr)[i]
                : (long long)reinterpret_cast<const int*>(ptr)[i];
  }
};

// Where one sequence lives.
struct SeqSpan {
  long long bos;         // first row
  int len;               // rows
  long long chunk_base;  // global index of its first chunk
  int n_chunks;
};

struct SeqLayout {
  IndexTable cu;             // null ptr -> fixed length
  IndexTable chunk_offsets;  // used only with cu
  int T;                     // rows per sequence when fixed length
  __device__ __forceinline__ SeqSpan span(int n) const {
    SeqSpan s;
    if (cu.ptr) {
      s.bos = cu[n];
      s.len = (int)(cu[n + 1] - s.bos);
      s.chunk_base = chunk_offsets[n];
    } else {
      s.bos = (long long)n * T;
      s.len = T;
      s.chunk_base = (long long)n * ((T + CHUNK - 1) / CHUNK);
    }
    s.n_chunks = (s.len + CHUNK - 1) / CHUNK;
    return s;
  }
};

// ---- small PTX wrappers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// 16-byte global->shared copy; when !pred the destination is zero-filled and nothing is read.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool pred) {
  int n = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem_dst)),
               "l"(gmem_src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4],
                                               const uint32_t b0, const uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp(float x) { return exp2f(x * 1.4426950408889634f); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  bf162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void st_bf16x2(bf16* p, float lo, float hi) {
  *reinterpret_cast<bf162*>(p) = __floats2bfloat162_rn(lo, hi);
}
__device__ __forceinline__ float2 ld_bf16x2(const bf16* p) {
  return __bfloat1622float2(*reinterpret_cast<const bf162*>(p));
}

// 4 x 4 transpose of 32-bit words across the four lanes of a quad (lanes 4n .. 4n+3): on return
// w[m] of lane j holds what w[j] of lane m held.  Two butterfly steps, four shuffles; the whole
// warp must call it.
__device__ __forceinline__ void quad_transpose(uint32_t* w, int lane) {
  const bool b0 = lane & 1, b1 = lane & 2;
  uint32_t r;
  r = __shfl_xor_sync(0xffffffffu, b0 ? w[0] : w[1], 1);
  if (b0) w[0] = r; else w[1] = r;
  r = __shfl_xor_sync(0xffffffffu, b0 ? w[2] : w[3], 1);
  if (b0) w[2] = r; else w[3] = r;
  r = __shfl_xor_sync(0xffffffffu, b1 ? w[0] : w[2], 2);
  if (b1) w[0] = r; else w[2] = r;
  r = __shfl_xor_sync(0xffffffffu, b1 ? w[1] : w[3], 2);
  if (b1) w[1] = r; else w[3] = r;
}

// ---- warp-level tile GEMM on shared-memory operands -----------------------------------------
// acc[mt][nt] (+)= op(A) * op(B) for a warp tile of (MT*16) x (NT*8), reduction length KT*16.
//   A_TRANS = false: A is stored [m][k] (row stride lda), `As` points at (m0, 0).
//   A_TRANS = true : A is stored [k][m],                  `As` points at (0, m0).
//   B_NMAJOR = false: B is stored [n][k] (row stride ldb), `Bs` points at (n0, 0).
//   B_NMAJOR = true : B is stored [k][n],                  `Bs` points at (0, n0).
// Row strides must be multiples of 8 elements (16-byte rows for ldmatrix).
// Fragment ownership of acc[mt][nt][i]: row = mt*16 + lane/4 + (i/2)*8, col = nt*8 + (lane%4)*2 + i%2.
template <int MT, int NT, int KT, bool A_TRANS, bool B_NMAJOR>
__device__ __forceinline__ void warp_gemm(float (&acc)[MT][NT][4], const bf16* As, int lda,
                                          const bf16* Bs, int ldb, int lane) {
  static_assert(NT % 2 == 0, "NT must be even");
  const int r8 = lane & 7, sel1 = (lane >> 3) & 1, sel2 = lane >> 4;
#pragma unroll
  for (int kt = 0; kt < KT; ++kt) {
    uint32_t a[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (!A_TRANS) {
        ldmatrix_x4(a[mt], As + (mt * 16 + r8 + sel1 * 8) * lda + kt * 16 + sel2 * 8);
      } else {
        ldmatrix_x4_trans(a[mt], As + (kt * 16 + r8 + sel2 * 8) * lda + mt * 16 + sel1 * 8);
      }
    }
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      if (!B_NMAJOR) {
        ldmatrix_x4(b, Bs + (np * 16 + r8 + sel2 * 8) * ldb + kt * 16 + sel1 * 8);
      } else {
        ldmatrix_x4_trans(b, Bs + (kt * 16 + r8 + sel1 * 8) * ldb + np * 16 + sel2 * 8);
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        mma_bf16_16816(acc[mt][2 * np], a[mt], b[0], b[1]);
        mma_bf16_16816(acc[mt][2 * np + 1], a[mt], b[2], b[3]);
      }
    }
  }
}

template <int MT, int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[MT][NT][4]) {
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
}

// Asynchronously copy a [rows<=64] x [COLS] bf16 tile (global row stride `g_stride` elements)
// into shared memory with row stride LDS; rows >= valid are zero-filled.
template <int COLS, int LDS, int NTHREADS>
__device__ __forceinline__ void load_tile_async(bf16* s, const bf16* g, long long g_stride,
                                                int valid, int tid) {
  constexpr int SEGS = COLS / 8;  // 16-byte segments per row
  for (int i = tid; i < CHUNK * SEGS; i += NTHREADS) {
    int r = i / SEGS, c = (i % SEGS) * 8;
    bool ok = r < valid;
    const bf16* src = g + (long long)(ok ? r : 0) * g_stride + c;
    cp_async16(s + r * LDS + c, src, ok);
  }
}

__device__ __forceinline__ float load_beta(const void* beta, int beta_is_f32, long long idx) {
  return beta_is_f32 ? reinterpret_cast<const float*>(beta)[idx]
                     : __bfloat162float(reinterpret_cast<const bf16*>(beta)[idx]);
}

}  // namespace fqla
