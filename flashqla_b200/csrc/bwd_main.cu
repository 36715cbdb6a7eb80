// Chunk-parallel part of the gated-delta-rule backward: given the per-chunk states h (entering
// each chunk) and state gradients dh (leaving each chunk), every (chunk, value head) is
// independent.  One CTA per (chunk, value head) computes, in the notation of the reference's
// tests/ref_gdr.py:427-600 (torch_chunk_dqkwg_bwd followed by torch_chunk_wy_bwd):
//
//   ds  = scale * G * (dO Vn^T)                      G[r][c] = exp(g_r - g_c), r >= c
//   dq  = scale * exp(g) * (dO h^T) + ds K
//   dk  = exp(g_last - g) * (Vn dh^T) + ds^T Q
//   dw  = -du h^T
//   dA  = strict_lower((dw K^T) * beta_c exp(g_c) + (du V^T) * beta_c)
//   dk += (A^T dw) * beta exp(g);   dv = (A^T du) * beta
//   dA3 = -(A^T dA A^T) * G (strict lower)
//   dk += (dA3 K) * beta + (diag(beta) dA3)^T K
//   dbeta, dg: the row/column reductions of the same products
//
// which is what the reference's blackwell/fused_bwd.py:595-862 evaluates inside its sequential
// loop.  Outputs: dq, dk per VALUE head (summed over each GVA group afterwards), dv, dbeta and
// the pre-cumsum dg.  mma.sync implementation: 16 tile products, eight cooperating warps.
#include "common.cuh"
#include "fqla_internal.h"

namespace fqla {

struct BwdMainParams {
  const bf16* q;
  const bf16* k;
  const bf16* v;
  const bf16* vnew;
  const bf16* A;
  const float* g;
  const void* beta;
  int beta_is_f32;
  const bf16* dO;
  const bf16* du;
  const bf16* h;
  const bf16* dh;
  bf16* dq;   // [rows, Hv, D]
  bf16* dk;   // [rows, Hv, D]
  bf16* dv;   // [rows, Hv, D]
  float* db;  // [rows, Hv]
  float* dg;  // [rows, Hv]
  int Hq, Hv;
  float scale;
  SeqLayout lay;
  IndexTable chunk_indices;
};

template <int D>
struct BwdMainSmem {
  static constexpr int LDK = D + 8;
  static constexpr int LDA = CHUNK + 8;
  static constexpr int ROW_TILE = CHUNK * LDK;
  static constexpr int SQ_TILE = D * LDK;
  static constexpr int A_TILE = CHUNK * LDA;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + ROW_TILE;
  static constexpr int OFF_V = OFF_K + ROW_TILE;
  static constexpr int OFF_VN = OFF_V + ROW_TILE;
  static constexpr int OFF_DO = OFF_VN + ROW_TILE;
  static constexpr int OFF_DU = OFF_DO + ROW_TILE;
  static constexpr int OFF_H = OFF_DU + ROW_TILE;   // later reused for dw
  static constexpr int OFF_DH = OFF_H + SQ_TILE;
  static constexpr int OFF_A = OFF_DH + SQ_TILE;
  static constexpr int OFF_DS = OFF_A + A_TILE;     // ds, later beta-scaled dA3
  static constexpr int OFF_DA = OFF_DS + A_TILE;    // dA, later dA3
  static constexpr int OFF_T = OFF_DA + A_TILE;     // A^T dA
  static constexpr int BF16_ELEMS = OFF_T + A_TILE;
  static constexpr int VEC_FLOATS = 6 * CHUNK + 4;  // g, gamma, rho, beta, dg, db, dg_last
  static constexpr int BYTES = BF16_ELEMS * 2 + VEC_FLOATS * 4;
};

// acc rows rA (e<2) and rA+8 (e>=2): add sum over the warp tile's columns of acc*other into dst[row]
template <int NT, typename F>
__device__ __forceinline__ void row_reduce_add(float* dst, int rA, int lane, F elem) {
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    s0 += elem(nt, 0) + elem(nt, 1);
    s1 += elem(nt, 2) + elem(nt, 3);
  }
  s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
  s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
  if ((lane & 3) == 0) {
    atomicAdd(dst + rA, s0);
    atomicAdd(dst + rA + 8, s1);
  }
}

// column sums of a warp tile with NT n-tiles starting at column c0: dst[col] += sign * sum_rows
template <int NT, typename F>
__device__ __forceinline__ void col_reduce_add(float* dst, int c0, int lane, float sign, F elem) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float s = elem(nt, j) + elem(nt, j + 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 16);
      if (lane < 4) atomicAdd(dst + c0 + nt * 8 + lane * 2 + j, sign * s);
    }
}

template <int D>
__global__ void __launch_bounds__(256, 1) bwd_main_kernel(const BwdMainParams p) {
  using L = BwdMainSmem<D>;
  constexpr int LDK = L::LDK, LDA = L::LDA;
  constexpr int NTD = D / 16;  // n-tiles per warp for 64 x D outputs (D/2 columns per warp)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sm = reinterpret_cast<bf16*>(smem_raw);
  bf16 *sQ = sm + L::OFF_Q, *sK = sm + L::OFF_K, *sV = sm + L::OFF_V, *sVn = sm + L::OFF_VN;
  bf16 *sDO = sm + L::OFF_DO, *sDU = sm + L::OFF_DU, *sH = sm + L::OFF_H, *sDH = sm + L::OFF_DH;
  bf16 *sA = sm + L::OFF_A, *sDs = sm + L::OFF_DS, *sDA = sm + L::OFF_DA, *sT = sm + L::OFF_T;
  bf16* sDw = sH;
  float* sG = reinterpret_cast<float*>(smem_raw + L::BF16_ELEMS * 2);
  float* sGam = sG + CHUNK;
  float* sRho = sGam + CHUNK;
  float* sBeta = sRho + CHUNK;
  float* sDg = sBeta + CHUNK;
  float* sDb = sDg + CHUNK;
  float* sDgLast = sDb + CHUNK;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp & 3, wn = warp >> 2;
  const int hv = blockIdx.y, hq = hv / (p.Hv / p.Hq);
  int seq, ci;
  if (p.lay.cu.ptr) {
    seq = (int)p.chunk_indices[2 * blockIdx.x];
    ci = (int)p.chunk_indices[2 * blockIdx.x + 1];
  } else {
    int per = (p.lay.T + CHUNK - 1) / CHUNK;
    seq = blockIdx.x / per;
    ci = blockIdx.x % per;
  }
  const SeqSpan sp = p.lay.span(seq);
  const long long row0 = sp.bos + (long long)ci * CHUNK;
  const int valid = min(CHUNK, sp.len - ci * CHUNK);
  const long long qk_stride = (long long)p.Hq * D, v_stride = (long long)p.Hv * D;
  const long long vbase = (row0 * p.Hv + hv) * D;

  // ---- loads: group 0 = what phase 2 needs, group 1 = the rest
  load_tile_async<D, LDK, 256>(sDO, p.dO + vbase, v_stride, valid, tid);
  load_tile_async<D, LDK, 256>(sVn, p.vnew + vbase, v_stride, valid, tid);
  load_tile_async<D, LDK, 256>(sDU, p.du + vbase, v_stride, valid, tid);
  {
    const long long hoff = ((sp.chunk_base + ci) * p.Hv + hv) * (long long)D * D;
    constexpr int SEGS = D / 8;
    for (int i = tid; i < D * SEGS; i += 256) {
      int r = i / SEGS, c = (i % SEGS) * 8;
      cp_async16(sH + r * LDK + c, p.h + hoff + (long long)r * D + c, true);
      cp_async16(sDH + r * LDK + c, p.dh + hoff + (long long)r * D + c, true);
    }
  }
  load_tile_async<D, LDK, 256>(sQ, p.q + (row0 * p.Hq + hq) * D, qk_stride, valid, tid);
  load_tile_async<D, LDK, 256>(sK, p.k + (row0 * p.Hq + hq) * D, qk_stride, valid, tid);
  cp_async_commit();
  load_tile_async<D, LDK, 256>(sV, p.v + vbase, v_stride, valid, tid);
  load_tile_async<CHUNK, LDA, 256>(sA, p.A + (row0 * p.Hv + hv) * CHUNK, (long long)p.Hv * CHUNK,
                                   valid, tid);
  cp_async_commit();
  if (tid < CHUNK) {
    int r = min(tid, valid - 1);
    float gv = p.g[(row0 + r) * p.Hv + hv];
    float gl = p.g[(row0 + valid - 1) * p.Hv + hv];
    sG[tid] = gv;
    sGam[tid] = fast_exp(gv);
    sRho[tid] = fast_exp(gl - gv);
    sBeta[tid] = tid < valid ? load_beta(p.beta, p.beta_is_f32, (row0 + tid) * p.Hv + hv) : 0.f;
    sDg[tid] = 0.f;
    sDb[tid] = 0.f;
    if (tid == 0) *sDgLast = 0.f;
  }
  cp_async_wait<1>();
  __syncthreads();

  const int rA = 16 * wm + (lane >> 2);
  const int cD = (D / 2) * wn + (lane & 3) * 2;   // column of fragment element (nt=0, e even) in 64 x D tiles
  const int c64 = 32 * wn + (lane & 3) * 2;       // same for 64 x 64 tiles
  float dq[1][NTD][4], dk[1][NTD][4];
  zero_acc(dq);
  zero_acc(dk);

  // =================== phase 2: products with h and dh ===================
  warp_gemm<1, NTD, D / 16, false, false>(dq, sDO + 16 * wm * LDK, LDK, sH + (D / 2) * wn * LDK,
                                          LDK, lane);
  warp_gemm<1, NTD, D / 16, false, false>(dk, sVn + 16 * wm * LDK, LDK, sDH + (D / 2) * wn * LDK,
                                          LDK, lane);
#pragma unroll
  for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int r = rA + (e >> 1) * 8;
      dq[0][nt][e] *= p.scale * sGam[r];
      dk[0][nt][e] *= sRho[r];
    }
  // dg += rowsum(q*dq) - rowsum(k*dk);  dg_last += sum(k*dk)
  {
    float kdk_total;
    {
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = rA + hh * 8, c = cD + nt * 8;
          float2 qq = ld_bf16x2(sQ + r * LDK + c), kk = ld_bf16x2(sK + r * LDK + c);
          float t = qq.x * dq[0][nt][2 * hh] + qq.y * dq[0][nt][2 * hh + 1];
          float u = kk.x * dk[0][nt][2 * hh] + kk.y * dk[0][nt][2 * hh + 1];
          if (hh == 0) s0 += t - u; else s1 += t - u;
        }
      s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
      s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
      s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
      if ((lane & 3) == 0) {
        atomicAdd(sDg + rA, s0);
        atomicAdd(sDg + rA + 8, s1);
      }
      // total of k*dk over the warp tile
      float kt = 0.f;
#pragma unroll
      for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = rA + hh * 8, c = cD + nt * 8;
          float2 kk = ld_bf16x2(sK + r * LDK + c);
          kt += kk.x * dk[0][nt][2 * hh] + kk.y * dk[0][nt][2 * hh + 1];
        }
      kdk_total = kt;
    }
    // gamma_last * sum(h * dh) over the whole D x D tile
    float hd = 0.f;
    for (int i = tid; i < D * (D / 2); i += 256) {
      int r = i / (D / 2), c = (i % (D / 2)) * 2;
      float2 a = ld_bf16x2(sH + r * LDK + c), b = ld_bf16x2(sDH + r * LDK + c);
      hd += a.x * b.x + a.y * b.y;
    }
    float tot = kdk_total + sGam[CHUNK - 1] * hd;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, d);
    if (lane == 0) atomicAdd(sDgLast, tot);
  }
  // dw = -du h^T (kept in registers until h is dead)
  float dw[1][NTD][4];
  zero_acc(dw);
  warp_gemm<1, NTD, D / 16, false, false>(dw, sDU + 16 * wm * LDK, LDK, sH + (D / 2) * wn * LDK,
                                          LDK, lane);
  // ds = scale * G * (dO Vn^T);  ds2 = ds * (Q K^T)
  {
    float ds[1][4][4], qk[1][4][4];
    zero_acc(ds);
    zero_acc(qk);
    warp_gemm<1, 4, D / 16, false, false>(ds, sDO + 16 * wm * LDK, LDK, sVn + 32 * wn * LDK, LDK,
                                          lane);
    warp_gemm<1, 4, D / 16, false, false>(qk, sQ + 16 * wm * LDK, LDK, sK + 32 * wn * LDK, LDK,
                                          lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int r = rA + (e >> 1) * 8, c = c64 + nt * 8 + (e & 1);
        float x = r >= c ? p.scale * ds[0][nt][e] * fast_exp(sG[r] - sG[c]) : 0.f;
        ds[0][nt][e] = x;
        qk[0][nt][e] *= x;  // ds2
      }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        st_bf16x2(sDs + (rA + hh * 8) * LDA + c64 + nt * 8, ds[0][nt][2 * hh],
                  ds[0][nt][2 * hh + 1]);
    row_reduce_add<4>(sDg, rA, lane, [&](int nt, int e) { return qk[0][nt][e]; });
    col_reduce_add<4>(sDg, 32 * wn, lane, -1.f, [&](int nt, int e) { return qk[0][nt][e]; });
  }
  cp_async_wait<0>();
  __syncthreads();  // h, dh dead; ds visible; v and A landed

  // =================== phase 3: dq, dk += ds products; stage dw ===================
#pragma unroll
  for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
      st_bf16x2(sDw + (rA + hh * 8) * LDK + cD + nt * 8, -dw[0][nt][2 * hh],
                -dw[0][nt][2 * hh + 1]);
  warp_gemm<1, NTD, CHUNK / 16, false, true>(dq, sDs + 16 * wm * LDA, LDA, sK + (D / 2) * wn, LDK,
                                             lane);
  warp_gemm<1, NTD, CHUNK / 16, true, true>(dk, sDs + 16 * wm, LDA, sQ + (D / 2) * wn, LDK, lane);
#pragma unroll
  for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = rA + hh * 8;
      if (r < valid)
        st_bf16x2(p.dq + vbase + (long long)r * v_stride + cD + nt * 8, dq[0][nt][2 * hh],
                  dq[0][nt][2 * hh + 1]);
    }
  __syncthreads();  // dw visible

  // =================== phase 4: dA, A^T dw, A^T du ===================
  {
    float x1[1][4][4], x2[1][4][4];
    zero_acc(x1);
    zero_acc(x2);
    warp_gemm<1, 4, D / 16, false, false>(x1, sDw + 16 * wm * LDK, LDK, sK + 32 * wn * LDK, LDK,
                                          lane);
    warp_gemm<1, 4, D / 16, false, false>(x2, sDU + 16 * wm * LDK, LDK, sV + 32 * wn * LDK, LDK,
                                          lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = rA + hh * 8, c = c64 + nt * 8;
        float a = r > c ? sBeta[c] * (sGam[c] * x1[0][nt][2 * hh] + x2[0][nt][2 * hh]) : 0.f;
        float b = r > c + 1
                      ? sBeta[c + 1] * (sGam[c + 1] * x1[0][nt][2 * hh + 1] + x2[0][nt][2 * hh + 1])
                      : 0.f;
        st_bf16x2(sDA + r * LDA + c, a, b);
      }
  }
  {
    float t1[1][NTD][4];
    zero_acc(t1);
    warp_gemm<1, NTD, CHUNK / 16, true, true>(t1, sA + 16 * wm, LDA, sDw + (D / 2) * wn, LDK, lane);
    // dk += t1 * beta*gamma ; db += gamma * rowsum(t1*k) ; dg += beta*gamma*rowsum(t1*k)
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = rA + hh * 8, c = cD + nt * 8;
        float2 kk = ld_bf16x2(sK + r * LDK + c);
        float a = t1[0][nt][2 * hh], b = t1[0][nt][2 * hh + 1];
        float f = sBeta[r] * sGam[r];
        dk[0][nt][2 * hh] += f * a;
        dk[0][nt][2 * hh + 1] += f * b;
        float t = kk.x * a + kk.y * b;
        if (hh == 0) s0 += t; else s1 += t;
      }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if ((lane & 3) == 0) {
      atomicAdd(sDb + rA, sGam[rA] * s0);
      atomicAdd(sDb + rA + 8, sGam[rA + 8] * s1);
      atomicAdd(sDg + rA, sBeta[rA] * sGam[rA] * s0);
      atomicAdd(sDg + rA + 8, sBeta[rA + 8] * sGam[rA + 8] * s1);
    }
  }
  {
    float t2[1][NTD][4];
    zero_acc(t2);
    warp_gemm<1, NTD, CHUNK / 16, true, true>(t2, sA + 16 * wm, LDA, sDU + (D / 2) * wn, LDK, lane);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = rA + hh * 8, c = cD + nt * 8;
        float2 vv = ld_bf16x2(sV + r * LDK + c);
        float a = t2[0][nt][2 * hh], b = t2[0][nt][2 * hh + 1];
        float t = vv.x * a + vv.y * b;
        if (hh == 0) s0 += t; else s1 += t;
        if (r < valid)
          st_bf16x2(p.dv + vbase + (long long)r * v_stride + c, sBeta[r] * a, sBeta[r] * b);
      }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if ((lane & 3) == 0) {
      atomicAdd(sDb + rA, s0);
      atomicAdd(sDb + rA + 8, s1);
    }
  }
  __syncthreads();  // dA visible

  // =================== phase 5: dA3 = -(A^T dA A^T) * G ===================
  {
    float t[1][4][4];
    zero_acc(t);
    warp_gemm<1, 4, CHUNK / 16, true, true>(t, sA + 16 * wm, LDA, sDA + 32 * wn, LDA, lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        st_bf16x2(sT + (rA + hh * 8) * LDA + c64 + nt * 8, t[0][nt][2 * hh], t[0][nt][2 * hh + 1]);
  }
  __syncthreads();  // T visible; all reads of dA done
  {
    float d3[1][4][4], kk[1][4][4];
    zero_acc(d3);
    zero_acc(kk);
    warp_gemm<1, 4, CHUNK / 16, false, false>(d3, sT + 16 * wm * LDA, LDA, sA + 32 * wn * LDA, LDA,
                                              lane);
    warp_gemm<1, 4, D / 16, false, false>(kk, sK + 16 * wm * LDK, LDK, sK + 32 * wn * LDK, LDK,
                                          lane);
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int r = rA + (e >> 1) * 8, c = c64 + nt * 8 + (e & 1);
        float x = r > c ? -d3[0][nt][e] * fast_exp(sG[r] - sG[c]) : 0.f;
        d3[0][nt][e] = x;
        kk[0][nt][e] *= x * sBeta[r];  // dA3 * (beta_r k_r.k_c)
      }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = rA + hh * 8, c = c64 + nt * 8;
        st_bf16x2(sDA + r * LDA + c, d3[0][nt][2 * hh], d3[0][nt][2 * hh + 1]);
        st_bf16x2(sDs + r * LDA + c, sBeta[r] * d3[0][nt][2 * hh], sBeta[r] * d3[0][nt][2 * hh + 1]);
      }
    row_reduce_add<4>(sDg, rA, lane, [&](int nt, int e) { return kk[0][nt][e]; });
    col_reduce_add<4>(sDg, 32 * wn, lane, -1.f, [&](int nt, int e) { return kk[0][nt][e]; });
  }
  __syncthreads();  // dA3 and its beta-scaled copy visible

  // =================== phase 6: dk += (dA3 K) beta + (beta dA3)^T K ===================
  {
    float t3[1][NTD][4];
    zero_acc(t3);
    warp_gemm<1, NTD, CHUNK / 16, false, true>(t3, sDA + 16 * wm * LDA, LDA, sK + (D / 2) * wn, LDK,
                                               lane);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = rA + hh * 8, c = cD + nt * 8;
        float2 kk = ld_bf16x2(sK + r * LDK + c);
        float a = t3[0][nt][2 * hh], b = t3[0][nt][2 * hh + 1];
        dk[0][nt][2 * hh] += sBeta[r] * a;
        dk[0][nt][2 * hh + 1] += sBeta[r] * b;
        float t = kk.x * a + kk.y * b;
        if (hh == 0) s0 += t; else s1 += t;
      }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if ((lane & 3) == 0) {
      atomicAdd(sDb + rA, s0);
      atomicAdd(sDb + rA + 8, s1);
    }
  }
  warp_gemm<1, NTD, CHUNK / 16, true, true>(dk, sDs + 16 * wm, LDA, sK + (D / 2) * wn, LDK, lane);
#pragma unroll
  for (int nt = 0; nt < NTD; ++nt)
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      int r = rA + hh * 8;
      if (r < valid)
        st_bf16x2(p.dk + vbase + (long long)r * v_stride + cD + nt * 8, dk[0][nt][2 * hh],
                  dk[0][nt][2 * hh + 1]);
    }
  __syncthreads();
  if (tid < valid) {
    float dgv = sDg[tid];
    if (tid == valid - 1) dgv += *sDgLast;
    p.dg[(row0 + tid) * p.Hv + hv] = dgv;
    p.db[(row0 + tid) * p.Hv + hv] = sDb[tid];
  }
}

template <int D>
static int launch_bwd_main(const BwdMainParams& p, long long n_chunks, cudaStream_t st) {
  using L = BwdMainSmem<D>;
  int rc = configure_smem((const void*)bwd_main_kernel<D>, L::BYTES);
  if (rc != 0) return rc;
  bwd_main_kernel<D><<<dim3((unsigned)n_chunks, p.Hv), 256, L::BYTES, st>>>(p);
  return (int)cudaGetLastError();
}

// tcgen05 version for K = V = 128 (bwd_main_tc.cu)
int launch_bwd_main_tc(const void* q, const void* k, const void* v, const void* vnew, const void* A,
                       const float* g, const void* beta, int beta_is_f32, const void* dO,
                       const void* du, const void* h, const void* dh, void* dq, void* dk, void* dv,
                       float* db, float* dg, int tiled, int Hq, int Hv, long long T_rows, long long n_chunks,
                       float scale, SeqLayout lay, IndexTable chunk_indices, cudaStream_t st);
}  // namespace fqla
using namespace fqla;

extern "C" int fqla_bwd_main(const void* q, const void* k, const void* v, const void* vnew,
                             const void* A, const float* g_cum, const void* beta,
                             int beta_is_f32, const void* dO, const void* du, const void* h,
                             const void* dh, void* dq, void* dk, void* dv, float* db, float* dg,
                             int B, int T, int Hq, int Hv, int D, float scale,
                             const void* cu_seqlens, const void* chunk_offsets,
                             const void* chunk_indices, int idx_is64, long long num_chunks,
                             int operand_tiles, void* stream) {
  if (!q || !k || !v || !vnew || !A || !g_cum || !beta || !dO || !du || !h || !dh || !dq ||
      !dk || !dv || !db || !dg || Hq <= 0 || Hv % Hq)
    return FQLA_ERR_INVALID_ARG;
  if (cu_seqlens && (!chunk_offsets || !chunk_indices || B != 1)) return FQLA_ERR_INVALID_ARG;
  BwdMainParams p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v;
  p.vnew = (const bf16*)vnew; p.A = (const bf16*)A; p.g = g_cum; p.beta = beta;
  p.beta_is_f32 = beta_is_f32; p.dO = (const bf16*)dO; p.du = (const bf16*)du;
  p.h = (const bf16*)h; p.dh = (const bf16*)dh; p.dq = (bf16*)dq; p.dk = (bf16*)dk;
  p.dv = (bf16*)dv; p.db = db; p.dg = dg; p.Hq = Hq; p.Hv = Hv; p.scale = scale;
  p.lay = SeqLayout{{cu_seqlens, idx_is64}, {chunk_offsets, idx_is64}, T};
  p.chunk_indices = IndexTable{chunk_indices, idx_is64};
  long long n = cu_seqlens ? num_chunks : (long long)B * ((T + CHUNK - 1) / CHUNK);
  if (n <= 0) return FQLA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  static const bool force_legacy = getenv("FQLA_FORCE_MMA_SYNC") != nullptr;
  if (D == 128 && !force_legacy)
    return launch_bwd_main_tc(q, k, v, vnew, A, g_cum, beta, beta_is_f32, dO, du, h, dh, dq, dk, dv,
                              db, dg, operand_tiles, Hq, Hv, (long long)B * T, n, scale, p.lay,
                              p.chunk_indices, st);
  if (operand_tiles) return FQLA_ERR_UNSUPPORTED_DIM;  // only the tcgen05 kernel reads tiles
  if (D == 128) return launch_bwd_main<128>(p, n, st);
  if (D == 64) return launch_bwd_main<64>(p, n, st);
  return FQLA_ERR_UNSUPPORTED_DIM;
}
