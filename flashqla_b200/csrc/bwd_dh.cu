// Reverse chunk recurrence of the gated delta rule: the gradient of the recurrent state.
//
// One CTA walks the chunks of one (sequence or segment, value head, 64-wide value slice) from
// the last to the first.  With dS [D x BV] the fp32 gradient with respect to the state LEAVING
// the chunk (registers, bf16 copy in shared memory as tensor-core operand):
//     emit dh_c = dS (bf16)
//     w   = A (beta * exp(g) * K)                                     (64 x D, FLA's w)
//     P   = scale * (Q K^T) * exp(g_r - g_c)  for r >= c              (64 x 64)
//     dv  = exp(g_last - g) * (K dS) + P^T dO                         (64 x BV) -> emitted (du)
//     dS <- exp(g_last) dS + Q^T (scale * exp(g) * dO) - w^T dv
// After the first chunk dS is the gradient of the initial state.  This is the recurrence of the
// reference's tests/ref_gdr.py:352-424 (torch_chunk_gdr_bwd, with torch_chunk_dv_bwd :302-349
// folded in); the reference's kernels compute it inside blackwell/fused_bwd.py:336-474 and, for
// context parallelism, in blackwell/cp_bwd.py:16-589.
//
// mma.sync implementation, eight cooperating warps, cp.async double buffering.
#include "common.cuh"
#include "fqla_internal.h"

namespace fqla {

struct BwdDhParams {
  const bf16* q;
  const bf16* k;
  const bf16* A;
  const float* g;
  const void* beta;
  int beta_is_f32;
  const bf16* dO;
  const float* dht;  // [N, Hv, D, D] or null
  bf16* dh;          // [chunks, Hv, D, D] or null
  bf16* du;          // [rows, Hv, D] or null
  float* dh0;        // [N, Hv, D, D] or null
  const int* warm;   // [N, Hv] or null: walk only the first warm[n,hv] chunks (dh0-only pass);
                     // a negative entry skips the (sequence, head) altogether
  const int* order;  // [N] or null: block index -> sequence (longest first shortens the tail)
  const int* run_mask;  // [N, Hv] or null: pairs whose entry differs from run_value are skipped
  int run_value;
  int N, Hq, Hv;
  float scale;
  SeqLayout lay;
};

template <int D, int BV>
struct BwdDhSmem {
  static constexpr int LDK = D + 8;
  static constexpr int LDV = BV + 8;
  static constexpr int LDA = CHUNK + 8;
  static constexpr int QK_TILE = CHUNK * LDK;
  static constexpr int V_TILE = CHUNK * LDV;
  static constexpr int A_TILE = CHUNK * LDA;
  static constexpr int OFF_Q = 0;                     // 2 stages
  static constexpr int OFF_K = OFF_Q + 2 * QK_TILE;   // 2 stages
  static constexpr int OFF_DO = OFF_K + 2 * QK_TILE;  // 2 stages
  static constexpr int OFF_A = OFF_DO + 2 * V_TILE;   // 2 stages
  static constexpr int OFF_KBG = OFF_A + 2 * A_TILE;
  static constexpr int OFF_W = OFF_KBG + QK_TILE;
  static constexpr int OFF_DS = OFF_W + QK_TILE;      // D x LDV
  static constexpr int OFF_DOG = OFF_DS + D * LDV;
  static constexpr int OFF_NDV = OFF_DOG + V_TILE;
  static constexpr int OFF_P = OFF_NDV + V_TILE;
  static constexpr int BF16_ELEMS = OFF_P + A_TILE;
  static constexpr int VEC_FLOATS = 4 * CHUNK;
  static constexpr int BYTES = BF16_ELEMS * 2 + VEC_FLOATS * 4;
};

template <int D, int BV>
__global__ void __launch_bounds__(256, 1) bwd_dh_kernel(const BwdDhParams p) {
  using L = BwdDhSmem<D, BV>;
  constexpr int LDK = L::LDK, LDV = L::LDV, LDA = L::LDA;
  constexpr int NTV = BV / 16;  // n-tiles (of 8) per warp for 64 x BV outputs: BV/2 columns
  constexpr int MTS = D / 64;   // m-tiles (of 16) per warp for the D x BV state: D/4 rows
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sm = reinterpret_cast<bf16*>(smem_raw);
  float* sG = reinterpret_cast<float*>(smem_raw + L::BF16_ELEMS * 2);
  float* sGam = sG + CHUNK;
  float* sRho = sGam + CHUNK;
  float* sBeta = sRho + CHUNK;
  bf16* sKbg = sm + L::OFF_KBG;
  bf16* sW = sm + L::OFF_W;
  bf16* sDS = sm + L::OFF_DS;
  bf16* sDOg = sm + L::OFF_DOG;
  bf16* sNdv = sm + L::OFF_NDV;
  bf16* sP = sm + L::OFF_P;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp & 3, wn = warp >> 2;
  const int hv = blockIdx.x % p.Hv;
  const int n = p.order ? p.order[blockIdx.x / p.Hv] : (int)(blockIdx.x / p.Hv);
  const int hq = hv / (p.Hv / p.Hq);
  const int v0 = blockIdx.y * BV;
  if (p.run_mask && p.run_mask[n * p.Hv + hv] != p.run_value) return;  // uniform per CTA
  const SeqSpan sp = p.lay.span(n);
  int c_end = sp.n_chunks;  // exclusive
  if (p.warm) {
    const int w = p.warm[n * p.Hv + hv];
    if (w < 0) return;  // nothing is wanted of this (sequence, head): no output is written
    c_end = min(sp.n_chunks, w);
  }

  float dS[MTS][NTV][4];
  const long long state_off = ((long long)n * p.Hv + hv) * D * D;
#pragma unroll
  for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int r = (16 * MTS) * wm + mt * 16 + (lane >> 2) + (e >> 1) * 8;
        int c = v0 + (BV / 2) * wn + nt * 8 + (lane & 3) * 2 + (e & 1);
        dS[mt][nt][e] =
            (p.dht && c_end == sp.n_chunks) ? p.dht[state_off + (long long)r * D + c] : 0.f;
      }
  auto store_state_copy = [&]() {
#pragma unroll
    for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = (16 * MTS) * wm + mt * 16 + (lane >> 2) + hh * 8;
          int c = (BV / 2) * wn + nt * 8 + (lane & 3) * 2;
          st_bf16x2(sDS + r * LDV + c, dS[mt][nt][2 * hh], dS[mt][nt][2 * hh + 1]);
        }
  };
  store_state_copy();

  const long long qk_stride = (long long)p.Hq * D, v_stride = (long long)p.Hv * D;
  auto prefetch = [&](int c, int stage) {
    long long row0 = sp.bos + (long long)c * CHUNK;
    int valid = min(CHUNK, sp.len - c * CHUNK);
    load_tile_async<D, LDK, 256>(sm + L::OFF_Q + stage * L::QK_TILE,
                                 p.q + (row0 * p.Hq + hq) * D, qk_stride, valid, tid);
    load_tile_async<D, LDK, 256>(sm + L::OFF_K + stage * L::QK_TILE,
                                 p.k + (row0 * p.Hq + hq) * D, qk_stride, valid, tid);
    load_tile_async<BV, LDV, 256>(sm + L::OFF_DO + stage * L::V_TILE,
                                  p.dO + (row0 * p.Hv + hv) * D + v0, v_stride, valid, tid);
    load_tile_async<CHUNK, LDA, 256>(sm + L::OFF_A + stage * L::A_TILE,
                                     p.A + (row0 * p.Hv + hv) * CHUNK,
                                     (long long)p.Hv * CHUNK, valid, tid);
  };
  auto fetch_gb = [&](int c, float& gval, float& bval) {
    if (tid < CHUNK) {
      long long row0 = sp.bos + (long long)c * CHUNK;
      int valid = min(CHUNK, sp.len - c * CHUNK);
      int r = min(tid, valid - 1);
      gval = p.g[(row0 + r) * p.Hv + hv];
      bval = tid < valid ? load_beta(p.beta, p.beta_is_f32, (row0 + tid) * p.Hv + hv) : 0.f;
    }
  };

  float g_next = 0.f, b_next = 0.f;
  if (c_end > 0) {
    prefetch(c_end - 1, 0);
    fetch_gb(c_end - 1, g_next, b_next);
  }
  cp_async_commit();

  for (int c = c_end - 1; c >= 0; --c) {
    const int stage = (c_end - 1 - c) & 1;
    const long long row0 = sp.bos + (long long)c * CHUNK;
    const int valid = min(CHUNK, sp.len - c * CHUNK);
    bf16* sQ = sm + L::OFF_Q + stage * L::QK_TILE;
    bf16* sK = sm + L::OFF_K + stage * L::QK_TILE;
    bf16* sDO = sm + L::OFF_DO + stage * L::V_TILE;
    bf16* sA = sm + L::OFF_A + stage * L::A_TILE;

    if (tid < CHUNK) { sG[tid] = g_next; sBeta[tid] = b_next; }
    cp_async_wait<0>();
    __syncthreads();
    if (c > 0) {
      prefetch(c - 1, stage ^ 1);
      fetch_gb(c - 1, g_next, b_next);
    }
    cp_async_commit();
    if (tid < CHUNK) {
      float gl = sG[CHUNK - 1];
      sGam[tid] = fast_exp(sG[tid]);
      sRho[tid] = fast_exp(gl - sG[tid]);
    }
    if (p.dh) {
      bf16* dst = p.dh + ((sp.chunk_base + c) * p.Hv + hv) * (long long)D * D + v0;
      constexpr int SEGS = BV / 8;
      for (int i = tid; i < D * SEGS; i += 256) {
        int r = i / SEGS, cc = (i % SEGS) * 8;
        *reinterpret_cast<uint4*>(dst + (long long)r * D + cc) =
            *reinterpret_cast<const uint4*>(sDS + r * LDV + cc);
      }
    }
    __syncthreads();

    // ---------------- phase A ----------------
    const int rA = 16 * wm + (lane >> 2);
    // beta*gamma*K and scale*gamma*dO as bf16 operands (elementwise, all threads)
    for (int i = tid; i < CHUNK * (D / 2); i += 256) {
      int r = i / (D / 2), cc = (i % (D / 2)) * 2;
      float2 kk = ld_bf16x2(sK + r * LDK + cc);
      float f = sBeta[r] * sGam[r];
      st_bf16x2(sKbg + r * LDK + cc, f * kk.x, f * kk.y);
    }
    for (int i = tid; i < CHUNK * (BV / 2); i += 256) {
      int r = i / (BV / 2), cc = (i % (BV / 2)) * 2;
      float2 d = ld_bf16x2(sDO + r * LDV + cc);
      float f = p.scale * sGam[r];
      st_bf16x2(sDOg + r * LDV + cc, f * d.x, f * d.y);
    }
    {
      float P[1][4][4];
      zero_acc(P);
      warp_gemm<1, 4, D / 16, false, false>(P, sQ + 16 * wm * LDK, LDK, sK + 32 * wn * LDK, LDK,
                                            lane);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = rA + hh * 8, cc = 32 * wn + nt * 8 + (lane & 3) * 2;
          float gr = sG[r];
          float x0 = r >= cc ? p.scale * P[0][nt][2 * hh] * fast_exp(gr - sG[cc]) : 0.f;
          float x1 = r >= cc + 1 ? p.scale * P[0][nt][2 * hh + 1] * fast_exp(gr - sG[cc + 1]) : 0.f;
          st_bf16x2(sP + r * LDA + cc, x0, x1);
        }
    }
    float dv[1][NTV][4];
    zero_acc(dv);
    warp_gemm<1, NTV, D / 16, false, true>(dv, sK + 16 * wm * LDK, LDK, sDS + (BV / 2) * wn, LDV,
                                           lane);
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) dv[0][nt][e] *= sRho[rA + (e >> 1) * 8];
    __syncthreads();

    // ---------------- phase B: w, dv ----------------
    {
      float Wt[1][D / 16][4];
      zero_acc(Wt);
      warp_gemm<1, D / 16, CHUNK / 16, false, true>(Wt, sA + 16 * wm * LDA, LDA,
                                                    sKbg + (D / 2) * wn, LDK, lane);
#pragma unroll
      for (int nt = 0; nt < D / 16; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = rA + hh * 8, cc = (D / 2) * wn + nt * 8 + (lane & 3) * 2;
          st_bf16x2(sW + r * LDK + cc, Wt[0][nt][2 * hh], Wt[0][nt][2 * hh + 1]);
        }
    }
    warp_gemm<1, NTV, CHUNK / 16, true, true>(dv, sP + 16 * wm, LDA, sDO + (BV / 2) * wn, LDV,
                                              lane);
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        int r = rA + hh * 8, cc = (BV / 2) * wn + nt * 8 + (lane & 3) * 2;
        float a = dv[0][nt][2 * hh], b = dv[0][nt][2 * hh + 1];
        st_bf16x2(sNdv + r * LDV + cc, -a, -b);
        if (p.du && r < valid) st_bf16x2(p.du + ((row0 + r) * p.Hv + hv) * D + v0 + cc, a, b);
      }
    __syncthreads();

    // ---------------- phase C: dS update ----------------
    {
      const float gl = sGam[CHUNK - 1];
#pragma unroll
      for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
        for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) dS[mt][nt][e] *= gl;
      warp_gemm<MTS, NTV, CHUNK / 16, true, true>(dS, sQ + (16 * MTS) * wm, LDK, sDOg + (BV / 2) * wn, LDV,
                                                lane);
      warp_gemm<MTS, NTV, CHUNK / 16, true, true>(dS, sW + (16 * MTS) * wm, LDK, sNdv + (BV / 2) * wn, LDV,
                                                lane);
    }
    store_state_copy();  // last read in phase A, two barriers ago
  }

  if (p.dh0) {
#pragma unroll
    for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = (16 * MTS) * wm + mt * 16 + (lane >> 2) + hh * 8;
          int c = v0 + (BV / 2) * wn + nt * 8 + (lane & 3) * 2;
          *reinterpret_cast<float2*>(p.dh0 + state_off + (long long)r * D + c) =
              make_float2(dS[mt][nt][2 * hh], dS[mt][nt][2 * hh + 1]);
        }
  }
}

template <int D>
static int launch_bwd_dh(const BwdDhParams& p, cudaStream_t st) {
  constexpr int BV = 64;
  using L = BwdDhSmem<D, BV>;
  int rc = configure_smem((const void*)bwd_dh_kernel<D, BV>, L::BYTES);
  if (rc != 0) return rc;
  dim3 grid((unsigned)(p.N * p.Hv), D / BV);
  bwd_dh_kernel<D, BV><<<grid, 256, L::BYTES, st>>>(p);
  return (int)cudaGetLastError();
}

// tcgen05 version for K = V = 128, full walks only (bwd_dh_tc.cu)
int launch_bwd_dh_tc(const void* q, const void* k, const void* A, const float* g, const void* beta,
                     int beta_is_f32, const void* dO, const float* dht, void* dh, void* du,
                     float* dh0, int tiled, const int* lead, const int* order, const int* run_mask,
                     int run_value, int N, int Hq, int Hv,
                     long long T_rows, float scale, SeqLayout lay, cudaStream_t st);

}  // namespace fqla

using namespace fqla;

extern "C" int fqla_bwd_dh(const void* q, const void* k, const void* A, const float* g_cum,
                           const void* beta, int beta_is_f32, const void* dO, const float* dht,
                           void* dh, void* du, float* dh0, const int* warm_chunks,
                           const int* lead_chunks, const int* seq_order, const int* run_mask,
                           int run_value, int B, int T, int Hq, int Hv, int D, float scale,
                           const void* cu_seqlens,
                           const void* chunk_offsets, int idx_is64, int N, int operand_tiles,
                           void* stream) {
  if (!q || !k || !A || !g_cum || !beta || !dO || Hq <= 0 || Hv % Hq)
    return FQLA_ERR_INVALID_ARG;
  if (cu_seqlens && (!chunk_offsets || B != 1)) return FQLA_ERR_INVALID_ARG;
  if (warm_chunks && (dh || du)) return FQLA_ERR_INVALID_ARG;
  if (lead_chunks && warm_chunks) return FQLA_ERR_INVALID_ARG;
  BwdDhParams p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.A = (const bf16*)A; p.g = g_cum;
  p.beta = beta; p.beta_is_f32 = beta_is_f32; p.dO = (const bf16*)dO; p.dht = dht;
  p.dh = (bf16*)dh; p.du = (bf16*)du; p.dh0 = dh0; p.warm = warm_chunks; p.order = seq_order;
  p.run_mask = run_mask; p.run_value = run_value;
  p.N = cu_seqlens ? N : B; p.Hq = Hq; p.Hv = Hv; p.scale = scale;
  p.lay = SeqLayout{{cu_seqlens, idx_is64}, {chunk_offsets, idx_is64}, T};
  if (p.N <= 0) return FQLA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  static const bool force_legacy = getenv("FQLA_FORCE_MMA_SYNC") != nullptr;
  if (D == 128 && !warm_chunks && !force_legacy)
    return launch_bwd_dh_tc(q, k, A, g_cum, beta, beta_is_f32, dO, dht, dh, du, dh0,
                            operand_tiles, lead_chunks, seq_order, run_mask, run_value, p.N, Hq, Hv, (long long)B * T, scale, p.lay,
                            st);
  // only the tcgen05 kernel writes tiles or leads out
  if (operand_tiles || lead_chunks) return FQLA_ERR_UNSUPPORTED_DIM;
  if (D == 128) return launch_bwd_dh<128>(p, st);
  if (D == 64) return launch_bwd_dh<64>(p, st);
  return FQLA_ERR_UNSUPPORTED_DIM;
}
