// Sequential chunk recurrence of the gated delta rule, forward direction.
//
// One CTA walks the chunks of one (sequence or segment, value head, 64-wide slice of the value
// dimension) in order.  Per chunk, with S [D x BV] the fp32 state entering the chunk (registers)
// and a bf16 copy of it in shared memory as the tensor-core operand:
//     P  = scale * (Q K^T) * exp(g_r - g_c)  for r >= c                (64 x 64)
//     W  = beta * (V - exp(g) * (K S))                                 (64 x BV)
//     Vn = A W                       (A = gated inverse from kkt_solve; Vn is FLA's v_new)
//     O  = scale * exp(g) * (Q S) + P Vn
//     S <- exp(g_last) S + K^T (exp(g_last - g) * Vn)
// This is the computation of the reference's blackwell/fused_fwd.py:22-772 (fused forward) and
// blackwell/prepare_h.py:17-666 (state-only pass); the transition matrix of prepare_h.py:322-362
// falls out of the same loop by running extra slices whose state starts at the identity and
// whose V is zero.
//
// This translation unit is the mma.sync (legacy tensor core) implementation: all eight warps
// cooperate on each product in turn, operands staged by cp.async with the next chunk's tiles in
// flight.  It supports D = 64 and D = 128.
#include <cstdlib>

#include "common.cuh"
#include "fqla_internal.h"

namespace fqla {

// tcgen05 implementation of the full forward (fwd_tc.cu)
int launch_fwd_tc(const void* q, const void* k, const void* v, const void* A, const float* g,
                  const void* beta, int beta_is_f32, const float* h0, float* ht, void* o, void* h,
                  void* vnew, int tiled, const int* lead, const int* order, const int* run_mask,
                  int run_value, int N, int Hq, int Hv, long long T_rows, float scale,
                  SeqLayout lay, cudaStream_t st);

struct FwdSeqParams {
  const bf16* q;      // may be null (state-only pass)
  const bf16* k;
  const bf16* v;
  const bf16* A;
  const float* g;     // chunk-local cumsum
  const void* beta;
  int beta_is_f32;
  const float* h0;    // [N, Hv, D, D] or null
  float* ht;          // [N, Hv, D, D] or null
  bf16* o;            // [rows, Hv, D] or null
  bf16* h;            // [chunks, Hv, D, D] or null
  bf16* vnew;         // [rows, Hv, D] or null
  float* M;           // [N, Hv, D, D] or null: transition matrix (state_end = local + M state_0)
  const int* warm;    // [N, Hv] or null: process only the last warm[n,hv] chunks (state-only)
  const int* m_mask;  // [N, Hv] or null: compute M only where non-zero
  const int* order;   // [N] or null: block index -> sequence (longest first shortens the tail)
  const int* run_mask;  // [N, Hv] or null: pairs whose entry differs from run_value are skipped
  int run_value;
  int N, Hq, Hv;
  long long T_rows;   // total rows of the token axis (for zero-filling the tail of o)
  float scale;
  SeqLayout lay;
};

template <int D, int BV>
struct FwdSeqSmem {
  static constexpr int LDK = D + 8;    // q, k tiles
  static constexpr int LDV = BV + 8;   // v, W, Vn tiles and the state copy
  static constexpr int LDA = CHUNK + 8;
  static constexpr int QK_TILE = CHUNK * LDK;
  static constexpr int V_TILE = CHUNK * LDV;
  static constexpr int A_TILE = CHUNK * LDA;
  static constexpr int S_TILE = D * LDV;
  // element (bf16) offsets
  static constexpr int OFF_Q = 0;                        // 2 stages
  static constexpr int OFF_K = OFF_Q + 2 * QK_TILE;      // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * QK_TILE;      // 2 stages
  static constexpr int OFF_A = OFF_V + 2 * V_TILE;       // 2 stages
  static constexpr int OFF_S = OFF_A + 2 * A_TILE;
  static constexpr int OFF_W = OFF_S + S_TILE;
  static constexpr int OFF_VN = OFF_W + V_TILE;
  static constexpr int OFF_VR = OFF_VN + V_TILE;
  static constexpr int OFF_P = OFF_VR + V_TILE;
  static constexpr int BF16_ELEMS = OFF_P + A_TILE;
  static constexpr int VEC_FLOATS = 4 * CHUNK;           // g, gamma, rho, beta
  static constexpr int BYTES = BF16_ELEMS * 2 + VEC_FLOATS * 4;
};

template <int D, int BV>
__global__ void __launch_bounds__(256, 1) fwd_seq_kernel(const FwdSeqParams p) {
  using L = FwdSeqSmem<D, BV>;
  constexpr int LDK = L::LDK, LDV = L::LDV, LDA = L::LDA;
  constexpr int NTV = BV / 16;  // n-tiles (of 8) per warp for 64 x BV outputs: BV/2 columns
  constexpr int MTS = D / 64;   // m-tiles (of 16) per warp for the D x BV state: D/4 rows
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sm = reinterpret_cast<bf16*>(smem_raw);
  float* sG = reinterpret_cast<float*>(smem_raw + L::BF16_ELEMS * 2);
  float* sGam = sG + CHUNK;
  float* sRho = sGam + CHUNK;
  float* sBeta = sRho + CHUNK;
  bf16* sS = sm + L::OFF_S;
  bf16* sW = sm + L::OFF_W;
  bf16* sVn = sm + L::OFF_VN;
  bf16* sVr = sm + L::OFF_VR;
  bf16* sP = sm + L::OFF_P;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp & 3, wn = warp >> 2;
  const int hv = blockIdx.x % p.Hv;
  const int n = p.order ? p.order[blockIdx.x / p.Hv] : (int)(blockIdx.x / p.Hv);
  const int hq = hv / (p.Hv / p.Hq);
  constexpr int V_SLICES = D / BV;
  const bool m_slice = (int)blockIdx.y >= V_SLICES;  // transition-matrix slice
  const int v0 = (m_slice ? (int)blockIdx.y - V_SLICES : (int)blockIdx.y) * BV;
  const bool with_q = p.q != nullptr && !m_slice;
  const SeqSpan sp = p.lay.span(n);
  if (p.run_mask && p.run_mask[n * p.Hv + hv] != p.run_value) return;  // uniform per CTA
  if (m_slice && p.m_mask && p.m_mask[n * p.Hv + hv] == 0) return;
  if (!m_slice && !p.ht && !p.o && !p.h && !p.vnew) return;          // nothing asked of this slice

  int c_begin = 0;
  if (p.warm) {
    const int w = p.warm[n * p.Hv + hv];
    if (w < 0) return;  // nothing is wanted of this (sequence, head): no output is written
    c_begin = max(0, sp.n_chunks - w);
  }

  // ---- state in registers: rows 32*wm + mt*16 + ..., cols (BV/2)*wn + nt*8 + ...
  float S[MTS][NTV][4];
  const long long state_off = ((long long)n * p.Hv + hv) * D * D;
#pragma unroll
  for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
    for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int r = (16 * MTS) * wm + mt * 16 + (lane >> 2) + (e >> 1) * 8;
        int c = v0 + (BV / 2) * wn + nt * 8 + (lane & 3) * 2 + (e & 1);
        float x = 0.f;
        if (m_slice) x = (r == c) ? 1.f : 0.f;
        else if (p.h0 && c_begin == 0) x = p.h0[state_off + (long long)r * D + c];
        S[mt][nt][e] = x;
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
          st_bf16x2(sS + r * LDV + c, S[mt][nt][2 * hh], S[mt][nt][2 * hh + 1]);
        }
  };
  store_state_copy();

  const long long qk_stride = (long long)p.Hq * D, v_stride = (long long)p.Hv * D;
  auto prefetch = [&](int c, int stage) {
    long long row0 = sp.bos + (long long)c * CHUNK;
    int valid = min(CHUNK, sp.len - c * CHUNK);
    if (with_q)
      load_tile_async<D, LDK, 256>(sm + L::OFF_Q + stage * L::QK_TILE,
                                   p.q + (row0 * p.Hq + hq) * D, qk_stride, valid, tid);
    load_tile_async<D, LDK, 256>(sm + L::OFF_K + stage * L::QK_TILE,
                                 p.k + (row0 * p.Hq + hq) * D, qk_stride, valid, tid);
    if (!m_slice)
      load_tile_async<BV, LDV, 256>(sm + L::OFF_V + stage * L::V_TILE,
                                    p.v + (row0 * p.Hv + hv) * D + v0, v_stride, valid, tid);
    load_tile_async<CHUNK, LDA, 256>(sm + L::OFF_A + stage * L::A_TILE,
                                     p.A + (row0 * p.Hv + hv) * CHUNK,
                                     (long long)p.Hv * CHUNK, valid, tid);
  };
  // per-row gate and beta of a chunk, fetched one chunk ahead into registers (threads 0..63)
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
  if (c_begin < sp.n_chunks) {
    prefetch(c_begin, 0);
    fetch_gb(c_begin, g_next, b_next);
  }
  cp_async_commit();

  for (int c = c_begin; c < sp.n_chunks; ++c) {
    const int stage = (c - c_begin) & 1;
    const long long row0 = sp.bos + (long long)c * CHUNK;
    const int valid = min(CHUNK, sp.len - c * CHUNK);
    bf16* sQ = sm + L::OFF_Q + stage * L::QK_TILE;
    bf16* sK = sm + L::OFF_K + stage * L::QK_TILE;
    bf16* sV = sm + L::OFF_V + stage * L::V_TILE;
    bf16* sA = sm + L::OFF_A + stage * L::A_TILE;

    if (tid < CHUNK) { sG[tid] = g_next; sBeta[tid] = b_next; }
    cp_async_wait<0>();
    __syncthreads();  // tiles of chunk c, sS, sG visible; previous chunk's reads all done
    if (c + 1 < sp.n_chunks) {
      prefetch(c + 1, stage ^ 1);
      fetch_gb(c + 1, g_next, b_next);
    }
    cp_async_commit();
    if (tid < CHUNK) {
      float gl = sG[CHUNK - 1];
      sGam[tid] = fast_exp(sG[tid]);
      sRho[tid] = fast_exp(gl - sG[tid]);
    }
    // per-chunk state out (bf16), straight from the operand copy
    if (p.h && !m_slice) {
      bf16* hdst = p.h + ((sp.chunk_base + c) * p.Hv + hv) * (long long)D * D + v0;
      constexpr int SEGS = BV / 8;
      for (int i = tid; i < D * SEGS; i += 256) {
        int r = i / SEGS, cc = (i % SEGS) * 8;
        *reinterpret_cast<uint4*>(hdst + (long long)r * D + cc) =
            *reinterpret_cast<const uint4*>(sS + r * LDV + cc);
      }
    }
    __syncthreads();  // gamma / rho visible

    // ---------------- phase A: P, W, O_inter ----------------
    const int rA = 16 * wm + (lane >> 2);  // fragment rows rA, rA+8
    float O[1][NTV][4];
    if (with_q) {
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
      zero_acc(O);
      warp_gemm<1, NTV, D / 16, false, true>(O, sQ + 16 * wm * LDK, LDK, sS + (BV / 2) * wn, LDV,
                                             lane);
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) O[0][nt][e] *= p.scale * sGam[rA + (e >> 1) * 8];
    }
    {
      float U[1][NTV][4];
      zero_acc(U);
      warp_gemm<1, NTV, D / 16, false, true>(U, sK + 16 * wm * LDK, LDK, sS + (BV / 2) * wn, LDV,
                                             lane);
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = rA + hh * 8, cc = (BV / 2) * wn + nt * 8 + (lane & 3) * 2;
          float2 vv = m_slice ? make_float2(0.f, 0.f) : ld_bf16x2(sV + r * LDV + cc);
          float gm = sGam[r], bt = sBeta[r];
          st_bf16x2(sW + r * LDV + cc, bt * (vv.x - gm * U[0][nt][2 * hh]),
                    bt * (vv.y - gm * U[0][nt][2 * hh + 1]));
        }
    }
    __syncthreads();

    // ---------------- phase B: Vn = A W ----------------
    {
      float Vn[1][NTV][4];
      zero_acc(Vn);
      warp_gemm<1, NTV, CHUNK / 16, false, true>(Vn, sA + 16 * wm * LDA, LDA, sW + (BV / 2) * wn,
                                                 LDV, lane);
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = rA + hh * 8, cc = (BV / 2) * wn + nt * 8 + (lane & 3) * 2;
          float a = Vn[0][nt][2 * hh], b = Vn[0][nt][2 * hh + 1], rho = sRho[r];
          st_bf16x2(sVn + r * LDV + cc, a, b);
          st_bf16x2(sVr + r * LDV + cc, rho * a, rho * b);
          if (p.vnew && !m_slice && r < valid)
            st_bf16x2(p.vnew + ((row0 + r) * p.Hv + hv) * D + v0 + cc, a, b);
        }
    }
    __syncthreads();

    // ---------------- phase C: O += P Vn ; S update ----------------
    if (with_q && p.o) {
      warp_gemm<1, NTV, CHUNK / 16, false, true>(O, sP + 16 * wm * LDA, LDA, sVn + (BV / 2) * wn,
                                                 LDV, lane);
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = rA + hh * 8, cc = (BV / 2) * wn + nt * 8 + (lane & 3) * 2;
          if (r < valid)
            st_bf16x2(p.o + ((row0 + r) * p.Hv + hv) * D + v0 + cc, O[0][nt][2 * hh],
                      O[0][nt][2 * hh + 1]);
        }
    }
    {
      const float gl = sGam[CHUNK - 1];
#pragma unroll
      for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
        for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) S[mt][nt][e] *= gl;
      warp_gemm<MTS, NTV, CHUNK / 16, true, true>(S, sK + (16 * MTS) * wm, LDK, sVr + (BV / 2) * wn, LDV,
                                                lane);
    }
    // The old state copy was last read in phase A, two barriers ago: safe to overwrite.
    store_state_copy();
  }

  // ---- final state / transition matrix out (fp32)
  float* dst = m_slice ? p.M : p.ht;
  if (dst) {
#pragma unroll
    for (int mt = 0; mt < MTS; ++mt)
#pragma unroll
      for (int nt = 0; nt < NTV; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          int r = (16 * MTS) * wm + mt * 16 + (lane >> 2) + hh * 8;
          int c = v0 + (BV / 2) * wn + nt * 8 + (lane & 3) * 2;
          *reinterpret_cast<float2*>(dst + state_off + (long long)r * D + c) =
              make_float2(S[mt][nt][2 * hh], S[mt][nt][2 * hh + 1]);
        }
  }
  // rows of o past the last sequence's end come out zero
  if (p.o && !m_slice && p.lay.cu.ptr && n == p.N - 1) {
    long long end = sp.bos + sp.len;
    constexpr int SEGS = BV / 8;
    for (long long i = tid; i < (p.T_rows - end) * SEGS; i += 256) {
      long long r = end + i / SEGS;
      int cc = (int)(i % SEGS) * 8;
      *reinterpret_cast<uint4*>(p.o + (r * p.Hv + hv) * D + v0 + cc) = make_uint4(0, 0, 0, 0);
    }
  }
}

template <int D>
static int launch_fwd_seq(const FwdSeqParams& p, cudaStream_t st) {
  constexpr int BV = 64;
  using L = FwdSeqSmem<D, BV>;
  int rc = configure_smem((const void*)fwd_seq_kernel<D, BV>, L::BYTES);
  if (rc != 0) return rc;
  dim3 grid((unsigned)(p.N * p.Hv), (D / BV) * (p.M ? 2 : 1));
  fwd_seq_kernel<D, BV><<<grid, 256, L::BYTES, st>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace fqla

using namespace fqla;

extern "C" int fqla_fwd_seq(const void* q, const void* k, const void* v, const void* A,
                            const float* g_cum, const void* beta, int beta_is_f32,
                            const float* h0, float* ht, void* o, void* h, void* vnew, float* M,
                            const int* warm_chunks, const int* m_mask, const int* lead_chunks,
                            const int* seq_order, const int* run_mask, int run_value, int B, int T,
                            int Hq, int Hv, int D, float scale, const void* cu_seqlens,
                            const void* chunk_offsets, int idx_is64, int N, int operand_tiles,
                            void* stream) {
  if (!k || !v || !A || !g_cum || !beta || Hq <= 0 || Hv % Hq) return FQLA_ERR_INVALID_ARG;
  if (cu_seqlens && (!chunk_offsets || B != 1)) return FQLA_ERR_INVALID_ARG;
  if (o && !q) return FQLA_ERR_INVALID_ARG;
  if (warm_chunks && (q || h || vnew)) return FQLA_ERR_INVALID_ARG;
  if (lead_chunks && (warm_chunks || M || m_mask)) return FQLA_ERR_INVALID_ARG;
  FwdSeqParams p;
  p.q = (const bf16*)q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.A = (const bf16*)A;
  p.g = g_cum; p.beta = beta; p.beta_is_f32 = beta_is_f32;
  p.h0 = h0; p.ht = ht; p.o = (bf16*)o; p.h = (bf16*)h; p.vnew = (bf16*)vnew; p.M = M;
  p.warm = warm_chunks;
  p.m_mask = m_mask;
  p.order = seq_order;
  p.run_mask = run_mask;
  p.run_value = run_value;
  p.N = cu_seqlens ? N : B; p.Hq = Hq; p.Hv = Hv;
  p.T_rows = (long long)B * T;
  p.scale = scale;
  p.lay = SeqLayout{{cu_seqlens, idx_is64}, {chunk_offsets, idx_is64}, T};
  if (p.N <= 0) return FQLA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // The full forward (q and o present, K = V = 128) and the recomputation of the per-chunk
  // states and v_new for the backward pass (neither q nor o) run on the tcgen05 kernel;
  // state-only passes, transition matrices and D = 64 run on the mma.sync kernel in this file.
  static const bool force_legacy = getenv("FQLA_FORCE_MMA_SYNC") != nullptr;
  const bool full = q && o, recompute = !q && !o && (h || vnew);
  if (D == 128 && (full || recompute) && !M && !warm_chunks && !m_mask && !force_legacy)
    return launch_fwd_tc(q, k, v, A, g_cum, beta, beta_is_f32, h0, ht, o, h, vnew, operand_tiles,
                         lead_chunks, seq_order, run_mask, run_value, p.N, Hq, Hv, p.T_rows, scale,
                         p.lay, st);
  if (operand_tiles || lead_chunks) return FQLA_ERR_UNSUPPORTED_DIM;  // tcgen05 kernel only
  if (D == 128) return launch_fwd_seq<128>(p, st);
  if (D == 64) return launch_fwd_seq<64>(p, st);
  return FQLA_ERR_UNSUPPORTED_DIM;
}
