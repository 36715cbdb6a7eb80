// Reverse chunk recurrence of the gated delta rule (gradient of the recurrent state) on Blackwell
// tensor cores, K = V = 128.  Same mathematics and outputs as bwd_dh.cu (reference:
// tests/ref_gdr.py:302-424; the reference's kernels compute it inside
// blackwell/fused_bwd.py:336-474): one CTA walks the chunks of one (sequence or segment, value
// head) from the last to the first.
//
// The state gradient is kept transposed, dS^T [v][k], fp32 in tensor memory (128 lanes = value
// index).  Per chunk, with Kc/Qc/dOc/Ac the chunk's tiles:
//     emit dh_c = dS                                   (bf16; also the operand copy in smem)
//     X1^T = dS^T Kc^T                  [v][tok]       on the chain
//     X2^T = dOc^T Pg                   [v][tok]       Pg = scale * G .* (Qc Kc^T), lower tri.
//     dv^T = rho .* X1^T + X2^T                        -> bf16 operand, emitted as du
//     w    = (Ac diag(beta gamma)) Kc   [tok][k]
//     dS^T <- gamma_last dS^T - dv^T w + dOc^T (scale gamma .* Qc)
// Six roles as in the forward kernel (fwd_tc.cu): warp 0 issues every tcgen05.mma, warp 1 runs the
// TMA pipeline (two stages of q, k, dO, A) and the per-row vectors, warps 2-3 scale A and q,
// warps 4-7 own the state (operand copy, decay, dh / dh0 output), warps 8-11 turn X1, X2 and w
// into operands (and write du), warps 12-15 build Pg.  All waits are bounded mbarrier waits.
#include <cuda.h>

#include "common.cuh"
#include "fqla_internal.h"
#include "tc05.cuh"

namespace fqla {

using namespace tc;

// set to 1 when a CTA of this file's kernel abandoned a bounded wait
__device__ int g_bwd_dh_status = 0;

struct BwdDhTcParams {
  const float* g;
  const void* beta;
  int beta_is_f32;
  const float* dht;  // [N, Hv, D, D] or null
  bf16* dh;          // [chunks, Hv, D, D] or null
  bf16* du;          // [rows, Hv, D] or null
  float* dh0;        // [N, Hv, D, D] or null
  int N, Hq, Hv;
  float scale;
  SeqLayout lay;
  int tiled;  // dh and du are written as operand tiles (dh^T, du^T per chunk) by TMA
  const int* order;  // [N] or null: block index -> sequence (longest first shortens the tail)
  // [N, Hv] or null: lead-out.  A CTA with lead > 0 starts from a ZERO state gradient `lead`
  // chunks after the end of its segment (those rows are the head of segment n + 1 of the same
  // sequence), walks them without output and enters its own last chunk with the gradient it
  // would have been handed, up to what the gates let through of anything later.  dht is ignored
  // for such a CTA.
  const int* lead;
  // [N, Hv] or null: a CTA whose entry differs from run_value returns at once
  const int* run_mask;
  int run_value;
};

namespace bdtc {
constexpr int D = 128;
constexpr int TILE = 16384, TILE_A = 8192;
constexpr int STAGE_BYTES = 3 * TILE + TILE_A;  // q, k, dO, A
constexpr int OFF_STAGE = 0;
constexpr int OFF_ST = 2 * STAGE_BYTES;   // dS^T copy, 2 blocks of [128 x 128B]
constexpr int OFF_DVT = OFF_ST + 32768;   // dv^T   [128 x 128B]
constexpr int OFF_W = OFF_DVT + 16384;    // w      2 blocks of [64 x 128B]
constexpr int OFF_P = OFF_W + 16384;      // Pg     [64 x 128B]
constexpr int OFF_APP = OFF_P + 8192;     // A diag(beta gamma)
constexpr int OFF_QS = OFF_APP + 8192;    // scale gamma .* q, 2 blocks of [64 x 128B]
constexpr int OFF_VEC = OFF_QS + TILE;
constexpr int VEC_SLOT_FLOATS = 5 * CHUNK;
constexpr int OFF_BAR = OFF_VEC + 4 * VEC_SLOT_FLOATS * 4;
constexpr int N_BARS = 24;
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;
constexpr uint32_t TM_S = 0, TM_X1 = 128, TM_X2 = 192, TM_P = 256, TM_W = 384;
enum { FULL0 = 0, FULL1, EMPTY0, EMPTY1, S_COPY, S_DEC, X1_DONE, X2_DONE, S_DONE, P_DONE, W_DONE,
       DV_READY, W_READY, P_READY, AP_READY, QS_READY, PRIV,
       // the A tile and the per-row vectors of a chunk travel one chunk ahead of q, k, dO
       FULLA0, FULLA1, EMPTYA0, EMPTYA1, PRIVA };
enum { V_G = 0, V_BG = 1, V_RHO = 2, V_SGAM = 3, V_GL = 4 };
}  // namespace bdtc

__device__ __forceinline__ uint32_t scale2(uint32_t packed, float lo, float hi) {
  float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&packed));
  return pack_bf16(f.x * lo, f.y * hi);
}

__global__ void __launch_bounds__(512, 1)
bwd_dh_tc_kernel(const BwdDhTcParams p, const __grid_constant__ CUtensorMap map_q,
                 const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_do,
                 const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_dh,
                 const __grid_constant__ CUtensorMap map_du) {
  using namespace bdtc;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);
  float* vec = reinterpret_cast<float*>(smem + OFF_VEC);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hv = blockIdx.x % p.Hv;
  const int n = p.order ? p.order[blockIdx.x / p.Hv] : (int)(blockIdx.x / p.Hv);
  const int hq = hv / (p.Hv / p.Hq);
  if (p.run_mask && p.run_mask[n * p.Hv + hv] != p.run_value) return;  // uniform per CTA
  const SeqSpan sp = p.lay.span(n);
  // iteration `it` handles chunk n_it - 1 - it of the segment; chunks >= sp.n_chunks are the
  // lead-out chunks (whole chunks, except possibly the very last one of the sequence)
  const int lead = (p.lead && sp.n_chunks > 0) ? p.lead[n * p.Hv + hv] : 0;
  const int n_it = sp.n_chunks + lead;
  const int len_ext = sp.len + (lead > 0 ? min(lead * CHUNK, p.lay.span(n + 1).len) : 0);

  if (tid == 0) {
    mbar_init(&bars[FULL0], 1);
    mbar_init(&bars[FULL1], 1);
    mbar_init(&bars[EMPTY0], 1 + 2);  // MMA commit + the two scaling warps
    mbar_init(&bars[EMPTY1], 1 + 2);
    mbar_init(&bars[S_COPY], 128);
    mbar_init(&bars[S_DEC], 128);
    mbar_init(&bars[X1_DONE], 1);
    mbar_init(&bars[X2_DONE], 1);
    mbar_init(&bars[S_DONE], 1);
    mbar_init(&bars[P_DONE], 1);
    mbar_init(&bars[W_DONE], 1);
    mbar_init(&bars[DV_READY], 128);
    mbar_init(&bars[W_READY], 128);
    mbar_init(&bars[P_READY], 128);
    mbar_init(&bars[AP_READY], 2);
    mbar_init(&bars[QS_READY], 2);
    mbar_init(&bars[PRIV], 1);
    mbar_init(&bars[FULLA0], 1);
    mbar_init(&bars[FULLA1], 1);
    mbar_init(&bars[EMPTYA0], 2);  // the two scaling warps, the only readers of the raw A tile
    mbar_init(&bars[EMPTYA1], 2);
    mbar_init(&bars[PRIVA], 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_do);
    tma_prefetch_desc(&map_a);
  }
  // Pg is lower triangular: zeroed once, only the column groups that can be non-zero are rewritten
  for (int i = tid; i < 8192 / 16; i += 512)
    *reinterpret_cast<uint4*>(smem + OFF_P + i * 16) = make_uint4(0, 0, 0, 0);
  fence_proxy_async();
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
  const long long state_off = ((long long)n * p.Hv + hv) * D * D;
  bool ok = true;
  auto WAIT = [&](int idx, uint32_t parity) { return mbar_wait(&bars[idx], parity, abort_flag); };

  if (warp >= 4 && warp < 8) {
    // =============================== state group ===============================
    const int v = tid - 128;
#pragma unroll 1
    for (int k0 = 0; k0 < D; k0 += 32) {
      float x[32];
#pragma unroll
      for (int j = 0; j < 32; ++j)
        x[j] = (p.dht && lead == 0) ? p.dht[state_off + (long long)(k0 + j) * D + v] : 0.f;
      tmem_st32(tmem + lane_sel + TM_S + k0, x);
    }
    tmem_st_wait();
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1, c = n_it - 1 - it;
      if (it > 0) ok = WAIT(S_DONE, (it - 1) & 1);
      if (!ok) break;
      tc_fence_after();
      bf16* hdst = (p.dh && it >= lead)
                       ? p.dh + ((sp.chunk_base + c) * p.Hv + hv) * (long long)D * D : nullptr;
#pragma unroll 1
      for (int kb = 0; kb < 2; ++kb) {
        float x[32], y[32];
        tmem_ld32(tmem + lane_sel + TM_S + kb * 64, x);
        tmem_ld32(tmem + lane_sel + TM_S + kb * 64 + 32, y);
        tmem_ld_wait();
        unsigned char* row = smem + OFF_ST + kb * 16384 + v * 128;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          *reinterpret_cast<uint4*>(row + ((cc ^ (v & 7)) << 4)) =
              make_uint4(pack_bf16(x[8 * cc + 0], x[8 * cc + 1]), pack_bf16(x[8 * cc + 2], x[8 * cc + 3]),
                         pack_bf16(x[8 * cc + 4], x[8 * cc + 5]), pack_bf16(x[8 * cc + 6], x[8 * cc + 7]));
          *reinterpret_cast<uint4*>(row + (((cc + 4) ^ (v & 7)) << 4)) =
              make_uint4(pack_bf16(y[8 * cc + 0], y[8 * cc + 1]), pack_bf16(y[8 * cc + 2], y[8 * cc + 3]),
                         pack_bf16(y[8 * cc + 4], y[8 * cc + 5]), pack_bf16(y[8 * cc + 6], y[8 * cc + 7]));
        }
        if (hdst && !p.tiled) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            hdst[(long long)(kb * 64 + j) * D + v] = __float2bfloat16(x[j]);
            hdst[(long long)(kb * 64 + 32 + j) * D + v] = __float2bfloat16(y[j]);
          }
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[S_COPY]);
      // off the chain: decay in place
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (!ok) break;
      const float gl = vec[(it & 3) * VEC_SLOT_FLOATS + V_GL * CHUNK];
#pragma unroll 1
      for (int kb = 0; kb < 2; ++kb) {
        float x[32], y[32];
        tmem_ld32(tmem + lane_sel + TM_S + kb * 64, x);
        tmem_ld32(tmem + lane_sel + TM_S + kb * 64 + 32, y);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          x[j] *= gl;
          y[j] *= gl;
        }
        tmem_st32(tmem + lane_sel + TM_S + kb * 64, x);
        tmem_st32(tmem + lane_sel + TM_S + kb * 64 + 32, y);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[S_DEC]);
    }
    if (ok && n_it > 0) ok = WAIT(S_DONE, (n_it - 1) & 1);
    if (ok && p.dh0) {
      tc_fence_after();
#pragma unroll 1
      for (int k0 = 0; k0 < D; k0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_S + k0, x);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) p.dh0[state_off + (long long)(k0 + j) * D + v] = x[j];
      }
    }
  } else if (warp >= 8 && warp < 12) {
    // =============================== dv / w group ===============================
    const int v = tid - 256;
    const int wq = warp & 3;
    const int tok_w = 16 * wq + lane;  // lanes 0-15 of each quarter hold a row of w
    auto convert_w = [&](int it) {
      if (!WAIT(W_DONE, it & 1)) return false;
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_W + c0, x);
        tmem_ld_wait();
        if (lane < 16) {
          unsigned char* row = smem + OFF_W + (c0 >> 6) * 8192 + tok_w * 128;
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
            *reinterpret_cast<uint4*>(row + (((((c0 & 63) >> 3) + cc) ^ (tok_w & 7)) << 4)) =
                make_uint4(pack_bf16(x[8 * cc + 0], x[8 * cc + 1]), pack_bf16(x[8 * cc + 2], x[8 * cc + 3]),
                           pack_bf16(x[8 * cc + 4], x[8 * cc + 5]), pack_bf16(x[8 * cc + 6], x[8 * cc + 7]));
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[W_READY]);
      return true;
    };
    if (n_it > 0) ok = convert_w(0);
    for (int it = 0; it < n_it && ok; ++it) {
      const int c = n_it - 1 - it;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = min(CHUNK, len_ext - c * CHUNK);
      ok = WAIT(FULL0 + (it & 1), (it >> 1) & 1) && WAIT(X2_DONE, it & 1) && WAIT(X1_DONE, it & 1);
      if (!ok) break;
      tc_fence_after();
      const float* rho = vec + (it & 3) * VEC_SLOT_FLOATS + V_RHO * CHUNK;
      unsigned char* row = smem + OFF_DVT + v * 128;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {  // 32 tokens per round
        float x[32], y[32];
        tmem_ld32(tmem + lane_sel + TM_X1 + 32 * h, x);
        tmem_ld32(tmem + lane_sel + TM_X2 + 32 * h, y);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 r = *reinterpret_cast<const float4*>(rho + 32 * h + j);
          x[j] = r.x * x[j] + y[j];
          x[j + 1] = r.y * x[j + 1] + y[j + 1];
          x[j + 2] = r.z * x[j + 2] + y[j + 2];
          x[j + 3] = r.w * x[j + 3] + y[j + 3];
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
          *reinterpret_cast<uint4*>(row + (((4 * h + cc) ^ (v & 7)) << 4)) =
              make_uint4(pack_bf16(x[8 * cc + 0], x[8 * cc + 1]), pack_bf16(x[8 * cc + 2], x[8 * cc + 3]),
                         pack_bf16(x[8 * cc + 4], x[8 * cc + 5]), pack_bf16(x[8 * cc + 6], x[8 * cc + 7]));
        if (h == 1) {  // operand complete, accumulators read: hand over before the global stores
          fence_proxy_async();
          tc_fence_before();
          mbar_arrive(&bars[DV_READY]);
        }
        if (p.du && !p.tiled && it >= lead) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (32 * h + j < valid)
              p.du[((row0 + 32 * h + j) * p.Hv + hv) * D + v] = __float2bfloat16(x[j]);
        }
      }
      if (it + 1 < n_it) ok = convert_w(it + 1);
    }
  } else if (warp >= 12) {
    // =============================== Pg group ===============================
    const int wq = warp & 3;
    const int row_a = 16 * wq + (lane >> 2), row_b = row_a + 8, cp = 2 * (lane & 3);
    const uint32_t lanes_p = (uint32_t)(wq * 32) << 16;
    const float log2_scale = log2f(p.scale);
    for (int it = 0; it < n_it && ok; ++it) {
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      ok = WAIT(FULL0 + (it & 1), (it >> 1) & 1) && WAIT(P_DONE, it & 1);
      if (ok && it > 0) ok = WAIT(X2_DONE, (it - 1) & 1);  // the previous Pg tile has been consumed
      if (!ok) break;
      tc_fence_after();
      const float ga2 = vs[V_G * CHUNK + row_a] * 1.4426950408889634f + log2_scale;
      const float gb2 = vs[V_G * CHUNK + row_b] * 1.4426950408889634f + log2_scale;
      float x[32];
      tmem_ld_16x64(tmem + lanes_p + TM_P, x);
      tmem_ld_wait();
      unsigned char* pa = smem + OFF_P + row_a * 128 + cp * 2;
      unsigned char* pb = smem + OFF_P + row_b * 128 + cp * 2;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i > 2 * wq + 1) continue;
        const float2 gc = *reinterpret_cast<const float2*>(vs + V_G * CHUNK + 8 * i + cp);
        const int col = 8 * i + cp;
        const float e0 = -1.4426950408889634f * gc.x, e1 = -1.4426950408889634f * gc.y;
        const float a0 = col <= row_a ? x[4 * i] * exp2f(e0 + ga2) : 0.f;
        const float a1 = col + 1 <= row_a ? x[4 * i + 1] * exp2f(e1 + ga2) : 0.f;
        const float b0 = col <= row_b ? x[4 * i + 2] * exp2f(e0 + gb2) : 0.f;
        const float b1 = col + 1 <= row_b ? x[4 * i + 3] * exp2f(e1 + gb2) : 0.f;
        *reinterpret_cast<uint32_t*>(pa + ((i ^ (row_a & 7)) << 4)) = pack_bf16(a0, a1);
        *reinterpret_cast<uint32_t*>(pb + ((i ^ (row_b & 7)) << 4)) = pack_bf16(b0, b1);
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[P_READY]);
    }
  } else if (warp == 0) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t ID_P = idesc_bf16(64, 64, 0, 0);
      constexpr uint32_t ID_X1 = idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t ID_X2 = idesc_bf16(128, 64, 1, 1);
      constexpr uint32_t ID_W = idesc_bf16(64, 128, 0, 1);
      constexpr uint32_t ID_UPD_W = idesc_bf16(128, 128, 0, 1) | (1u << 13);  // A negated
      constexpr uint32_t ID_UPD_Q = idesc_bf16(128, 128, 1, 1);
      const uint32_t st_lo = desc_lo_kmajor(smem + OFF_ST), dvt_lo = desc_lo_kmajor(smem + OFF_DVT);
      const uint32_t wmn_lo = desc_lo_mnmajor(smem + OFF_W, 8192), pmn_lo = desc_lo_mnmajor(smem + OFF_P, 8192);
      const uint32_t app_lo = desc_lo_kmajor(smem + OFF_APP);
      const uint32_t qsmn_lo = desc_lo_mnmajor(smem + OFF_QS, 8192);
      const uint32_t q0_lo = desc_lo_kmajor(smem + OFF_STAGE);
      const uint32_t k0_lo = desc_lo_kmajor(smem + OFF_STAGE + TILE);
      const uint32_t kmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + TILE, 8192);
      const uint32_t domn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + 2 * TILE, 8192);
      constexpr uint32_t STAGE_LO = STAGE_BYTES >> 4;
      auto issue_w = [&](uint32_t so) {
        umma_group<4, 2, 0, 128, 0, false>(tmem + TM_W, app_lo, kmn0_lo + so, ID_W);
        umma_commit(&bars[W_DONE]);
      };
      auto issue_p = [&](uint32_t so) {
        umma_group<8, 2, 512, 2, 512, false>(tmem + TM_P, q0_lo + so, k0_lo + so, ID_P);
        umma_commit(&bars[P_DONE]);
      };
      auto issue_x2 = [&](uint32_t so) {
        umma_group<4, 128, 0, 128, 0, false>(tmem + TM_X2, domn0_lo + so, pmn_lo, ID_X2);
        umma_commit(&bars[X2_DONE]);
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t so = s ? STAGE_LO : 0u, so_next = s ? 0u : STAGE_LO;
        if (it == 0) {
          ok = WAIT(FULL0, 0) && WAIT(AP_READY, 0);
          if (!ok) break;
          tc_fence_after();
          issue_w(0);
          issue_p(0);
          ok = WAIT(P_READY, 0);
          if (!ok) break;
          tc_fence_after();
          issue_x2(0);
        }
        ok = WAIT(S_COPY, it & 1);
        if (!ok) break;
        tc_fence_after();
        // X1^T = dS^T K^T   (on the chain)
        umma_group<8, 2, 1024, 2, 512, false>(tmem + TM_X1, st_lo, k0_lo + so, ID_X1);
        tma_store_wait_read();  // du^T of the chunk before has left its tile
        umma_commit(&bars[X1_DONE]);
        const int y_tile = (int)(((sp.chunk_base + (n_it - 1 - it)) * p.Hv + hv) * D);
        if (p.tiled && p.dh && it >= lead) {  // the operand copy of dS^T is dh of this chunk
          tma_store_2d(&map_dh, 0, y_tile, smem + OFF_ST);
          tma_store_2d(&map_dh, 64, y_tile, smem + OFF_ST + 16384);
          tma_store_commit();
        }
        if (it + 1 < n_it) {
          ok = WAIT(FULL0 + (s ^ 1), ((it + 1) >> 1) & 1);
          if (!ok) break;
          issue_p(so_next);  // the Pg group has read P of this chunk (P_READY waited below/earlier)
        }
        ok = WAIT(W_READY, it & 1) && WAIT(QS_READY, it & 1) && WAIT(S_DEC, it & 1) &&
             WAIT(DV_READY, it & 1);
        if (!ok) break;
        tc_fence_after();
        // dS^T <- dS^T - dv^T w + dO^T (scale gamma q)
        umma_group<4, 2, 0, 128, 0, true>(tmem + TM_S, dvt_lo, wmn_lo, ID_UPD_W);
        umma_group<4, 128, 0, 128, 0, true>(tmem + TM_S, domn0_lo + so, qsmn_lo, ID_UPD_Q);
        tma_store_wait_read();  // the dS^T tile may be rewritten after this
        umma_commit(&bars[S_DONE]);
        if (p.tiled && p.du && it >= lead) {
          tma_store_2d(&map_du, 0, y_tile, smem + OFF_DVT);
          tma_store_commit();
        }
        umma_commit(&bars[EMPTY0 + s]);
        if (it + 1 < n_it) {
          ok = WAIT(AP_READY, (it + 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_w(so_next);
          ok = WAIT(P_READY, (it + 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_x2(so_next);
        }
      }
      tma_store_wait_all();
    }
  } else if (warp == 1) {
    // =============================== producer ===============================
    float g_r[2] = {0.f, 0.f}, b_r[2] = {0.f, 0.f}, gl_r = 0.f;
    auto fetch = [&](int it) {
      const int c = n_it - 1 - it;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = min(CHUNK, len_ext - c * CHUNK);
      gl_r = p.g[(row0 + valid - 1) * p.Hv + hv];
#pragma unroll
      for (int z = 0; z < 2; ++z) {
        int r = 2 * lane + z, rc = min(r, valid - 1);
        g_r[z] = p.g[(row0 + rc) * p.Hv + hv];
        b_r[z] = r < valid ? load_beta(p.beta, p.beta_is_f32, (row0 + r) * p.Hv + hv) : 0.f;
      }
    };
    // vectors and A tile of the chunk of iteration j (its stage's A buffer is free once the
    // scaling warps have read it)
    auto a_part = [&](int j) {
      const int sj = j & 1, c = n_it - 1 - j;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = min(CHUNK, len_ext - c * CHUNK);
      if (j >= 2 && !WAIT(EMPTYA0 + sj, ((j >> 1) - 1) & 1)) return false;
      float* vs = vec + (j & 3) * VEC_SLOT_FLOATS;
#pragma unroll
      for (int z = 0; z < 2; ++z) {
        int r = 2 * lane + z;
        float gam = fast_exp(g_r[z]);
        vs[V_G * CHUNK + r] = g_r[z];
        vs[V_BG * CHUNK + r] = b_r[z] * gam;
        vs[V_RHO * CHUNK + r] = fast_exp(gl_r - g_r[z]);
        vs[V_SGAM * CHUNK + r] = p.scale * gam;
      }
      if (lane == 0) vs[V_GL * CHUNK] = fast_exp(gl_r);
      __syncwarp();
      unsigned char* dst = smem + OFF_STAGE + sj * STAGE_BYTES + 3 * TILE;
      const bool partial = valid < CHUNK;
      uint64_t* bar = partial ? &bars[PRIVA] : &bars[FULLA0 + sj];
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, TILE_A);
        tma_load_2d(dst, &map_a, hv * CHUNK, (int)row0, bar);
      }
      if (partial) {
        // only the last chunk of a sequence (the first one walked) can be partial: used once
        if (!WAIT(PRIVA, 0)) return false;
        for (int i = lane; i < (CHUNK - valid) * 8; i += 32)
          *reinterpret_cast<uint4*>(dst + (valid + (i >> 3)) * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[FULLA0 + sj]);
      }
      return true;
    };
    if (n_it > 0) {
      fetch(0);
      ok = a_part(0);
      if (n_it > 1) fetch(1);
    }
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1, c = n_it - 1 - it;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = min(CHUNK, len_ext - c * CHUNK);
      if (it >= 2) {
        ok = WAIT(EMPTY0 + s, ((it >> 1) - 1) & 1);
        if (!ok) break;
      }
      unsigned char* st = smem + OFF_STAGE + s * STAGE_BYTES;
      const bool partial = valid < CHUNK;
      uint64_t* bar = partial ? &bars[PRIV] : &bars[FULL0 + s];
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, STAGE_BYTES - TILE_A);
        const int y = (int)row0;
        tma_load_2d(st + TILE, &map_k, hq * D, y, bar);
        tma_load_2d(st + TILE + 8192, &map_k, hq * D + 64, y, bar);
        tma_load_2d(st, &map_q, hq * D, y, bar);
        tma_load_2d(st + 8192, &map_q, hq * D + 64, y, bar);
        tma_load_2d(st + 2 * TILE, &map_do, hv * D, y, bar);
        tma_load_2d(st + 2 * TILE + 8192, &map_do, hv * D + 64, y, bar);
      }
      if (partial) {
        ok = WAIT(PRIV, 0);
        if (!ok) break;
        for (int blk = 0; blk < 6; ++blk) {
          unsigned char* base = st + blk * 8192;
          for (int i = lane; i < (CHUNK - valid) * 8; i += 32)
            *reinterpret_cast<uint4*>(base + (valid + (i >> 3)) * 128 + ((i & 7) << 4)) =
                make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[FULL0 + s]);
      }
      // the next chunk's vectors and A tile go out a whole chunk before its q, k, dO; slot
      // (it + 1) % 4 of the vectors was last read for the chunk of iteration it - 3, which the wait
      // on the stage of iteration it - 2 above has seen finished
      if (it + 1 < n_it) {
        ok = a_part(it + 1);
        if (ok && it + 2 < n_it) fetch(it + 2);
      }
    }
  } else {
    // =============================== scaling warps (2, 3) ===============================
    // A'' = A diag(beta gamma) (columns): thread t owns the 8 columns 8 (t%8) .. of the rows
    // t/8 + 8 i, its scale factors stay in registers and the eight threads of a row touch one
    // 128-byte line per access.  q' = scale gamma .* q (rows): one thread per row, rotated order.
    const int r = tid - 64;
    const int c8 = r & 7, r0 = r >> 3, pc_a = c8 ^ r0;
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      ok = WAIT(FULLA0 + s, (it >> 1) & 1);
      if (ok && it > 0) ok = WAIT(W_DONE, (it - 1) & 1);  // w of the chunk before has been issued and is done
      if (!ok) break;
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      const unsigned char* stg = smem + OFF_STAGE + s * STAGE_BYTES;
      const unsigned char* src = stg + 3 * TILE;
      const float4 g0 = *reinterpret_cast<const float4*>(vs + V_BG * CHUNK + 8 * c8);
      const float4 g1 = *reinterpret_cast<const float4*>(vs + V_BG * CHUNK + 8 * c8 + 4);
#pragma unroll 4
      for (int i = 0; i < 8; ++i) {
        const int off = (r0 + 8 * i) * 128 + pc_a * 16;
        const uint4 a = *reinterpret_cast<const uint4*>(src + off);
        *reinterpret_cast<uint4*>(smem + OFF_APP + off) =
            make_uint4(scale2(a.x, g0.x, g0.y), scale2(a.y, g0.z, g0.w), scale2(a.z, g1.x, g1.y),
                       scale2(a.w, g1.z, g1.w));
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars[AP_READY]);
        mbar_arrive(&bars[EMPTYA0 + s]);  // the A tile of this stage is no longer read
      }
      // q' has one buffer: the state update of the chunk before must have read it; q has landed
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (ok && it > 0) ok = WAIT(S_DONE, (it - 1) & 1);
      if (!ok) break;
      const float sg = vs[V_SGAM * CHUNK + r];
      unsigned char* qs = smem + OFF_QS;
#pragma unroll 1
      for (int q16 = 0; q16 < 16; ++q16) {
        const int blk = q16 >> 3, pc = (q16 + r) & 7;
        const uint4 a = *reinterpret_cast<const uint4*>(stg + blk * 8192 + r * 128 + pc * 16);
        *reinterpret_cast<uint4*>(qs + blk * 8192 + r * 128 + pc * 16) =
            make_uint4(scale2(a.x, sg, sg), scale2(a.y, sg, sg), scale2(a.z, sg, sg), scale2(a.w, sg, sg));
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars[QS_READY]);
        mbar_arrive(&bars[EMPTY0 + s]);
      }
    }
  }

  // ---- teardown ----
  if (!ok) *abort_flag = 1;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicCAS(&g_bwd_dh_status, 0, 1);
}

int bwd_dh_tc_status(int* out, int reset) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_bwd_dh_status, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  *out = v;
  if (reset && v != 0) {
    int z = 0;
    e = cudaMemcpyToSymbol(g_bwd_dh_status, &z, sizeof(int));
  }
  return (int)e;
}

// ---- host side --------------------------------------------------------------------------------
int make_tile_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, int box_rows);

int launch_bwd_dh_tc(const void* q, const void* k, const void* A, const float* g, const void* beta,
                     int beta_is_f32, const void* dO, const float* dht, void* dh, void* du,
                     float* dh0, int tiled, const int* lead, const int* order, const int* run_mask,
                     int run_value, int N, int Hq, int Hv,
                     long long T_rows, float scale, SeqLayout lay, cudaStream_t st) {
  using namespace bdtc;
  CUtensorMap mq, mk, mdo, ma, mdh, mdu;
  int rc;
  if ((rc = make_tile_map(&mq, q, T_rows, (long long)Hq * D, 64))) return rc;
  if ((rc = make_tile_map(&mk, k, T_rows, (long long)Hq * D, 64))) return rc;
  if ((rc = make_tile_map(&mdo, dO, T_rows, (long long)Hv * D, 64))) return rc;
  if ((rc = make_tile_map(&ma, A, T_rows, (long long)Hv * CHUNK, 64))) return rc;
  mdh = mq;
  mdu = mq;
  if (tiled) {
    // an upper bound of the chunk count: the maps only have to cover what the kernel stores
    const long long max_chunks = (T_rows + CHUNK - 1) / CHUNK + N;
    if (dh && (rc = make_tile_map(&mdh, dh, max_chunks * Hv * D, D, 128))) return rc;
    if (du && (rc = make_tile_map(&mdu, du, max_chunks * Hv * D, CHUNK, 128))) return rc;
  }
  BwdDhTcParams p;
  p.tiled = tiled;
  p.order = order;
  p.lead = lead;
  p.run_mask = run_mask;
  p.run_value = run_value;
  p.g = g; p.beta = beta; p.beta_is_f32 = beta_is_f32; p.dht = dht;
  p.dh = (bf16*)dh; p.du = (bf16*)du; p.dh0 = dh0;
  p.N = N; p.Hq = Hq; p.Hv = Hv; p.scale = scale; p.lay = lay;
  rc = configure_smem((const void*)bwd_dh_tc_kernel, SMEM_BYTES);
  if (rc != 0) return rc;
  bwd_dh_tc_kernel<<<(unsigned)(N * Hv), 512, SMEM_BYTES, st>>>(p, mq, mk, mdo, ma, mdh, mdu);
  return (int)cudaGetLastError();
}

}  // namespace fqla
