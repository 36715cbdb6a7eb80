// Sequential forward recurrence of the gated delta rule on Blackwell tensor cores:
// TMA-fed tcgen05.mma with all accumulators in tensor memory, warp-specialised.
//
// One CTA (512 threads) walks the chunks of one (sequence or segment, value head), K = V = 128.
// Everything is kept TRANSPOSED so that the 128-wide value dimension sits on the MMA M axis
// (tensor-memory lane = value index v, one thread per lane):
//     U^T  [v x tok]  = S^T K^T                    (A = bf16 copy of S^T, B = K tile, K-major)
//     W^T             = beta_tok (V^T - gamma_tok U^T)                  (CUDA cores, V group)
//     Vn^T [v x tok]  = W^T A^T                    (B = A tile, K-major)
//     O^T  [v x tok]  = s gamma_tok (S^T Q^T)  +  Vn^T Pg^T             (two accumulators)
//     S^T  [v x k]    = gamma_last S^T + (rho Vn)^T K                   (B = K tile, MN-major)
//     P    [tok x tok'] = Q K^T  (M = 64),  Pg = s P exp(g_tok - g_tok') for tok >= tok'
// which is the algebra of the reference's blackwell/fused_fwd.py:349-596 with the gate folded
// into A (see kkt_solve).
//
// Warp roles (thread ranges):
//     0-127   S group : fp32 master state in tensor memory; per chunk writes the bf16 operand copy
//                       of S^T to shared memory, decays S^T in place, emits h / the final state
//     128-255 V group : U^T -> W^T, Vn^T -> Vn^T and rho-scaled copies (MMA operands), v_new out
//     256-383 O group : P -> Pg (operand), output epilogue  o = s gamma O1 + O2
//     warp 12 : issues every tcgen05.mma (one elected lane)
//     warp 13 : producer: per-chunk gate vectors, TMA loads of the q, k, v, A tiles (2 stages),
//               zero-fill of the rows past the end of a partial last chunk
// Synchronisation is by mbarriers only; every wait is bounded and reports through a status word.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "fqla_internal.h"
#include "tc05.cuh"

namespace fqla {

using namespace tc;

__device__ int g_device_status = 0;
// Diagnostics (FQLA_PROFILE=1): cycles the first CTA's role leaders spent waiting per barrier,
// [role 0..4][barrier 0..15], plus [5][0] = total cycles of the CTA.
__device__ long long g_wait_profile[6 * 16];  // 0 ok; otherwise the code of the first bounded wait that gave up

struct FwdTcParams {
  const float* g;
  const void* beta;
  int beta_is_f32;
  const float* h0;
  float* ht;
  bf16* o;
  bf16* h;
  bf16* vnew;
  int N, Hq, Hv;
  long long T_rows;
  float scale;
  SeqLayout lay;
  int profile;
};

namespace fwdtc {
constexpr int D = 128;
constexpr int TILE_QK = 16384, TILE_V = 16384, TILE_A = 8192;
constexpr int STAGE_BYTES = 2 * TILE_QK + TILE_V + TILE_A;  // 57344
constexpr int OFF_STAGE = 0;
constexpr int OFF_ST = 2 * STAGE_BYTES;          // S^T copy, 2 blocks of [128 x 128B]
constexpr int OFF_WT = OFF_ST + 32768;           // W^T   [128 x 128B]
constexpr int OFF_VNT = OFF_WT + 16384;          // Vn^T
constexpr int OFF_VRT = OFF_VNT + 16384;         // rho * Vn^T
constexpr int OFF_P = OFF_VRT + 16384;           // Pg    [64 x 128B]
constexpr int OFF_VEC = OFF_P + 8192;            // 4 slots x 5 vectors x 64 floats
constexpr int VEC_SLOT_FLOATS = 5 * CHUNK;
constexpr int OFF_BAR = OFF_VEC + 4 * VEC_SLOT_FLOATS * 4;
constexpr int N_BARS = 20;
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;  // + slack for 1024-byte alignment of the base
// tensor-memory columns
constexpr uint32_t TM_S = 0, TM_UV = 128, TM_O1 = 192, TM_O2 = 256, TM_P = 320;
// barrier indices
enum { FULL0 = 0, FULL1, EMPTY0, EMPTY1, S_COPY, S_DEC, U_DONE, VN_DONE, S_DONE, P_DONE, O_DONE,
       W_READY, VR_READY, P_READY, O_FREE, PRIV };
// vector indices inside a slot
enum { V_G = 0, V_GAM = 1, V_RHO = 2, V_BETA = 3, V_SGAM = 4 };
}  // namespace fwdtc

__global__ void __launch_bounds__(512, 1)
fwd_tc_kernel(const FwdTcParams p, const __grid_constant__ CUtensorMap map_q,
              const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const __grid_constant__ CUtensorMap map_a) {
  using namespace fwdtc;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);
  float* vec = reinterpret_cast<float*>(smem + OFF_VEC);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x / p.Hv, hv = blockIdx.x % p.Hv;
  const int hq = hv / (p.Hv / p.Hq);
  const SeqSpan sp = p.lay.span(n);
  const int n_it = sp.n_chunks;

  if (tid == 0) {
    mbar_init(&bars[FULL0], 1);
    mbar_init(&bars[FULL1], 1);
    mbar_init(&bars[EMPTY0], 1 + 128);  // MMA commit + V group
    mbar_init(&bars[EMPTY1], 1 + 128);
    mbar_init(&bars[S_COPY], 128);
    mbar_init(&bars[S_DEC], 128);
    mbar_init(&bars[U_DONE], 1);
    mbar_init(&bars[VN_DONE], 1);
    mbar_init(&bars[S_DONE], 1);
    mbar_init(&bars[P_DONE], 1);
    mbar_init(&bars[O_DONE], 1);
    mbar_init(&bars[W_READY], 128);
    mbar_init(&bars[VR_READY], 128);
    mbar_init(&bars[P_READY], 128);
    mbar_init(&bars[O_FREE], 128);
    mbar_init(&bars[PRIV], 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_a);
  }
  if (warp == 12) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;  // this warp's lane quarter
  const long long state_off = ((long long)n * p.Hv + hv) * D * D;
  bool ok = true;
  long long waited[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) waited[i] = 0;
  const long long t_start = clock64();
  long long t_sec = 0;
  auto WAIT = [&](int idx, uint32_t parity) {
    if (!p.profile) return mbar_wait(&bars[idx], parity, abort_flag);
    long long t0 = clock64();
    bool r = mbar_wait(&bars[idx], parity, abort_flag);
    waited[idx] += clock64() - t0;
    return r;
  };

  if (warp < 4) {
    // =============================== S group ===============================
    const int v = tid;  // lane of tensor memory = value index
    // initial state -> tensor memory (S^T[v][k] = h0[k][v])
    for (int k0 = 0; k0 < D; k0 += 32) {
      float x[32];
#pragma unroll
      for (int j = 0; j < 32; ++j)
        x[j] = p.h0 ? p.h0[state_off + (long long)(k0 + j) * D + v] : 0.f;
      tmem_st32(tmem + lane_sel + TM_S + k0, x);
    }
    tmem_st_wait();
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      if (it > 0) ok = WAIT(S_DONE, (it - 1) & 1);
      if (!ok) break;
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (!ok) break;
      tc_fence_after();
      const float gl = vec[(it & 3) * VEC_SLOT_FLOATS + V_GAM * CHUNK + CHUNK - 1];
      bf16* hdst = p.h ? p.h + ((sp.chunk_base + it) * p.Hv + hv) * (long long)D * D : nullptr;
      for (int k0 = 0; k0 < D; k0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_S + k0, x);
        tmem_ld_wait();
        unsigned char* row = smem + OFF_ST + (k0 >> 6) * 16384 + v * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // 4 chunks of 8 k values
          uint4 pk;
          pk.x = pack_bf16(x[8 * c + 0], x[8 * c + 1]);
          pk.y = pack_bf16(x[8 * c + 2], x[8 * c + 3]);
          pk.z = pack_bf16(x[8 * c + 4], x[8 * c + 5]);
          pk.w = pack_bf16(x[8 * c + 6], x[8 * c + 7]);
          int ch = ((k0 & 63) >> 3) + c;
          *reinterpret_cast<uint4*>(row + ((ch ^ (v & 7)) << 4)) = pk;
        }
        if (hdst) {
#pragma unroll
          for (int j = 0; j < 32; ++j) hdst[(long long)(k0 + j) * D + v] = __float2bfloat16(x[j]);
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) x[j] *= gl;
        tmem_st32(tmem + lane_sel + TM_S + k0, x);
      }
      fence_proxy_async();
      mbar_arrive(&bars[S_COPY]);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[S_DEC]);
    }
    if (ok && n_it > 0) ok = WAIT(S_DONE, (n_it - 1) & 1);
    if (ok && p.ht) {
      tc_fence_after();
      for (int k0 = 0; k0 < D; k0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_S + k0, x);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) p.ht[state_off + (long long)(k0 + j) * D + v] = x[j];
      }
    }
  } else if (warp < 8) {
    // =============================== V group ===============================
    const int v = tid - 128;
    const int vblk = v >> 6, vch = (v & 63) >> 3, vsub = (v & 7) * 2;
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      const long long row0 = sp.bos + (long long)it * CHUNK;
      const int valid = min(CHUNK, sp.len - it * CHUNK);
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (!ok) break;
      ok = WAIT(U_DONE, it & 1);
      if (!ok) break;
      tc_fence_after();
      t_sec = clock64();
      const unsigned char* vt = smem + OFF_STAGE + s * STAGE_BYTES + 2 * TILE_QK + vblk * 8192;
      for (int t0 = 0; t0 < CHUNK; t0 += 32) {
        float u[32];
        tmem_ld32(tmem + lane_sel + TM_UV + t0, u);
        tmem_ld_wait();
        unsigned char* row = smem + OFF_WT + v * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float wv[2];
#pragma unroll
            for (int z = 0; z < 2; ++z) {
              int j = 8 * c + 2 * e + z, tok = t0 + j;
              float vv = __bfloat162float(*reinterpret_cast<const bf16*>(
                  vt + tok * 128 + ((vch ^ (tok & 7)) << 4) + vsub));
              wv[z] = vs[V_BETA * CHUNK + tok] * (vv - vs[V_GAM * CHUNK + tok] * u[j]);
            }
            w[e] = pack_bf16(wv[0], wv[1]);
          }
          int ch = (t0 >> 3) + c;
          *reinterpret_cast<uint4*>(row + ((ch ^ (v & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[W_READY]);
      if (p.profile) waited[S_COPY] += clock64() - t_sec;
      ok = WAIT(VN_DONE, it & 1);
      t_sec = clock64();
      if (!ok) break;
      tc_fence_after();
      for (int t0 = 0; t0 < CHUNK; t0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_UV + t0, x);
        tmem_ld_wait();
        unsigned char* rown = smem + OFF_VNT + v * 128;
        unsigned char* rowr = smem + OFF_VRT + v * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t a[4], b[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            int j = 8 * c + 2 * e, tok = t0 + j;
            a[e] = pack_bf16(x[j], x[j + 1]);
            b[e] = pack_bf16(vs[V_RHO * CHUNK + tok] * x[j], vs[V_RHO * CHUNK + tok + 1] * x[j + 1]);
          }
          int sw = (((t0 >> 3) + c) ^ (v & 7)) << 4;
          *reinterpret_cast<uint4*>(rown + sw) = make_uint4(a[0], a[1], a[2], a[3]);
          *reinterpret_cast<uint4*>(rowr + sw) = make_uint4(b[0], b[1], b[2], b[3]);
        }
        if (p.vnew) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (t0 + j < valid)
              p.vnew[((row0 + t0 + j) * p.Hv + hv) * D + v] = __float2bfloat16(x[j]);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[VR_READY]);
      if (p.profile) waited[S_DEC] += clock64() - t_sec;
      mbar_arrive(&bars[EMPTY0 + s]);
    }
  } else if (warp < 12) {
    // =============================== O group ===============================
    const int v = tid - 256;
    const int wq = warp & 3;
    auto epilogue = [&](int it) {
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      const long long row0 = sp.bos + (long long)it * CHUNK;
      const int valid = min(CHUNK, sp.len - it * CHUNK);
      for (int t0 = 0; t0 < CHUNK; t0 += 32) {
        float a[32], b[32];
        tmem_ld32(tmem + lane_sel + TM_O1 + t0, a);
        tmem_ld32(tmem + lane_sel + TM_O2 + t0, b);
        tmem_ld_wait();
        if (t0 + 32 >= CHUNK) {  // all tensor-memory reads of this chunk's output are done
          tc_fence_before();
          mbar_arrive(&bars[O_FREE]);
        }
        if (p.o) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (t0 + j < valid)
              p.o[((row0 + t0 + j) * p.Hv + hv) * D + v] =
                  __float2bfloat16(vs[V_SGAM * CHUNK + t0 + j] * a[j] + b[j]);
        }
      }
    };
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (!ok) break;
      if (it > 0) {
        ok = WAIT(O_DONE, (it - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        { long long t_e = clock64(); epilogue(it - 1); if (p.profile) waited[S_COPY] += clock64() - t_e; }
      }
      ok = WAIT(P_DONE, it & 1);
      if (!ok) break;
      tc_fence_after();
      t_sec = clock64();
      // P is an M = 64 accumulator: row tok lives in lane (tok % 16) + 32 * (tok / 16)
      const int tok = 16 * wq + (lane & 15);
      const float gt = vs[V_G * CHUNK + tok];
      for (int c0 = 0; c0 < CHUNK; c0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_P + c0, x);
        tmem_ld_wait();
        if (lane < 16) {
          unsigned char* row = smem + OFF_P + tok * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float pv[2];
#pragma unroll
              for (int z = 0; z < 2; ++z) {
                int col = c0 + 8 * c + 2 * e + z;
                pv[z] = tok >= col ? p.scale * x[8 * c + 2 * e + z] *
                                         fast_exp(gt - vs[V_G * CHUNK + col])
                                   : 0.f;
              }
              w[e] = pack_bf16(pv[0], pv[1]);
            }
            int ch = (c0 >> 3) + c;
            *reinterpret_cast<uint4*>(row + ((ch ^ (tok & 7)) << 4)) =
                make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[P_READY]);
      if (p.profile) waited[S_DEC] += clock64() - t_sec;
    }
    if (ok && n_it > 0) {
      ok = WAIT(O_DONE, (n_it - 1) & 1);
      if (ok) {
        tc_fence_after();
        epilogue(n_it - 1);
      }
    }
    // rows of o past the end of the last packed sequence come out zero
    if (p.o && p.lay.cu.ptr && n == p.N - 1) {
      for (long long r = sp.bos + sp.len; r < p.T_rows; ++r)
        p.o[(r * p.Hv + hv) * D + v] = __float2bfloat16(0.f);
    }
  } else if (warp == 12) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t ID_P = idesc_bf16(64, 64, 0, 0);
      constexpr uint32_t ID_N64 = idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t ID_S = idesc_bf16(128, 128, 0, 1);
      auto stage = [&](int s) { return smem + OFF_STAGE + s * STAGE_BYTES; };
      auto issue_p = [&](int s) {
        const unsigned char* q = stage(s);
        const unsigned char* k = stage(s) + TILE_QK;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma(tmem + TM_P, desc_kmajor(q + (j >> 2) * 8192 + (j & 3) * 32),
               desc_kmajor(k + (j >> 2) * 8192 + (j & 3) * 32), ID_P, j > 0);
        umma_commit(&bars[P_DONE]);
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const unsigned char* q = stage(s);
        const unsigned char* k = stage(s) + TILE_QK;
        const unsigned char* a = stage(s) + 2 * TILE_QK + TILE_V;
        ok = WAIT(FULL0 + s, (it >> 1) & 1);
        if (!ok) break;
        tc_fence_after();
        if (it == 0) issue_p(0);
        ok = WAIT(S_COPY, it & 1);
        if (!ok) break;
        tc_fence_after();
        // U^T = S^T K^T
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma(tmem + TM_UV, desc_kmajor(smem + OFF_ST + (j >> 2) * 16384 + (j & 3) * 32),
               desc_kmajor(k + (j >> 2) * 8192 + (j & 3) * 32), ID_N64, j > 0);
        umma_commit(&bars[U_DONE]);
        if (it > 0) {
          ok = WAIT(O_FREE, (it - 1) & 1);
          if (!ok) break;
          tc_fence_after();
        }
        // O1^T = S^T Q^T
#pragma unroll
        for (int j = 0; j < 8; ++j)
          umma(tmem + TM_O1, desc_kmajor(smem + OFF_ST + (j >> 2) * 16384 + (j & 3) * 32),
               desc_kmajor(q + (j >> 2) * 8192 + (j & 3) * 32), ID_N64, j > 0);
        ok = WAIT(W_READY, it & 1);
        if (!ok) break;
        tc_fence_after();
        // Vn^T = W^T A^T
#pragma unroll
        for (int j = 0; j < 4; ++j)
          umma(tmem + TM_UV, desc_kmajor(smem + OFF_WT + j * 32), desc_kmajor(a + j * 32), ID_N64,
               j > 0);
        umma_commit(&bars[VN_DONE]);
        ok = WAIT(VR_READY, it & 1);
        if (!ok) break;
        ok = WAIT(S_DEC, it & 1);
        if (!ok) break;
        tc_fence_after();
        // S^T += (rho Vn)^T K      (B = K tile read MN-major: contraction over its 64 rows)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          umma(tmem + TM_S, desc_kmajor(smem + OFF_VRT + j * 32), desc_mnmajor(k + j * 2048, 8192),
               ID_S, true);
        umma_commit(&bars[S_DONE]);
        ok = WAIT(P_READY, it & 1);
        if (!ok) break;
        tc_fence_after();
        // O2^T = Vn^T Pg^T
#pragma unroll
        for (int j = 0; j < 4; ++j)
          umma(tmem + TM_O2, desc_kmajor(smem + OFF_VNT + j * 32),
               desc_kmajor(smem + OFF_P + j * 32), ID_N64, j > 0);
        umma_commit(&bars[O_DONE]);
        umma_commit(&bars[EMPTY0 + s]);
        if (it + 1 < n_it) {
          ok = WAIT(FULL0 + (s ^ 1), ((it + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_p(s ^ 1);
        }
      }
    }
  } else if (warp == 13) {
    // =============================== producer ===============================
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      const long long row0 = sp.bos + (long long)it * CHUNK;
      const int valid = min(CHUNK, sp.len - it * CHUNK);
      if (it >= 2) {
        ok = WAIT(EMPTY0 + s, ((it >> 1) - 1) & 1);
        if (!ok) break;
      }
      float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      const float g_last = p.g[(row0 + valid - 1) * p.Hv + hv];
#pragma unroll
      for (int z = 0; z < 2; ++z) {
        int r = 2 * lane + z, rc = min(r, valid - 1);
        float gv = p.g[(row0 + rc) * p.Hv + hv];
        float bv = r < valid ? load_beta(p.beta, p.beta_is_f32, (row0 + r) * p.Hv + hv) : 0.f;
        float gam = fast_exp(gv);
        vs[V_G * CHUNK + r] = gv;
        vs[V_GAM * CHUNK + r] = gam;
        vs[V_RHO * CHUNK + r] = fast_exp(g_last - gv);
        vs[V_BETA * CHUNK + r] = bv;
        vs[V_SGAM * CHUNK + r] = p.scale * gam;
      }
      __syncwarp();
      unsigned char* st = smem + OFF_STAGE + s * STAGE_BYTES;
      const bool partial = valid < CHUNK;
      uint64_t* bar = partial ? &bars[PRIV] : &bars[FULL0 + s];
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, STAGE_BYTES);
        const int y = (int)row0;
        tma_load_2d(st + TILE_QK, &map_k, hq * D, y, bar);
        tma_load_2d(st + TILE_QK + 8192, &map_k, hq * D + 64, y, bar);
        tma_load_2d(st, &map_q, hq * D, y, bar);
        tma_load_2d(st + 8192, &map_q, hq * D + 64, y, bar);
        tma_load_2d(st + 2 * TILE_QK, &map_v, hv * D, y, bar);
        tma_load_2d(st + 2 * TILE_QK + 8192, &map_v, hv * D + 64, y, bar);
        tma_load_2d(st + 2 * TILE_QK + TILE_V, &map_a, hv * CHUNK, y, bar);
      }
      if (partial) {
        // rows past the sequence end belong to the next sequence: wait for the copy, zero them
        ok = WAIT(PRIV, 0);  // used at most once per CTA (last chunk)
        if (!ok) break;
        for (int blk = 0; blk < 7; ++blk) {
          unsigned char* base = st + blk * 8192;
          for (int i = lane; i < (CHUNK - valid) * 8; i += 32)
            *reinterpret_cast<uint4*>(base + (valid + (i >> 3)) * 128 + ((i & 7) << 4)) =
                make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[FULL0 + s]);
      }
    }
  }

  if (p.profile && blockIdx.x == 0 && (tid == 0 || tid == 128 || tid == 256 || tid == 384 || tid == 416)) {
    int role = tid == 0 ? 0 : tid == 128 ? 1 : tid == 256 ? 2 : tid == 384 ? 3 : 4;
    for (int i = 0; i < 16; ++i) g_wait_profile[role * 16 + i] = waited[i];
    if (tid == 0) g_wait_profile[5 * 16] = clock64() - t_start;
  }
  // ---- teardown: everybody meets, then the allocating warp frees tensor memory
  if (!ok) *abort_flag = 1;
  tc_fence_before();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicCAS(&g_device_status, 0, 1);
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess)
      f = nullptr;
    return (EncodeTiledFn)f;
  }();
  return fn;
}

// 2-D bf16 tensor [rows][cols] (row pitch = cols), box = 64 columns x 64 rows, 128-byte swizzle.
static int make_map(CUtensorMap* m, const void* ptr, long long rows, long long cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return FQLA_ERR_INVALID_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, 64};
  cuuint32_t es[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FQLA_ERR_INVALID_ARG;
}

int launch_fwd_tc(const void* q, const void* k, const void* v, const void* A, const float* g,
                  const void* beta, int beta_is_f32, const float* h0, float* ht, void* o, void* h,
                  void* vnew, int N, int Hq, int Hv, long long T_rows, float scale, SeqLayout lay,
                  cudaStream_t st) {
  using namespace fwdtc;
  CUtensorMap mq, mk, mv, ma;
  int rc;
  if ((rc = make_map(&mq, q, T_rows, (long long)Hq * D))) return rc;
  if ((rc = make_map(&mk, k, T_rows, (long long)Hq * D))) return rc;
  if ((rc = make_map(&mv, v, T_rows, (long long)Hv * D))) return rc;
  if ((rc = make_map(&ma, A, T_rows, (long long)Hv * CHUNK))) return rc;
  FwdTcParams p;
  p.g = g; p.beta = beta; p.beta_is_f32 = beta_is_f32; p.h0 = h0; p.ht = ht;
  p.o = (bf16*)o; p.h = (bf16*)h; p.vnew = (bf16*)vnew;
  p.N = N; p.Hq = Hq; p.Hv = Hv; p.T_rows = T_rows; p.scale = scale; p.lay = lay;
  static const bool profile = getenv("FQLA_PROFILE") != nullptr;
  p.profile = profile ? 1 : 0;
  rc = configure_smem((const void*)fwd_tc_kernel, SMEM_BYTES);
  if (rc != 0) return rc;
  fwd_tc_kernel<<<(unsigned)(N * Hv), 512, SMEM_BYTES, st>>>(p, mq, mk, mv, ma);
  return (int)cudaGetLastError();
}

}  // namespace fqla

extern "C" int fqla_debug_wait_profile(long long* out96) {
  return (int)cudaMemcpyFromSymbol(out96, fqla::g_wait_profile, sizeof(long long) * 96);
}

extern "C" int fqla_device_status(int* out, int reset) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, fqla::g_device_status, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  if (out) *out = v;
  if (reset && v != 0) {
    int z = 0;
    e = cudaMemcpyToSymbol(fqla::g_device_status, &z, sizeof(int));
  }
  return (int)e;
}
