// Sequential forward recurrence of the gated delta rule on Blackwell tensor cores:
// TMA-fed tcgen05.mma with all accumulators in tensor memory, warp-specialised.
//
// One CTA (512 threads) walks the chunks of one (sequence or segment, value head), K = V = 128.
// The state path is kept TRANSPOSED so that the 128-wide value dimension sits on the MMA M axis
// (tensor-memory lane = value index v, one thread per lane); the output path is not (M = 64 rows
// = tokens, so that a thread owns one contiguous output row):
//     VT   [v x tok]    = V^T            (A = V tile read MN-major, B = identity: a transpose)
//     U^T  [v x tok]    = S^T K^T        (A = bf16 copy of S^T, B = K tile)
//     W^T               = beta_tok VT - (beta gamma)_tok U^T                 (V group)
//     Vn^T [v x tok]    = W^T A^T        (B = A tile)
//     S^T  [v x k]      = gamma_last S^T + (rho Vn)^T K        (B = K tile read MN-major)
//     P    [tok x tok'] = Q K^T,  Pg = s P exp(g_tok - g_tok') for tok >= tok'      (O group)
//     O    [tok x v]    = s gamma_tok (Q S) + Pg Vn            (two M = 64 accumulators)
// which is the algebra of the reference's blackwell/fused_fwd.py:349-596 with the gate folded
// into A (see kkt_solve).
//
// Warp roles (thread ranges):
//     0-127   S group : fp32 master state in tensor memory; per chunk writes the bf16 operand copy
//                       of S^T to shared memory, decays S^T in place, emits h / the final state
//     128-255 V group : U^T, VT -> W^T;  Vn^T -> Vn^T and rho-scaled copies (MMA operands)
//     256-383 O group : P -> Pg (operand); output epilogue o = s gamma O1 + O2, 16-byte stores
//     warp 12 : issues every tcgen05.mma (one elected lane), descriptors precomputed
//     warp 13 : producer: per-chunk gate vectors (fetched one chunk ahead), TMA loads of the
//               q, k, v, A tiles (2 stages), zero-fill of rows past the end of a partial chunk
// Synchronisation is by mbarriers only; every wait is bounded and reports through a status word.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "fqla_internal.h"
#include "tc05.cuh"

namespace fqla {

using namespace tc;

// 0 = ok; 1 after some kernel abandoned a bounded wait (its outputs are then invalid)
__device__ int g_device_status = 0;
// Diagnostics (FQLA_PROFILE=1): cycles the first CTA's role leaders spent per barrier wait and
// per section, [role 0..4][slot 0..15], plus [5][0] = total cycles of the CTA.
__device__ long long g_wait_profile[6 * 16];

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
constexpr int OFF_I = OFF_P + 8192;              // identity [64 x 128B]
constexpr int OFF_VEC = OFF_I + 8192;            // 4 slots x 6 vectors x 64 floats
constexpr int VEC_SLOT_FLOATS = 6 * CHUNK;
constexpr int OFF_BAR = OFF_VEC + 4 * VEC_SLOT_FLOATS * 4;
constexpr int N_BARS = 20;
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;  // + slack for 1024-byte alignment of the base
// tensor-memory columns.  P shares the columns of O1 in the upper half-lanes: an M = 64
// accumulator only occupies lanes 0-15 of each 32-lane quarter, a second one fits at lane +16.
constexpr uint32_t TM_S = 0, TM_UV = 128, TM_VT = 192, TM_O1 = 256, TM_O2 = 384;
constexpr uint32_t TM_P = TM_O1 + (16u << 16);
// barrier indices
enum { FULL0 = 0, FULL1, EMPTY0, EMPTY1, S_COPY, S_DEC, U_DONE, VN_DONE, S_DONE, P_DONE, O_DONE,
       W_READY, VR_READY, P_READY, O_FREE, PRIV };
// vectors inside a slot; V_GL holds gamma_last at [0]
enum { V_G = 0, V_BETA = 1, V_BG = 2, V_RHO = 3, V_SGAM = 4, V_GL = 5 };
}  // namespace fwdtc

__global__ void __launch_bounds__(512, 1)
fwd_tc_kernel(const FwdTcParams p, const __grid_constant__ CUtensorMap map_q,
              const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const __grid_constant__ CUtensorMap map_a) {
  using namespace fwdtc;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
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
    mbar_init(&bars[EMPTY0], 1);  // the MMA commit: tiles are read by tensor-core operations only
    mbar_init(&bars[EMPTY1], 1);
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
  // identity tile (B operand of the V transpose), written once
  for (int i = tid; i < CHUNK * 8; i += 512) {
    int r = i >> 3, ch = i & 7;
    uint4 z = make_uint4(0, 0, 0, 0);
    if (ch == (r >> 3)) {
      uint32_t one = (r & 1) ? 0x3F800000u : 0x00003F80u;  // bf16 1.0 in the high / low half
      (&z.x)[(r & 7) >> 1] = one;
    }
    *reinterpret_cast<uint4*>(smem + OFF_I + r * 128 + ((ch ^ (r & 7)) << 4)) = z;
  }
  fence_proxy_async();
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
      if (p.profile) t_sec = clock64();
      const float gl = vec[(it & 3) * VEC_SLOT_FLOATS + V_GL * CHUNK];
      bf16* hdst = p.h ? p.h + ((sp.chunk_base + it) * p.Hv + hv) * (long long)D * D : nullptr;
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {  // 64 columns (one operand block) per round
        float x[32], y[32];
        tmem_ld32(tmem + lane_sel + TM_S + kb * 64, x);
        tmem_ld32(tmem + lane_sel + TM_S + kb * 64 + 32, y);
        tmem_ld_wait();
        unsigned char* row = smem + OFF_ST + kb * 16384 + v * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          *reinterpret_cast<uint4*>(row + ((c ^ (v & 7)) << 4)) =
              make_uint4(pack_bf16(x[8 * c + 0], x[8 * c + 1]), pack_bf16(x[8 * c + 2], x[8 * c + 3]),
                         pack_bf16(x[8 * c + 4], x[8 * c + 5]), pack_bf16(x[8 * c + 6], x[8 * c + 7]));
          *reinterpret_cast<uint4*>(row + (((c + 4) ^ (v & 7)) << 4)) =
              make_uint4(pack_bf16(y[8 * c + 0], y[8 * c + 1]), pack_bf16(y[8 * c + 2], y[8 * c + 3]),
                         pack_bf16(y[8 * c + 4], y[8 * c + 5]), pack_bf16(y[8 * c + 6], y[8 * c + 7]));
        }
        if (hdst) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            hdst[(long long)(kb * 64 + j) * D + v] = __float2bfloat16(x[j]);
            hdst[(long long)(kb * 64 + 32 + j) * D + v] = __float2bfloat16(y[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          x[j] *= gl;
          y[j] *= gl;
        }
        tmem_st32(tmem + lane_sel + TM_S + kb * 64, x);
        tmem_st32(tmem + lane_sel + TM_S + kb * 64 + 32, y);
      }
      fence_proxy_async();
      mbar_arrive(&bars[S_COPY]);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[S_DEC]);
      if (p.profile) waited[S_COPY] += clock64() - t_sec;
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
      if (p.profile) t_sec = clock64();
#pragma unroll
      for (int t0 = 0; t0 < CHUNK; t0 += 32) {
        float u[32], vt[32];
        long long t_l = p.profile ? clock64() : 0;
        tmem_ld32(tmem + lane_sel + TM_UV + t0, u);
        tmem_ld32(tmem + lane_sel + TM_VT + t0, vt);
        tmem_ld_wait();
        if (p.profile) waited[P_DONE] += clock64() - t_l;
        unsigned char* row = smem + OFF_WT + v * 128;
        const float4* b4 = reinterpret_cast<const float4*>(vs + V_BETA * CHUNK + t0);
        const float4* g4 = reinterpret_cast<const float4*>(vs + V_BG * CHUNK + t0);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float4 b0 = b4[2 * c], b1 = b4[2 * c + 1], g0 = g4[2 * c], g1 = g4[2 * c + 1];
          const float* uu = u + 8 * c;
          const float* vv = vt + 8 * c;
          uint4 w;
          w.x = pack_bf16(b0.x * vv[0] - g0.x * uu[0], b0.y * vv[1] - g0.y * uu[1]);
          w.y = pack_bf16(b0.z * vv[2] - g0.z * uu[2], b0.w * vv[3] - g0.w * uu[3]);
          w.z = pack_bf16(b1.x * vv[4] - g1.x * uu[4], b1.y * vv[5] - g1.y * uu[5]);
          w.w = pack_bf16(b1.z * vv[6] - g1.z * uu[6], b1.w * vv[7] - g1.w * uu[7]);
          *reinterpret_cast<uint4*>(row + ((((t0 >> 3) + c) ^ (v & 7)) << 4)) = w;
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[W_READY]);
      if (p.profile) waited[S_COPY] += clock64() - t_sec;
      ok = WAIT(VN_DONE, it & 1);
      if (!ok) break;
      tc_fence_after();
      if (p.profile) t_sec = clock64();
#pragma unroll
      for (int t0 = 0; t0 < CHUNK; t0 += 32) {
        float x[32];
        long long t_l = p.profile ? clock64() : 0;
        tmem_ld32(tmem + lane_sel + TM_UV + t0, x);
        tmem_ld_wait();
        if (p.profile) waited[O_DONE] += clock64() - t_l;
        unsigned char* rown = smem + OFF_VNT + v * 128;
        unsigned char* rowr = smem + OFF_VRT + v * 128;
        const float4* r4 = reinterpret_cast<const float4*>(vs + V_RHO * CHUNK + t0);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float4 r0 = r4[2 * c], r1 = r4[2 * c + 1];
          const float* xx = x + 8 * c;
          int sw = (((t0 >> 3) + c) ^ (v & 7)) << 4;
          *reinterpret_cast<uint4*>(rown + sw) =
              make_uint4(pack_bf16(xx[0], xx[1]), pack_bf16(xx[2], xx[3]), pack_bf16(xx[4], xx[5]),
                         pack_bf16(xx[6], xx[7]));
          *reinterpret_cast<uint4*>(rowr + sw) =
              make_uint4(pack_bf16(r0.x * xx[0], r0.y * xx[1]), pack_bf16(r0.z * xx[2], r0.w * xx[3]),
                         pack_bf16(r1.x * xx[4], r1.y * xx[5]), pack_bf16(r1.z * xx[6], r1.w * xx[7]));
        }
        if (p.vnew) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (t0 + j < valid)
              p.vnew[((row0 + t0 + j) * p.Hv + hv) * D + v] = __float2bfloat16(x[j]);
        }
      }
      long long t_f = p.profile ? clock64() : 0;
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[VR_READY]);
      if (p.profile) waited[S_DEC] += clock64() - t_sec;
      if (p.profile) waited[P_READY] += clock64() - t_f;
    }
  } else if (warp < 12) {
    // =============================== O group ===============================
    const int wq = warp & 3;
    const int tok_o = 16 * wq + (lane & 15);  // lanes 0-15: a row of O;  lanes 16-31: a row of P
    auto epilogue = [&](int it) {
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      const long long row0 = sp.bos + (long long)it * CHUNK;
      const int valid = min(CHUNK, sp.len - it * CHUNK);
      const float sg = vs[V_SGAM * CHUNK + tok_o];
      bf16* orow = p.o ? p.o + ((row0 + tok_o) * p.Hv + hv) * D : nullptr;
      const bool write = lane < 16 && tok_o < valid && orow != nullptr;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float a[32], b[32];
        tmem_ld32(tmem + lane_sel + TM_O1 + c0, a);
        tmem_ld32(tmem + lane_sel + TM_O2 + c0, b);
        tmem_ld_wait();
        if (c0 + 32 >= D) {  // all tensor-memory reads of this chunk's output are done
          tc_fence_before();
          mbar_arrive(&bars[O_FREE]);
        }
        if (write) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float* aa = a + 8 * c;
            const float* bb = b + 8 * c;
            *reinterpret_cast<uint4*>(orow + c0 + 8 * c) = make_uint4(
                pack_bf16(sg * aa[0] + bb[0], sg * aa[1] + bb[1]),
                pack_bf16(sg * aa[2] + bb[2], sg * aa[3] + bb[3]),
                pack_bf16(sg * aa[4] + bb[4], sg * aa[5] + bb[5]),
                pack_bf16(sg * aa[6] + bb[6], sg * aa[7] + bb[7]));
          }
        }
      }
    };
    const float log2_scale = log2f(p.scale);
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (!ok) break;
      if (it > 0) {
        ok = WAIT(O_DONE, (it - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        if (p.profile) t_sec = clock64();
        epilogue(it - 1);
        if (p.profile) waited[S_COPY] += clock64() - t_sec;
      }
      ok = WAIT(P_DONE, it & 1);
      if (!ok) break;
      tc_fence_after();
      if (p.profile) t_sec = clock64();
      // Pg = s P exp(g_tok - g_col) = P exp2((g_tok - g_col) log2e + log2 s), col <= tok
      const float gt2 = vs[V_G * CHUNK + tok_o] * 1.4426950408889634f + log2_scale;
#pragma unroll
      for (int c0 = 0; c0 < CHUNK; c0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_O1 + c0, x);  // lanes 16-31 of the quarter hold P
        tmem_ld_wait();
        if (lane >= 16) {
          unsigned char* row = smem + OFF_P + tok_o * 128;
          const float4* g4 = reinterpret_cast<const float4*>(vs + V_G * CHUNK + c0);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float4 ga = g4[2 * c], gb = g4[2 * c + 1];
            const float gc[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
            float pv[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              int col = c0 + 8 * c + e;
              float ex = exp2f(fmaf(gc[e], -1.4426950408889634f, gt2));
              pv[e] = col <= tok_o ? x[8 * c + e] * ex : 0.f;
            }
            *reinterpret_cast<uint4*>(row + ((((c0 >> 3) + c) ^ (tok_o & 7)) << 4)) =
                make_uint4(pack_bf16(pv[0], pv[1]), pack_bf16(pv[2], pv[3]), pack_bf16(pv[4], pv[5]),
                           pack_bf16(pv[6], pv[7]));
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
      const long long end = sp.bos + sp.len;
      for (long long i = tid - 256; i < (p.T_rows - end) * 16; i += 128)
        *reinterpret_cast<uint4*>(p.o + ((end + (i >> 4)) * p.Hv + hv) * D + (i & 15) * 8) =
            make_uint4(0, 0, 0, 0);
    }
  } else if (warp == 12) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t ID_P = idesc_bf16(64, 64, 0, 0);
      constexpr uint32_t ID_O = idesc_bf16(64, 128, 0, 0);
      constexpr uint32_t ID_U = idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t ID_VT = idesc_bf16(128, 64, 1, 0);
      constexpr uint32_t ID_S = idesc_bf16(128, 128, 0, 1);
      // low descriptor words of every operand tile (see umma_lo); steps are 32-bit adds
      const uint32_t st_lo = desc_lo_kmajor(smem + OFF_ST), wt_lo = desc_lo_kmajor(smem + OFF_WT);
      const uint32_t vnt_lo = desc_lo_kmajor(smem + OFF_VNT), vrt_lo = desc_lo_kmajor(smem + OFF_VRT);
      const uint32_t p_lo = desc_lo_kmajor(smem + OFF_P), i_lo = desc_lo_kmajor(smem + OFF_I);
      const uint32_t q0_lo = desc_lo_kmajor(smem + OFF_STAGE);
      const uint32_t k0_lo = desc_lo_kmajor(smem + OFF_STAGE + TILE_QK);
      const uint32_t a0_lo = desc_lo_kmajor(smem + OFF_STAGE + 2 * TILE_QK + TILE_V);
      const uint32_t kmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + TILE_QK, 8192);
      const uint32_t vmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + 2 * TILE_QK, 8192);
      constexpr uint32_t STAGE_LO = STAGE_BYTES >> 4;
      auto issue_p_vt = [&](uint32_t so) {  // so = stage offset in descriptor units
        umma_group<8, 2, 512, 2, 512, false>(tmem + TM_P, q0_lo + so, k0_lo + so, ID_P);
        umma_commit(&bars[P_DONE]);
        // VT = V^T: A = V tile read MN-major (16 rows per step), B = identity
        umma_group<4, 128, 0, 2, 0, false>(tmem + TM_VT, vmn0_lo + so, i_lo, ID_VT);
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t so = s ? STAGE_LO : 0u, so_next = s ? 0u : STAGE_LO;
        ok = WAIT(FULL0 + s, (it >> 1) & 1);
        if (!ok) break;
        tc_fence_after();
        if (it == 0) issue_p_vt(0);
        ok = WAIT(S_COPY, it & 1);
        if (!ok) break;
        tc_fence_after();
        if (p.profile) t_sec = clock64();
        // U^T = S^T K^T
        umma_group<8, 2, 1024, 2, 512, false>(tmem + TM_UV, st_lo, k0_lo + so, ID_U);
        umma_commit(&bars[U_DONE]);
        if (p.profile) waited[U_DONE] += clock64() - t_sec;
        if (it > 0) {
          ok = WAIT(O_FREE, (it - 1) & 1);
          if (!ok) break;
          tc_fence_after();
        }
        if (p.profile) t_sec = clock64();
        // O1 = Q S      (B = S^T copy: N = v rows, K = k)
        umma_group<8, 2, 512, 2, 1024, false>(tmem + TM_O1, q0_lo + so, st_lo, ID_O);
        if (p.profile) waited[O_DONE] += clock64() - t_sec;
        ok = WAIT(W_READY, it & 1);
        if (!ok) break;
        tc_fence_after();
        if (p.profile) t_sec = clock64();
        // Vn^T = W^T A^T
        umma_group<4, 2, 0, 2, 0, false>(tmem + TM_UV, wt_lo, a0_lo + so, ID_U);
        umma_commit(&bars[VN_DONE]);
        if (p.profile) waited[VN_DONE] += clock64() - t_sec;
        ok = WAIT(VR_READY, it & 1);
        if (!ok) break;
        ok = WAIT(S_DEC, it & 1);
        if (!ok) break;
        tc_fence_after();
        if (p.profile) t_sec = clock64();
        // S^T += (rho Vn)^T K      (B = K tile read MN-major: contraction over its 64 rows)
        umma_group<4, 2, 0, 128, 0, true>(tmem + TM_S, vrt_lo, kmn0_lo + so, ID_S);
        umma_commit(&bars[S_DONE]);
        if (p.profile) waited[S_DONE] += clock64() - t_sec;
        ok = WAIT(P_READY, it & 1);
        if (!ok) break;
        tc_fence_after();
        if (p.profile) t_sec = clock64();
        // O2 = Pg Vn     (B = Vn^T copy: N = v rows, K = tok')
        umma_group<4, 2, 0, 2, 0, false>(tmem + TM_O2, p_lo, vnt_lo, ID_O);
        umma_commit(&bars[O_DONE]);
        umma_commit(&bars[EMPTY0 + s]);
        if (p.profile) waited[EMPTY0] += clock64() - t_sec;
        if (it + 1 < n_it) {
          ok = WAIT(FULL0 + (s ^ 1), ((it + 1) >> 1) & 1);
          if (!ok) break;
          tc_fence_after();
          if (p.profile) t_sec = clock64();
          issue_p_vt(so_next);
          if (p.profile) waited[P_DONE] += clock64() - t_sec;
        }
      }
    }
  } else if (warp == 13) {
    // =============================== producer ===============================
    float g_r[2] = {0.f, 0.f}, b_r[2] = {0.f, 0.f}, gl_r = 0.f;
    auto fetch = [&](int it) {
      const long long row0 = sp.bos + (long long)it * CHUNK;
      const int valid = min(CHUNK, sp.len - it * CHUNK);
      gl_r = p.g[(row0 + valid - 1) * p.Hv + hv];
#pragma unroll
      for (int z = 0; z < 2; ++z) {
        int r = 2 * lane + z, rc = min(r, valid - 1);
        g_r[z] = p.g[(row0 + rc) * p.Hv + hv];
        b_r[z] = r < valid ? load_beta(p.beta, p.beta_is_f32, (row0 + r) * p.Hv + hv) : 0.f;
      }
    };
    if (n_it > 0) fetch(0);
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      const long long row0 = sp.bos + (long long)it * CHUNK;
      const int valid = min(CHUNK, sp.len - it * CHUNK);
      if (it >= 2) {
        ok = WAIT(EMPTY0 + s, ((it >> 1) - 1) & 1);
        if (!ok) break;
      }
      float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
#pragma unroll
      for (int z = 0; z < 2; ++z) {
        int r = 2 * lane + z;
        float gam = fast_exp(g_r[z]);
        vs[V_G * CHUNK + r] = g_r[z];
        vs[V_BETA * CHUNK + r] = b_r[z];
        vs[V_BG * CHUNK + r] = b_r[z] * gam;
        vs[V_RHO * CHUNK + r] = fast_exp(gl_r - g_r[z]);
        vs[V_SGAM * CHUNK + r] = p.scale * gam;
      }
      if (lane == 0) vs[V_GL * CHUNK] = fast_exp(gl_r);
      __syncwarp();
      unsigned char* st = smem + OFF_STAGE + s * STAGE_BYTES;
      const bool partial = valid < CHUNK;
      uint64_t* bar = partial ? &bars[PRIV] : &bars[FULL0 + s];
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, STAGE_BYTES);
        const int y = (int)row0;
        tma_load_2d(st + TILE_QK, &map_k, hq * D, y, bar);
        tma_load_2d(st + TILE_QK + 8192, &map_k, hq * D + 64, y, bar);
        tma_load_2d(st + 2 * TILE_QK, &map_v, hv * D, y, bar);
        tma_load_2d(st + 2 * TILE_QK + 8192, &map_v, hv * D + 64, y, bar);
        tma_load_2d(st, &map_q, hq * D, y, bar);
        tma_load_2d(st + 8192, &map_q, hq * D + 64, y, bar);
        tma_load_2d(st + 2 * TILE_QK + TILE_V, &map_a, hv * CHUNK, y, bar);
      }
      if (it + 1 < n_it) fetch(it + 1);  // in flight while this warp waits for the next free stage
      if (partial) {
        // rows past the sequence end belong to the next sequence: wait for the copy, zero them
        ok = WAIT(PRIV, 0);  // only the last chunk of a sequence can be partial: used once
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

  if (p.profile && blockIdx.x == 0 &&
      (tid == 0 || tid == 128 || tid == 256 || tid == 384 || tid == 416)) {
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
