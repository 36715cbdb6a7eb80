// Sequential forward recurrence of the gated delta rule on Blackwell tensor cores:
// TMA-fed tcgen05.mma with all accumulators in tensor memory, warp-specialised.
//
// One CTA (512 threads) walks the chunks of one (sequence or segment, value head), K = V = 128.
// Per chunk, with S [K x V] the fp32 state entering the chunk, A the gated inverse from
// kkt_solve, g the chunk-local cumulative log gate (gamma = exp g, rho = exp(g_last - g)):
//
//   off the serial chain, prepared one chunk ahead (WY form, FLA's w and u):
//     A'  = A diag(beta),  A'' = A diag(beta gamma)                               (prep warps)
//     u^T [v x tok] = V^T A'^T          (A operand = V tile read MN-major)        -> TM_UV
//     w   [tok x k] = A'' K             (B operand = K tile read MN-major)        -> TM_W -> smem
//     P   [tok x tok'] = Q K^T,  Pg = s P exp(g_tok - g_tok') for tok >= tok'     (O group)
//   on the chain (two products):
//     Vn^T [v x tok] = u^T - S^T w^T    (A = bf16 copy of S^T, negated; accumulates onto u^T)
//     S^T  [v x k]   = gamma_last S^T + (rho Vn)^T K     (B = K tile read MN-major)
//   output:
//     O [tok x v] = s gamma_tok (Q S) + Pg Vn      (two M = 64 accumulators, one thread per row)
//
// The state path is kept TRANSPOSED so that the 128-wide value dimension sits on the MMA M axis
// (tensor-memory lane = value index, one thread per lane).  This is the algebra of the
// reference's blackwell/fused_fwd.py:349-596 (and the X/Y form of prepare_h.py:312-318) with the
// gate folded into A.
//
// Warp roles (thread ranges):
//     128-255 S group : fp32 master state in tensor memory; per chunk writes the bf16 operand copy
//                       of S^T to shared memory (on the chain), then decays S^T in place
//     256-383 V group : Vn^T -> rho-scaled and plain bf16 operand copies; w -> bf16 operand tile
//     384-511 O group : P -> Pg (operand); output epilogue o = s gamma O1 + O2
//     warp 0  : issues every tcgen05.mma (one elected lane)
//     warp 1  : producer: per-chunk gate vectors (fetched one chunk ahead), TMA loads of the
//               q, k, v, A tiles (2 stages), zero-fill of rows past the end of a partial chunk
//     64-127  prep    : one thread per chunk row: A' and A'' tiles
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
// per section, [role 0..5][slot 0..23], plus [6][0] = total cycles of the CTA.
__device__ long long g_wait_profile[7 * 24];
// Diagnostics: (1 << 24 | warp << 16 | barrier << 8 | parity) of the first wait that was given up
__device__ int g_fwd_abort_info = 0;

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
  int tiled;  // h and vnew are written as operand tiles (h^T per chunk, v_new^T per chunk) by TMA
  // [N, Hv] or null: lead-in.  A CTA with lead > 0 starts from a ZERO state `lead` chunks before
  // its sequence (segment) and walks those chunks state-only (no q, no output, nothing stored):
  // the rows just before a segment are the tail of the segment before it, whose influence dies
  // out within `lead` chunks.  h0 is ignored for such a CTA.
  const int* lead;
};

namespace fwdtc {
constexpr int D = 128;
constexpr int TILE_QK = 16384, TILE_V = 16384, TILE_A = 8192;
constexpr int STAGE_BYTES = 2 * TILE_QK + TILE_V + TILE_A;  // 57344
constexpr int OFF_STAGE = 0;
constexpr int OFF_ST = 2 * STAGE_BYTES;          // S^T copy, 2 blocks of [128 x 128B]
constexpr int OFF_VNT = OFF_ST + 32768;          // Vn^T  [128 x 128B]
constexpr int OFF_W = OFF_VNT + 16384;           // w     2 blocks of [64 x 128B]
constexpr int OFF_VRT = OFF_W + 16384;           // rho-scaled Vn^T [128 x 128B]
constexpr int OFF_P = OFF_VRT + 16384;            // Pg    [64 x 128B]
constexpr int OFF_AP = OFF_P + 8192;             // A diag(beta)
constexpr int OFF_APP = OFF_AP + 8192;           // A diag(beta gamma)
constexpr int OFF_VEC = OFF_APP + 8192;          // 4 slots x 6 vectors x 64 floats
constexpr int VEC_SLOT_FLOATS = 6 * CHUNK;
constexpr int OFF_BAR = OFF_VEC + 4 * VEC_SLOT_FLOATS * 4;
constexpr int N_BARS = 30;
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;  // + slack for 1024-byte alignment of the base
// tensor-memory columns.  An M = 64 accumulator only occupies lanes 0-15 of each 32-lane
// quarter, so a second one fits at lane +16 of the same columns: P under O1, w under O2.
constexpr uint32_t TM_S = 0, TM_UV = 128, TM_O1 = 256, TM_O2 = 384;
constexpr uint32_t TM_P = TM_O1 + (16u << 16), TM_W = TM_O2 + (16u << 16);
// barrier indices
enum { FULL0 = 0, FULL1, EMPTY0, EMPTY1, S_COPY, S_DEC, VN_DONE, S_DONE, P_DONE, O_DONE, W_DONE,
       VN_READY, W_READY, P_READY, O_FREE, AP_READY, VR_READY, PRIV,
       SEC_A = 18, SEC_B, SEC_C, SEC_D, SEC_E, SEC_F,  // SEC_*: profiling slots only
       // the A tile and the per-row vectors of a chunk travel one chunk ahead of q, k, v
       FULLA0 = 24, FULLA1, EMPTYA0, EMPTYA1, PRIVA };
// vectors inside a slot; V_GL holds gamma_last at [0]
enum { V_G = 0, V_BETA = 1, V_BG = 2, V_RHO = 3, V_SGAM = 4, V_GL = 5 };
}  // namespace fwdtc

__device__ __forceinline__ uint32_t scale_bf16x2(uint32_t packed, float lo, float hi) {
  float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&packed));
  return pack_bf16(f.x * lo, f.y * hi);
}

// PROFILE: wait/section cycle counters (diagnostics).  EXTRA: per-chunk state and v_new outputs.
// Both are compiled out of the common instantiation: the six roles run six different code
// regions at once, and the kernel is sensitive to its instruction-cache footprint.
// NO_O: state-only walk (recomputation for the backward pass): no q, no output products, the
// output warps stay idle.
template <bool PROFILE, bool EXTRA, bool NO_O>
__global__ void __launch_bounds__(512, 1)
fwd_tc_kernel(const FwdTcParams p, const __grid_constant__ CUtensorMap map_q,
              const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_h,
              const __grid_constant__ CUtensorMap map_vn) {
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
  // iteration j handles chunk c = j - lead of the sequence; c < 0 are the lead-in chunks
  const int lead = p.lead ? p.lead[n * p.Hv + hv] : 0;
  const int n_it = sp.n_chunks == 0 ? 0 : sp.n_chunks + lead;

  if (tid == 0) {
    mbar_init(&bars[FULL0], 1);
    mbar_init(&bars[FULL1], 1);
    mbar_init(&bars[EMPTY0], 1);  // MMA commit
    mbar_init(&bars[EMPTY1], 1);
    mbar_init(&bars[FULLA0], 1);
    mbar_init(&bars[FULLA1], 1);
    mbar_init(&bars[EMPTYA0], 2);  // the two prep warps, the only readers of the raw A tile
    mbar_init(&bars[EMPTYA1], 2);
    mbar_init(&bars[PRIVA], 1);
    mbar_init(&bars[S_COPY], 128);
    mbar_init(&bars[S_DEC], 128);
    mbar_init(&bars[VN_DONE], 1);
    mbar_init(&bars[S_DONE], 1);
    mbar_init(&bars[P_DONE], 1);
    mbar_init(&bars[O_DONE], 1);
    mbar_init(&bars[W_DONE], 1);
    mbar_init(&bars[VN_READY], 128);
    mbar_init(&bars[W_READY], 128);
    mbar_init(&bars[P_READY], 128);
    mbar_init(&bars[O_FREE], 128);
    mbar_init(&bars[AP_READY], 2);
    mbar_init(&bars[VR_READY], 128);
    mbar_init(&bars[PRIV], 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_a);
  }
  // Pg is lower triangular: its tile is zeroed once, the O group only ever rewrites the column
  // groups that can be non-zero for its rows
  for (int i = tid; i < 8192 / 16; i += 512)
    *reinterpret_cast<uint4*>(smem + OFF_P + i * 16) = make_uint4(0, 0, 0, 0);
  fence_proxy_async();
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;  // this warp's lane quarter
  const long long state_off = ((long long)n * p.Hv + hv) * D * D;
  bool ok = true;
  long long waited[24];
#pragma unroll
  for (int i = 0; i < 24; ++i) waited[i] = 0;
  const long long t_start = clock64();
  long long t_sec = 0;
  auto WAIT = [&](int idx, uint32_t parity) {
    if constexpr (!PROFILE) {
      const bool r = mbar_wait(&bars[idx], parity, abort_flag);
      if (!r) atomicCAS(&g_fwd_abort_info, 0, (1 << 24) | (warp << 16) | (idx << 8) | (int)parity);
      return r;
    } else {
      long long t0 = clock64();
      bool r = mbar_wait(&bars[idx], parity, abort_flag);
      if (idx < 24) waited[idx] += clock64() - t0;
      return r;
    }
  };
#define SEC_BEGIN() do { if constexpr (PROFILE) t_sec = clock64(); } while (0)
#define SEC_END(slot) do { if constexpr (PROFILE) waited[slot] += clock64() - t_sec; } while (0)

  // Role of each warp.  The MMA issuer is warp 0 and the producer warp 1 on purpose: among the
  // warps of one scheduler the oldest (lowest id) wins when several are ready, and these two
  // single-thread roles must never queue behind the arithmetic of the compute groups.
  if (warp >= 4 && warp < 8) {
    // =============================== S group ===============================
    const int v = tid - 128;  // lane of tensor memory = value index
    // initial state -> tensor memory (S^T[v][k] = h0[k][v])
#pragma unroll 1
    for (int k0 = 0; k0 < D; k0 += 32) {
      float x[32];
#pragma unroll
      for (int j = 0; j < 32; ++j)
        x[j] = (p.h0 && lead == 0) ? p.h0[state_off + (long long)(k0 + j) * D + v] : 0.f;
      tmem_st32(tmem + lane_sel + TM_S + k0, x);
    }
    tmem_st_wait();
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      if (it > 0) ok = WAIT(S_DONE, (it - 1) & 1);
      if (!ok) break;
      tc_fence_after();
      SEC_BEGIN();
      bf16* hdst = (EXTRA && p.h && it >= lead)
                       ? p.h + ((sp.chunk_base + (it - lead)) * p.Hv + hv) * (long long)D * D : nullptr;
      // on the chain: the bf16 operand copy of S^T
#pragma unroll 1
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
        if (EXTRA && hdst && !p.tiled) {
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
      SEC_END(SEC_A);
      // off the chain: decay in place, needed only by the state update at the end of the chunk
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (!ok) break;
      SEC_BEGIN();
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
      SEC_END(SEC_B);
    }
    if (ok && n_it > 0) ok = WAIT(S_DONE, (n_it - 1) & 1);
    if (ok && p.ht) {
      tc_fence_after();
#pragma unroll 1
      for (int k0 = 0; k0 < D; k0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_S + k0, x);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) p.ht[state_off + (long long)(k0 + j) * D + v] = x[j];
      }
    }
  } else if (warp >= 8 && warp < 12) {
    // =============================== V group ===============================
    const int v = tid - 256;
    const int wq = warp & 3;
    const int tok_w = 16 * wq + (lane & 15);  // lanes 16-31 of each quarter hold a row of w
    // w of chunk `it` (tensor memory, M = 64 layout at lane +16) -> bf16 operand tile
    auto convert_w = [&](int it) {
      if (!WAIT(W_DONE, it & 1)) return false;
      tc_fence_after();
      SEC_BEGIN();
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_O2 + c0, x);
        tmem_ld_wait();
        if (lane >= 16) {
          unsigned char* row = smem + OFF_W + (c0 >> 6) * 8192 + tok_w * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(row + (((((c0 & 63) >> 3) + c) ^ (tok_w & 7)) << 4)) =
                make_uint4(pack_bf16(x[8 * c + 0], x[8 * c + 1]), pack_bf16(x[8 * c + 2], x[8 * c + 3]),
                           pack_bf16(x[8 * c + 4], x[8 * c + 5]), pack_bf16(x[8 * c + 6], x[8 * c + 7]));
        }
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[W_READY]);
      SEC_END(SEC_B);
      return true;
    };
    if (n_it > 0) ok = convert_w(0);
    for (int it = 0; it < n_it && ok; ++it) {
      const int c = it - lead;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = c < 0 ? 0 : min(CHUNK, sp.len - c * CHUNK);  // 0: nothing is stored
      ok = WAIT(FULL0 + (it & 1), (it >> 1) & 1) && WAIT(VN_DONE, it & 1);
      if (!ok) break;
      tc_fence_after();
      SEC_BEGIN();
      {
        float x[32], y[32];
        tmem_ld32(tmem + lane_sel + TM_UV, x);
        tmem_ld32(tmem + lane_sel + TM_UV + 32, y);
        tmem_ld_wait();
        // first the rho-scaled copy (operand of the state update, on the chain) ...
        const float* rho = vec + (it & 3) * VEC_SLOT_FLOATS + V_RHO * CHUNK;
        unsigned char* rowr = smem + OFF_VRT + v * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float4 r0 = *reinterpret_cast<const float4*>(rho + 8 * c);
          const float4 r1 = *reinterpret_cast<const float4*>(rho + 8 * c + 4);
          const float4 r2 = *reinterpret_cast<const float4*>(rho + 32 + 8 * c);
          const float4 r3 = *reinterpret_cast<const float4*>(rho + 32 + 8 * c + 4);
          *reinterpret_cast<uint4*>(rowr + ((c ^ (v & 7)) << 4)) = make_uint4(
              pack_bf16(r0.x * x[8 * c + 0], r0.y * x[8 * c + 1]),
              pack_bf16(r0.z * x[8 * c + 2], r0.w * x[8 * c + 3]),
              pack_bf16(r1.x * x[8 * c + 4], r1.y * x[8 * c + 5]),
              pack_bf16(r1.z * x[8 * c + 6], r1.w * x[8 * c + 7]));
          *reinterpret_cast<uint4*>(rowr + (((c + 4) ^ (v & 7)) << 4)) = make_uint4(
              pack_bf16(r2.x * y[8 * c + 0], r2.y * y[8 * c + 1]),
              pack_bf16(r2.z * y[8 * c + 2], r2.w * y[8 * c + 3]),
              pack_bf16(r3.x * y[8 * c + 4], r3.y * y[8 * c + 5]),
              pack_bf16(r3.z * y[8 * c + 6], r3.w * y[8 * c + 7]));
        }
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(&bars[VR_READY]);
        SEC_END(SEC_A);
        // ... then the plain copy (operand of the output product)
        unsigned char* row = smem + OFF_VNT + v * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          *reinterpret_cast<uint4*>(row + ((c ^ (v & 7)) << 4)) =
              make_uint4(pack_bf16(x[8 * c + 0], x[8 * c + 1]), pack_bf16(x[8 * c + 2], x[8 * c + 3]),
                         pack_bf16(x[8 * c + 4], x[8 * c + 5]), pack_bf16(x[8 * c + 6], x[8 * c + 7]));
          *reinterpret_cast<uint4*>(row + (((c + 4) ^ (v & 7)) << 4)) =
              make_uint4(pack_bf16(y[8 * c + 0], y[8 * c + 1]), pack_bf16(y[8 * c + 2], y[8 * c + 3]),
                         pack_bf16(y[8 * c + 4], y[8 * c + 5]), pack_bf16(y[8 * c + 6], y[8 * c + 7]));
        }
        fence_proxy_async();
        mbar_arrive(&bars[VN_READY]);
        if (EXTRA && p.vnew && !p.tiled) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (j < valid) p.vnew[((row0 + j) * p.Hv + hv) * D + v] = __float2bfloat16(x[j]);
            if (32 + j < valid)
              p.vnew[((row0 + 32 + j) * p.Hv + hv) * D + v] = __float2bfloat16(y[j]);
          }
        }
      }
      if (it + 1 < n_it) ok = convert_w(it + 1);
    }
  } else if (warp >= 12) {
    if constexpr (!NO_O) {
    // =============================== O group ===============================
    // M = 64 accumulators are read with the 16-lane shape: lane l of warp q owns rows
    // 16q + l/4 and 16q + l/4 + 8, and in every group of 8 columns the pair 2*(l%4), +1.
    const int wq = warp & 3;
    const int row_a = 16 * wq + (lane >> 2), row_b = row_a + 8, cp = 2 * (lane & 3);
    const uint32_t lanes_o = (uint32_t)(wq * 32) << 16;        // O1 / O2: lanes 0-15 of the quarter
    const uint32_t lanes_p = (uint32_t)(wq * 32 + 16) << 16;   // P: lanes 16-31
    // c counts the chunks of the sequence itself; the lead-in chunks (iterations j < lead) have no
    // output products, so the barriers of this group's products are phased by c, while stages and
    // vector slots follow the iteration j = c + lead
    auto epilogue = [&](int c) {
      const float* vs = vec + ((c + lead) & 3) * VEC_SLOT_FLOATS;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = min(CHUNK, sp.len - c * CHUNK);
      const float sg_a = vs[V_SGAM * CHUNK + row_a], sg_b = vs[V_SGAM * CHUNK + row_b];
      bf16* o_a = p.o + ((row0 + row_a) * p.Hv + hv) * D + cp;
      bf16* o_b = p.o + ((row0 + row_b) * p.Hv + hv) * D + cp;
      const bool wr_a = p.o != nullptr && row_a < valid, wr_b = p.o != nullptr && row_b < valid;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 64) {
        float a[32], b[32];
        tmem_ld_16x64(tmem + lanes_o + TM_O1 + c0, a);
        tmem_ld_16x64(tmem + lanes_o + TM_O2 + c0, b);
        tmem_ld_wait();
        if (c0 + 64 >= D) {  // all tensor-memory reads of this chunk's output are done
          tc_fence_before();
          mbar_arrive(&bars[O_FREE]);
        }
        // A lane holds one column pair of every group of 8 columns; the four lanes of a quad
        // (same rows) exchange words (4 x 4 transposes, two butterfly steps each) so that each
        // lane ends up with 8 consecutive columns: a store instruction then writes 64 contiguous
        // bytes of 8 rows instead of 16 bytes of 8 rows.
        uint32_t wa[8], wb[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          wa[i] = pack_bf16(sg_a * a[4 * i] + b[4 * i], sg_a * a[4 * i + 1] + b[4 * i + 1]);
          wb[i] = pack_bf16(sg_b * a[4 * i + 2] + b[4 * i + 2], sg_b * a[4 * i + 3] + b[4 * i + 3]);
        }
#pragma unroll
        for (int h4 = 0; h4 < 8; h4 += 4) {
          quad_transpose(wa + h4, lane);
          quad_transpose(wb + h4, lane);
          // lane j of the quad now holds columns c0 + 8 h4 + 8 j .. + 7 (o_a, o_b include 2 j)
          if (wr_a)
            *reinterpret_cast<uint4*>(o_a + c0 + 8 * h4 + 3 * cp) = make_uint4(wa[h4], wa[h4 + 1], wa[h4 + 2], wa[h4 + 3]);
          if (wr_b)
            *reinterpret_cast<uint4*>(o_b + c0 + 8 * h4 + 3 * cp) = make_uint4(wb[h4], wb[h4 + 1], wb[h4 + 2], wb[h4 + 3]);
        }
      }
    };
    const float log2_scale = log2f(p.scale);
    const int n_out = n_it - lead;  // chunks with output
    for (int it = 0; it < n_out && ok; ++it) {
      const int j = it + lead;
      const float* vs = vec + (j & 3) * VEC_SLOT_FLOATS;
      // (after a lead-in of four or more chunks the first of these waits may see an older phase of
      // the same parity; the wait for this chunk's P below is what orders the reads)
      ok = WAIT(FULL0 + (j & 1), (j >> 1) & 1);
      if (!ok) break;
      if (it > 0) {
        ok = WAIT(O_DONE, (it - 1) & 1);
        if (!ok) break;
        tc_fence_after();
        SEC_BEGIN();
        epilogue(it - 1);
        SEC_END(SEC_A);
      }
      ok = WAIT(P_DONE, it & 1);
      if (!ok) break;
      tc_fence_after();
      SEC_BEGIN();
      // Pg = s P exp(g_row - g_col) = P exp2((g_row - g_col) log2e + log2 s), col <= row
      {
        const float ga2 = vs[V_G * CHUNK + row_a] * 1.4426950408889634f + log2_scale;
        const float gb2 = vs[V_G * CHUNK + row_b] * 1.4426950408889634f + log2_scale;
        float x[32];
        tmem_ld_16x64(tmem + lanes_p + TM_O1, x);
        tmem_ld_wait();
        unsigned char* pa = smem + OFF_P + row_a * 128 + cp * 2;
        unsigned char* pb = smem + OFF_P + row_b * 128 + cp * 2;
        // column groups entirely above this warp's rows stay zero (written once at start)
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
      }
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(&bars[P_READY]);
      SEC_END(SEC_B);
    }
    if (ok && n_out > 0) {
      ok = WAIT(O_DONE, (n_out - 1) & 1);
      if (ok) {
        tc_fence_after();
        epilogue(n_out - 1);
      }
    }
    // rows of o past the end of the last packed sequence come out zero
    if (p.o && p.lay.cu.ptr && n == p.N - 1) {
      const long long end = sp.bos + sp.len;
      for (long long i = tid - 384; i < (p.T_rows - end) * 16; i += 128)
        *reinterpret_cast<uint4*>(p.o + ((end + (i >> 4)) * p.Hv + hv) * D + (i & 15) * 8) =
            make_uint4(0, 0, 0, 0);
    }
    }  // !NO_O
  } else if (warp == 0) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t ID_P = idesc_bf16(64, 64, 0, 0);
      constexpr uint32_t ID_O = idesc_bf16(64, 128, 0, 0);
      constexpr uint32_t ID_UT = idesc_bf16(128, 64, 1, 0);            // A = V tile, MN-major
      constexpr uint32_t ID_W = idesc_bf16(64, 128, 0, 1);             // B = K tile, MN-major
      constexpr uint32_t ID_VN = idesc_bf16(128, 64, 0, 0) | (1u << 13);  // A negated
      constexpr uint32_t ID_S = idesc_bf16(128, 128, 0, 1);
      // low descriptor words of every operand tile (see umma_lo); steps are 32-bit adds
      const uint32_t st_lo = desc_lo_kmajor(smem + OFF_ST), vnt_lo = desc_lo_kmajor(smem + OFF_VNT);
      const uint32_t w_lo = desc_lo_kmajor(smem + OFF_W), p_lo = desc_lo_kmajor(smem + OFF_P);
      const uint32_t ap_lo = desc_lo_kmajor(smem + OFF_AP), app_lo = desc_lo_kmajor(smem + OFF_APP);
      const uint32_t vrt_lo = desc_lo_kmajor(smem + OFF_VRT);
      const uint32_t q0_lo = desc_lo_kmajor(smem + OFF_STAGE);
      const uint32_t k0_lo = desc_lo_kmajor(smem + OFF_STAGE + TILE_QK);
      const uint32_t kmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + TILE_QK, 8192);
      const uint32_t vmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + 2 * TILE_QK, 8192);
      constexpr uint32_t STAGE_LO = STAGE_BYTES >> 4;
      auto issue_u_w = [&](uint32_t so) {  // so = stage offset in descriptor units
        umma_group<4, 128, 0, 2, 0, false>(tmem + TM_UV, vmn0_lo + so, ap_lo, ID_UT);
        umma_group<4, 2, 0, 128, 0, false>(tmem + TM_W, app_lo, kmn0_lo + so, ID_W);
        umma_commit(&bars[W_DONE]);
      };
      auto issue_p = [&](uint32_t so) {
        umma_group<8, 2, 512, 2, 512, false>(tmem + TM_P, q0_lo + so, k0_lo + so, ID_P);
        umma_commit(&bars[P_DONE]);
      };
      auto store_vn = [&](int it) {  // after VN_READY: the v_new^T tile is complete
        if (p.tiled && p.vnew && it >= lead) {
          tma_store_2d(&map_vn, 0, (int)(((sp.chunk_base + (it - lead)) * p.Hv + hv) * D), smem + OFF_VNT);
          tma_store_commit();
        }
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1;
        const uint32_t so = s ? STAGE_LO : 0u, so_next = s ? 0u : STAGE_LO;
        if (it == 0) {
          ok = WAIT(FULL0, 0) && WAIT(AP_READY, 0);
          if (!ok) break;
          tc_fence_after();
          issue_u_w(0);
        }
        ok = WAIT(S_COPY, it & 1) && WAIT(W_READY, it & 1);
        if (!ok) break;
        tc_fence_after();
        SEC_BEGIN();
        // Vn^T = u^T - S^T w^T   (accumulates onto u^T)
        umma_group<8, 2, 1024, 2, 512, true>(tmem + TM_UV, st_lo, w_lo, ID_VN);
        if constexpr (EXTRA) tma_store_wait_read();  // v_new^T of the chunk before has left its tile
        umma_commit(&bars[VN_DONE]);
        if constexpr (EXTRA) {
          if (p.tiled && p.h && it >= lead) {  // the operand copy of S^T is the state entering this chunk
            const int y = (int)(((sp.chunk_base + (it - lead)) * p.Hv + hv) * D);
            tma_store_2d(&map_h, 0, y, smem + OFF_ST);
            tma_store_2d(&map_h, 64, y, smem + OFF_ST + 16384);
            tma_store_commit();
          }
        }
        SEC_END(SEC_A);
        const int c = it - lead;  // < 0: lead-in chunk, no output products
        if (!NO_O && c >= 0) {
          if (c > 0) {
            ok = WAIT(O_FREE, (c - 1) & 1);
            if (!ok) break;
            tc_fence_after();
          }
          SEC_BEGIN();
          // O1 = Q S      (B = S^T copy: N = v rows, K = k)
          umma_group<8, 2, 512, 2, 1024, false>(tmem + TM_O1, q0_lo + so, st_lo, ID_O);
          // P of this chunk goes here, into the time the value group needs for Vn: the output
          // group turns it into Pg while the state update runs (it read P of the chunk before
          // ahead of the output product issued at the end of the previous iteration)
          issue_p(so);
          SEC_END(SEC_B);
        }
        ok = WAIT(VR_READY, it & 1) && WAIT(S_DEC, it & 1);
        if (!ok) break;
        tc_fence_after();
        SEC_BEGIN();
        // S^T += (rho Vn)^T K      (B = K tile read MN-major: contraction over its 64 rows)
        umma_group<4, 2, 0, 128, 0, true>(tmem + TM_S, vrt_lo, kmn0_lo + so, ID_S);
        if constexpr (EXTRA) tma_store_wait_read();  // the S^T tile may be rewritten after this
        umma_commit(&bars[S_DONE]);
        umma_commit(&bars[EMPTY0 + s]);  // last product that reads this stage
        SEC_END(SEC_C);
        if (it + 1 < n_it) {
          ok = WAIT(FULL0 + (s ^ 1), ((it + 1) >> 1) & 1) && WAIT(AP_READY, (it + 1) & 1) &&
               WAIT(VN_READY, it & 1);  // the V group has read Vn^T out of TM_UV
          if (!ok) break;
          tc_fence_after();
          SEC_BEGIN();
          issue_u_w(so_next);
          SEC_END(SEC_D);
          if constexpr (EXTRA) store_vn(it);
        }
        ok = (NO_O || c < 0 || WAIT(P_READY, c & 1)) && (it + 1 < n_it || WAIT(VN_READY, it & 1));
        if (!ok) break;
        tc_fence_after();
        if constexpr (EXTRA) {
          if (it + 1 >= n_it) store_vn(it);
        }
        if (!NO_O && c >= 0) {
          SEC_BEGIN();
          // O2 = Pg Vn     (B = Vn^T copy: N = v rows, K = tok')
          umma_group<4, 2, 0, 2, 0, false>(tmem + TM_O2, p_lo, vnt_lo, ID_O);
          umma_commit(&bars[O_DONE]);
          SEC_END(SEC_E);
        }
      }
      if constexpr (EXTRA) tma_store_wait_all();
    }
  } else if (warp == 1) {
    // =============================== producer ===============================
    float g_r[2] = {0.f, 0.f}, b_r[2] = {0.f, 0.f}, gl_r = 0.f;
    // (lead-in chunks, c < 0, are whole chunks of the rows before the sequence)
    auto fetch = [&](int it) {
      const int c = it - lead;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = c < 0 ? CHUNK : min(CHUNK, sp.len - c * CHUNK);
      gl_r = p.g[(row0 + valid - 1) * p.Hv + hv];
#pragma unroll
      for (int z = 0; z < 2; ++z) {
        int r = 2 * lane + z, rc = min(r, valid - 1);
        g_r[z] = p.g[(row0 + rc) * p.Hv + hv];
        b_r[z] = r < valid ? load_beta(p.beta, p.beta_is_f32, (row0 + r) * p.Hv + hv) : 0.f;
      }
    };
    // vectors and A tile of chunk j (its stage's A buffer is free once the prep warps have read it)
    auto a_part = [&](int j) {
      const int sj = j & 1, c = j - lead;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = c < 0 ? CHUNK : min(CHUNK, sp.len - c * CHUNK);
      if (j >= 2 && !WAIT(EMPTYA0 + sj, ((j >> 1) - 1) & 1)) return false;
      float* vs = vec + (j & 3) * VEC_SLOT_FLOATS;
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
      unsigned char* dst = smem + OFF_STAGE + sj * STAGE_BYTES + 2 * TILE_QK + TILE_V;
      const bool partial = valid < CHUNK;
      uint64_t* bar = partial ? &bars[PRIVA] : &bars[FULLA0 + sj];
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, TILE_A);
        tma_load_2d(dst, &map_a, hv * CHUNK, (int)row0, bar);
      }
      if (partial) {
        // rows past the sequence end belong to the next sequence: wait for the copy, zero them
        // (only the last chunk of a sequence can be partial: the private barrier is used once)
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
      const int s = it & 1, c = it - lead;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = c < 0 ? CHUNK : min(CHUNK, sp.len - c * CHUNK);
      const bool with_q = !NO_O && c >= 0;
      if (it >= 2) {
        ok = WAIT(EMPTY0 + s, ((it >> 1) - 1) & 1);
        if (!ok) break;
      }
      unsigned char* st = smem + OFF_STAGE + s * STAGE_BYTES;
      const bool partial = valid < CHUNK;
      uint64_t* bar = partial ? &bars[PRIV] : &bars[FULL0 + s];
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, STAGE_BYTES - TILE_A - (with_q ? 0 : TILE_QK));
        const int y = (int)row0;
        tma_load_2d(st + TILE_QK, &map_k, hq * D, y, bar);
        tma_load_2d(st + TILE_QK + 8192, &map_k, hq * D + 64, y, bar);
        tma_load_2d(st + 2 * TILE_QK, &map_v, hv * D, y, bar);
        tma_load_2d(st + 2 * TILE_QK + 8192, &map_v, hv * D + 64, y, bar);
        if (with_q) {
          tma_load_2d(st, &map_q, hq * D, y, bar);
          tma_load_2d(st + 8192, &map_q, hq * D + 64, y, bar);
        }
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
      // The next chunk's vectors and A tile go out now, a whole chunk before its q, k, v: the
      // q, k, v stage of chunk it + 1 is still in use, but the prep warps can start on A early.
      // (Slot (it + 1) % 4 of the vectors was last read for chunk it - 3, which the wait on the
      // stage of chunk it - 2 above has seen finished.)
      if (it + 1 < n_it) {
        ok = a_part(it + 1);
        if (ok && it + 2 < n_it) fetch(it + 2);
      }
    }
  } else {
    // =============================== prep (warps 2, 3) ===============================
    // A' = A diag(beta), A'' = A diag(beta gamma).  Thread t owns the 8 columns 8 (t%8) .. of the
    // rows t/8 + 8 i: its 16 scale factors stay in registers, and the eight threads of a row touch
    // the eight 16-byte pieces of that row (one 128-byte line per access, conflict-free).
    const int t = tid - 64, c8 = t & 7, r0 = t >> 3;
    const int pc = c8 ^ r0;  // physical piece: rows r0 + 8 i all have (row & 7) == r0
    for (int it = 0; it < n_it && ok; ++it) {
      const int s = it & 1;
      ok = WAIT(FULLA0 + s, (it >> 1) & 1);
      if (ok && it > 0) ok = WAIT(W_DONE, (it - 1) & 1);  // u, w of the chunk before are done
      if (!ok) break;
      SEC_BEGIN();
      const float* vs = vec + (it & 3) * VEC_SLOT_FLOATS;
      const float4 b0 = *reinterpret_cast<const float4*>(vs + V_BETA * CHUNK + 8 * c8);
      const float4 b1 = *reinterpret_cast<const float4*>(vs + V_BETA * CHUNK + 8 * c8 + 4);
      const float4 g0 = *reinterpret_cast<const float4*>(vs + V_BG * CHUNK + 8 * c8);
      const float4 g1 = *reinterpret_cast<const float4*>(vs + V_BG * CHUNK + 8 * c8 + 4);
      const unsigned char* src = smem + OFF_STAGE + s * STAGE_BYTES + 2 * TILE_QK + TILE_V;
#pragma unroll 4
      for (int i = 0; i < 8; ++i) {
        const int off = (r0 + 8 * i) * 128 + pc * 16;
        const uint4 a = *reinterpret_cast<const uint4*>(src + off);
        *reinterpret_cast<uint4*>(smem + OFF_AP + off) =
            make_uint4(scale_bf16x2(a.x, b0.x, b0.y), scale_bf16x2(a.y, b0.z, b0.w),
                       scale_bf16x2(a.z, b1.x, b1.y), scale_bf16x2(a.w, b1.z, b1.w));
        *reinterpret_cast<uint4*>(smem + OFF_APP + off) =
            make_uint4(scale_bf16x2(a.x, g0.x, g0.y), scale_bf16x2(a.y, g0.z, g0.w),
                       scale_bf16x2(a.z, g1.x, g1.y), scale_bf16x2(a.w, g1.z, g1.w));
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars[AP_READY]);
        mbar_arrive(&bars[EMPTYA0 + s]);  // the A tile of this stage is no longer read here
      }
      SEC_END(SEC_A);
    }
  }

  if (PROFILE && blockIdx.x == 0 && (tid % 128 == 0 || tid == 32 || tid == 64)) {
    int role = tid == 128 ? 0 : tid == 256 ? 1 : tid == 384 ? 2 : tid == 0 ? 3 : tid == 32 ? 4 : 5;
    for (int i = 0; i < 24; ++i) g_wait_profile[role * 24 + i] = waited[i];
    if (tid == 128) g_wait_profile[6 * 24] = clock64() - t_start;
  }
#undef SEC_BEGIN
#undef SEC_END
  // ---- teardown: everybody meets, then the allocating warp frees tensor memory
  if (!ok) *abort_flag = 1;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicCAS(&g_device_status, 0, 1);
}

// ---- host side --------------------------------------------------------------------------------
// 2-D bf16 tensor [rows][cols] (row pitch = cols), box = 64 columns x box_rows rows, 128-byte
// swizzle; recently used maps are served from a small host-side table (bwd_main_tc.cu).
int make_tile_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, int box_rows);

static int make_map(CUtensorMap* m, const void* ptr, long long rows, long long cols) {
  return make_tile_map(m, ptr, rows, cols, 64);
}

int launch_fwd_tc(const void* q, const void* k, const void* v, const void* A, const float* g,
                  const void* beta, int beta_is_f32, const float* h0, float* ht, void* o, void* h,
                  void* vnew, int tiled, const int* lead, int N, int Hq, int Hv, long long T_rows,
                  float scale, SeqLayout lay, cudaStream_t st) {
  using namespace fwdtc;
  CUtensorMap mq, mk, mv, ma, mh, mvn;
  int rc;
  // without q (recomputation of h and v_new for the backward pass) the state-only variant runs;
  // its q map is never used and only has to be a valid map
  if ((rc = make_map(&mq, q ? q : k, T_rows, (long long)Hq * D))) return rc;
  if ((rc = make_map(&mk, k, T_rows, (long long)Hq * D))) return rc;
  if ((rc = make_map(&mv, v, T_rows, (long long)Hv * D))) return rc;
  if ((rc = make_map(&ma, A, T_rows, (long long)Hv * CHUNK))) return rc;
  mh = mq;
  mvn = mq;
  if (tiled) {
    // an upper bound of the chunk count: the maps only have to cover what the kernel stores
    const long long max_chunks = (T_rows + CHUNK - 1) / CHUNK + N;
    if (h && (rc = make_tile_map(&mh, h, max_chunks * Hv * D, D, 128))) return rc;
    if (vnew && (rc = make_tile_map(&mvn, vnew, max_chunks * Hv * D, CHUNK, 128))) return rc;
  }
  FwdTcParams p;
  p.tiled = tiled;
  p.lead = lead;
  p.g = g; p.beta = beta; p.beta_is_f32 = beta_is_f32; p.h0 = h0; p.ht = ht;
  p.o = (bf16*)o; p.h = (bf16*)h; p.vnew = (bf16*)vnew;
  p.N = N; p.Hq = Hq; p.Hv = Hv; p.T_rows = T_rows; p.scale = scale; p.lay = lay;
  p.profile = 0;
  const bool extra = h != nullptr || vnew != nullptr;
  auto launch = [&](auto kernel) {
    int err = configure_smem((const void*)kernel, SMEM_BYTES);
    if (err != 0) return err;
    kernel<<<(unsigned)(N * Hv), 512, SMEM_BYTES, st>>>(p, mq, mk, mv, ma, mh, mvn);
    return (int)cudaGetLastError();
  };
#ifdef FQLA_DIAGNOSTICS  // wait/section cycle counters of the first CTA (development builds only)
  static const bool profile = getenv("FQLA_PROFILE") != nullptr;
  p.profile = profile ? 1 : 0;
  if (p.profile) return launch(fwd_tc_kernel<true, true, false>);
#endif
  if (!q && !o) return launch(fwd_tc_kernel<false, true, true>);  // recomputation of h, v_new
  if (extra) return launch(fwd_tc_kernel<false, true, false>);
  return launch(fwd_tc_kernel<false, false, false>);
}

}  // namespace fqla

#ifdef FQLA_DIAGNOSTICS
extern "C" int fqla_debug_abort_info(int* out) {
  return (int)cudaMemcpyFromSymbol(out, fqla::g_fwd_abort_info, sizeof(int));
}

extern "C" int fqla_debug_wait_profile(long long* out168) {
  return (int)cudaMemcpyFromSymbol(out168, fqla::g_wait_profile, sizeof(long long) * 7 * 24);
}
#endif

namespace fqla {
// Self-test of the bounded-wait path: one thread waits on an mbarrier that nobody ever arrives
// at, with a budget of `tries` suspended tries of at most 1 ms each.  The wait gives up, the
// kernel sets the device status word exactly as a product kernel does, and returns.
__global__ void wait_timeout_selftest_kernel(uint32_t tries) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(&bar, 0, &abort_flag, tries);
  __syncthreads();
  if (threadIdx.x == 0 && (!ok || abort_flag)) atomicCAS(&g_device_status, 0, 1);
}
}  // namespace fqla

extern "C" int fqla_selftest_wait_timeout(int tries, void* stream) {
  if (tries < 1 || tries > 100) return FQLA_ERR_INVALID_ARG;
  fqla::wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((uint32_t)tries);
  return (int)cudaGetLastError();
}

namespace fqla {
int bwd_main_tc_status(int* out, int reset);
int bwd_dh_tc_status(int* out, int reset);
}

extern "C" int fqla_device_status(int* out, int reset) {
  int v = 0, w = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, fqla::g_device_status, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  int u = 0;
  int rc = fqla::bwd_main_tc_status(&w, reset);
  if (rc != 0) return rc;
  rc = fqla::bwd_dh_tc_status(&u, reset);
  if (rc != 0) return rc;
  if (out) *out = v | w | u;
  if (reset && v != 0) {
    int z = 0;
    e = cudaMemcpyToSymbol(fqla::g_device_status, &z, sizeof(int));
  }
  return (int)e;
}
