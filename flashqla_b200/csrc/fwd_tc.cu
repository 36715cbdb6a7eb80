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
//     w^T [k x tok] = K^T A''^T         (A operand = K tile read MN-major)        -> TM_PW -> smem
//     P   [tok x tok'] = Q K^T,  Pg = s P exp(g_tok - g_tok') for tok >= tok'     (O group)
//   on the chain (two products):
//     Vn^T [v x tok] = u^T - S^T w^T    (A = bf16 copy of S^T, negated; accumulates onto u^T)
//     S^T  [v x k]   = gamma_last S^T + (rho Vn)^T K     (B = K tile read MN-major)
//   output, transposed so that it shares the A operands of the chain:
//     O1^T [v x tok] = S^T Q^T,   O2^T [v x tok] = Vn^T Pg^T,   o = s gamma_tok O1 + O2
//
// The state path is kept TRANSPOSED: the 128-wide value dimension sits on the MMA M axis
// (tensor-memory lane = value index, one thread per lane), so every product but P has M = 128.
// Every operand that a read-out warp derives from an accumulator - the bf16 copy of S^T, Vn^T and
// rho Vn^T - goes back into TENSOR MEMORY (two bf16 per 32-bit column) and is consumed as the A
// operand of the next product straight from there (tcgen05.mma with A in tensor memory): the
// chunk-to-chunk chain never touches shared memory, and the tensor pipe, which is bound by the
// shared-memory fetch of its operands, reads half as much.  This is the algebra of the
// reference's blackwell/fused_fwd.py:349-596 (and the X/Y form of prepare_h.py:312-318) with the
// gate folded into A.
//
// Warp roles (thread ranges):
//     128-255 S group : fp32 master state in tensor memory; per chunk packs the bf16 operand copy
//                       of S^T into tensor memory (on the chain), then decays S^T in place
//     256-383 V group : Vn^T -> rho-scaled and plain bf16 operand copies (tensor memory);
//                       w^T -> bf16 operand tile (shared memory)
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

#ifdef FQLA_DIAGNOSTICS
// Development builds only: clock stamps of the role leaders of CTA 0 over a window of chunks,
// [role 0..5][chunk in window 0..15][tag 0..9].
__device__ long long g_fwd_trace[6 * 16 * 10];
__device__ int g_trace_cta = 0;               // which CTA records the role trace
__device__ long long g_cta_cycles[2 * 1024];  // per CTA: SM id, cycles from entry to exit
// chain issuer of CTA 0 and CTA 77: clock at the start of every chunk, [cta 0/1][chunk 0..127];
// entries 126, 127: kernel entry and exit of that CTA
__device__ long long g_fwd_chunk_clock[2 * 128];
#define FQLA_CHUNK_CLOCK(idx)                                                              \
  do {                                                                                     \
    if ((blockIdx.x == 0 || blockIdx.x == 77) && (idx) < 128)                              \
      g_fwd_chunk_clock[(blockIdx.x == 0 ? 0 : 128) + (idx)] = clock64();                  \
  } while (0)
#define FQLA_TRACE(role, tag)                                                         \
  do {                                                                                \
    if (blockIdx.x == g_trace_cta && it >= 24 && it < 40)                             \
      g_fwd_trace[((role) * 16 + (it - 24)) * 10 + (tag)] = clock64();               \
  } while (0)
#else
#define FQLA_TRACE(role, tag) do { } while (0)
#define FQLA_CHUNK_CLOCK(idx) do { } while (0)
#endif

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
  int tiled;  // h and vnew are written as operand tiles (h^T per chunk, v_new^T per chunk) by TMA
  // [N, Hv] or null: lead-in.  A CTA with lead > 0 starts from a ZERO state `lead` chunks before
  // its sequence (segment) and walks those chunks state-only (no q, no output, nothing stored):
  // the rows just before a segment are the tail of the segment before it, whose influence dies
  // out within `lead` chunks.  h0 is ignored for such a CTA.
  const int* lead;
  // [N, Hv] or null: a CTA whose entry differs from run_value returns at once, reading and
  // writing nothing (two launches can share one set of outputs, each taking its own pairs)
  const int* run_mask;
  int run_value;
  // [N] or null: the CTAs of block index i / Hv walk sequence order[i].  Blocks start in index
  // order, so a table that lists the longest sequences first shortens the tail of a ragged batch.
  const int* order;
};

namespace fwdtc {
constexpr int D = 128;
constexpr int TILE_QK = 16384, TILE_V = 16384, TILE_A = 8192;
constexpr int STAGE_BYTES = 2 * TILE_QK + TILE_V + TILE_A;  // 57344
constexpr int OFF_STAGE = 0;
constexpr int OFF_W = 2 * STAGE_BYTES;           // w^T   [128 k rows x 128B (64 tokens)]
constexpr int OFF_P = OFF_W + 16384;             // Pg    [64 x 128B]
constexpr int OFF_AP = OFF_P + 8192;             // A diag(beta)
constexpr int OFF_APP = OFF_AP + 8192;           // A diag(beta gamma)
constexpr int OFF_O = OFF_APP + 8192;            // o tile [64 tok x 128 v] bf16, source of its TMA store
constexpr int OFF_VEC = OFF_O + 16384;           // 4 slots x 6 vectors x 64 floats
constexpr int VEC_SLOT_FLOATS = 6 * CHUNK;
constexpr int OFF_BAR = OFF_VEC + 4 * VEC_SLOT_FLOATS * 4;
constexpr int N_BARS = 32;
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;
// only the variants that hand per-chunk tiles to the backward pass keep shared-memory copies of
// S^T and Vn^T (the sources of their TMA stores)
constexpr int OFF_ST = (OFF_MISC + 16 + 1023) / 1024 * 1024;  // S^T copy, 2 blocks of [128 x 128B]
constexpr int OFF_VNT = OFF_ST + 32768;                       // Vn^T  [128 x 128B]
constexpr int SMEM_BYTES = OFF_ST + 1024;  // + slack for 1024-byte alignment of the base
constexpr int SMEM_BYTES_EXTRA = OFF_VNT + 16384 + 1024;
// tensor-memory columns (512).  The bf16 operands hold two elements per column.
constexpr uint32_t TM_S = 0;      // S^T fp32                      128 columns
constexpr uint32_t TM_SB = 128;   // S^T bf16 (A operand, K = 128)  64 columns
constexpr uint32_t TM_UV = 192;   // u^T, then Vn^T fp32            64 columns
constexpr uint32_t TM_VNB = 256;  // Vn^T bf16 (A operand, K = 64)  32 columns
constexpr uint32_t TM_VRB = 288;  // rho Vn^T bf16                  32 columns
constexpr uint32_t TM_O1 = 320;   // O1^T fp32                      64 columns
constexpr uint32_t TM_O2 = 384;   // O2^T fp32                      64 columns
// P (M = 64: lanes 0-15 of each quarter) and w^T of the NEXT chunk (M = 128) take turns in the
// same columns: w^T is issued only after the output group has read P, and the next P only after
// the value group has turned w^T into its operand tile (the chain's first product waits for it).
constexpr uint32_t TM_PW = 448;
// barrier indices
enum { FULL0 = 0, FULL1, EMPTY0, EMPTY1, S_COPY, S_DEC, VN_DONE, S_DONE, P_DONE, O_DONE, W_DONE,
       VB_READY, W_READY, P_READY, O_FREE, AP_READY, PRIV,
       // the A tile and the per-row vectors of a chunk travel one chunk ahead of q, k, v
       FULLA0, FULLA1, EMPTYA0, EMPTYA1, PRIVA,
       // tile outputs: the shared-memory copies of S^T / Vn^T are complete
       ST_READY, VN_READY,
       // the output product that reads the packed copy of S^T has completed
       SB_FREE };
// vectors inside a slot; V_GL holds gamma_last at [0]
enum { V_G = 0, V_BETA = 1, V_BG = 2, V_RHO = 3, V_SGAM = 4, V_GL = 5 };
}  // namespace fwdtc

__device__ __forceinline__ uint32_t scale_bf16x2(uint32_t packed, float lo, float hi) {
  float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&packed));
  return pack_bf16(f.x * lo, f.y * hi);
}

// EXTRA: per-chunk state and v_new outputs (compiled out of the common instantiation: the six
// roles run six different code regions at once, and the kernel is sensitive to its
// instruction-cache footprint).  NO_O: state-only walk (recomputation for the backward pass): no q,
// no output products, the output warps stay idle.
template <bool EXTRA, bool NO_O>
__global__ void __launch_bounds__(512, 1)
fwd_tc_kernel(const FwdTcParams p, const __grid_constant__ CUtensorMap map_q,
              const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_h,
              const __grid_constant__ CUtensorMap map_vn, const __grid_constant__ CUtensorMap map_o) {
  using namespace fwdtc;
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
  // iteration j handles chunk c = j - lead of the sequence; c < 0 are the lead-in chunks
  const int lead = p.lead ? p.lead[n * p.Hv + hv] : 0;
  const int n_it = sp.n_chunks == 0 ? 0 : sp.n_chunks + lead;
  const bool tile_h = EXTRA && p.tiled && p.h, tile_vn = EXTRA && p.tiled && p.vnew;

  if (tid == 0) FQLA_CHUNK_CLOCK(126);
#ifdef FQLA_DIAGNOSTICS
  const long long g_fwd_chunk_clock_entry = clock64();
#endif
  if (tid == 0) {
    mbar_init(&bars[FULL0], 1);
    mbar_init(&bars[FULL1], 1);
    mbar_init(&bars[EMPTY0], 2);  // MMA commits of the two issuing threads
    mbar_init(&bars[EMPTY1], 2);
    mbar_init(&bars[SB_FREE], 1);
    mbar_init(&bars[FULLA0], 1);
    mbar_init(&bars[FULLA1], 1);
    mbar_init(&bars[EMPTYA0], 128);  // the output group, the only reader of the raw A tile
    mbar_init(&bars[EMPTYA1], 128);
    mbar_init(&bars[PRIVA], 1);
    mbar_init(&bars[S_COPY], 128);
    mbar_init(&bars[S_DEC], 128);
    mbar_init(&bars[VN_DONE], 1);
    mbar_init(&bars[S_DONE], 1);
    mbar_init(&bars[P_DONE], 1);
    mbar_init(&bars[O_DONE], 1);
    mbar_init(&bars[W_DONE], 1);
    mbar_init(&bars[VB_READY], 128);
    mbar_init(&bars[W_READY], 128);
    mbar_init(&bars[P_READY], 128);
    mbar_init(&bars[O_FREE], 128);
    mbar_init(&bars[AP_READY], 128);
    mbar_init(&bars[PRIV], 1);
    mbar_init(&bars[ST_READY], 128);
    mbar_init(&bars[VN_READY], 128);
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
  auto WAIT = [&](int idx, uint32_t parity) { return mbar_wait(&bars[idx], parity, abort_flag); };


  // Role of each warp.  The MMA issuer is warp 0 and the producer warp 1 on purpose: among the
  // warps of one scheduler the oldest (lowest id) wins when several are ready, and these two
  // single-thread roles must never queue behind the arithmetic of the compute groups.
  if (warp >= 4 && warp < 8) {
    // =============================== S group ===============================
    const int v = tid - 128;  // lane of tensor memory = value index
    // initial state -> tensor memory (S^T[v][k] = h0[k][v]); a lead-in starts from zero
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
      if (v == 0) FQLA_TRACE(0, 0);
      if (it > 0) ok = WAIT(S_DONE, (it - 1) & 1);
      // the output product of the chunk before, issued by the other thread, has read the copy
      if (!NO_O && ok && it - 1 >= lead) ok = WAIT(SB_FREE, (it - 1 - lead) & 1);
      if (!ok) break;
      tc_fence_after();
      if (v == 0) FQLA_TRACE(0, 1);
      // on the chain: the bf16 operand copy of S^T, packed back into tensor memory.  (The products
      // that read the copy of the chunk before were issued ahead of the state update whose
      // completion was just waited for, and the tensor pipe runs in issue order.)
#pragma unroll 1
      for (int k0 = 0; k0 < D; k0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_S + k0, x);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
        tmem_st16(tmem + lane_sel + TM_SB + (k0 >> 1), pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[S_COPY]);
      if (v == 0) FQLA_TRACE(0, 2);
      if constexpr (EXTRA) {
        // off the chain: the state entering this chunk as an output
        if (p.h && it >= lead) {
          bf16* hdst = p.h + ((sp.chunk_base + (it - lead)) * p.Hv + hv) * (long long)D * D;
#pragma unroll 1
          for (int kb = 0; kb < 2; ++kb) {  // 64 columns (one operand block) per round
            float x[32], y[32];
            tmem_ld32(tmem + lane_sel + TM_S + kb * 64, x);
            tmem_ld32(tmem + lane_sel + TM_S + kb * 64 + 32, y);
            tmem_ld_wait();
            if (p.tiled) {
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
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                hdst[(long long)(kb * 64 + j) * D + v] = __float2bfloat16(x[j]);
                hdst[(long long)(kb * 64 + 32 + j) * D + v] = __float2bfloat16(y[j]);
              }
            }
          }
          if (p.tiled) {
            fence_proxy_async();
            mbar_arrive(&bars[ST_READY]);
          }
        }
      }
      // off the chain: decay in place, needed only by the state update at the end of the chunk
      ok = WAIT(FULL0 + s, (it >> 1) & 1);
      if (!ok) break;
      if (v == 0) FQLA_TRACE(0, 3);
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
      if (v == 0) FQLA_TRACE(0, 4);
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
    const int v = tid - 256;  // tensor-memory lane: value index for Vn^T, key index for w^T
    // w^T of chunk `it` (tensor memory, [k][tok]) -> bf16 operand tile, row k = 64 tokens
    auto convert_w = [&](int it) {
      if (!WAIT(W_DONE, it & 1)) return false;
      tc_fence_after();
      float x[32], y[32];
      tmem_ld32(tmem + lane_sel + TM_PW, x);
      tmem_ld32(tmem + lane_sel + TM_PW + 32, y);
      tmem_ld_wait();
      tc_fence_before();
      unsigned char* row = smem + OFF_W + v * 128;
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
      mbar_arrive(&bars[W_READY]);
      return true;
    };
    if (n_it > 0) ok = convert_w(0);
    for (int it = 0; it < n_it && ok; ++it) {
      const int c = it - lead;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = c < 0 ? 0 : min(CHUNK, sp.len - c * CHUNK);  // 0: nothing is stored
      if (v == 0) FQLA_TRACE(1, 0);
      ok = WAIT(FULL0 + (it & 1), (it >> 1) & 1) && WAIT(VN_DONE, it & 1);
      if (!ok) break;
      // the output product that reads Vn^T of the chunk before is issued by the other thread
      if (!NO_O && c >= 1 && !WAIT(O_DONE, (c - 1) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (v == 0) FQLA_TRACE(1, 1);
      const float* rho = vec + (it & 3) * VEC_SLOT_FLOATS + V_RHO * CHUNK;
      // on the chain: Vn^T as the two bf16 operands (rho-scaled for the state update, plain for
      // the output product), 32 tokens = 16 packed columns at a time
#pragma unroll 1
      for (int t0 = 0; t0 < CHUNK; t0 += 32) {
        float x[32];
        tmem_ld32(tmem + lane_sel + TM_UV + t0, x);
        tmem_ld_wait();
        uint32_t pr[16], pn[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 r = *reinterpret_cast<const float4*>(rho + t0 + 4 * i);
          pr[2 * i] = pack_bf16(r.x * x[4 * i], r.y * x[4 * i + 1]);
          pr[2 * i + 1] = pack_bf16(r.z * x[4 * i + 2], r.w * x[4 * i + 3]);
          pn[2 * i] = pack_bf16(x[4 * i], x[4 * i + 1]);
          pn[2 * i + 1] = pack_bf16(x[4 * i + 2], x[4 * i + 3]);
        }
        tmem_st16(tmem + lane_sel + TM_VRB + (t0 >> 1), pr);
        tmem_st16(tmem + lane_sel + TM_VNB + (t0 >> 1), pn);
        if constexpr (EXTRA) {
          if (p.vnew && c >= 0) {
            if (p.tiled) {  // the tile of the TMA store (the store of the chunk before has read it)
              unsigned char* row = smem + OFF_VNT + v * 128;
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<uint4*>(row + ((((t0 >> 3) + q4) ^ (v & 7)) << 4)) =
                    make_uint4(pn[4 * q4], pn[4 * q4 + 1], pn[4 * q4 + 2], pn[4 * q4 + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (t0 + j < valid)
                  p.vnew[((row0 + t0 + j) * p.Hv + hv) * D + v] = __float2bfloat16(x[j]);
            }
          }
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[VB_READY]);
      if (v == 0) FQLA_TRACE(1, 2);
      if constexpr (EXTRA) {
        if (tile_vn && c >= 0) {
          fence_proxy_async();
          mbar_arrive(&bars[VN_READY]);
        }
      }
      if (it + 1 < n_it) ok = convert_w(it + 1);
      if (v == 0) FQLA_TRACE(1, 3);
    }
  } else if (warp >= 12) {
    // =============================== O group ===============================
    // Per chunk: the epilogue of the chunk before, Pg of this chunk, and A' = A diag(beta),
    // A'' = A diag(beta gamma) of the NEXT chunk (the scaled tiles the issuing thread needs for
    // u^T, w^T at the end of this chunk).  The state-only variant keeps only the last part.
    // P is an M = 64 accumulator read with the 16-lane shape: lane l of warp q owns rows
    // 16q + l/4 and 16q + l/4 + 8, and in every group of 8 columns the pair 2*(l%4), +1.
    const int wq = warp & 3;
    const int v = tid - 384;
    const int row_a = 16 * wq + (lane >> 2), row_b = row_a + 8, cp = 2 * (lane & 3);
    const uint32_t lanes_p = (uint32_t)(wq * 32) << 16;  // P: lanes 0-15 of the quarter
    // c counts the chunks of the sequence itself; the lead-in chunks (iterations j < lead) have no
    // output products, so the barriers of this group's products are phased by c, while stages and
    // vector slots follow the iteration j = c + lead
    // The output tile leaves through shared memory and one TMA store per 64-column box: a
    // read-out thread owns one value index of all 64 tokens, and global stores of that shape (two
    // 64-byte pieces per warp instruction) are an order of magnitude slower than the rest of the
    // chunk.  Only a sequence's ragged last chunk is written with plain stores, row by row.
    auto epilogue = [&](int c) {
      const int it = c + lead;  // (trace window index)
      const float* sg = vec + (it & 3) * VEC_SLOT_FLOATS + V_SGAM * CHUNK;
      const long long row0 = sp.bos + (long long)c * CHUNK;
      const int valid = min(CHUNK, sp.len - c * CHUNK);
      if (v == 0) tma_store_wait_read();  // the store of the chunk before has read the tile
      asm volatile("bar.sync 1, 128;" ::: "memory");
      // The accumulators hold o transposed ([value index][token]).  Read with the 16-lane shape, a
      // lane gets mma-style fragments: rows l/4 and l/4 + 8 of a 16-row half, token pairs
      // 8 i + 2 (l%4), +1.  stmatrix with .trans writes each 8 x 8 fragment block transposed, i.e.
      // as eight 16-byte pieces "8 value indices of one token": the tile comes out token-major
      // without a single shuffle.
      const int l4 = lane & 3, mtx = lane >> 3, r8 = lane & 7;
      float2 sgv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) sgv[i] = *reinterpret_cast<const float2*>(sg + 8 * i + 2 * l4);
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        if (v == 0) FQLA_TRACE(2, h ? 7 : 5);
        const uint32_t lanes = (uint32_t)(wq * 32 + 16 * h) << 16;
        float a[32], b[32];
        tmem_ld_16x64(tmem + lanes + TM_O1, a);
        tmem_ld_16x64(tmem + lanes + TM_O2, b);
        tmem_ld_wait();
        if (v == 0) FQLA_TRACE(2, h ? 8 : 6);
        if (h == 1) {  // all tensor-memory reads of this chunk's output are done
          tc_fence_before();
          mbar_arrive(&bars[O_FREE]);
        }
        // this lane supplies the address of row r8 of matrix mtx of every store: matrices 0, 1 are
        // the two 8-row blocks of token block i, matrices 2, 3 those of token block i + 1
        const int pv = ((wq & 1) * 32 + 16 * h) >> 3;  // 16-byte piece of rows 0-7 inside the box
        const uint32_t base = s32(smem + OFF_O + (wq >> 1) * 8192) +
                              (uint32_t)((8 * (mtx >> 1) + r8) * 128 + (((pv + (mtx & 1)) ^ r8) << 4));
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          uint32_t w[4];
#pragma unroll
          for (int z = 0; z < 2; ++z) {
            const float2 s2 = sgv[i + z];
            const float* aa = a + 4 * (i + z);
            const float* bb = b + 4 * (i + z);
            w[2 * z] = pack_bf16(s2.x * aa[0] + bb[0], s2.y * aa[1] + bb[1]);
            w[2 * z + 1] = pack_bf16(s2.x * aa[2] + bb[2], s2.y * aa[3] + bb[3]);
          }
          stmatrix_x4_trans(base + (uint32_t)(i * 1024), w[0], w[1], w[2], w[3]);
        }
      }
      fence_proxy_async();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (valid == CHUNK) {
        if (v == 0) {
          tma_store_2d(&map_o, hv * D, (int)row0, smem + OFF_O);
          tma_store_2d(&map_o, hv * D + 64, (int)row0, smem + OFF_O + 8192);
          tma_store_commit();
        }
      } else {
        // 16 pieces of 16 bytes per row; piece pc of row r sits at pc ^ (r & 7) inside its box
        for (int i = v; i < valid * 16; i += 128) {
          const int r = i >> 4, pc = i & 15;
          const uint4 w = *reinterpret_cast<const uint4*>(smem + OFF_O + (pc >> 3) * 8192 + r * 128 +
                                                          (((pc & 7) ^ (r & 7)) << 4));
          *reinterpret_cast<uint4*>(p.o + ((row0 + r) * p.Hv + hv) * D + pc * 8) = w;
        }
      }
    };
    // A', A'': thread t owns the 8 columns 8 (t%8) .. of the rows t/8 + 16 i: its 16 scale factors
    // stay in registers, and the eight threads of a row touch the eight 16-byte pieces of that row
    // (one 128-byte line per access, conflict-free)
    auto scale_a = [&](int j) {
      const int sj = j & 1, c8 = v & 7, r0 = v >> 3;
      const int pc = c8 ^ (r0 & 7);  // physical piece: rows r0 + 16 i all have (row & 7) == r0 & 7
      if (!WAIT(FULLA0 + sj, (j >> 1) & 1)) return false;
      if (j > 0 && !WAIT(W_DONE, (j - 1) & 1)) return false;  // u, w of the chunk before are done
      const float* vs = vec + (j & 3) * VEC_SLOT_FLOATS;
      const float4 b0 = *reinterpret_cast<const float4*>(vs + V_BETA * CHUNK + 8 * c8);
      const float4 b1 = *reinterpret_cast<const float4*>(vs + V_BETA * CHUNK + 8 * c8 + 4);
      const float4 g0 = *reinterpret_cast<const float4*>(vs + V_BG * CHUNK + 8 * c8);
      const float4 g1 = *reinterpret_cast<const float4*>(vs + V_BG * CHUNK + 8 * c8 + 4);
      const unsigned char* src = smem + OFF_STAGE + sj * STAGE_BYTES + 2 * TILE_QK + TILE_V;
      uint4 a[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        a[i] = *reinterpret_cast<const uint4*>(src + (r0 + 16 * i) * 128 + pc * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int off = (r0 + 16 * i) * 128 + pc * 16;
        *reinterpret_cast<uint4*>(smem + OFF_AP + off) =
            make_uint4(scale_bf16x2(a[i].x, b0.x, b0.y), scale_bf16x2(a[i].y, b0.z, b0.w),
                       scale_bf16x2(a[i].z, b1.x, b1.y), scale_bf16x2(a[i].w, b1.z, b1.w));
        *reinterpret_cast<uint4*>(smem + OFF_APP + off) =
            make_uint4(scale_bf16x2(a[i].x, g0.x, g0.y), scale_bf16x2(a[i].y, g0.z, g0.w),
                       scale_bf16x2(a[i].z, g1.x, g1.y), scale_bf16x2(a[i].w, g1.z, g1.w));
      }
      fence_proxy_async();
      mbar_arrive(&bars[AP_READY]);
      mbar_arrive(&bars[EMPTYA0 + sj]);  // the A tile of this stage is no longer read here
      return true;
    };
    const float log2_scale = log2f(p.scale);
    if (n_it > 0) ok = scale_a(0);
    for (int j = 0; j < n_it && ok; ++j) {
      const int it = j - lead;  // chunk of the sequence; < 0: lead-in, no output
      if (!NO_O && it >= 0) {
        const float* vs = vec + (j & 3) * VEC_SLOT_FLOATS;
        // the epilogue of the chunk before first: the issuing thread needs its accumulators free
        // (O_FREE) for this chunk's first output product
        if (it > 0) {
          ok = WAIT(O_DONE, (it - 1) & 1);
          if (!ok) break;
          tc_fence_after();
          epilogue(it - 1);
        }
        ok = WAIT(FULL0 + (j & 1), (j >> 1) & 1) && WAIT(P_DONE, it & 1);
        if (!ok) break;
        tc_fence_after();
        // Pg = s P exp(g_row - g_col) = P exp2((g_row - g_col) log2e + log2 s), col <= row
        {
          const float ga2 = vs[V_G * CHUNK + row_a] * 1.4426950408889634f + log2_scale;
          const float gb2 = vs[V_G * CHUNK + row_b] * 1.4426950408889634f + log2_scale;
          float x[32];
          tmem_ld_16x64(tmem + lanes_p + TM_PW, x);
          tmem_ld_wait();
          tc_fence_before();
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
        mbar_arrive(&bars[P_READY]);
      }
      if (j + 1 < n_it) ok = scale_a(j + 1);
    }
    if constexpr (!NO_O) {
      const int n_out = n_it - lead;  // chunks with output
      if (ok && n_out > 0) {
        ok = WAIT(O_DONE, (n_out - 1) & 1);
        if (ok) {
          tc_fence_after();
          epilogue(n_out - 1);
        }
      }
      if (v == 0) tma_store_wait_all();
      // rows of o past the end of the last packed sequence come out zero
      if (p.o && p.lay.cu.ptr && n == p.N - 1) {
        const long long end = sp.bos + sp.len;
        for (long long i = tid - 384; i < (p.T_rows - end) * 16; i += 128)
          *reinterpret_cast<uint4*>(p.o + ((end + (i >> 4)) * p.Hv + hv) * D + (i & 15) * 8) =
              make_uint4(0, 0, 0, 0);
      }
    }
  } else if (warp == 0 || warp == 1) {
    // =============================== MMA issuers ===============================
    // Two threads issue, each with its own waits and its own tcgen05.commit (a commit covers the
    // MMAs of the committing thread only):
    //   warp 0, the chain: Vn^T and the state update, nothing else: twelve MMAs per chunk;
    //   warp 1, everything off the chain: P, O1^T, O2^T and u^T / w^T of the next chunk.  It is the
    //           one that waits for the output group, so the chain never stands behind an epilogue.
    // The tensor pipe runs products in issue order whoever issued them; the extra barriers
    // (SB_FREE, the O_DONE wait of the value group) cover what one thread's program order would.
    constexpr uint32_t ID_P = idesc_bf16(64, 64, 0, 0);
    constexpr uint32_t ID_UT = idesc_bf16(128, 64, 1, 0);            // A = V / K tile, MN-major
    constexpr uint32_t ID_VN = idesc_bf16(128, 64, 0, 1) | (1u << 13);  // A negated; B = w^T tile
    constexpr uint32_t ID_OT = idesc_bf16(128, 64, 0, 0);            // A from tensor memory
    constexpr uint32_t ID_S = idesc_bf16(128, 128, 0, 1);
    constexpr uint32_t STAGE_LO = STAGE_BYTES >> 4;
    if (warp == 0 && lane == 0) {
      auto SPIN = [&](int idx, uint32_t parity) { return mbar_wait_spin(&bars[idx], parity, abort_flag); };
      // low descriptor words of every operand tile (see umma_lo); steps are 32-bit adds
      const uint32_t wmn_lo = desc_lo_mnmajor(smem + OFF_W, 16384);
      const uint32_t kmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + TILE_QK, 8192);
      auto store_vn = [&](int it) {  // after VN_READY: the v_new^T tile is complete
        tma_store_2d(&map_vn, 0, (int)(((sp.chunk_base + (it - lead)) * p.Hv + hv) * D), smem + OFF_VNT);
        tma_store_commit();
      };
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1, c = it - lead;  // c < 0: lead-in chunk
        const uint32_t so = s ? STAGE_LO : 0u;
        FQLA_TRACE(3, 0);
        if (it < 126) FQLA_CHUNK_CLOCK(it);
        ok = SPIN(S_COPY, it & 1) && SPIN(W_READY, it & 1);
        if (!ok) break;
        tc_fence_after();
        FQLA_TRACE(3, 1);
        // Vn^T = u^T - S^T w^T   (accumulates onto u^T; A = packed S^T in tensor memory)
        umma_ts_group<8, 8, 128, true>(tmem + TM_UV, tmem + TM_SB, wmn_lo, ID_VN);
        if constexpr (EXTRA) tma_store_wait_read();  // v_new^T of the chunk before has left its tile
        umma_commit(&bars[VN_DONE]);
        FQLA_TRACE(3, 2);
        if constexpr (EXTRA) {
          if (tile_h && c >= 0) {  // the state entering this chunk, as an operand tile
            ok = WAIT(ST_READY, c & 1);
            if (!ok) break;
            const int y = (int)(((sp.chunk_base + c) * p.Hv + hv) * D);
            tma_store_2d(&map_h, 0, y, smem + OFF_ST);
            tma_store_2d(&map_h, 64, y, smem + OFF_ST + 16384);
            tma_store_commit();
          }
        }
        FQLA_TRACE(3, 3);
        ok = SPIN(VB_READY, it & 1) && SPIN(S_DEC, it & 1);
        if (!ok) break;
        tc_fence_after();
        FQLA_TRACE(3, 4);
        // S^T += (rho Vn)^T K      (A = packed rho Vn^T; B = K tile read MN-major)
        umma_ts_group<4, 8, 128, true>(tmem + TM_S, tmem + TM_VRB, kmn0_lo + so, ID_S);
        if constexpr (EXTRA) tma_store_wait_read();  // the S^T tile may be rewritten after this
        umma_commit(&bars[S_DONE]);
        umma_commit(&bars[EMPTY0 + s]);  // this thread's last product that reads the stage
        FQLA_TRACE(3, 5);
        if constexpr (EXTRA) {
          if (tile_vn && c >= 0) {
            ok = WAIT(VN_READY, c & 1);
            if (!ok) break;
            store_vn(it);
          }
        }
        FQLA_TRACE(3, 8);
      }
      if constexpr (EXTRA) tma_store_wait_all();
    } else if (warp == 1 && lane == 0) {
      const uint32_t p_lo = desc_lo_kmajor(smem + OFF_P);
      const uint32_t q0_lo = desc_lo_kmajor(smem + OFF_STAGE);
      const uint32_t k0_lo = desc_lo_kmajor(smem + OFF_STAGE + TILE_QK);
      const uint32_t ap_lo = desc_lo_kmajor(smem + OFF_AP), app_lo = desc_lo_kmajor(smem + OFF_APP);
      const uint32_t kmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + TILE_QK, 8192);
      const uint32_t vmn0_lo = desc_lo_mnmajor(smem + OFF_STAGE + 2 * TILE_QK, 8192);
      auto issue_u_w = [&](uint32_t so) {  // so = stage offset in descriptor units
        umma_group<4, 128, 0, 2, 0, false>(tmem + TM_UV, vmn0_lo + so, ap_lo, ID_UT);
        umma_group<4, 128, 0, 2, 0, false>(tmem + TM_PW, kmn0_lo + so, app_lo, ID_UT);
        umma_commit(&bars[W_DONE]);
      };
      if (n_it > 0) {
        ok = WAIT(FULL0, 0) && WAIT(AP_READY, 0);
        if (ok) {
          tc_fence_after();
          issue_u_w(0);
        }
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it & 1, c = it - lead;
        const uint32_t so = s ? STAGE_LO : 0u, so_next = s ? 0u : STAGE_LO;
        const bool with_o = !NO_O && c >= 0;
        if (with_o) {
          // P = Q K^T goes first: the output group turns it into Pg while everything else runs.
          // Its columns held w^T of this chunk until the value group made the operand tile of it.
          ok = WAIT(W_READY, it & 1);
          if (!ok) break;
          tc_fence_after();
          umma_group<8, 2, 512, 2, 512, false>(tmem + TM_PW, q0_lo + so, k0_lo + so, ID_P);
          umma_commit(&bars[P_DONE]);
          // O1^T = S^T Q^T   (A = packed S^T; B = q tile, K-major)
          ok = WAIT(S_COPY, it & 1) && (c == 0 || WAIT(O_FREE, (c - 1) & 1));
          if (!ok) break;
          tc_fence_after();
          umma_ts_group_kmajor_b<8>(tmem + TM_O1, tmem + TM_SB, q0_lo + so, ID_OT);
          umma_commit(&bars[SB_FREE]);
        }
        // this thread's products that read the stage (u^T, w^T of this chunk, issued a chunk ago,
        // and the two above) are all issued
        umma_commit(&bars[EMPTY0 + s]);
        if (with_o) {
          // O2^T = Vn^T Pg^T   (A = packed Vn^T; B = Pg, K-major)
          ok = WAIT(P_READY, c & 1) && WAIT(VB_READY, it & 1);
          if (!ok) break;
          tc_fence_after();
          umma_ts_group<4, 8, 2, false>(tmem + TM_O2, tmem + TM_VNB, p_lo, ID_OT);
          umma_commit(&bars[O_DONE]);
        }
        if (it + 1 < n_it) {
          // u^T and w^T of the next chunk: u^T overwrites Vn^T (read by the value group:
          // VB_READY), w^T overwrites P (read by the output group: P_READY above)
          ok = WAIT(FULL0 + (s ^ 1), ((it + 1) >> 1) & 1) && WAIT(AP_READY, (it + 1) & 1) &&
               WAIT(VB_READY, it & 1);
          if (!ok) break;
          tc_fence_after();
          issue_u_w(so_next);
        }
      }
    }
  } else if (warp == 2) {
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
  }

  // ---- teardown: everybody meets, then the allocating warp frees tensor memory
  if (!ok) *abort_flag = 1;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicCAS(&g_device_status, 0, 1);
  if (tid == 0) FQLA_CHUNK_CLOCK(127);
#ifdef FQLA_DIAGNOSTICS
  if (tid == 0 && blockIdx.x < 1024) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    g_cta_cycles[2 * blockIdx.x] = smid;
    g_cta_cycles[2 * blockIdx.x + 1] = clock64() - g_fwd_chunk_clock_entry;
  }
#endif
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
                  void* vnew, int tiled, const int* lead, const int* order, const int* run_mask,
                  int run_value, int N, int Hq, int Hv, long long T_rows, float scale,
                  SeqLayout lay, cudaStream_t st) {
  using namespace fwdtc;
  CUtensorMap mq, mk, mv, ma, mh, mvn, mo;
  int rc;
  // without q (recomputation of h and v_new for the backward pass) the state-only variant runs;
  // its q map is never used and only has to be a valid map
  if ((rc = make_map(&mq, q ? q : k, T_rows, (long long)Hq * D))) return rc;
  if ((rc = make_map(&mk, k, T_rows, (long long)Hq * D))) return rc;
  if ((rc = make_map(&mv, v, T_rows, (long long)Hv * D))) return rc;
  if ((rc = make_map(&ma, A, T_rows, (long long)Hv * CHUNK))) return rc;
  mh = mq;
  mvn = mq;
  mo = mq;
  if (o && (rc = make_map(&mo, o, T_rows, (long long)Hv * D))) return rc;
  if (tiled) {
    // an upper bound of the chunk count: the maps only have to cover what the kernel stores
    const long long max_chunks = (T_rows + CHUNK - 1) / CHUNK + N;
    if (h && (rc = make_tile_map(&mh, h, max_chunks * Hv * D, D, 128))) return rc;
    if (vnew && (rc = make_tile_map(&mvn, vnew, max_chunks * Hv * D, CHUNK, 128))) return rc;
  }
  FwdTcParams p;
  p.tiled = tiled;
  p.lead = lead;
  p.order = order;
  p.run_mask = run_mask;
  p.run_value = run_value;
  p.g = g; p.beta = beta; p.beta_is_f32 = beta_is_f32; p.h0 = h0; p.ht = ht;
  p.o = (bf16*)o; p.h = (bf16*)h; p.vnew = (bf16*)vnew;
  p.N = N; p.Hq = Hq; p.Hv = Hv; p.T_rows = T_rows; p.scale = scale; p.lay = lay;
  const bool extra = h != nullptr || vnew != nullptr;
  auto launch = [&](auto kernel, int smem_bytes) {
    int err = configure_smem((const void*)kernel, smem_bytes);
    if (err != 0) return err;
    kernel<<<(unsigned)(N * Hv), 512, smem_bytes, st>>>(p, mq, mk, mv, ma, mh, mvn, mo);
    return (int)cudaGetLastError();
  };
  if (!q && !o) return launch(fwd_tc_kernel<true, true>, SMEM_BYTES_EXTRA);  // recomputation of h, v_new
  if (extra) return launch(fwd_tc_kernel<true, false>, SMEM_BYTES_EXTRA);
  return launch(fwd_tc_kernel<false, false>, SMEM_BYTES);
}

}  // namespace fqla

#ifdef FQLA_DIAGNOSTICS
extern "C" int fqla_debug_fwd_trace(long long* out960) {
  return (int)cudaMemcpyFromSymbol(out960, fqla::g_fwd_trace, sizeof(long long) * 960);
}
extern "C" int fqla_debug_cta_cycles(long long* out2048, int trace_cta) {
  cudaMemcpyToSymbol(fqla::g_trace_cta, &trace_cta, sizeof(int));
  return (int)cudaMemcpyFromSymbol(out2048, fqla::g_cta_cycles, sizeof(long long) * 2048);
}
extern "C" int fqla_debug_fwd_chunk_clock(long long* out256) {
  return (int)cudaMemcpyFromSymbol(out256, fqla::g_fwd_chunk_clock, sizeof(long long) * 256);
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
