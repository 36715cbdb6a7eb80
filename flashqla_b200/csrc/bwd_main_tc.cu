// Chunk-parallel part of the gated-delta-rule backward on Blackwell tensor cores (K = V = 128).
//
// Same mathematics and same outputs as bwd_main.cu (the reference's tests/ref_gdr.py:427-600,
// evaluated by the reference kernels inside blackwell/fused_bwd.py:595-862).  Persistent CTAs
// (one per SM) walk the work items (chunk, value head).  All sixteen tile products are
// tcgen05.mma with M = 64 (rows = tokens) and fp32 accumulators in tensor memory; two M = 64
// accumulators share each column range (lanes +0 and +16 of every 32-lane quarter).
//
// Roles: warp 16 issues every product and every TMA load (one elected thread).  Warps 0-7 (chain
// group) read the 64-wide accumulators (16-lane shape) and write the intermediate operands (dw,
// ds, dA, T, dA3) back to shared memory as bf16 tiles; warps 8-15 (bulk group) do what is off the
// dependent chain: the h.dh sum, dq1 | dk1 (scaled in place in tensor memory), dv and the final
// dq | dk, read in the 32-lane shape with 16-byte shared and global accesses.  The sides are
// coupled by one mbarrier per product group (commit -> read-out) and one per operand tile
// (written -> may be multiplied), so that the chain
//     dw -> dA -> T = A^T dA -> dA3 -> (beta dA3) K, (beta dA3)^T K
// never waits for the bulk work.  Row scalings ride on operands where they can (A diag(beta),
// A diag(beta gamma) are written over the dead v tile; dk is one accumulator fed by four
// products).  Operand tiles of the next item are fetched as soon as the buffers of the current
// one are dead (k has two buffers).
#include <cuda.h>

#include "common.cuh"
#include "fqla_internal.h"
#include <mutex>

#include "tc05.cuh"

namespace fqla {

using namespace tc;

// set to 1 when a CTA of this file's kernel abandoned a bounded wait; read through
// fqla_device_status together with the forward kernel's word
__device__ int g_bwd_main_status = 0;

struct BwdMainTcParams {
  const float* g;
  const void* beta;
  int beta_is_f32;
  bf16* dq;
  bf16* dk;
  bf16* dv;
  float* db;
  float* dg;
  int Hq, Hv;
  float scale;
  SeqLayout lay;
  IndexTable chunk_indices;
  long long n_chunks;
};

namespace bmtc {
constexpr int D = 128;
constexpr int N_EPI = 512;       // read-out threads: 16 warps = 4 lane quarters x 4 column quarters
constexpr int NT = N_EPI + 32;   // + the issue warp
constexpr int ROW_TILE = 16384;  // [64 x 128] bf16 as two 64-column blocks
constexpr int SQ_TILE = 32768;   // [128 x 128] bf16 as two 64-column blocks of 128 rows
constexpr int OFF_Q = 0, OFF_K = OFF_Q + ROW_TILE;  // k: two buffers
constexpr int OFF_V = OFF_K + 2 * ROW_TILE;
constexpr int OFF_VN = OFF_V + ROW_TILE, OFF_DO = OFF_VN + ROW_TILE, OFF_DU = OFF_DO + ROW_TILE;
constexpr int OFF_H = OFF_DU + ROW_TILE;
constexpr int OFF_DH = OFF_H + SQ_TILE;
constexpr int OFF_A = OFF_DH + SQ_TILE;
constexpr int OFF_DS = OFF_A + 8192;        // ds, later diag(beta) dA3
constexpr int OFF_DA = OFF_DS + 8192;       // dA, then T = A^T dA, then dA3
constexpr int OFF_DW = OFF_DA + 8192;       // -du h^T
// g, gamma, rho, beta (64 floats each); per-warp partial sums of dg (rows: 4 column quarters x 64,
// columns: 4 lane quarters x 64), of db (rows 4 x 64, two column terms 4 x 64 each) and of the
// chunk total (16)
constexpr int OFF_VEC = OFF_DW + ROW_TILE;
constexpr int OFF_BAR = OFF_VEC + (4 * 64 + 5 * 256 + 512 + 16) * 4;
constexpr int N_BARS = 20;
constexpr int OFF_MISC = OFF_BAR + N_BARS * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;
// the operand tiles of one item arrive in three groups, in the order their buffers become free
constexpr uint32_t TX_A = 2 * SQ_TILE + 3 * ROW_TILE;  // h, dh, dO, v_new, k (other buffer)
constexpr uint32_t TX_B = 3 * ROW_TILE;                // du, q, v
constexpr uint32_t TX_C = 8192;                        // A
// tensor memory: (column, lane half) of every accumulator
constexpr uint32_t HI = 16u << 16;
constexpr uint32_t T_DQ1 = 0, T_DK1 = 0 + HI, T_DW = 256;   // dq1 | dk1 share columns (lane halves)
constexpr uint32_t T_DQ2 = 128, T_DK2 = 128 + HI;        // ds K | the four-product dk sum share columns
constexpr uint32_t T_T2 = 256 + HI, T_DS = 384 + HI, T_QK = 448 + HI;
constexpr uint32_t T_X1 = 256, T_X2 = 320;            // after dw has been read
constexpr uint32_t T_T = 384 + HI, T_KK = 448 + HI;    // after ds, qk have been read
constexpr uint32_t T_D3 = 256;                         // after x1 has been read
enum {
  L_A = 0, L_B, L_C,                                       // TMA groups landed
  C_DW, C_DSQK, C_1B, C_X, C_2B, C_T, C_D3, C_5,           // product groups complete (commit)
  R_ZERO, R_END,                     // all 16 read-out warps -> issue warp
  R_DW, R_DS, R_DA, R_T, R_D3,       // the 8 warps of the chain group -> issue warp
  R_HD, R_E4                         // the 8 warps of the bulk group -> issue warp
};
}  // namespace bmtc

// 16 lanes x 32 (x4) or 16 (x2) columns: register 4i+e of lane l holds row l/4 + 8*(e>>1),
// column 8i + 2(l%4) + (e&1)
__device__ __forceinline__ void tmem_ld_16x32(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_16x16(uint32_t taddr, float (&v)[8]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void epi_barrier() {  // the 16 read-out warps only
  asm volatile("bar.sync 1, 512;" ::: "memory");
}

// Persistent: CTA b handles work items b, b + gridDim.x, ...; item w = (chunk w / Hv, head w % Hv),
// so neighbouring CTAs share q and k of a grouped-value-attention group through L2.
// TILED: h, dh, vnew and du arrive in the operand layouts written by the sequential kernels
// (h^T, dh^T as [V][K] per chunk; vnew^T, du^T as [V][64] per chunk) instead of row-major.
template <bool TILED>
__global__ void __launch_bounds__(bmtc::NT, 1)
bwd_main_tc_kernel(const BwdMainTcParams p, const __grid_constant__ CUtensorMap map_q,
                   const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const __grid_constant__ CUtensorMap map_vn, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_du, const __grid_constant__ CUtensorMap map_h,
                   const __grid_constant__ CUtensorMap map_dh, const __grid_constant__ CUtensorMap map_a) {
  using namespace bmtc;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);
  volatile int* stop_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 8);  // [2], by item parity
  // per-row vectors g, gamma, rho, beta of an item: two buffers (item parity), the second one
  // behind the column sums
  float* sVec0 = reinterpret_cast<float*>(smem + OFF_VEC);
  float* sRowDg = sVec0 + 256;
  float* sColDg = sRowDg + 256;
  float* sRowDb = sColDg + 256;
  float* sColC1 = sRowDb + 256;
  float* sVec1 = sColC1 + 256;
  float* sRowW = sVec1 + 256;  // row terms of the 128-wide steps: [column quarter x lane half][row]
  float* sLast = sRowW + 512;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long total = p.n_chunks * p.Hv;

  struct Item {
    long long row0, chunk_id;
    int valid, hv, hq;
  };
  auto decode = [&](long long w) {
    Item t;
    const long long cidx = w / p.Hv;
    t.hv = (int)(w % p.Hv);
    t.hq = t.hv / (p.Hv / p.Hq);
    int seq, ci;
    if (p.lay.cu.ptr) {
      seq = (int)p.chunk_indices[2 * cidx];
      ci = (int)p.chunk_indices[2 * cidx + 1];
    } else {
      const int per = (p.lay.T + CHUNK - 1) / CHUNK;
      seq = (int)(cidx / per);
      ci = (int)(cidx % per);
    }
    const SeqSpan sp = p.lay.span(seq);
    t.row0 = sp.bos + (long long)ci * CHUNK;
    // clamped: a table row that does not belong to its sequence must not index outside the tiles
    t.valid = max(1, min(CHUNK, sp.len - ci * CHUNK));
    t.chunk_id = sp.chunk_base + ci;
    return t;
  };

  if (tid == 0) {
    for (int i = L_A; i <= C_5; ++i) mbar_init(&bars[i], 1);
    mbar_init(&bars[R_ZERO], N_EPI / 32);
    mbar_init(&bars[R_END], N_EPI / 32);
    for (int i = R_DW; i <= R_E4; ++i) mbar_init(&bars[i], N_EPI / 64);
    *abort_flag = 0;
    stop_flag[0] = 0;
    stop_flag[1] = 0;
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  auto WAIT = [&](int idx, uint32_t parity) { return mbar_wait(&bars[idx], parity, abort_flag); };

  if (warp == N_EPI / 32) {
    // ====================== issue warp: TMA loads and every tcgen05.mma ======================
    if (lane == 0) {
      auto load_a = [&](const Item& t, int kbuf) {
        const int y = (int)t.row0, ys = (int)((t.chunk_id * p.Hv + t.hv) * D);
        mbar_arrive_expect_tx(&bars[L_A], TX_A);
        tma_load_2d(smem + OFF_DU - ROW_TILE, &map_do, t.hv * D, y, &bars[L_A]);  // = OFF_DO
        tma_load_2d(smem + OFF_DO + 8192, &map_do, t.hv * D + 64, y, &bars[L_A]);
        tma_load_2d(smem + OFF_H, &map_h, 0, ys, &bars[L_A]);
        tma_load_2d(smem + OFF_H + 16384, &map_h, 64, ys, &bars[L_A]);
        if constexpr (TILED) {
          tma_load_2d(smem + OFF_VN, &map_vn, 0, ys, &bars[L_A]);
        } else {
          tma_load_2d(smem + OFF_VN, &map_vn, t.hv * D, y, &bars[L_A]);
          tma_load_2d(smem + OFF_VN + 8192, &map_vn, t.hv * D + 64, y, &bars[L_A]);
        }
        tma_load_2d(smem + OFF_K + kbuf * ROW_TILE, &map_k, t.hq * D, y, &bars[L_A]);
        tma_load_2d(smem + OFF_K + kbuf * ROW_TILE + 8192, &map_k, t.hq * D + 64, y, &bars[L_A]);
        tma_load_2d(smem + OFF_DH, &map_dh, 0, ys, &bars[L_A]);
        tma_load_2d(smem + OFF_DH + 16384, &map_dh, 64, ys, &bars[L_A]);
      };
      auto load_b = [&](const Item& t) {
        const int y = (int)t.row0;
        mbar_arrive_expect_tx(&bars[L_B], TX_B);
        if constexpr (TILED) {
          tma_load_2d(smem + OFF_DU, &map_du, 0, (int)((t.chunk_id * p.Hv + t.hv) * D), &bars[L_B]);
        } else {
          tma_load_2d(smem + OFF_DU, &map_du, t.hv * D, y, &bars[L_B]);
          tma_load_2d(smem + OFF_DU + 8192, &map_du, t.hv * D + 64, y, &bars[L_B]);
        }
        tma_load_2d(smem + OFF_Q, &map_q, t.hq * D, y, &bars[L_B]);
        tma_load_2d(smem + OFF_Q + 8192, &map_q, t.hq * D + 64, y, &bars[L_B]);
        tma_load_2d(smem + OFF_V, &map_v, t.hv * D, y, &bars[L_B]);
        tma_load_2d(smem + OFF_V + 8192, &map_v, t.hv * D + 64, y, &bars[L_B]);
      };
      auto load_c = [&](const Item& t) {
        mbar_arrive_expect_tx(&bars[L_C], TX_C);
        tma_load_2d(smem + OFF_A, &map_a, t.hv * CHUNK, (int)t.row0, &bars[L_C]);
      };
      // descriptors (low words)
      const uint32_t q_lo = desc_lo_kmajor(smem + OFF_Q), v_lo = desc_lo_kmajor(smem + OFF_V);
      const uint32_t k_lo0 = desc_lo_kmajor(smem + OFF_K), kmn_lo0 = desc_lo_mnmajor(smem + OFF_K, 8192);
      const uint32_t vn_lo = desc_lo_kmajor(smem + OFF_VN);
      const uint32_t do_lo = desc_lo_kmajor(smem + OFF_DO), du_lo = desc_lo_kmajor(smem + OFF_DU);
      const uint32_t h_lo = desc_lo_kmajor(smem + OFF_H), dh_lo = desc_lo_kmajor(smem + OFF_DH);
      const uint32_t a_lo = desc_lo_kmajor(smem + OFF_A), ds_lo = desc_lo_kmajor(smem + OFF_DS);
      const uint32_t da_lo = desc_lo_kmajor(smem + OFF_DA), dw_lo = desc_lo_kmajor(smem + OFF_DW);
      const uint32_t qmn_lo = desc_lo_mnmajor(smem + OFF_Q, 8192);
      const uint32_t dumn_lo = desc_lo_mnmajor(smem + OFF_DU, 8192), dwmn_lo = desc_lo_mnmajor(smem + OFF_DW, 8192);
      const uint32_t amn_lo = desc_lo_mnmajor(smem + OFF_A, 8192), dsmn_lo = desc_lo_mnmajor(smem + OFF_DS, 8192);
      const uint32_t damn_lo = desc_lo_mnmajor(smem + OFF_DA, 8192);
      const uint32_t a1mn_lo = desc_lo_mnmajor(smem + OFF_V, 8192), a2mn_lo = desc_lo_mnmajor(smem + OFF_V + 8192, 8192);
      // operand-tile layouts: [V rows][K or token columns], read MN-major, contraction over rows
      const uint32_t hT_lo = desc_lo_mnmajor(smem + OFF_H, 16384), dhT_lo = desc_lo_mnmajor(smem + OFF_DH, 16384);
      const uint32_t vnT_lo = desc_lo_mnmajor(smem + OFF_VN, 16384), duT_lo = desc_lo_mnmajor(smem + OFF_DU, 16384);
      constexpr uint32_t ID_KK_128 = idesc_bf16(64, 128, 0, 0), ID_KK_64 = idesc_bf16(64, 64, 0, 0);
      constexpr uint32_t ID_KM_128 = idesc_bf16(64, 128, 0, 1), ID_MM_128 = idesc_bf16(64, 128, 1, 1);
      constexpr uint32_t ID_MM_64 = idesc_bf16(64, 64, 1, 1);
      constexpr uint32_t ID_KM_64 = idesc_bf16(64, 64, 0, 1), ID_MK_64 = idesc_bf16(64, 64, 1, 0);
      constexpr uint32_t ID_MK_128 = idesc_bf16(64, 128, 1, 0);
      constexpr uint32_t KBUF_LO = ROW_TILE >> 4;

      Item cur = decode(blockIdx.x);
      load_a(cur, 0);
      load_b(cur);
      load_c(cur);
      bool ok = true;
      uint32_t it = 0;
#pragma unroll 1
      for (long long w = blockIdx.x; w < total && ok; w += gridDim.x, ++it) {
        const uint32_t ph = it & 1;
        const bool has_next = w + gridDim.x < total;
        Item nxt = cur;
        if (has_next) nxt = decode(w + gridDim.x);
        const uint32_t k_lo = k_lo0 + (ph ? KBUF_LO : 0u), kmn_lo = kmn_lo0 + (ph ? KBUF_LO : 0u);
        // the read-out warps have finished the previous item (accumulators free) and have zeroed
        // the rows past the sequence end in this item's tiles (which also means: tiles landed)
        // A full chunk needs no zero fill: its first products start as soon as its tiles have
        // landed, while the bulk group still finishes the previous item (the accumulators they
        // write were last read by the chain group, whose R_D3 this thread has seen; dq1 | dk1 come
        // after R_DW of this item, which the read-out warps only give after the previous item).
        if (cur.valid == CHUNK) ok = WAIT(L_A, ph) && WAIT(L_B, ph);
        else ok = (it == 0 || WAIT(R_END, (it - 1) & 1)) && WAIT(R_ZERO, ph);
        if (!ok) break;
        tc_fence_after();
        // ---- products that need only loaded tiles ----
        if constexpr (TILED) {
          umma_group<8, 128, 512, 128, 512, false>(tmem + T_DW, duT_lo, hT_lo, ID_MM_128);
        } else {
          umma_group<8, 2, 512, 2, 1024, false>(tmem + T_DW, du_lo, h_lo, ID_KK_128);
        }
        umma_commit(&bars[C_DW]);
        if constexpr (TILED) {
          umma_group<8, 2, 512, 128, 512, false>(tmem + T_DS, do_lo, vnT_lo, ID_KM_64);
        } else {
          umma_group<8, 2, 512, 2, 512, false>(tmem + T_DS, do_lo, vn_lo, ID_KK_64);
        }
        umma_group<8, 2, 512, 2, 512, false>(tmem + T_QK, q_lo, k_lo, ID_KK_64);
        umma_commit(&bars[C_DSQK]);
        // ---- dw is an operand now: the pieces of dA, and A^T dw, A^T du ----
        ok = WAIT(R_DW, ph);
        if (!ok) break;
        tc_fence_after();
        umma_group<8, 2, 512, 2, 512, false>(tmem + T_X1, dw_lo, k_lo, ID_KK_64);
        if constexpr (TILED) umma_group<8, 128, 512, 2, 512, false>(tmem + T_X2, duT_lo, v_lo, ID_MK_64);
        else umma_group<8, 2, 512, 2, 512, false>(tmem + T_X2, du_lo, v_lo, ID_KK_64);
        umma_commit(&bars[C_X]);
        // products off the dependent chain go behind the ones the read-out is waiting for
        if constexpr (TILED) {
          umma_group<8, 2, 512, 128, 512, false>(tmem + T_DQ1, do_lo, hT_lo, ID_KM_128);
          umma_group<8, 128, 512, 128, 512, false>(tmem + T_DK1, vnT_lo, dhT_lo, ID_MM_128);
        } else {
          umma_group<8, 2, 512, 2, 1024, false>(tmem + T_DQ1, do_lo, h_lo, ID_KK_128);
          umma_group<8, 2, 512, 2, 1024, false>(tmem + T_DK1, vn_lo, dh_lo, ID_KK_128);
        }
        umma_commit(&bars[C_1B]);
        // ---- ds is an operand now ----
        ok = WAIT(R_DS, ph);
        if (!ok) break;
        tc_fence_after();
        umma_group<4, 2, 0, 128, 0, false>(tmem + T_DQ2, ds_lo, kmn_lo, ID_KM_128);
        umma_group<4, 128, 0, 128, 0, false>(tmem + T_DK2, dsmn_lo, qmn_lo, ID_MM_128);
        umma_group<8, 2, 512, 2, 512, false>(tmem + T_KK, k_lo, k_lo, ID_KK_64);  // qk has been read
        // h, dh, dO, v_new are dead once the first products are complete and the h.dh sum is done
        if (has_next) {
          ok = WAIT(C_1B, ph) && WAIT(R_HD, ph);
          if (!ok) break;
          load_a(nxt, (int)(ph ^ 1));
        }
        // ---- dA -> T = A^T dA (and K K^T) ----
        ok = WAIT(R_DA, ph);
        if (!ok) break;
        tc_fence_after();
        umma_group<4, 128, 0, 128, 0, false>(tmem + T_T, amn_lo, damn_lo, ID_MM_64);
        umma_commit(&bars[C_T]);
        // with A' = A diag(beta) and A'' = A diag(beta gamma) (written over the dead v tile):
        // dk += A''^T dw (onto ds^T q), dv = A'^T du -- the row scalings ride on the operands
        umma_group<4, 128, 0, 128, 0, true>(tmem + T_DK2, a2mn_lo, dwmn_lo, ID_MM_128);
        if constexpr (TILED) umma_group<4, 128, 0, 2, 0, false>(tmem + T_T2, a1mn_lo, du_lo, ID_MK_128);
        else umma_group<4, 128, 0, 128, 0, false>(tmem + T_T2, a1mn_lo, dumn_lo, ID_MM_128);
        umma_commit(&bars[C_2B]);
        // ---- T -> d3 = T A^T ----
        ok = WAIT(R_T, ph);
        if (!ok) break;
        tc_fence_after();
        umma_group<4, 2, 0, 2, 0, false>(tmem + T_D3, da_lo, a_lo, ID_KK_64);
        umma_commit(&bars[C_D3]);
        // The bulk group is past its first read-out (always waited for: its threads combine the
        // partial sums of the previous item before that, and the last products of this item let
        // the group overwrite those sums).
        ok = WAIT(R_E4, ph);
        if (!ok) break;
        if (has_next) {
          // du, q, v are dead once their products are complete and the bulk group has used q
          ok = WAIT(C_2B, ph);
          if (!ok) break;
          load_b(nxt);
          ok = WAIT(C_D3, ph);  // last product that reads A
          if (!ok) break;
          load_c(nxt);
        }
        // ---- beta dA3 is an operand now ----
        ok = WAIT(R_D3, ph);
        if (!ok) break;
        tc_fence_after();
        // dk += (beta dA3) K + (beta dA3)^T K, onto the same accumulator
        umma_group<4, 2, 0, 128, 0, true>(tmem + T_DK2, ds_lo, kmn_lo, ID_KM_128);
        umma_group<4, 128, 0, 128, 0, true>(tmem + T_DK2, dsmn_lo, kmn_lo, ID_MM_128);
        umma_commit(&bars[C_5]);
        cur = nxt;
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ====================== read-out warps ======================
    // Two groups of eight warps.  The CHAIN group (warps 0-7) serves the dependent chain
    // dw -> dA -> T -> dA3 (plus ds, which it gets for free from the same kind of tile): it reads
    // the 64-wide accumulators in the 16-lane shape (lane l of warp (qd, half) owns rows
    // 16 qd + l/4 (+8), column pairs 32 half + 8 i + 2 (l%4)).  The BULK group (warps 8-15) does
    // everything that is off the chain: the h.dh sum, the scaling of dq1 | dk1 (written back to
    // tensor memory), dv, and the final dq | dk.  It reads the 128-wide accumulators in the
    // 32-lane shape, which returns the accumulator at lanes +0 and the one at lanes +16 of the
    // same columns at once: lane l owns row 16 qd + l%16 of the lower (l < 16) or upper one, 32
    // consecutive columns per pass; shared and global memory are touched 16 bytes at a time.
    const bool chain = warp < 8;
    const int gw = warp & 7, qd = gw & 3, half = gw >> 2;
    const int row_a = 16 * qd + (lane >> 2), row_b = row_a + 8, cp = 2 * (lane & 3);
    const int row_w = 16 * qd + (lane & 15);
    const bool hi = lane >= 16;
    const uint32_t lanes = (uint32_t)(qd * 32) << 16;
    const int c64 = 32 * half;    // first column of this warp in 64-wide tiles (chain group)
    const int c128 = 64 * half;   // first column of this warp in 128-wide tiles
    // byte offset of this thread's 16-byte piece (pass, j) (8 columns) inside a [64 x 128] row tile
    const int piece_base = half * 8192 + row_w * 128;
    auto piece = [&](int pass, int j) { return piece_base + (((4 * pass + j) ^ (row_w & 7)) << 4); };
    auto quad_sum = [&](float x) {
      x += __shfl_xor_sync(0xffffffffu, x, 1);
      x += __shfl_xor_sync(0xffffffffu, x, 2);
      return x;
    };
    auto col_sum = [&](float x) {
      x += __shfl_xor_sync(0xffffffffu, x, 4);
      x += __shfl_xor_sync(0xffffffffu, x, 8);
      x += __shfl_xor_sync(0xffffffffu, x, 16);
      return x;
    };
    auto st_tile64 = [&](int off, int row, int col, float lo, float hi2) {
      *reinterpret_cast<uint32_t*>(smem + off + sw128_offset(row, col)) = pack_bf16(lo, hi2);
    };
    auto pack8 = [&](const float* x) {
      return make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
    };
    // 32 consecutive columns of this thread's output row (x, fp32) go out as bf16. A thread owns a
    // row, so a plain 16-byte store per thread would touch 32 lines per instruction; the four
    // lanes of a quad first exchange their 16-byte pieces (a 4 x 4 transpose, two butterfly
    // steps), after which each store instruction writes 64 contiguous bytes of 8 rows.
    // base = offset of the row of lane 0 of the quad (+ the 32-column block), row_q = that row.
    auto store_rows = [&](bf16* out, long long base, int row_q, int valid_rows, const float* x) {  // whole warp
      uint4 pc[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) pc[j] = pack8(x + 8 * j);
      const bool b0 = lane & 1, b1 = lane & 2;
      auto xchg = [&](uint4& keep_if0, uint4& keep_if1, bool bit, int mask) {
        // lanes with bit clear keep keep_if0 and send keep_if1; lanes with bit set the reverse
        uint4 snd = bit ? keep_if0 : keep_if1, rcv;
        rcv.x = __shfl_xor_sync(0xffffffffu, snd.x, mask);
        rcv.y = __shfl_xor_sync(0xffffffffu, snd.y, mask);
        rcv.z = __shfl_xor_sync(0xffffffffu, snd.z, mask);
        rcv.w = __shfl_xor_sync(0xffffffffu, snd.w, mask);
        if (bit) keep_if0 = rcv; else keep_if1 = rcv;
      };
      xchg(pc[0], pc[1], b0, 1);
      xchg(pc[2], pc[3], b0, 1);
      xchg(pc[0], pc[2], b1, 2);
      xchg(pc[1], pc[3], b1, 2);
      // pc[j] now holds piece (lane & 3) of row row_q + j
      const long long pitch = (long long)p.Hv * D;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (row_q + j < valid_rows)
          *reinterpret_cast<uint4*>(out + base + j * pitch + 8 * (lane & 3)) = pc[j];
    };
    // this warp's part of a tile (or of the accumulators) is done: tell the issue warp
    auto signal = [&](int bar) {
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars[bar]);
    };
    auto zero_rows = [&](int off, int n_blocks, int valid) {
      for (int blk = 0; blk < n_blocks; ++blk) {
        unsigned char* base = smem + off + blk * 8192;
        for (int i = tid; i < (CHUNK - valid) * 8; i += N_EPI)
          *reinterpret_cast<uint4*>(base + (valid + (i >> 3)) * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
      }
    };
    // The vectors of the next item are fetched a whole item ahead.  beta stays in its raw form
    // until it is used: a conversion right behind the load would make the thread wait for it.
    float pre_g = 0.f, pre_gl = 0.f;
    uint32_t pre_beta_raw = 0;
    auto fetch_vectors = [&](const Item& t) {
      if (tid < CHUNK) {
        const int r = min(tid, t.valid - 1);
        const long long i = (t.row0 + r) * p.Hv + t.hv;
        pre_g = p.g[i];
        pre_gl = p.g[(t.row0 + t.valid - 1) * p.Hv + t.hv];
        pre_beta_raw = p.beta_is_f32 ? reinterpret_cast<const uint32_t*>(p.beta)[i]
                                     : (uint32_t)reinterpret_cast<const unsigned short*>(p.beta)[i];
      }
    };
    // the fetched vectors of item t go to buffer `buf` (threads 0..63; published by a barrier)
    auto write_vectors = [&](const Item& t, float* buf) {
      if (tid < CHUNK) {
        buf[tid] = pre_g;
        buf[64 + tid] = fast_exp(pre_g);
        buf[128 + tid] = fast_exp(pre_gl - pre_g);
        buf[192 + tid] =
            tid < t.valid ? __uint_as_float(p.beta_is_f32 ? pre_beta_raw : pre_beta_raw << 16) : 0.f;
      }
    };
    // dg, db of a finished item from the partial sums in shared memory (threads 256..319, which
    // would otherwise idle until the first wide products are complete)
    auto combine = [&](long long first, int n_rows) {  // first = row0 * Hv + hv of the item
      const int r = tid - N_EPI / 2;
      if (r >= 0 && r < n_rows) {
        float dgv = 0.f, dbv = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          dgv += sRowW[j * 64 + r] - sColDg[j * 64 + r];
          dbv += sColC1[j * 64 + r];
        }
        dgv += sRowDg[r] + sRowDg[64 + r];
        dbv += sRowDb[r] + sRowDb[64 + r];
        if (r == n_rows - 1) {
#pragma unroll
          for (int j = 0; j < 8; ++j) dgv += sLast[j];
        }
        p.dg[first + (long long)r * p.Hv] = dgv;
        p.db[first + (long long)r * p.Hv] = dbv;
      }
    };
    Item cur = decode(blockIdx.x);
    long long prev_first = 0;
    int prev_rows = 0;
    fetch_vectors(cur);
    write_vectors(cur, sVec0);
    epi_barrier();
    uint32_t it = 0;
    bool stopped = false;
#pragma unroll 1
    for (long long w = blockIdx.x; w < total; w += gridDim.x, ++it) {
      const uint32_t ph = it & 1;
      const bool has_next = w + gridDim.x < total;
      Item nxt = cur;
      if (has_next) nxt = decode(w + gridDim.x);
      const int valid = cur.valid;
      const int koff = OFF_K + (int)ph * ROW_TILE;
      const float* sG = ph ? sVec1 : sVec0;
      const float *sGam = sG + 64, *sRho = sG + 128, *sBeta = sG + 192;
      bool ok = WAIT(L_A, ph) && WAIT(L_B, ph) && WAIT(L_C, ph);
      if (ok && valid < CHUNK) {
        zero_rows(OFF_Q, 2, valid);
        zero_rows(koff, 2, valid);
        zero_rows(OFF_A, 1, valid);
        if constexpr (TILED) {  // the transposed tiles already hold zeros past the sequence end
          zero_rows(OFF_V, 2, valid);
          zero_rows(OFF_DO, 2, valid);
        } else {
          zero_rows(OFF_V, 8, valid);  // v, v_new, dO, du
        }
      }
      signal(R_ZERO);
      if (has_next) fetch_vectors(nxt);
      float acc_last = 0.f;

      if (chain) {
        // ===================== chain group =====================
        const float g_a = sG[row_a], g_b = sG[row_b];
        const float beta_a = sBeta[row_a], beta_b = sBeta[row_b];
        // row sums (dg, db) and column sums (dg; the two column terms that come from A^T dw and
        // A^T du) of this thread; reduced across lanes once, at the end of the item
        float acc_dg_a = 0.f, acc_dg_b = 0.f, acc_db_a = 0.f, acc_db_b = 0.f;
        float acc_col[8], acc_dbc[8];  // per column: dg terms (to subtract), db terms
#pragma unroll
        for (int j = 0; j < 8; ++j) acc_col[j] = acc_dbc[j] = 0.f;

        // ---- E1: dw = -du h^T as an operand tile (lower lanes of the 32-lane shape) ----
        ok = ok && WAIT(C_DW, ph);
        if (ok) {
          tc_fence_after();
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            float x[32];
            tmem_ld32(tmem + lanes + T_DW + c128 + 32 * pass, x);
            tmem_ld_wait();
            if (!hi) {
#pragma unroll
              for (int j = 0; j < 32; ++j) x[j] = -x[j];
#pragma unroll
              for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(smem + OFF_DW + piece(pass, j)) = pack8(x + 8 * j);
            }
          }
        }
        signal(R_DW);

        // ---- E2: ds = scale * G * (dO Vn^T); ds2 = ds * (Q K^T) ----
        ok = ok && WAIT(C_DSQK, ph);
        if (ok) {
          tc_fence_after();
          float ds[16], qk[16];
          tmem_ld_16x32(tmem + lanes + T_DS + c64, ds);
          tmem_ld_16x32(tmem + lanes + T_QK + c64, qk);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = c64 + 8 * i + cp;
            const float gc0 = sG[col], gc1 = sG[col + 1];
            const float a0 = col <= row_a ? p.scale * ds[4 * i] * fast_exp(g_a - gc0) : 0.f;
            const float a1 = col + 1 <= row_a ? p.scale * ds[4 * i + 1] * fast_exp(g_a - gc1) : 0.f;
            const float b0 = col <= row_b ? p.scale * ds[4 * i + 2] * fast_exp(g_b - gc0) : 0.f;
            const float b1 = col + 1 <= row_b ? p.scale * ds[4 * i + 3] * fast_exp(g_b - gc1) : 0.f;
            st_tile64(OFF_DS, row_a, col, a0, a1);
            st_tile64(OFF_DS, row_b, col, b0, b1);
            const float s0 = a0 * qk[4 * i], s1 = a1 * qk[4 * i + 1], s2 = b0 * qk[4 * i + 2], s3 = b1 * qk[4 * i + 3];
            acc_dg_a += s0 + s1;
            acc_dg_b += s2 + s3;
            acc_col[2 * i] += s0 + s2;
            acc_col[2 * i + 1] += s1 + s3;
          }
        }
        signal(R_DS);

        // ---- E3: dA = strict_lower(beta_c (gamma_c x1 + x2)); A' = A diag(beta), A'' = A diag(beta gamma) ----
        ok = ok && WAIT(C_X, ph);
        if (ok) {
          tc_fence_after();
          float x1[16], x2[16];
          tmem_ld_16x32(tmem + lanes + T_X1 + c64, x1);
          tmem_ld_16x32(tmem + lanes + T_X2 + c64, x2);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = c64 + 8 * i + cp;
            const float b0 = sBeta[col], b1 = sBeta[col + 1], g0 = sGam[col], g1 = sGam[col + 1];
            st_tile64(OFF_DA, row_a, col, col < row_a ? b0 * (g0 * x1[4 * i] + x2[4 * i]) : 0.f,
                      col + 1 < row_a ? b1 * (g1 * x1[4 * i + 1] + x2[4 * i + 1]) : 0.f);
            st_tile64(OFF_DA, row_b, col, col < row_b ? b0 * (g0 * x1[4 * i + 2] + x2[4 * i + 2]) : 0.f,
                      col + 1 < row_b ? b1 * (g1 * x1[4 * i + 3] + x2[4 * i + 3]) : 0.f);
            // rowsum((A^T dw) k)[r] = sum_s A[s][r] x1[s][r], rowsum((A^T du) v)[r] = sum_s A[s][r] x2[s][r]
            const float2 A_a = ld_bf16x2(reinterpret_cast<const bf16*>(smem + OFF_A + sw128_offset(row_a, col)));
            const float2 A_b = ld_bf16x2(reinterpret_cast<const bf16*>(smem + OFF_A + sw128_offset(row_b, col)));
            // column r: db += gamma_r c1 + c2, dg += beta_r gamma_r c1 (entered with a minus sign
            // into the column sums, which the final step subtracts)
            const float c1a = A_a.x * x1[4 * i] + A_b.x * x1[4 * i + 2];
            const float c1b = A_a.y * x1[4 * i + 1] + A_b.y * x1[4 * i + 3];
            acc_dbc[2 * i] += g0 * c1a + A_a.x * x2[4 * i] + A_b.x * x2[4 * i + 2];
            acc_dbc[2 * i + 1] += g1 * c1b + A_a.y * x2[4 * i + 1] + A_b.y * x2[4 * i + 3];
            acc_col[2 * i] -= b0 * g0 * c1a;
            acc_col[2 * i + 1] -= b1 * g1 * c1b;
            // the v tile is dead (its product is part of this group): A' and A'' go there
            st_tile64(OFF_V, row_a, col, A_a.x * b0, A_a.y * b1);
            st_tile64(OFF_V, row_b, col, A_b.x * b0, A_b.y * b1);
            st_tile64(OFF_V + 8192, row_a, col, A_a.x * b0 * g0, A_a.y * b1 * g1);
            st_tile64(OFF_V + 8192, row_b, col, A_b.x * b0 * g0, A_b.y * b1 * g1);
          }
        }
        signal(R_DA);

        // ---- E5: T = A^T dA as an operand tile (over dA, which the product has consumed) ----
        ok = ok && WAIT(C_T, ph);
        if (ok) {
          tc_fence_after();
          float t[16];
          tmem_ld_16x32(tmem + lanes + T_T + c64, t);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = c64 + 8 * i + cp;
            st_tile64(OFF_DA, row_a, col, t[4 * i], t[4 * i + 1]);
            st_tile64(OFF_DA, row_b, col, t[4 * i + 2], t[4 * i + 3]);
          }
        }
        signal(R_T);

        // ---- E7: beta dA3 = -beta G d3 (over ds) as an operand tile; its dg and db terms ----
        ok = ok && WAIT(C_D3, ph);
        if (ok) {
          tc_fence_after();
          float d3[16], kk[16];
          tmem_ld_16x32(tmem + lanes + T_D3 + c64, d3);
          tmem_ld_16x32(tmem + lanes + T_KK + c64, kk);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = c64 + 8 * i + cp;
            const float gc0 = sG[col], gc1 = sG[col + 1];
            const float a0 = col < row_a ? -d3[4 * i] * fast_exp(g_a - gc0) : 0.f;
            const float a1 = col + 1 < row_a ? -d3[4 * i + 1] * fast_exp(g_a - gc1) : 0.f;
            const float b0 = col < row_b ? -d3[4 * i + 2] * fast_exp(g_b - gc0) : 0.f;
            const float b1 = col + 1 < row_b ? -d3[4 * i + 3] * fast_exp(g_b - gc1) : 0.f;
            st_tile64(OFF_DS, row_a, col, beta_a * a0, beta_a * a1);
            st_tile64(OFF_DS, row_b, col, beta_b * b0, beta_b * b1);
            // db += rowsum((dA3 K) k) = rowsum(dA3 * (K K^T)); the dg terms carry the beta factor
            const float u0 = a0 * kk[4 * i], u1 = a1 * kk[4 * i + 1], u2 = b0 * kk[4 * i + 2], u3 = b1 * kk[4 * i + 3];
            acc_db_a += u0 + u1;
            acc_db_b += u2 + u3;
            const float s0 = u0 * beta_a, s1 = u1 * beta_a, s2 = u2 * beta_b, s3 = u3 * beta_b;
            acc_dg_a += s0 + s1;
            acc_dg_b += s2 + s3;
            acc_col[2 * i] += s0 + s2;
            acc_col[2 * i + 1] += s1 + s3;
          }
        }
        signal(R_D3);
        signal(R_END);  // this group no longer touches the accumulators or the tiles of the item
        // The partial-sum slots were read for the previous item by threads of the bulk group, which
        // arrive on R_E4 of this item only after that: long complete by now.
        ok = ok && WAIT(R_E4, ph);
        // one reduction per quantity, one plain store per (warp, row or column): no atomics
        acc_dg_a = quad_sum(acc_dg_a);
        acc_dg_b = quad_sum(acc_dg_b);
        acc_db_a = quad_sum(acc_db_a);
        acc_db_b = quad_sum(acc_db_b);
        if ((lane & 3) == 0) {
          sRowDg[half * 64 + row_a] = acc_dg_a;
          sRowDg[half * 64 + row_b] = acc_dg_b;
          sRowDb[half * 64 + row_a] = acc_db_a;
          sRowDb[half * 64 + row_b] = acc_db_b;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float c = col_sum(acc_col[j]);
          const float c1 = col_sum(acc_dbc[j]);
          if (lane < 4) {
            const int col = c64 + 8 * (j >> 1) + cp + (j & 1);
            sColDg[qd * 64 + col] = c;
            sColC1[qd * 64 + col] = c1;
          }
        }
      } else {
        // ===================== bulk group =====================
        // gamma_last * sum(h * dh) over the whole 128 x 128 tiles (plain shared-memory reads)
        if (ok) {
          float hd = 0.f;
          for (int i = tid - N_EPI / 2; i < SQ_TILE / 16; i += N_EPI / 2) {
            const uint4 a = *reinterpret_cast<const uint4*>(smem + OFF_H + i * 16);
            const uint4 b = *reinterpret_cast<const uint4*>(smem + OFF_DH + i * 16);
            const uint32_t* pa = &a.x;
            const uint32_t* pb = &b.x;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float2 fa = __bfloat1622float2(*reinterpret_cast<const bf162*>(&pa[e]));
              float2 fb = __bfloat1622float2(*reinterpret_cast<const bf162*>(&pb[e]));
              hd += fa.x * fb.x + fa.y * fb.y;
            }
          }
          acc_last += sGam[CHUNK - 1] * hd;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[R_HD]);
        if (it > 0) combine(prev_first, prev_rows);  // fits into the wait for the first wide products
        const float f_w = hi ? sRho[row_w] : p.scale * sGam[row_w];
        const int row_q = row_w - (lane & 3);  // row of lane 0 of this quad
        const long long out_q = ((cur.row0 + row_q) * p.Hv + cur.hv) * D + c128;
        float acc_w = 0.f;

        // ---- E4: dq1 = scale gamma (dO h^T) on the lower lanes, dk1 = rho (Vn dh^T) on the upper;
        //      scaled in place (written back to tensor memory), with their dg terms ----
        ok = ok && WAIT(C_1B, ph);
        if (ok) {
          tc_fence_after();
          const unsigned char* tile = smem + (hi ? koff : OFF_Q);
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            float x[32];
            tmem_ld32(tmem + lanes + T_DQ1 + c128 + 32 * pass, x);
            tmem_ld_wait();
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 raw = *reinterpret_cast<const uint4*>(tile + piece(pass, j));
              const uint32_t* pr = &raw.x;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 t = __bfloat1622float2(*reinterpret_cast<const bf162*>(&pr[e]));
                x[8 * j + 2 * e] *= f_w;
                x[8 * j + 2 * e + 1] *= f_w;
                s += t.x * x[8 * j + 2 * e] + t.y * x[8 * j + 2 * e + 1];
              }
            }
            tmem_st32(tmem + lanes + T_DQ1 + c128 + 32 * pass, x);
            // dg += rowsum(q dq1) - rowsum(k dk1); the chunk total gets + sum(k dk1)
            acc_w += hi ? -s : s;
            if (hi) acc_last += s;
          }
          tmem_st_wait();
        }
        signal(R_E4);  // q (and this item's k for this group) are no longer read from shared memory

        // ---- E6: dv = A'^T du (upper lanes), already row-scaled by beta ----
        ok = ok && WAIT(C_2B, ph);
        if (ok) {
          tc_fence_after();
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            float x[32];
            tmem_ld32(tmem + lanes + (T_T2 & 0xFFFFu) + c128 + 32 * pass, x);
            tmem_ld_wait();
            store_rows(p.dv, out_q + 32 * pass, row_q, hi ? valid : 0, x);  // dv sits on the upper lanes
          }
        }

        // ---- E8: dq = dq1 + ds K (lower lanes); dk = dk1 + [ds^T q + A''^T dw + (beta dA3) K + (beta dA3)^T K] ----
        ok = ok && WAIT(C_5, ph);
        if (ok) {
          tc_fence_after();
          bf16* out = hi ? p.dk : p.dq;
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            float x[32], y[32];
            tmem_ld32(tmem + lanes + T_DQ1 + c128 + 32 * pass, x);
            tmem_ld32(tmem + lanes + T_DQ2 + c128 + 32 * pass, y);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) x[j] += y[j];
            store_rows(out, out_q + 32 * pass, row_q, valid, x);
          }
        }
        signal(R_END);  // accumulators and k of this item are free
        sRowW[(2 * half + (hi ? 1 : 0)) * 64 + row_w] = acc_w;
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) acc_last += __shfl_xor_sync(0xffffffffu, acc_last, d);
        if (lane == 0) sLast[gw] = acc_last;
      }
      // One barrier per item: every contribution to dg, db of this item is in, and the vectors of
      // the next item are in place (other buffer).  The stop flag alternates as well, so that it
      // is read by all before it can be written again.
      if (has_next) write_vectors(nxt, ph ? sVec0 : sVec1);
      if (!ok) *abort_flag = 1;
      if (tid == 0) stop_flag[ph] = *abort_flag;
      epi_barrier();
      prev_first = cur.row0 * p.Hv + cur.hv;
      prev_rows = cur.valid;
      cur = nxt;
      if (stop_flag[ph]) {  // written before the barrier by one thread: uniform
        stopped = true;
        break;
      }
    }
    if (it > 0 && !stopped) combine(prev_first, prev_rows);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && *abort_flag) atomicCAS(&g_bwd_main_status, 0, 1);
}

int bwd_main_tc_status(int* out, int reset) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_bwd_main_status, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  *out = v;
  if (reset && v != 0) {
    int z = 0;
    e = cudaMemcpyToSymbol(g_bwd_main_status, &z, sizeof(int));
  }
  return (int)e;
}


// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D bf16 tensor map, rows x cols (row-major), box = 64 columns x box_rows rows, 128-byte swizzle.
// Encoding a map costs about a microsecond on the host and a launch needs four to nine of them, so
// the last maps are kept in a small table keyed by (pointer, shape, box): a steady-state step that
// reuses its buffers (a framework's caching allocator, a CUDA graph's private pool) encodes nothing.
// A map only describes addresses and extents, so an entry stays valid when the buffer is freed and
// an equal allocation returns at the same address.
int make_tile_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, int box_rows) {
  static EncodeTiledFn2 fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess)
      f = nullptr;
    return (EncodeTiledFn2)f;
  }();
  if (!fn) return FQLA_ERR_INVALID_ARG;
  struct Entry {
    const void* ptr;
    long long rows, cols;
    int box_rows, used;
    CUtensorMap map;
  };
  constexpr int N_ENTRIES = 128;
  static Entry table[N_ENTRIES] = {};
  static std::mutex lock;
  const uint64_t hsh = ((uint64_t)(uintptr_t)ptr >> 8) * 0x9E3779B97F4A7C15ull ^
                       ((uint64_t)rows * 0xC2B2AE3D27D4EB4Full) ^ ((uint64_t)cols << 17) ^
                       (uint64_t)box_rows;
  Entry& e = table[(hsh >> 32) % N_ENTRIES];
  {
    std::lock_guard<std::mutex> hold(lock);
    if (e.used && e.ptr == ptr && e.rows == rows && e.cols == cols && e.box_rows == box_rows) {
      *m = e.map;
      return 0;
    }
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return FQLA_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> hold(lock);
  e.ptr = ptr; e.rows = rows; e.cols = cols; e.box_rows = box_rows; e.map = *m; e.used = 1;
  return 0;
}

int launch_bwd_main_tc(const void* q, const void* k, const void* v, const void* vnew, const void* A,
                       const float* g, const void* beta, int beta_is_f32, const void* dO,
                       const void* du, const void* h, const void* dh, void* dq, void* dk, void* dv,
                       float* db, float* dg, int tiled, int Hq, int Hv, long long T_rows, long long n_chunks,
                       float scale, SeqLayout lay, IndexTable chunk_indices, cudaStream_t st) {
  using namespace bmtc;
  CUtensorMap mq, mk, mv, mvn, mdo, mdu, mh, mdh, ma;
  int rc;
  if ((rc = make_tile_map(&mq, q, T_rows, (long long)Hq * D, 64))) return rc;
  if ((rc = make_tile_map(&mk, k, T_rows, (long long)Hq * D, 64))) return rc;
  if ((rc = make_tile_map(&mv, v, T_rows, (long long)Hv * D, 64))) return rc;
  if (tiled) {
    if ((rc = make_tile_map(&mvn, vnew, n_chunks * Hv * D, CHUNK, 128))) return rc;
    if ((rc = make_tile_map(&mdu, du, n_chunks * Hv * D, CHUNK, 128))) return rc;
  } else {
    if ((rc = make_tile_map(&mvn, vnew, T_rows, (long long)Hv * D, 64))) return rc;
    if ((rc = make_tile_map(&mdu, du, T_rows, (long long)Hv * D, 64))) return rc;
  }
  if ((rc = make_tile_map(&mdo, dO, T_rows, (long long)Hv * D, 64))) return rc;
  if ((rc = make_tile_map(&mh, h, n_chunks * Hv * D, D, 128))) return rc;
  if ((rc = make_tile_map(&mdh, dh, n_chunks * Hv * D, D, 128))) return rc;
  if ((rc = make_tile_map(&ma, A, T_rows, (long long)Hv * CHUNK, 64))) return rc;
  BwdMainTcParams p;
  p.g = g; p.beta = beta; p.beta_is_f32 = beta_is_f32;
  p.dq = (bf16*)dq; p.dk = (bf16*)dk; p.dv = (bf16*)dv; p.db = db; p.dg = dg;
  p.Hq = Hq; p.Hv = Hv; p.scale = scale; p.lay = lay; p.chunk_indices = chunk_indices;
  p.n_chunks = n_chunks;
  rc = configure_smem(tiled ? (const void*)bwd_main_tc_kernel<true> : (const void*)bwd_main_tc_kernel<false>,
                      SMEM_BYTES);
  if (rc != 0) return rc;
  int dev = 0, n_sm = 0;  // per launch: the current device may differ from call to call
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev);
  if (n_sm <= 0) n_sm = 148;
  const long long total = n_chunks * Hv;
  const unsigned grid = (unsigned)(total < n_sm ? total : n_sm);
  if (tiled)
    bwd_main_tc_kernel<true><<<grid, NT, SMEM_BYTES, st>>>(p, mq, mk, mv, mvn, mdo, mdu, mh, mdh, ma);
  else
    bwd_main_tc_kernel<false><<<grid, NT, SMEM_BYTES, st>>>(p, mq, mk, mv, mvn, mdo, mdu, mh, mdh, ma);
  return (int)cudaGetLastError();
}

}  // namespace fqla
