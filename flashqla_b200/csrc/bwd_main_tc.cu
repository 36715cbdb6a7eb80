// Chunk-parallel part of the gated-delta-rule backward on Blackwell tensor cores (K = V = 128).
//
// Same mathematics and same outputs as bwd_main.cu (the reference's tests/ref_gdr.py:427-600,
// evaluated by the reference kernels inside blackwell/fused_bwd.py:595-862): one CTA per
// (chunk, value head), 256 threads.  All sixteen tile products are tcgen05.mma with M = 64 (rows
// = tokens) and fp32 accumulators in tensor memory; operand tiles arrive by TMA (128-byte
// swizzle), intermediate operands (ds, dw, dA, ...) are written back to shared memory as bf16 by
// the threads that read the accumulators.  The work is five rounds of
//     one thread issues a batch of products -> commit -> everybody waits on the mbarrier ->
//     every warp reads its quarter of the accumulators (16-lane shape) and does the elementwise
//     work of the round -> fence -> __syncthreads
// Two M = 64 accumulators share each column range (lanes +0 and +16 of every 32-lane quarter).
#include <cuda.h>

#include "common.cuh"
#include "fqla_internal.h"
#include "tc05.cuh"

namespace fqla {

using namespace tc;

// set to 1 when a CTA of this file's kernel abandoned a bounded wait; read through
// fqla_device_status together with the forward kernel's word
__device__ int g_bwd_main_status = 0;
// Diagnostics (FQLA_PROFILE=1): clock of CTA (0,0) at the end of every step of the kernel
__device__ long long g_bwd_main_profile[16];

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
  int profile;
};

namespace bmtc {
constexpr int D = 128;
constexpr int NT = 512;          // threads: 16 warps = 4 lane quarters x 4 column quarters
constexpr int ROW_TILE = 16384;  // [64 x 128] bf16 as two 64-column blocks
constexpr int SQ_TILE = 32768;   // [128 x 128] bf16 as two 64-column blocks of 128 rows
constexpr int OFF_Q = 0, OFF_K = OFF_Q + ROW_TILE, OFF_V = OFF_K + ROW_TILE;
constexpr int OFF_VN = OFF_V + ROW_TILE, OFF_DO = OFF_VN + ROW_TILE, OFF_DU = OFF_DO + ROW_TILE;
constexpr int OFF_H = OFF_DU + ROW_TILE;
constexpr int OFF_DH = OFF_H + SQ_TILE;
constexpr int OFF_A = OFF_DH + SQ_TILE;
constexpr int OFF_DS = OFF_A + 8192;       // ds, later T = A^T dA
constexpr int OFF_DA = OFF_DS + 8192;
constexpr int OFF_D3 = OFF_DA + 8192;      // dA3
constexpr int OFF_D3B = OFF_D3 + 8192;     // diag(beta) dA3
constexpr int OFF_DW = OFF_D3B + 8192;     // -du h^T
constexpr int OFF_VEC = OFF_DW + ROW_TILE;  // g, gamma, rho, beta, dg, db (64 floats each) + dg_last
constexpr int OFF_BAR = OFF_VEC + (6 * 64 + 4) * 4;
constexpr int OFF_MISC = OFF_BAR + 8 * 8;
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;
// the operand tiles of one work item arrive in three groups, in the order their buffers of the
// previous item become free
constexpr uint32_t TX_A = 2 * SQ_TILE + 2 * ROW_TILE;  // h, dh, dO, v_new
constexpr uint32_t TX_B = 3 * ROW_TILE;                // du, q, v
constexpr uint32_t TX_C = ROW_TILE + 8192;             // k, A
// tensor memory: (column, lane half) of every accumulator
constexpr uint32_t HI = 16u << 16;
constexpr uint32_t T_DQ1 = 0, T_DK1 = 128, T_DW = 256, T_T1 = 384;
constexpr uint32_t T_DQ2 = 0 + HI, T_DK2 = 128 + HI, T_T2 = 256 + HI, T_DS = 384 + HI, T_QK = 448 + HI;
constexpr uint32_t T_X1 = 256, T_X2 = 320;            // after dw has been read
constexpr uint32_t T_T = 384 + HI, T_KK = 448 + HI;    // after ds, qk have been read
constexpr uint32_t T_D3 = 256;                         // after x1 has been read
constexpr uint32_t T_T3 = 0, T_DK5 = 0 + HI;           // after dq1, dq2 have been read
enum { BAR_LOAD_A = 0, BAR_LOAD_B, BAR_LOAD_C, BAR_MMA };
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
  float* sG = reinterpret_cast<float*>(smem + OFF_VEC);
  float* sGam = sG + 64;
  float* sRho = sGam + 64;
  float* sBeta = sRho + 64;
  float* sDg = sBeta + 64;
  float* sDb = sDg + 64;
  float* sDgLast = sDb + 64;

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
    t.valid = min(CHUNK, sp.len - ci * CHUNK);
    t.chunk_id = sp.chunk_base + ci;
    return t;
  };
  auto load_a = [&](const Item& t) {
    const int y = (int)t.row0, ys = (int)((t.chunk_id * p.Hv + t.hv) * D);
    mbar_arrive_expect_tx(&bars[BAR_LOAD_A], TX_A);
    tma_load_2d(smem + OFF_DO, &map_do, t.hv * D, y, &bars[BAR_LOAD_A]);
    tma_load_2d(smem + OFF_DO + 8192, &map_do, t.hv * D + 64, y, &bars[BAR_LOAD_A]);
    tma_load_2d(smem + OFF_H, &map_h, 0, ys, &bars[BAR_LOAD_A]);
    tma_load_2d(smem + OFF_H + 16384, &map_h, 64, ys, &bars[BAR_LOAD_A]);
    if constexpr (TILED) {
      tma_load_2d(smem + OFF_VN, &map_vn, 0, ys, &bars[BAR_LOAD_A]);
    } else {
      tma_load_2d(smem + OFF_VN, &map_vn, t.hv * D, y, &bars[BAR_LOAD_A]);
      tma_load_2d(smem + OFF_VN + 8192, &map_vn, t.hv * D + 64, y, &bars[BAR_LOAD_A]);
    }
    tma_load_2d(smem + OFF_DH, &map_dh, 0, ys, &bars[BAR_LOAD_A]);
    tma_load_2d(smem + OFF_DH + 16384, &map_dh, 64, ys, &bars[BAR_LOAD_A]);
  };
  auto load_b = [&](const Item& t) {
    const int y = (int)t.row0;
    mbar_arrive_expect_tx(&bars[BAR_LOAD_B], TX_B);
    if constexpr (TILED) {
      tma_load_2d(smem + OFF_DU, &map_du, 0, (int)((t.chunk_id * p.Hv + t.hv) * D), &bars[BAR_LOAD_B]);
    } else {
      tma_load_2d(smem + OFF_DU, &map_du, t.hv * D, y, &bars[BAR_LOAD_B]);
      tma_load_2d(smem + OFF_DU + 8192, &map_du, t.hv * D + 64, y, &bars[BAR_LOAD_B]);
    }
    tma_load_2d(smem + OFF_Q, &map_q, t.hq * D, y, &bars[BAR_LOAD_B]);
    tma_load_2d(smem + OFF_Q + 8192, &map_q, t.hq * D + 64, y, &bars[BAR_LOAD_B]);
    tma_load_2d(smem + OFF_V, &map_v, t.hv * D, y, &bars[BAR_LOAD_B]);
    tma_load_2d(smem + OFF_V + 8192, &map_v, t.hv * D + 64, y, &bars[BAR_LOAD_B]);
  };
  auto load_c = [&](const Item& t) {
    const int y = (int)t.row0;
    mbar_arrive_expect_tx(&bars[BAR_LOAD_C], TX_C);
    tma_load_2d(smem + OFF_K, &map_k, t.hq * D, y, &bars[BAR_LOAD_C]);
    tma_load_2d(smem + OFF_K + 8192, &map_k, t.hq * D + 64, y, &bars[BAR_LOAD_C]);
    tma_load_2d(smem + OFF_A, &map_a, t.hv * CHUNK, y, &bars[BAR_LOAD_C]);
  };
  // per-row scalars of an item, fetched one item ahead into registers by threads 0..63
  float pre_g = 0.f, pre_gl = 0.f, pre_beta = 0.f;
  auto fetch_vectors = [&](const Item& t) {
    if (tid < CHUNK) {
      const int r = min(tid, t.valid - 1);
      pre_g = p.g[(t.row0 + r) * p.Hv + t.hv];
      pre_gl = p.g[(t.row0 + t.valid - 1) * p.Hv + t.hv];
      pre_beta = tid < t.valid ? load_beta(p.beta, p.beta_is_f32, (t.row0 + tid) * p.Hv + t.hv) : 0.f;
    }
  };
  // rows past the end of the sequence belong to the next one: zero them in n_blocks 8 KB blocks
  auto zero_rows = [&](int off, int n_blocks, int valid) {
    for (int blk = 0; blk < n_blocks; ++blk) {
      unsigned char* base = smem + off + blk * 8192;
      for (int i = tid; i < (CHUNK - valid) * 8; i += NT)
        *reinterpret_cast<uint4*>(base + (valid + (i >> 3)) * 128 + ((i & 7) << 4)) = make_uint4(0, 0, 0, 0);
    }
  };

  if (tid == 0) {
    mbar_init(&bars[BAR_LOAD_A], 1);
    mbar_init(&bars[BAR_LOAD_B], 1);
    mbar_init(&bars[BAR_LOAD_C], 1);
    mbar_init(&bars[BAR_MMA], 1);
    *abort_flag = 0;
    *sDgLast = 0.f;
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const bool prof = p.profile && tid == 0 && blockIdx.x == 0;
  int stamp_i = 0;
  auto stamp = [&]() {
    if (prof && stamp_i < 16) g_bwd_main_profile[stamp_i++] = clock64();
  };
  stamp();

  Item cur = decode(blockIdx.x);  // the grid never exceeds the number of items
  if (tid == 0) {
    load_a(cur);
    load_b(cur);
    load_c(cur);
  }
  fetch_vectors(cur);

  // ---- descriptors (low words) ----
  const uint32_t q_lo = desc_lo_kmajor(smem + OFF_Q), k_lo = desc_lo_kmajor(smem + OFF_K);
  const uint32_t v_lo = desc_lo_kmajor(smem + OFF_V), vn_lo = desc_lo_kmajor(smem + OFF_VN);
  const uint32_t do_lo = desc_lo_kmajor(smem + OFF_DO), du_lo = desc_lo_kmajor(smem + OFF_DU);
  const uint32_t h_lo = desc_lo_kmajor(smem + OFF_H), dh_lo = desc_lo_kmajor(smem + OFF_DH);
  const uint32_t a_lo = desc_lo_kmajor(smem + OFF_A), ds_lo = desc_lo_kmajor(smem + OFF_DS);
  const uint32_t dw_lo = desc_lo_kmajor(smem + OFF_DW), d3_lo = desc_lo_kmajor(smem + OFF_D3);
  const uint32_t qmn_lo = desc_lo_mnmajor(smem + OFF_Q, 8192), kmn_lo = desc_lo_mnmajor(smem + OFF_K, 8192);
  const uint32_t dumn_lo = desc_lo_mnmajor(smem + OFF_DU, 8192), dwmn_lo = desc_lo_mnmajor(smem + OFF_DW, 8192);
  const uint32_t amn_lo = desc_lo_mnmajor(smem + OFF_A, 8192), dsmn_lo = desc_lo_mnmajor(smem + OFF_DS, 8192);
  const uint32_t damn_lo = desc_lo_mnmajor(smem + OFF_DA, 8192), d3bmn_lo = desc_lo_mnmajor(smem + OFF_D3B, 8192);
  constexpr uint32_t ID_KK_128 = idesc_bf16(64, 128, 0, 0), ID_KK_64 = idesc_bf16(64, 64, 0, 0);
  constexpr uint32_t ID_KM_128 = idesc_bf16(64, 128, 0, 1), ID_MM_128 = idesc_bf16(64, 128, 1, 1);
  constexpr uint32_t ID_MM_64 = idesc_bf16(64, 64, 1, 1);
  // operand-tile layouts: [V rows][K or token columns], read MN-major with the contraction over rows
  constexpr uint32_t ID_KM_64 = idesc_bf16(64, 64, 0, 1), ID_MK_64 = idesc_bf16(64, 64, 1, 0);
  constexpr uint32_t ID_MK_128 = idesc_bf16(64, 128, 1, 0);
  const uint32_t hT_lo = desc_lo_mnmajor(smem + OFF_H, 16384), dhT_lo = desc_lo_mnmajor(smem + OFF_DH, 16384);
  const uint32_t vnT_lo = desc_lo_mnmajor(smem + OFF_VN, 16384), duT_lo = desc_lo_mnmajor(smem + OFF_DU, 16384);

  // ---- per-thread coordinates in the 16-lane accumulator shape ----
  const int qd = warp & 3, cq = warp >> 2;
  const int row_a = 16 * qd + (lane >> 2), row_b = row_a + 8, cp = 2 * (lane & 3);
  const uint32_t lanes = (uint32_t)(qd * 32) << 16;
  const int c128 = 32 * cq, c64 = 16 * cq;   // first column of this warp in 128- / 64-wide tiles
  uint32_t phase = 0;
  bool ok = true;
  auto wait_mma = [&]() {
    bool r = mbar_wait(&bars[BAR_MMA], phase, abort_flag);
    phase ^= 1;
    tc_fence_after();
    return r;
  };
  // bf16 pair of a [64 x 128] row tile at (row, col), col even
  auto tile2 = [&](int off, int row, int col) {
    return ld_bf16x2(reinterpret_cast<const bf16*>(smem + off + (col >> 6) * 8192 + sw128_offset(row, col & 63)));
  };
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
  auto st_tile64 = [&](int off, int row, int col, float lo, float hi) {
    *reinterpret_cast<uint32_t*>(smem + off + sw128_offset(row, col)) = pack_bf16(lo, hi);
  };
  auto round_sync = [&]() {
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  };

#pragma unroll 1
  for (long long w = blockIdx.x; w < total && ok; w += gridDim.x) {
    const uint32_t lph = (uint32_t)((w / gridDim.x) & 1);
    const bool has_next = w + gridDim.x < total;
    Item nxt = cur;
    if (has_next) nxt = decode(w + gridDim.x);
    const int valid = cur.valid;
    if (tid < CHUNK) {
      sG[tid] = pre_g;
      sGam[tid] = fast_exp(pre_g);
      sRho[tid] = fast_exp(pre_gl - pre_g);
      sBeta[tid] = pre_beta;
      sDg[tid] = 0.f;
      sDb[tid] = 0.f;
    }
    ok = mbar_wait(&bars[BAR_LOAD_A], lph, abort_flag) && mbar_wait(&bars[BAR_LOAD_B], lph, abort_flag);
    if (ok && valid < CHUNK) {
      zero_rows(OFF_Q, 2, valid);
      if constexpr (TILED) {  // the transposed tiles already hold zeros past the sequence end
        zero_rows(OFF_V, 2, valid);
        zero_rows(OFF_DO, 2, valid);
      } else {
        zero_rows(OFF_V, 8, valid);  // v, v_new, dO, du
      }
    }
    round_sync();
    stamp();

    // ======================= round 1: products with h and dh, ds, qk =======================
    if (ok && tid == 0) {
      if constexpr (TILED) {
        umma_group<8, 128, 512, 128, 512, false>(tmem + T_DW, duT_lo, hT_lo, ID_MM_128);
        umma_group<8, 2, 512, 128, 512, false>(tmem + T_DS, do_lo, vnT_lo, ID_KM_64);
        umma_group<8, 2, 512, 128, 512, false>(tmem + T_DQ1, do_lo, hT_lo, ID_KM_128);
        umma_group<8, 128, 512, 128, 512, false>(tmem + T_DK1, vnT_lo, dhT_lo, ID_MM_128);
      } else {
        umma_group<8, 2, 512, 2, 1024, false>(tmem + T_DW, du_lo, h_lo, ID_KK_128);
        umma_group<8, 2, 512, 2, 512, false>(tmem + T_DS, do_lo, vn_lo, ID_KK_64);
        umma_group<8, 2, 512, 2, 1024, false>(tmem + T_DQ1, do_lo, h_lo, ID_KK_128);
        umma_group<8, 2, 512, 2, 1024, false>(tmem + T_DK1, vn_lo, dh_lo, ID_KK_128);
      }
    }
    // meanwhile: gamma_last * sum(h * dh) over the whole 128 x 128 tiles (plain shared-memory reads)
    if (ok) {
      float hd = 0.f;
      for (int i = tid; i < SQ_TILE / 16; i += NT) {
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
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) hd += __shfl_xor_sync(0xffffffffu, hd, d);
      if (lane == 0) atomicAdd(sDgLast, sGam[CHUNK - 1] * hd);
    }
    ok = ok && mbar_wait(&bars[BAR_LOAD_C], lph, abort_flag);
    if (ok && valid < CHUNK) {
      zero_rows(OFF_K, 2, valid);
      zero_rows(OFF_A, 1, valid);
      fence_proxy_async();
    }
    __syncthreads();
    if (ok && tid == 0) {
      umma_group<8, 2, 512, 2, 512, false>(tmem + T_QK, q_lo, k_lo, ID_KK_64);
      umma_commit(&bars[BAR_MMA]);
    }
    const float g_a = sG[row_a], g_b = sG[row_b];
    const float gam_a = sGam[row_a], gam_b = sGam[row_b];
    const float rho_a = sRho[row_a], rho_b = sRho[row_b];
    const float beta_a = sBeta[row_a], beta_b = sBeta[row_b];
    float dq1[16], dkacc[16];
    ok = ok && wait_mma();
    stamp();
    if (ok) {
      {  // dw = -du h^T as an operand tile
        float dw[16];
        tmem_ld_16x32(tmem + lanes + T_DW + c128, dw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = c128 + 8 * i + cp;
          unsigned char* base = smem + OFF_DW + (col >> 6) * 8192;
          *reinterpret_cast<uint32_t*>(base + sw128_offset(row_a, col & 63)) = pack_bf16(-dw[4 * i], -dw[4 * i + 1]);
          *reinterpret_cast<uint32_t*>(base + sw128_offset(row_b, col & 63)) = pack_bf16(-dw[4 * i + 2], -dw[4 * i + 3]);
        }
      }
      {  // ds = scale * G * (dO Vn^T); ds2 = ds * (Q K^T)
        float ds[8], qk[8];
        tmem_ld_16x16(tmem + lanes + T_DS + c64, ds);
        tmem_ld_16x16(tmem + lanes + T_QK + c64, qk);
        tmem_ld_wait();
        float rs_a = 0.f, rs_b = 0.f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int col = c64 + 8 * i + cp;
          const float gc0 = sG[col], gc1 = sG[col + 1];
          const float a0 = col <= row_a ? p.scale * ds[4 * i] * fast_exp(g_a - gc0) : 0.f;
          const float a1 = col + 1 <= row_a ? p.scale * ds[4 * i + 1] * fast_exp(g_a - gc1) : 0.f;
          const float b0 = col <= row_b ? p.scale * ds[4 * i + 2] * fast_exp(g_b - gc0) : 0.f;
          const float b1 = col + 1 <= row_b ? p.scale * ds[4 * i + 3] * fast_exp(g_b - gc1) : 0.f;
          st_tile64(OFF_DS, row_a, col, a0, a1);
          st_tile64(OFF_DS, row_b, col, b0, b1);
          const float s0 = a0 * qk[4 * i], s1 = a1 * qk[4 * i + 1], s2 = b0 * qk[4 * i + 2], s3 = b1 * qk[4 * i + 3];
          rs_a += s0 + s1;
          rs_b += s2 + s3;
          const float c0 = col_sum(s0 + s2), c1 = col_sum(s1 + s3);
          if (lane < 4) {
            atomicAdd(sDg + col, -c0);
            atomicAdd(sDg + col + 1, -c1);
          }
        }
        rs_a = quad_sum(rs_a);
        rs_b = quad_sum(rs_b);
        if ((lane & 3) == 0) {
          atomicAdd(sDg + row_a, rs_a);
          atomicAdd(sDg + row_b, rs_b);
        }
      }
      // dq1 = scale * gamma * (dO h^T), dg += rowsum(q * dq1)
      // dk1 = rho * (Vn dh^T), dg -= rowsum(k * dk1), dg_last += sum(k * dk1)
      tmem_ld_16x32(tmem + lanes + T_DQ1 + c128, dq1);
      tmem_ld_16x32(tmem + lanes + T_DK1 + c128, dkacc);
      tmem_ld_wait();
      float qa = 0.f, qb = 0.f, ka = 0.f, kb = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = c128 + 8 * i + cp;
        dq1[4 * i] *= p.scale * gam_a;
        dq1[4 * i + 1] *= p.scale * gam_a;
        dq1[4 * i + 2] *= p.scale * gam_b;
        dq1[4 * i + 3] *= p.scale * gam_b;
        dkacc[4 * i] *= rho_a;
        dkacc[4 * i + 1] *= rho_a;
        dkacc[4 * i + 2] *= rho_b;
        dkacc[4 * i + 3] *= rho_b;
        const float2 q_a = tile2(OFF_Q, row_a, col), q_b = tile2(OFF_Q, row_b, col);
        const float2 k_a = tile2(OFF_K, row_a, col), k_b = tile2(OFF_K, row_b, col);
        qa += q_a.x * dq1[4 * i] + q_a.y * dq1[4 * i + 1];
        qb += q_b.x * dq1[4 * i + 2] + q_b.y * dq1[4 * i + 3];
        ka += k_a.x * dkacc[4 * i] + k_a.y * dkacc[4 * i + 1];
        kb += k_b.x * dkacc[4 * i + 2] + k_b.y * dkacc[4 * i + 3];
      }
      qa = quad_sum(qa - ka);
      qb = quad_sum(qb - kb);
      float kt = ka + kb;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) kt += __shfl_xor_sync(0xffffffffu, kt, d);
      if ((lane & 3) == 0) {
        atomicAdd(sDg + row_a, qa);
        atomicAdd(sDg + row_b, qb);
      }
      if (lane == 0) atomicAdd(sDgLast, kt);
    }
    round_sync();
    stamp();

    // ======================= round 2: ds products, dA pieces, A^T dw, A^T du =======================
    if (ok && tid == 0) {
      if (has_next) load_a(nxt);  // h, dh, dO, v_new of this item are dead
      umma_group<8, 2, 512, 2, 512, false>(tmem + T_X1, dw_lo, k_lo, ID_KK_64);
      if constexpr (TILED) umma_group<8, 128, 512, 2, 512, false>(tmem + T_X2, duT_lo, v_lo, ID_MK_64);
      else umma_group<8, 2, 512, 2, 512, false>(tmem + T_X2, du_lo, v_lo, ID_KK_64);
      umma_group<4, 2, 0, 128, 0, false>(tmem + T_DQ2, ds_lo, kmn_lo, ID_KM_128);
      umma_group<4, 128, 0, 128, 0, false>(tmem + T_DK2, dsmn_lo, qmn_lo, ID_MM_128);
      umma_group<4, 128, 0, 128, 0, false>(tmem + T_T1, amn_lo, dwmn_lo, ID_MM_128);
      if constexpr (TILED) umma_group<4, 128, 0, 2, 0, false>(tmem + T_T2, amn_lo, du_lo, ID_MK_128);
      else umma_group<4, 128, 0, 128, 0, false>(tmem + T_T2, amn_lo, dumn_lo, ID_MM_128);
      umma_commit(&bars[BAR_MMA]);
    }
    if (has_next) fetch_vectors(nxt);
    const long long out_a = ((cur.row0 + row_a) * p.Hv + cur.hv) * D, out_b = ((cur.row0 + row_b) * p.Hv + cur.hv) * D;
    const bool wr_a = row_a < valid, wr_b = row_b < valid;
    ok = ok && wait_mma();
    stamp();
    if (ok) {
      {  // dA = strict_lower(beta_c (gamma_c x1 + x2))
        float x1[8], x2[8];
        tmem_ld_16x16(tmem + lanes + T_X1 + c64, x1);
        tmem_ld_16x16(tmem + lanes + T_X2 + c64, x2);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int col = c64 + 8 * i + cp;
          const float b0 = sBeta[col], b1 = sBeta[col + 1], g0 = sGam[col], g1 = sGam[col + 1];
          st_tile64(OFF_DA, row_a, col, col < row_a ? b0 * (g0 * x1[4 * i] + x2[4 * i]) : 0.f,
                    col + 1 < row_a ? b1 * (g1 * x1[4 * i + 1] + x2[4 * i + 1]) : 0.f);
          st_tile64(OFF_DA, row_b, col, col < row_b ? b0 * (g0 * x1[4 * i + 2] + x2[4 * i + 2]) : 0.f,
                    col + 1 < row_b ? b1 * (g1 * x1[4 * i + 3] + x2[4 * i + 3]) : 0.f);
        }
      }
    }
    // the dA tile is all the next product needs: hand it over before the rest of this round
    round_sync();
    if (ok && tid == 0) {
      umma_group<4, 128, 0, 128, 0, false>(tmem + T_T, amn_lo, damn_lo, ID_MM_64);
      umma_group<8, 2, 512, 2, 512, false>(tmem + T_KK, k_lo, k_lo, ID_KK_64);
      umma_commit(&bars[BAR_MMA]);
    }
    if (ok) {
      {  // dq = dq1 + ds K
        float x[16];
        tmem_ld_16x32(tmem + lanes + T_DQ2 + c128, x);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = c128 + 8 * i + cp;
          if (wr_a) *reinterpret_cast<uint32_t*>(p.dq + out_a + col) = pack_bf16(dq1[4 * i] + x[4 * i], dq1[4 * i + 1] + x[4 * i + 1]);
          if (wr_b) *reinterpret_cast<uint32_t*>(p.dq + out_b + col) = pack_bf16(dq1[4 * i + 2] + x[4 * i + 2], dq1[4 * i + 3] + x[4 * i + 3]);
        }
      }
      {  // dk += ds^T Q + beta gamma (A^T dw);  db += gamma rowsum(t1 k);  dg += beta gamma rowsum(t1 k)
        float x[16], t1[16];
        tmem_ld_16x32(tmem + lanes + T_DK2 + c128, x);
        tmem_ld_16x32(tmem + lanes + T_T1 + c128, t1);
        tmem_ld_wait();
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = c128 + 8 * i + cp;
          const float2 k_a = tile2(OFF_K, row_a, col), k_b = tile2(OFF_K, row_b, col);
          sa += k_a.x * t1[4 * i] + k_a.y * t1[4 * i + 1];
          sb += k_b.x * t1[4 * i + 2] + k_b.y * t1[4 * i + 3];
          dkacc[4 * i] += x[4 * i] + beta_a * gam_a * t1[4 * i];
          dkacc[4 * i + 1] += x[4 * i + 1] + beta_a * gam_a * t1[4 * i + 1];
          dkacc[4 * i + 2] += x[4 * i + 2] + beta_b * gam_b * t1[4 * i + 2];
          dkacc[4 * i + 3] += x[4 * i + 3] + beta_b * gam_b * t1[4 * i + 3];
        }
        sa = quad_sum(sa);
        sb = quad_sum(sb);
        if ((lane & 3) == 0) {
          atomicAdd(sDb + row_a, gam_a * sa);
          atomicAdd(sDb + row_b, gam_b * sb);
          atomicAdd(sDg + row_a, beta_a * gam_a * sa);
          atomicAdd(sDg + row_b, beta_b * gam_b * sb);
        }
      }
      {  // dv = beta (A^T du);  db += rowsum(t2 v)
        float t2[16];
        tmem_ld_16x32(tmem + lanes + T_T2 + c128, t2);
        tmem_ld_wait();
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = c128 + 8 * i + cp;
          const float2 v_a = tile2(OFF_V, row_a, col), v_b = tile2(OFF_V, row_b, col);
          sa += v_a.x * t2[4 * i] + v_a.y * t2[4 * i + 1];
          sb += v_b.x * t2[4 * i + 2] + v_b.y * t2[4 * i + 3];
          if (wr_a) *reinterpret_cast<uint32_t*>(p.dv + out_a + col) = pack_bf16(beta_a * t2[4 * i], beta_a * t2[4 * i + 1]);
          if (wr_b) *reinterpret_cast<uint32_t*>(p.dv + out_b + col) = pack_bf16(beta_b * t2[4 * i + 2], beta_b * t2[4 * i + 3]);
        }
        sa = quad_sum(sa);
        sb = quad_sum(sb);
        if ((lane & 3) == 0) {
          atomicAdd(sDb + row_a, sa);
          atomicAdd(sDb + row_b, sb);
        }
      }
    }
    stamp();

    // ======================= round 3: T = A^T dA, K K^T (issued above) =======================
    ok = ok && wait_mma();
    stamp();
    if (ok) {
      float t[8];
      tmem_ld_16x16(tmem + lanes + T_T + c64, t);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int col = c64 + 8 * i + cp;
        st_tile64(OFF_DS, row_a, col, t[4 * i], t[4 * i + 1]);
        st_tile64(OFF_DS, row_b, col, t[4 * i + 2], t[4 * i + 3]);
      }
    }
    round_sync();
    stamp();

    // ======================= round 4: d3 = T A^T =======================
    if (ok && tid == 0) {
      if (has_next) load_b(nxt);  // du, q, v of this item are dead
      umma_group<4, 2, 0, 2, 0, false>(tmem + T_D3, ds_lo, a_lo, ID_KK_64);
      umma_commit(&bars[BAR_MMA]);
    }
    ok = ok && wait_mma();
    stamp();
    if (ok) {
      float d3[8], kk[8];
      tmem_ld_16x16(tmem + lanes + T_D3 + c64, d3);
      tmem_ld_16x16(tmem + lanes + T_KK + c64, kk);
      tmem_ld_wait();
      float rs_a = 0.f, rs_b = 0.f;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int col = c64 + 8 * i + cp;
        const float gc0 = sG[col], gc1 = sG[col + 1];
        const float a0 = col < row_a ? -d3[4 * i] * fast_exp(g_a - gc0) : 0.f;
        const float a1 = col + 1 < row_a ? -d3[4 * i + 1] * fast_exp(g_a - gc1) : 0.f;
        const float b0 = col < row_b ? -d3[4 * i + 2] * fast_exp(g_b - gc0) : 0.f;
        const float b1 = col + 1 < row_b ? -d3[4 * i + 3] * fast_exp(g_b - gc1) : 0.f;
        st_tile64(OFF_D3, row_a, col, a0, a1);
        st_tile64(OFF_D3, row_b, col, b0, b1);
        st_tile64(OFF_D3B, row_a, col, beta_a * a0, beta_a * a1);
        st_tile64(OFF_D3B, row_b, col, beta_b * b0, beta_b * b1);
        const float s0 = a0 * beta_a * kk[4 * i], s1 = a1 * beta_a * kk[4 * i + 1];
        const float s2 = b0 * beta_b * kk[4 * i + 2], s3 = b1 * beta_b * kk[4 * i + 3];
        rs_a += s0 + s1;
        rs_b += s2 + s3;
        const float c0 = col_sum(s0 + s2), c1 = col_sum(s1 + s3);
        if (lane < 4) {
          atomicAdd(sDg + col, -c0);
          atomicAdd(sDg + col + 1, -c1);
        }
      }
      rs_a = quad_sum(rs_a);
      rs_b = quad_sum(rs_b);
      if ((lane & 3) == 0) {
        atomicAdd(sDg + row_a, rs_a);
        atomicAdd(sDg + row_b, rs_b);
      }
    }
    round_sync();
    stamp();

    // ======================= round 5: dA3 K and (beta dA3)^T K =======================
    if (ok && tid == 0) {
      umma_group<4, 2, 0, 128, 0, false>(tmem + T_T3, d3_lo, kmn_lo, ID_KM_128);
      umma_group<4, 128, 0, 128, 0, false>(tmem + T_DK5, d3bmn_lo, kmn_lo, ID_MM_128);
      umma_commit(&bars[BAR_MMA]);
    }
    ok = ok && wait_mma();
    stamp();
    if (ok) {
      float t3[16], x[16];
      tmem_ld_16x32(tmem + lanes + T_T3 + c128, t3);
      tmem_ld_16x32(tmem + lanes + T_DK5 + c128, x);
      tmem_ld_wait();
      float sa = 0.f, sb = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = c128 + 8 * i + cp;
        const float2 k_a = tile2(OFF_K, row_a, col), k_b = tile2(OFF_K, row_b, col);
        sa += k_a.x * t3[4 * i] + k_a.y * t3[4 * i + 1];
        sb += k_b.x * t3[4 * i + 2] + k_b.y * t3[4 * i + 3];
        if (wr_a)
          *reinterpret_cast<uint32_t*>(p.dk + out_a + col) =
              pack_bf16(dkacc[4 * i] + beta_a * t3[4 * i] + x[4 * i], dkacc[4 * i + 1] + beta_a * t3[4 * i + 1] + x[4 * i + 1]);
        if (wr_b)
          *reinterpret_cast<uint32_t*>(p.dk + out_b + col) =
              pack_bf16(dkacc[4 * i + 2] + beta_b * t3[4 * i + 2] + x[4 * i + 2], dkacc[4 * i + 3] + beta_b * t3[4 * i + 3] + x[4 * i + 3]);
      }
      sa = quad_sum(sa);
      sb = quad_sum(sb);
      if ((lane & 3) == 0) {
        atomicAdd(sDb + row_a, sa);
        atomicAdd(sDb + row_b, sb);
      }
    }
    tc_fence_before();
    ok = __syncthreads_and(ok);  // a wait given up by one thread ends the loop for all of them
    tc_fence_after();
    stamp();
    if (ok && tid == 0 && has_next) load_c(nxt);  // k, A of this item are dead
    if (tid < valid) {
      float dgv = sDg[tid];
      if (tid == valid - 1) {  // the only reader of the chunk total also clears it for the next item
        dgv += *sDgLast;
        *sDgLast = 0.f;
      }
      p.dg[(cur.row0 + tid) * p.Hv + cur.hv] = dgv;
      p.db[(cur.row0 + tid) * p.Hv + cur.hv] = sDb[tid];
    }
    cur = nxt;
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
  if (tid == 0 && (*abort_flag || !ok)) atomicCAS(&g_bwd_main_status, 0, 1);
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

}  // namespace fqla
extern "C" int fqla_debug_bwd_main_profile(long long* out16) {
  return (int)cudaMemcpyFromSymbol(out16, fqla::g_bwd_main_profile, sizeof(long long) * 16);
}
namespace fqla {

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D bf16 tensor map, rows x cols (row-major), box = 64 columns x box_rows rows, 128-byte swizzle
int make_tile_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, int box_rows) {
  static EncodeTiledFn2 fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess)
      f = nullptr;
    return (EncodeTiledFn2)f;
  }();
  if (!fn) return FQLA_ERR_INVALID_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                  box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FQLA_ERR_INVALID_ARG;
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
  static const bool profile = getenv("FQLA_PROFILE") != nullptr;
  p.profile = profile;
  rc = configure_smem(tiled ? (const void*)bwd_main_tc_kernel<true> : (const void*)bwd_main_tc_kernel<false>,
                      SMEM_BYTES);
  if (rc != 0) return rc;
  static const int n_sm = [] {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }();
  const long long total = n_chunks * Hv;
  const unsigned grid = (unsigned)(total < n_sm ? total : n_sm);
  if (tiled)
    bwd_main_tc_kernel<true><<<grid, NT, SMEM_BYTES, st>>>(p, mq, mk, mv, mvn, mdo, mdu, mh, mdh, ma);
  else
    bwd_main_tc_kernel<false><<<grid, NT, SMEM_BYTES, st>>>(p, mq, mk, mv, mvn, mdo, mdu, mh, mdh, ma);
  return (int)cudaGetLastError();
}

}  // namespace fqla
