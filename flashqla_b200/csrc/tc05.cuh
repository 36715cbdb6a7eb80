// Blackwell (sm_100a) building blocks: mbarrier, TMA (cp.async.bulk.tensor), tensor memory and
// tcgen05.mma wrappers, shared-memory matrix descriptors and the 128-byte swizzle used for every
// tensor-core operand tile in this library.
//
// Operand tile convention ("SW128 tile"): rows of 64 bf16 (128 bytes); 8 consecutive rows form a
// 1024-byte swizzle atom in which the 16-byte chunk c of row r is stored at chunk c ^ (r & 7).
// A tile base must be 1024-byte aligned.  This is exactly what TMA writes for a box of 64 bf16
// columns with CU_TENSOR_MAP_SWIZZLE_128B.  Wider matrices are stored as consecutive 64-column
// blocks (block stride = rows * 128 bytes).
//   * As a K-major operand (contraction along the 64 columns): SBO = 1024; a K step of 16
//     elements advances the start address by 32 bytes inside the block.
//   * As an MN-major operand (contraction along the rows): LBO = block stride, SBO = 1024; a
//     K step of 16 rows advances the start address by 2048 bytes.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace fqla {
namespace tc {

__device__ __forceinline__ uint32_t s32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- swizzle -------------------------------------------------------------------------------
// byte offset inside an SW128 tile of element (row, col), col in [0,64)
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
  return (uint32_t)(row * 128 + ((((col >> 3) ^ (row & 7)) << 4) | ((col & 7) << 1)));
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)),
               "r"(bytes)
               : "memory");
}
// One try: the thread is suspended by the hardware until the phase completes or the time hint
// (nanoseconds) runs out; no instructions are issued meanwhile, so waiting warps do not take
// issue slots from the warps they share a scheduler with.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(s32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Non-blocking test of a phase (about 13 cycles on B200 when the phase is complete; the bounded
// loop around the suspending form was measured at about 200 cycles even then).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(s32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: at most `budget` tries of up to 1 ms each.  Gives up as soon as *abort_flag
// (shared memory) is set; on its own timeout it sets *abort_flag so that every other role of the
// CTA leaves too.  Returns false when the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          volatile int* abort_flag, uint32_t budget = 2000) {
  if (mbar_test_wait(bar, parity)) return true;  // fast path: the phase is already complete
  // not unrolled: a kernel has dozens of wait sites and is larger than the instruction cache
#pragma unroll 1
  for (uint32_t i = 0; i < budget; ++i) {
    if (mbar_try_wait(bar, parity, 1000000u)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// Four 8 x 8 bf16 matrices from registers to shared memory, each stored TRANSPOSED: register i of
// lane l carries the elements (row l/4, columns 2(l%4), +1) of matrix i - the layout of an
// mma / 16x256b tensor-memory fragment - and lands at (row 2(l%4) + {0,1}, column l/4) of the
// stored matrix, whose row r (16 bytes) starts at the address given by lane 8i + r.
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t saddr, uint32_t r0, uint32_t r1,
                                                  uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(saddr),
               "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}

// The same bounded wait for a thread that is alone in its warp and on the critical path: it polls
// (about 13 cycles per test) for a while before it lets the hardware suspend it, because waking
// from the suspended form costs several hundred cycles.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity,
                                               volatile int* abort_flag) {
#pragma unroll 1
  for (int i = 0; i < 2048; ++i)
    if (mbar_test_wait(bar, parity)) return true;
  return mbar_wait(bar, parity, abort_flag);
}

// ---- proxy / tcgen05 fences ------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA -----------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%2, %3}], [%4];" ::"r"(s32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(s32(bar))
      : "memory");
}
// Tile store shared -> global (bulk async group of the issuing thread).  The shared-memory tile
// must have been written, fenced (fence.proxy.async) and handed over to the issuing thread.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y,
                                             const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map),
               "r"(x), "r"(y), "r"(s32(smem_src))
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// every store group committed so far by this thread has finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// ... and has been written to global memory
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------
// One warp allocates `ncols` (power of two >= 32) columns; the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(slot)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// 32 lanes x 32 consecutive columns -> 32 registers per thread (thread = lane of its warp's
// quarter of the tensor memory: warp w may only touch lanes 32*(w%4) .. 32*(w%4)+31).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 16 lanes x 64 consecutive columns spread over the 32 threads of a warp (the natural read of an
// M = 64 accumulator quarter): register 4i+e of lane l holds row l/4 + 8*(e>>1), column
// 8*i + 2*(l%4) + (e&1).  `taddr` names the first of the 16 lanes.
__device__ __forceinline__ void tmem_ld_16x64(uint32_t taddr, float (&v)[32]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 consecutive columns -> 16 registers per thread
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31]), "r"(taddr)
      : "memory");
}
// 32 lanes x 16 consecutive columns from 16 registers per thread (e.g. 32 packed bf16 per lane)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::"r"(r[0]),
      "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor for an SW128 tile (see the convention at the top).
//   bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset
//   >> 4, [46,48) version = 1, [61,64) layout type = 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint64_t desc_kmajor(const void* tile) {
  return smem_desc(s32(tile), 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor(const void* tile, uint32_t block_stride_bytes) {
  return smem_desc(s32(tile), block_stride_bytes, 1024);
}

// Instruction descriptor for kind::f16 with bf16 inputs and fp32 accumulation.
//   bits [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format, 15 A major
//   (0 = K, 1 = MN), 16 B major, [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                     uint32_t idesc, bool accumulate) {
  uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
      : "memory");
}
// Lean issue form.  Every descriptor of an SW128 tile has the same high word (SBO = 1024,
// version 1, 128-byte swizzle); the low word is (address >> 4) | (LBO >> 4) << 16, so a K step
// is one 32-bit add on a per-tile base kept in a register.  Few, mutually independent
// instructions per MMA matter: the issuing thread shares its scheduler with three busy warps
// and pays a scheduling delay for every dependent instruction.
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_kmajor(const void* tile) {
  return ((s32(tile) >> 4) & 0x3FFF) | (1u << 16);
}
__device__ __forceinline__ uint32_t desc_lo_mnmajor(const void* tile, uint32_t block_stride_bytes) {
  return ((s32(tile) >> 4) & 0x3FFF) | ((block_stride_bytes >> 4) << 16);
}
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                        uint32_t idesc) {
  if (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, 1, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(DESC_HI), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(DESC_HI), "r"(idesc)
        : "memory");
  }
}
// One product: NK K-steps; operand low words advance by A_STEP / B_STEP (units of 16 bytes) per
// step, plus A_BLK / B_BLK after every fourth step (next 64-column block of a K-major operand).
template <int NK, int A_STEP, int A_BLK, int B_STEP, int B_BLK, bool ACC_FIRST>
__device__ __forceinline__ void umma_group(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                           uint32_t idesc) {
#pragma unroll
  for (int j = 0; j < NK; ++j) {
    const uint32_t a = a_lo + (uint32_t)((j & 3) * A_STEP + (j >> 2) * A_BLK);
    const uint32_t b = b_lo + (uint32_t)((j & 3) * B_STEP + (j >> 2) * B_BLK);
    if (j == 0 && !ACC_FIRST) umma_lo<false>(d_tmem, a, b, idesc);
    else umma_lo<true>(d_tmem, a, b, idesc);
  }
}

// ---- A operand in tensor memory ("TS" form) -------------------------------------------------------
// The A matrix [M = 128 rows][K] sits in tensor memory: lane = row, one 32-bit column holds the
// two bf16 elements k = 2c (low half) and k = 2c + 1 (high half); a K step of 16 elements is 8
// columns.  It is written there with tcgen05.st by the thread that owns the lane.  B comes from
// shared memory as usual.  The product reads no shared memory for A: the tensor pipe, whose rate
// in the SS form is set by the 128 B/clk operand fetch, runs at its arithmetic rate.
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                           uint32_t idesc) {
  if (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, 1, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(DESC_HI), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(DESC_HI), "r"(idesc)
        : "memory");
  }
}
// NK K-steps; A advances A_COLS columns per step, B by B_STEP descriptor units (16 bytes) per step
// (an MN-major B tile: 128 = 16 rows; a K-major B tile of one 64-column block: 2).
template <int NK, int A_COLS, int B_STEP, bool ACC_FIRST>
__device__ __forceinline__ void umma_ts_group(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                              uint32_t idesc) {
#pragma unroll
  for (int j = 0; j < NK; ++j) {
    if (j == 0 && !ACC_FIRST) umma_ts_lo<false>(d_tmem, a_tmem, b_lo, idesc);
    else umma_ts_lo<true>(d_tmem, a_tmem + (uint32_t)(j * A_COLS), b_lo + (uint32_t)(j * B_STEP), idesc);
  }
}
// B = a K-major tile of NK / 4 blocks of 64 columns (block stride 8192 bytes), fresh accumulator.
template <int NK>
__device__ __forceinline__ void umma_ts_group_kmajor_b(uint32_t d_tmem, uint32_t a_tmem,
                                                       uint32_t b_lo, uint32_t idesc) {
#pragma unroll
  for (int j = 0; j < NK; ++j) {
    const uint32_t b = b_lo + (uint32_t)((j & 3) * 2 + (j >> 2) * 512);
    if (j == 0) umma_ts_lo<false>(d_tmem, a_tmem, b, idesc);
    else umma_ts_lo<true>(d_tmem, a_tmem + (uint32_t)(j * 8), b, idesc);
  }
}

// mbarrier arrives (count 1) once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   s32(bar))
               : "memory");
}

}  // namespace tc
}  // namespace fqla
