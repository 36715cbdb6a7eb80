/*
 * libfqla_sm100 - C ABI of the B200 (sm_100a) gated-delta-rule chunked-prefill kernels.
 *
 * This is the boundary a host framework binds to.  The reference project (QwenLM/FlashQLA)
 * has no native boundary: its kernels are TileLang functions called from Python.  Each entry
 * point below replaces one of those Python-level kernel wrappers; the wrapper it replaces is
 * cited by its path inside the reference project.
 *
 * Conventions
 *   - All pointers are device pointers unless said otherwise; the caller owns every buffer,
 *     the library never allocates.  Work is enqueued on `stream` (a cudaStream_t passed as
 *     void*) of the current device and the call returns at once.
 *   - Return value: 0 on success, a negative FQLA_ERR_* for arguments rejected on the host
 *     before any launch, or a positive cudaError_t reported by the launch.
 *   - Token axis: q, k are [B, T, Hq, D]; v, o, do, dv, vnew, du are [B, T, Hv, D]; g, beta,
 *     dg, db are [B, T, Hv]; A is [B, T, Hv, 64].  All bf16 except g/dg/db (fp32) and beta
 *     (bf16, or fp32 when beta_is_f32 != 0).  Hv must be a multiple of Hq; D is 64 or 128.
 *   - Packed variable-length input: B == 1, `cu_seqlens` [N+1] gives the sequence boundaries,
 *     `chunk_offsets` [N+1] the exclusive prefix sum of ceil(len/64), `chunk_indices`
 *     [num_chunks, 2] the (sequence, chunk-in-sequence) of every chunk.  The three tables share
 *     one integer type: int64 when idx_is64 != 0, else int32.  With cu_seqlens == NULL the
 *     input is B sequences of T rows and the tables are ignored.
 *   - States ([N, Hv, D, D], fp32) are indexed [key dim][value dim].  Per-chunk states h/dh are
 *     [total chunks, Hv, D, D] bf16.
 *   - g_cum is always the chunk-local cumulative sum of the log gates.
 */
#ifndef FQLA_H_
#define FQLA_H_

#ifdef __cplusplus
extern "C" {
#endif

#define FQLA_OK 0
#define FQLA_ERR_INVALID_ARG (-1)
#define FQLA_ERR_UNSUPPORTED_DIM (-2)
#define FQLA_ERR_TOO_LARGE (-3)

/* ABI version, bumped on any signature change. */
int fqla_version(void);
/* Human-readable text for a return value of this library (static storage). */
const char* fqla_status_string(int status);

/* Chunk-local prefix sum (reverse != 0: suffix sum) of g [B,T,H] fp32.
 * Replaces chunk_local_cumsum, flash_qla/ops/utils/cumsum.py:137-171. */
int fqla_chunk_local_cumsum(const float* g, float* out, int B, int T, int H,
                            const void* cu_seqlens, int idx_is64, int N,
                            const void* chunk_indices, long long num_chunks, int reverse,
                            void* stream);

/* A = (I + strict_lower(diag(beta) K K^T * exp(g_s - g_t)))^-1 per (chunk, value head); row t of
 * A holds row (t mod 64) of its chunk's matrix.
 * Replaces kkt_solve, flash_qla/ops/gated_delta_rule/chunk/blackwell/kkt_solve.py:284-324
 * (this library folds the gate into A, as the reference's tests/ref_gdr.py:77-140 does).
 * g_cum_out (optional): when given, g_cum is taken as the RAW per-token log gate and its
 * chunk-local cumulative sum (what fqla_chunk_local_cumsum computes) is formed in the same
 * kernel and written to g_cum_out on the rows that belong to sequences. */
int fqla_kkt_solve(const void* k, const void* beta, int beta_is_f32, const float* g_cum,
                   float* g_cum_out, void* A, int B, int T, int Hq, int Hv, int D,
                   const void* cu_seqlens, int idx_is64, const void* chunk_indices,
                   long long num_chunks, void* stream);

/* Sequential forward recurrence.  Optional outputs (NULL to skip): o, per-chunk states h,
 * vnew (the delta-rule corrected values, needed by the backward), final state ht, and the
 * transition matrix M (state_end = state_end|zero start + M state_start).  q may be NULL when
 * o is.  warm_chunks [N,Hv] (int32, optional, state-only calls): walk only the last
 * warm_chunks[n,hv] chunks of each sequence from a zero state.  m_mask [N,Hv] (int32,
 * optional): compute M only where non-zero.  operand_tiles != 0 (K = V = 128, no M, no
 * warm_chunks): h and vnew are written in the layout the backward kernels consume as tensor-core
 * operands, h as [chunks, Hv, V, K] (each state transposed) and vnew as [chunks, Hv, V, 64]
 * (each chunk transposed, rows past the sequence end zero); FQLA_ERR_UNSUPPORTED_DIM otherwise.
 * warm_chunks < 0 for a (sequence, head): nothing is computed or written for it.
 * lead_chunks [N,Hv] (int32, optional, K = V = 128, not together with warm_chunks, M, m_mask):
 * lead-in of a segment of a longer sequence.  Where lead_chunks[n,hv] > 0 the walk starts that
 * many chunks BEFORE the segment (those rows are the tail of the segment before it) from a zero
 * state, state-only, and only then enters the segment: the start state needs no separate pass.
 * h0 is ignored for such a (segment, head); outputs cover the segment's own rows only.  The
 * segment must start a whole number of chunks after the start of the sequence it was cut from
 * (A and g_cum are chunk-local quantities of that sequence) and at least lead_chunks[n,hv]
 * chunks after it.
 * seq_order [N] (int32, optional; a permutation of 0..N-1): the CTAs of block index i / Hv walk
 * sequence seq_order[i].  Blocks start in index order, so listing the longest sequences first
 * shortens the tail of a ragged batch; the results do not depend on it.
 * run_mask [N,Hv] (int32, optional) with run_value: only the (sequence, head) pairs with
 * run_mask[n,hv] == run_value are walked; nothing of the others is read or written, so two calls
 * with complementary values can fill one set of output buffers at different times.
 * Replaces fused_gdr_fwd (blackwell/fused_fwd.py:775-915) and fused_gdr_h
 * (blackwell/prepare_h.py:669-784). */
int fqla_fwd_seq(const void* q, const void* k, const void* v, const void* A, const float* g_cum,
                 const void* beta, int beta_is_f32, const float* h0, float* ht, void* o, void* h,
                 void* vnew, float* M, const int* warm_chunks, const int* m_mask,
                 const int* lead_chunks, const int* seq_order, const int* run_mask, int run_value,
                 int B, int T, int Hq, int Hv, int D, float scale, const void* cu_seqlens,
                 const void* chunk_offsets, int idx_is64, int N, int operand_tiles, void* stream);

/* Sequential reverse recurrence of the state gradient.  Optional outputs: per-chunk dh, du (the
 * gradient of vnew), dh0.  warm_chunks (optional, dh0-only calls): walk only the first
 * warm_chunks[n,hv] chunks from a zero gradient.  operand_tiles != 0 (K = V = 128, no
 * warm_chunks): dh is written as [chunks, Hv, V, K] and du as [chunks, Hv, V, 64], the operand
 * layouts of fqla_fwd_seq's h and vnew; FQLA_ERR_UNSUPPORTED_DIM otherwise.  lead_chunks
 * (optional, [N, Hv] int32, K = V = 128, not with warm_chunks): the mirror image of
 * fqla_fwd_seq's lead_chunks; sequence n is a segment of a longer sequence, whose following rows
 * belong to segment n + 1, and starts lead_chunks[n,hv] chunks after its end from a zero
 * gradient (dht is ignored for it) instead of being handed one; such a segment must end on a
 * chunk boundary, and segment n + 1 must hold at least lead_chunks[n,hv] chunks (its last one
 * may be partial).  seq_order, run_mask, run_value: as for fqla_fwd_seq.
 * Replaces fused_gdr_dh_ws (blackwell/cp_bwd.py:592-701) and the dS chain of fused_gdr_bwd
 * (blackwell/fused_bwd.py:336-474). */
int fqla_bwd_dh(const void* q, const void* k, const void* A, const float* g_cum, const void* beta,
                int beta_is_f32, const void* dO, const float* dht, void* dh, void* du, float* dh0,
                const int* warm_chunks, const int* lead_chunks, const int* seq_order,
                const int* run_mask, int run_value, int B, int T, int Hq, int Hv, int D,
                float scale, const void* cu_seqlens, const void* chunk_offsets, int idx_is64, int N,
                int operand_tiles, void* stream);

/* Chunk-parallel backward: dq, dk (per VALUE head, [B,T,Hv,D] bf16), dv, dbeta and the
 * pre-cumsum dg (both fp32 [B,T,Hv]) from h, dh, vnew and du.  operand_tiles != 0 (K = V = 128):
 * h, dh, vnew and du are in the operand layouts written by fqla_fwd_seq / fqla_bwd_dh with the
 * same flag.
 * Replaces the per-chunk body of fused_gdr_bwd (blackwell/fused_bwd.py:1325-1413). */
int fqla_bwd_main(const void* q, const void* k, const void* v, const void* vnew, const void* A,
                  const float* g_cum, const void* beta, int beta_is_f32, const void* dO,
                  const void* du, const void* h, const void* dh, void* dq, void* dk, void* dv,
                  float* db, float* dg, int B, int T, int Hq, int Hv, int D, float scale,
                  const void* cu_seqlens, const void* chunk_offsets, const void* chunk_indices,
                  int idx_is64, long long num_chunks, int operand_tiles, void* stream);

/* out[row, hq, :] = sum over the G value heads of group hq of in[row, hq*G + i, :] (bf16, fp32
 * accumulation).  Replaces group_reduce_vector, flash_qla/ops/utils/group_reduce.py:60-79. */
int fqla_group_reduce(const void* in, void* out, long long rows, int Hq, int G, int D,
                      void* stream);

/* Per (segment, head): number of chunks, counted from the segment end (from_start == 0) or start
 * (from_start != 0), after which the accumulated log gate is below `threshold`; fallback = 1
 * where the whole segment does not get there.  seg_cu_seqlens [n_seg+1].  keep (int32 [n_seg]
 * or NULL): segments with keep == 0 are skipped and get warm = fallback = 0 (the last segment of
 * a sequence hands nothing forward, the first nothing backward).
 * Replaces get_warmup_chunks / get_warmup_chunks_bidi, blackwell/cp_fwd.py:81-115, :224-264. */
int fqla_warmup_scan(const float* g_cum, int T, int Hv, const void* seg_cu_seqlens, int idx_is64,
                     int n_seg, float threshold, int from_start, const int* keep, int* warm,
                     int* fallback, void* stream);

/* Chain segment states of each raw sequence (segments seg_begin[r] .. seg_begin[r+1]-1):
 * reverse == 0: out[first] = raw[r] (or 0); out[i+1] = local[i] + use_m[i,hv] * M[i]   out[i]
 * reverse != 0: out[last]  = raw[r] (or 0); out[i-1] = local[i] + use_m[i,hv] * M[i]^T out[i]
 * All states fp32 [*, Hv, D, D]; use_m int32 [n_seg, Hv] or NULL (always apply M).
 * any_fallback (int32 [n_raw, Hv] or NULL, from fqla_segment_scan): where 0, only the edge
 * segment's entry of out is written (raw[r] or 0) and the chain is skipped.
 * seg_stride: 0 for packed local, M and use_m; otherwise the distance, in 4-byte words, between
 * the entries of consecutive segments in each of the three (they then point into the records of
 * one gathered buffer: no copy into packed tensors is needed).  raw and out are always packed.
 * Replaces correct_initial_states / correct_terminal_states, blackwell/cp_fwd.py:483-610. */
int fqla_merge_states(const float* local, const float* M, const int* use_m, const float* raw,
                      const int* seg_begin, const int* any_fallback, float* out, int n_raw, int Hv,
                      int D, int reverse, long long seg_stride, void* stream);

/* Row-wise L2 normalisation (the optional pre-op of q and k): y = x * rsqrt(sum x^2 + eps) in
 * the dtype of x, rstd [rows] fp32; and its gradient dx = (dy - <dy, y> y) * rstd, fp32.
 * Rows are contiguous, D even and <= 512.  dtype codes: 0 bf16, 1 fp16, 2 fp32.
 * Replaces l2norm_fwd / l2norm_bwd, flash_qla/utils/math.py:22-67 (torch.compile'd expressions
 * in the reference). */
int fqla_l2norm_fwd(const void* x, void* y, float* rstd, long long rows, int D, int dtype,
                    float eps, void* stream);
int fqla_l2norm_bwd(const void* y, const float* rstd, const void* dy, float* dx, long long rows,
                    int D, int y_dtype, int dy_dtype, void* stream);

/* The scan of fqla_warmup_scan for a whole split plan in one launch, plus the decision how each
 * segment gets its start state.  seg_begin [n_raw+1] (int32): first segment of every raw
 * sequence.  Outputs, all int32: warm, fallback [n_seg,Hv] as for fqla_warmup_scan (the segment
 * that hands nothing on gets 0 / 0); any_fallback [n_raw,Hv]: some segment of this (sequence,
 * head) never reaches the threshold; lead [n_seg,Hv]: where any_fallback is 0, the number of
 * chunks of the neighbouring segment (the one before it, forward; after it, from_start != 0) the
 * recurrence kernel walks first from a zero state (lead_chunks of fqla_fwd_seq), else 0;
 * exact_warm [n_seg,Hv]: warm where any_fallback is 1, else -1 (the warm_chunks of the separate
 * state-only pass, which then skips the segment).  With any_fallback given, fqla_merge_states
 * only copies the edge state of sequences without a chain.
 * Replaces get_warmup_chunks / get_warmup_chunks_bidi and the bookkeeping of
 * intra_card_cp_preprocess, chunk/cp_context.py:148-227. */
int fqla_segment_scan(const float* g_cum, int T, int Hv, const void* seg_cu_seqlens, int idx_is64,
                      const int* seg_begin, int n_raw, float threshold, int from_start, int* warm,
                      int* fallback, int* lead, int* exact_warm, int* any_fallback, void* stream);

/* Forward (o and, optionally, the final state ht) for hosts that cannot allocate device memory
 * where they call this library: an inference engine that gave all device memory to its own arena
 * at start-up, so that a later cudaMalloc stalls the device or simply fails, or a plugin that
 * only receives pointers and a stream from its framework.  No counterpart in the reference (its
 * wrappers allocate with torch on every call).
 *
 * The two intermediates of the forward (the chunk-local cumulative gate and the matrix A, which
 * fqla_kkt_solve otherwise writes into caller buffers) live in a fixed array inside the library
 * image, 4.125 MiB that every GPU loading the library holds until the process exits.  The call
 * runs the same kernels as fqla_kkt_solve (raw gate form) followed by fqla_fwd_seq and performs
 * no cudaMalloc, cudaFree or other allocating call.
 *   - g is the RAW per-token log gate [B,T,Hv] fp32; q, k, v, beta, h0, ht, o and the index
 *     tables are as for fqla_fwd_seq / fqla_kkt_solve; ht may be NULL.
 *   - Limit: B * T * Hv <= fqla_fwd_noalloc_max_pairs() (32768, e.g. 2048 tokens x 16 value
 *     heads); larger calls return FQLA_ERR_TOO_LARGE and launch nothing.
 *   - The first call on each device looks the array's device address up (with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on one device share the array and it keeps the previous call's contents (what
 *     must be clean is cleared by the call itself).  Two calls that may run at the same time on
 *     the GPU, from different streams or threads, race on it: order them on one stream or with
 *     events. */
int fqla_fwd_noalloc(const void* q, const void* k, const void* v, const float* g,
                     const void* beta, int beta_is_f32, const float* h0, float* ht, void* o,
                     int B, int T, int Hq, int Hv, int D, float scale, const void* cu_seqlens,
                     const void* chunk_offsets, const void* chunk_indices, int idx_is64, int N,
                     long long num_chunks, void* stream);
long long fqla_fwd_noalloc_max_pairs(void);

/* Host call: reads (and with reset != 0 clears) the device-side status word of the current
 * device.  It is non-zero after a kernel abandoned a bounded wait on one of its barriers; the
 * outputs of that launch are then invalid.  Synchronises the device.  No counterpart in the
 * reference (its kernels wait without bound). */
int fqla_device_status(int* out, int reset);

/* Self-test of the failure path every tensor-core kernel of this library shares: launches one
 * tiny kernel whose single waiter gives up on a barrier that nothing arrives at, after `tries`
 * (1..100) bounded tries of at most 1 ms each.  The kernel returns by itself and leaves the
 * device status word set, so fqla_device_status then reports 1 until it is reset.  Nothing
 * faults, traps or hangs.  No counterpart in the reference (its kernels wait without bound). */
int fqla_selftest_wait_timeout(int tries, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FQLA_H_ */
