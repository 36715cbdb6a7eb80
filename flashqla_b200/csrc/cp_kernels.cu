// Context-parallel helpers: when a sequence is cut into segments (inside one GPU, or across GPUs
// along T), every segment first computes its end state from a zero start ("local" state) and,
// where the gates do not let the past die out, the exact transition matrix M of the segment, so
// that   state_end = local + M * state_start.   The kernels here
//   * decide per (segment, head) how many trailing (forward) or leading (backward) chunks are
//     needed before the accumulated log-gate drops below a threshold, and
//   * chain the segments of each sequence:  start[i+1] = local[i] + M[i] start[i]  (forward) or
//     end[i-1] = local[i] + M[i]^T end[i]  (backward, for the state gradient).
// They replace the reference's blackwell/cp_fwd.py:10-221 (get_warmup_chunks, _bidi) and
// :268-480 (correct_h0, also used transposed for dht).
#include "common.cuh"
#include "fqla_internal.h"

namespace fqla {

// Whole-warp scan of one (segment, head).  Walks the chunk totals (the cumsum value on each
// chunk's last row) from the segment end backwards (forward pass) or from its start forwards
// (backward pass), 32 chunks per step: the lanes load in parallel, a warp prefix sum finds the
// first crossing.  Returns the chunk count in every lane; `reached` tells whether the threshold
// was crossed inside the segment.
__device__ __forceinline__ int scan_segment(const float* __restrict__ g_cum, int Hv, int hv,
                                            const SeqSpan sp, float threshold, int from_start,
                                            int lane, bool& reached_out) {
  float carry = 0.f;
  int n = sp.n_chunks;
  bool reached = false;
  for (int base = 0; base < sp.n_chunks && !reached; base += 32) {
    const int i = base + lane;
    const bool in = i < sp.n_chunks;
    float x = 0.f;
    if (in) {
      const int c = from_start ? i : sp.n_chunks - 1 - i;
      const int last_row = min(sp.len, (c + 1) * CHUNK) - 1;
      x = g_cum[(sp.bos + last_row) * Hv + hv];
    }
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    const unsigned hit = __ballot_sync(0xffffffffu, in && carry + x < threshold);
    if (hit) {
      n = base + __ffs(hit);
      reached = true;
    }
    carry += __shfl_sync(0xffffffffu, x, 31);
  }
  reached_out = reached;
  return n;
}

// One warp per (segment, head).  keep (optional, [n_seg]): segments with keep == 0 hand nothing
// on; they get warm = fallback = 0.
__global__ void __launch_bounds__(128)
warmup_scan_kernel(const float* __restrict__ g_cum, int Hv, SeqLayout lay, int n_seg,
                   float threshold, int from_start, const int* __restrict__ keep,
                   int* __restrict__ warm, int* __restrict__ fallback) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= n_seg * Hv) return;
  const int seg = item / Hv, hv = item % Hv;
  if (keep && keep[seg] == 0) {
    if (lane == 0) warm[item] = fallback[item] = 0;
    return;
  }
  bool reached;
  const int n = scan_segment(g_cum, Hv, hv, lay.span(seg), threshold, from_start, lane, reached);
  if (lane == 0) {
    warm[item] = n;
    fallback[item] = reached ? 0 : 1;
  }
}

// The scan for a whole split plan in one launch: one CTA per (raw sequence, head), its warps take
// the segments of that sequence in turn.  Besides warm / fallback per (segment, head) (same
// meaning as above; the segment that hands nothing on, last of its sequence forward or first
// backward, gets 0 / 0) it decides HOW each segment gets its start state:
//   * no segment of this (sequence, head) fell back (any_fb = 0): the recurrence kernel of segment
//     i simply starts lead[i] chunks early from a zero state (lead-in, forward: lead[i] =
//     warm[i - 1]; backward: lead[i] = warm[i + 1]); no local states, no merge chain;
//     exact_warm = -1 tells the separate state-only pass to skip the segment;
//   * otherwise (any_fb = 1) lead = 0 everywhere and exact_warm = warm: the state-only pass,
//     the transition matrices and the merge chain produce the exact start states.
__global__ void __launch_bounds__(256)
segment_scan_kernel(const float* __restrict__ g_cum, int Hv, SeqLayout lay,
                    const int* __restrict__ seg_begin, float threshold, int from_start,
                    int* __restrict__ warm, int* __restrict__ fallback, int* __restrict__ lead,
                    int* __restrict__ exact_warm, int* __restrict__ any_fb) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = blockIdx.x / Hv, hv = blockIdx.x % Hv;
  const int s0 = seg_begin[r], s1 = seg_begin[r + 1];
  int fb_any = 0;
  for (int seg = s0 + warp; seg < s1; seg += 8) {
    const bool hands_on = from_start ? seg > s0 : seg + 1 < s1;
    int n = 0;
    bool reached = true;
    if (hands_on) n = scan_segment(g_cum, Hv, hv, lay.span(seg), threshold, from_start, lane, reached);
    if (lane == 0) {
      warm[seg * Hv + hv] = n;
      fallback[seg * Hv + hv] = reached ? 0 : 1;
    }
    fb_any |= reached ? 0 : 1;
  }
  const int any = __syncthreads_or(fb_any);  // also orders the writes above for the reads below
  if (threadIdx.x == 0) any_fb[r * Hv + hv] = any;
  for (int seg = s0 + threadIdx.x; seg < s1; seg += blockDim.x) {
    const int giver = from_start ? seg + 1 : seg - 1;  // the segment whose tail/head leads in
    const bool has = from_start ? giver < s1 : giver >= s0;
    lead[seg * Hv + hv] = (!any && has) ? warm[giver * Hv + hv] : 0;
    exact_warm[seg * Hv + hv] = any ? warm[seg * Hv + hv] : -1;
  }
}

// Chain the segments of one raw sequence for one head and one 32-wide value slice.
// grid = (D/32, Hv, n_raw), 128 threads for D = 128 (thread a owns row a of the slice).
//   forward  (reverse = 0): out[first] = start_raw; out[i+1] = local[i] + useM[i] * M[i]   out[i]
//   backward (reverse = 1): out[last]  = end_raw;   out[i-1] = local[i] + useM[i] * M[i]^T out[i]
template <int D>
__global__ void __launch_bounds__(D) merge_kernel(const float* __restrict__ local,
                                                  const float* __restrict__ M,
                                                  const int* __restrict__ use_m,
                                                  const float* __restrict__ raw,
                                                  const int* __restrict__ seg_begin,
                                                  const int* __restrict__ any_fb,
                                                  float* __restrict__ out, int Hv, int reverse,
                                                  long long seg_stride, long long use_stride) {
  // seg_stride / use_stride: distance in 4-byte words between the entries of consecutive
  // segments in local and M / in use_m (packed tensors, or the records of a gathered buffer);
  // raw and out are always packed
  constexpr int BV = 32, BK = 32, LDC = BV + 1;
  // all global traffic is one 128-byte row segment per warp instruction; the padded row stride
  // keeps both the row-wise (warp = row) and the thread-owns-a-row accesses free of bank conflicts
  __shared__ float cur[D * LDC];
  // one staging buffer: the local state of the step, then D x BK panels of M, forward [a][j]
  // (row stride BK+1), reverse [j][a]
  __shared__ float panel[D * (BK + 1)];
  const int a = threadIdx.x, lane = a & 31, warp = a >> 5;
  const int v0 = blockIdx.x * BV, hv = blockIdx.y, r = blockIdx.z;
  const int s0 = seg_begin[r], s1 = seg_begin[r + 1];  // segments [s0, s1)
  if (s1 <= s0) return;
  auto state = [&](const float* base, int seg) {
    return base + (((long long)seg * Hv + hv) * D) * D;
  };
  auto strided = [&](const float* base, int seg) {
    return base + (long long)seg * seg_stride + ((long long)hv * D) * D;
  };
  if (any_fb && any_fb[r * Hv + hv] == 0) {
    // no chain for this (sequence, head): the recurrence kernel leads in by itself; only the
    // edge segment needs a state (the sequence's own initial state or final-state gradient)
    const float* src = raw ? state(raw, r) : nullptr;
    float* dst = const_cast<float*>(state(out, reverse ? s1 - 1 : s0));
    for (int row = warp; row < D; row += D / 32)
      dst[(long long)row * D + v0 + lane] = src ? src[(long long)row * D + v0 + lane] : 0.f;
    return;
  }
  // initial value
  {
    const float* src = raw ? state(raw, r) : nullptr;
    for (int row = warp; row < D; row += D / 32)
      cur[row * LDC + lane] = src ? src[(long long)row * D + v0 + lane] : 0.f;
  }
  __syncthreads();
  const int n = s1 - s0;
  // the local state (and the flag) of the next step are fetched one step ahead into registers:
  // the chain itself then only waits for shared memory
  constexpr int RPW = D / (D / 32);  // rows per warp
  float pre[RPW];
  int pre_m = 0;
  auto prefetch = [&](int step) {
    const int i = reverse ? s1 - 1 - step : s0 + step;
    const float* loc = strided(local, i);
#pragma unroll
    for (int t = 0; t < RPW; ++t) pre[t] = loc[(long long)(warp + t * (D / 32)) * D + v0 + lane];
    pre_m = use_m == nullptr ? 1 : use_m[(long long)i * use_stride + hv];
  };
  if (n > 1) prefetch(0);
  for (int step = 0; step < n; ++step) {
    const int i = reverse ? s1 - 1 - step : s0 + step;
    float* dst = const_cast<float*>(state(out, i));
    for (int row = warp; row < D; row += D / 32) dst[(long long)row * D + v0 + lane] = cur[row * LDC + lane];
    if (step == n - 1) break;
#pragma unroll
    for (int t = 0; t < RPW; ++t) panel[(warp + t * (D / 32)) * LDC + lane] = pre[t];
    const bool with_m = pre_m != 0;
    if (step + 1 < n - 1) prefetch(step + 1);
    __syncthreads();
    float acc[BV];
#pragma unroll
    for (int j = 0; j < BV; ++j) acc[j] = panel[a * LDC + j];
    if (with_m) {
      const float* m = strided(M, i);
      for (int b0 = 0; b0 < D; b0 += BK) {
        __syncthreads();  // the previous contents of the panel have been consumed
        if (!reverse) {
          // panel[a'][j] = M[a'][b0+j], one warp per row, coalesced
          for (int row = warp; row < D; row += D / 32)
            panel[row * (BK + 1) + lane] = m[(long long)row * D + b0 + lane];
        } else {
          // panel[j][a'] = M[b0+j][a']
          for (int j = 0; j < BK; ++j) panel[j * D + a] = m[(long long)(b0 + j) * D + a];
        }
        __syncthreads();
#pragma unroll 4
        for (int j = 0; j < BK; ++j) {
          float w = reverse ? panel[j * D + a] : panel[a * (BK + 1) + j];
#pragma unroll
          for (int vv = 0; vv < BV; ++vv) acc[vv] += w * cur[(b0 + j) * LDC + vv];
        }
      }
    }
    __syncthreads();  // every read of cur (and of the panel) is done
#pragma unroll
    for (int j = 0; j < BV; ++j) cur[a * LDC + j] = acc[j];
    __syncthreads();
  }
}

}  // namespace fqla

using namespace fqla;

extern "C" int fqla_warmup_scan(const float* g_cum, int T, int Hv, const void* seg_cu_seqlens,
                                int idx_is64, int n_seg, float threshold, int from_start,
                                const int* keep, int* warm, int* fallback, void* stream) {
  if (!g_cum || !seg_cu_seqlens || !warm || !fallback || Hv <= 0) return FQLA_ERR_INVALID_ARG;
  if (n_seg <= 0) return FQLA_OK;
  SeqLayout lay{{seg_cu_seqlens, idx_is64}, {seg_cu_seqlens, idx_is64}, T};
  const long long items = (long long)n_seg * Hv;
  warmup_scan_kernel<<<(unsigned)((items + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
      g_cum, Hv, lay, n_seg, threshold, from_start, keep, warm, fallback);
  return (int)cudaGetLastError();
}

extern "C" int fqla_segment_scan(const float* g_cum, int T, int Hv, const void* seg_cu_seqlens,
                                 int idx_is64, const int* seg_begin, int n_raw, float threshold,
                                 int from_start, int* warm, int* fallback, int* lead,
                                 int* exact_warm, int* any_fb, void* stream) {
  if (!g_cum || !seg_cu_seqlens || !seg_begin || !warm || !fallback || !lead || !exact_warm ||
      !any_fb || Hv <= 0)
    return FQLA_ERR_INVALID_ARG;
  if (n_raw <= 0) return FQLA_OK;
  SeqLayout lay{{seg_cu_seqlens, idx_is64}, {seg_cu_seqlens, idx_is64}, T};
  segment_scan_kernel<<<(unsigned)(n_raw * Hv), 256, 0, (cudaStream_t)stream>>>(
      g_cum, Hv, lay, seg_begin, threshold, from_start, warm, fallback, lead, exact_warm, any_fb);
  return (int)cudaGetLastError();
}

extern "C" int fqla_merge_states(const float* local, const float* M, const int* use_m,
                                 const float* raw, const int* seg_begin, const int* any_fb,
                                 float* out, int n_raw, int Hv, int D, int reverse,
                                 long long seg_stride, void* stream) {
  if (!local || !M || !seg_begin || !out || Hv <= 0 || seg_stride < 0) return FQLA_ERR_INVALID_ARG;
  if (n_raw <= 0) return FQLA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 128) {
    merge_kernel<128><<<dim3(128 / 32, Hv, n_raw), 128, 0, st>>>(
        local, M, use_m, raw, seg_begin, any_fb, out, Hv, reverse,
        seg_stride ? seg_stride : (long long)Hv * D * D, seg_stride ? seg_stride : Hv);
  } else if (D == 64) {
    merge_kernel<64><<<dim3(64 / 32, Hv, n_raw), 64, 0, st>>>(
        local, M, use_m, raw, seg_begin, any_fb, out, Hv, reverse,
        seg_stride ? seg_stride : (long long)Hv * D * D, seg_stride ? seg_stride : Hv);
  } else {
    return FQLA_ERR_UNSUPPORTED_DIM;
  }
  return (int)cudaGetLastError();
}
