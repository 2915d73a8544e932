// Beam-search step on the device, no host round trip:
//   beam_topk   one CTA of eight warps per (batch, beam) row: the row of int8 logits is streamed ONCE
//               with 16-byte loads, each warp taking every eighth 512-byte chunk; a 256-entry exp
//               table + float64 sums give the log-sum-exp, a warp-wide threshold + candidate buffer
//               per warp and a final merge give the exact top-k by (logit desc, token asc), emitted
//               with length-normalised scores.
//   beam_update one CTA per batch element: merges beam*beam candidates, rewrites the
//               token history and the KV-cache ancestry table in place (staged through
//               shared memory), updates probabilities/scores, counts finished beams and
//               advances the device-side step counter.
// Bookkeeping follows select_beam_rough_topk_i8I
// (lightseq/inference/kernels/transformerKernels_int8.cc.cu:1690-1844) and
// ker_refresh_result (lightseq/inference/kernels/transformerKernels.cc.cu:1398-1463);
// the rough threshold + global Thrust sort are replaced by an exact selection with a
// fixed tie-break (higher score, lower beam, lower token id).
#include <float.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"
#include "ctx.h"

namespace ls100 {

constexpr float LOGIT_THRESH_MIN = -64.f;   // lightseq/inference/kernels/transformerKernels.h:11
constexpr float MIN_LOG_PROB = -2000.f;     // transformerKernels.h:12
constexpr int MAX_BEAM = 8;

// One CTA per row, eight warps interleaved over the row's 512-byte chunks (a single warp per row leaves the
// machine idle and is bound by the latency of its one chunk in flight), ONE pass with 16-byte loads, two
// chunks per warp in flight. Per warp:
//  * sum of exp: every byte indexes a 256-entry table exp((q - 127) * s) in shared memory;
//    four independent fp32 partial sums per lane, combined in float64 at the end;
//  * top-k: the warp keeps ONE threshold (the k-th best value seen so far by the whole
//    warp). A 16-byte chunk is rejected with four SIMD byte compares; the rare bytes above
//    the threshold are appended (ballot-prefix, no atomics) to a shared-memory candidate
//    buffer of packed keys (value, then lower token id first), and when the buffer passes 32
//    entries the warp re-selects its k best with k arg-max rounds and raises the threshold.
//    Because the threshold reflects everything the warp has seen, only ~k*ln(V/k) bytes ever
//    take the slow path.
// log-sum-exp is taken relative to the largest representable logit (127 * s) instead of the
// row maximum; the reference's clamp of exp arguments at -64 can then never trigger, which
// the launcher enforces by requiring 254 * s <= 64.
constexpr int TOPK_WARPS = 8;
constexpr int TOPK_BUF = 512 + 64;  // one chunk can add 512 candidates while the threshold is still open

__device__ __forceinline__ int4 load_row16(const int8_t* lp, int off, int vocab) {
  if (off + 16 <= vocab) return *reinterpret_cast<const int4*>(lp + off);
  int w[4] = {(int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080};  // -128 = "no token"
  for (int j = 0; j < vocab - off; ++j) {
    const int byte = (int)(uint8_t)lp[off + j];
    w[j >> 2] = (w[j >> 2] & ~(0xff << ((j & 3) * 8))) | (byte << ((j & 3) * 8));
  }
  return make_int4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ unsigned topk_key(int val, int idx) {
  return ((unsigned)(val + 128) << 22) | (unsigned)(0x3fffff - idx);  // larger key = better candidate
}

// Re-selects the K best keys of buf[0 .. n) into buf[0 .. min(K, n)), best first. Returns the new
// threshold: the value of the K-th best, or -128 while fewer than K candidates exist.
template <int PER>
__device__ __forceinline__ int topk_flush_n(unsigned* buf, int n, int K, int lane, int* n_kept) {
  unsigned keys[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    keys[i] = (e < n) ? buf[e] : 0u;
  }
  __syncwarp();
  unsigned winner = 0;
  int thr = -128;
  for (int rnd = 0; rnd < K; ++rnd) {
    unsigned loc = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) loc = max(loc, keys[i]);
    unsigned best = loc;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if (best != 0u && loc == best) {  // keys are unique (token ids are), so exactly one lane owns it
#pragma unroll
      for (int i = 0; i < PER; ++i)
        if (keys[i] == best) keys[i] = 0u;
    }
    if (lane == rnd) winner = best;
    if (rnd == K - 1 && best != 0u) thr = (int)(best >> 22) - 128;
  }
  if (lane < K) buf[lane] = winner;
  __syncwarp();
  *n_kept = min(n, K);
  return thr;
}
// Almost every re-selection holds a few dozen keys (the current best K and the handful that passed the threshold
// since): two keys per lane then, the full buffer only after a chunk that arrived before any threshold existed.
__device__ __forceinline__ int topk_flush(unsigned* buf, int n, int K, int lane, int* n_kept) {
  if (n <= 64) return topk_flush_n<2>(buf, n, K, lane, n_kept);
  return topk_flush_n<(TOPK_BUF + 31) / 32>(buf, n, K, lane, n_kept);
}

__global__ void __launch_bounds__(32 * TOPK_WARPS) beam_topk_kernel(const ls100_beam_topk_args a) {
  __shared__ float s_lut[256];  // index = byte pattern (two's complement), value = exp((q - 127) * s); 0 for -128
  __shared__ unsigned s_buf[TOPK_WARPS][TOPK_BUF];
  __shared__ double s_sum[TOPK_WARPS];
  __shared__ int s_kept[TOPK_WARPS];
  __shared__ int s_thr;  // highest k-th-best value any warp of the row has established so far
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  if (threadIdx.x == 0) s_thr = -128;
  for (int i = threadIdx.x; i < 256; i += blockDim.x) {  // the table depends on the scale only: built before the wait
    const int q = (int)(int8_t)i;
    s_lut[i] = (q == -128) ? 0.f : expf(__fmul_rn((float)(q - 127), a.s_logits));
  }
  pdl_wait();
  __syncthreads();
  const int row = blockIdx.x;
  // this warp's first two chunks are requested before the step counter and the row's last token are known (a finished
  // row will not use them): the three reads then share one round trip instead of queueing behind each other
  const int8_t* lp = a.logits + (long long)row * a.ld_logits;
  const int4 none = make_int4((int)0x80808080, (int)0x80808080, (int)0x80808080, (int)0x80808080);
  int4 v1 = none, v2 = none;
  if (warp * 512 + lane * 16 < a.vocab) v1 = load_row16(lp, warp * 512 + lane * 16, a.vocab);
  if ((warp + TOPK_WARPS) * 512 + lane * 16 < a.vocab) v2 = load_row16(lp, (warp + TOPK_WARPS) * 512 + lane * 16, a.vocab);
  const int step = *a.step_ptr;
  const int K = a.beam;
  float* cs = a.cand_score + (long long)row * K;
  int32_t* ct = a.cand_token + (long long)row * K;
  if (step != 0 && a.alive[(long long)row * a.max_step + step] == a.end_id) {  // uniform over the CTA
    if (threadIdx.x < K) {  // a finished beam: one candidate, EOS, its frozen score (rank 0 of its row)
      cs[threadIdx.x] = (threadIdx.x == 0) ? __fsub_rn(a.seq_score[row], a.diverse_lambda) : -FLT_MAX;
      ct[threadIdx.x] = a.end_id;
    }
    return;
  }
  unsigned* buf = s_buf[warp];
  int n_buf = 0;   // entries in buf (the first ones are the current best list)
  int thr = -128;  // bytes strictly above thr are candidates
  unsigned add7 = 0x01010101u * 127u;
  float2 ps01 = make_float2(0.f, 0.f), ps23 = make_float2(0.f, 0.f);  // four running sums, added as two packed pairs
  const int n_chunks = (a.vocab + 511) / 512;
  // this warp's chunks: warp, warp + 8, ...; the next two are always in flight
  for (int ch = warp; ch < n_chunks; ch += TOPK_WARPS) {
    const int off = ch * 512 + lane * 16;
    const int4 v = v1;
    v1 = v2;
    v2 = none;
    if (off + 2 * TOPK_WARPS * 512 < a.vocab) v2 = load_row16(lp, off + 2 * TOPK_WARPS * 512, a.vocab);
    const unsigned w4[4] = {(unsigned)v.x, (unsigned)v.y, (unsigned)v.z, (unsigned)v.w};
    if (ch == warp) {
      // First chunk of this warp: without a threshold all of its 512 bytes would go through the candidate buffer.
      // The K-th largest of the 32 lanes' own maxima is a value that at least K bytes of the chunk reach, so
      // nothing below it can be among the row's K best (ties at it are kept: the test below is "strictly above").
      unsigned m = __vmaxs4(__vmaxs4(w4[0], w4[1]), __vmaxs4(w4[2], w4[3]));
      m = __vmaxs4(m, m >> 16);
      m = __vmaxs4(m, m >> 8);
      int cur = (int)(int8_t)(m & 0xffu), kth = -128;
      for (int r = 0; r < K; ++r) {
        kth = cur;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) kth = max(kth, __shfl_xor_sync(0xffffffffu, kth, o));
        const unsigned who = __ballot_sync(0xffffffffu, cur == kth);
        if (lane == __ffs(who) - 1) cur = -128;  // one instance leaves per round
      }
      if (kth - 1 > thr) {
        thr = kth - 1;
        add7 = 0x01010101u * (unsigned)(127 - max(thr, 0));
      }
    }
    {  // the other warps of the row raise the bar too: nothing below any warp's k-th best can be in the row's top k
      const int shared_thr = *((volatile int*)&s_thr);
      if (shared_thr > thr) {
        thr = shared_thr;
        add7 = 0x01010101u * (unsigned)(127 - max(thr, 0));
      }
    }
    // Bytes above the threshold. With thr >= 0 only bytes with a clear sign bit qualify and, for those, adding
    // (127 - thr) to the low seven bits carries into bit 7 exactly when the byte exceeds thr (no carry crosses a
    // byte): three logic/add operations per word. While thr < 0 every word goes to the exact path below.
    unsigned gt[4];
    unsigned hit = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      ps01 = f2_add(ps01, make_float2(s_lut[w4[w] & 0xff], s_lut[(w4[w] >> 8) & 0xff]));
      ps23 = f2_add(ps23, make_float2(s_lut[(w4[w] >> 16) & 0xff], s_lut[w4[w] >> 24]));
      gt[w] = ((w4[w] & 0x7f7f7f7fu) + add7) & ~w4[w] & 0x80808080u;
      hit |= gt[w];
    }
    if (thr < 0) hit = 1u;
    if (__ballot_sync(0xffffffffu, hit != 0u) != 0u) {  // rare once the threshold has risen, warp-uniform
      unsigned qbits = 0;
      if (thr < 0) {
        const unsigned thr4 = (unsigned)(thr & 0xff) * 0x01010101u;
#pragma unroll
        for (int w = 0; w < 4; ++w) gt[w] = __vcmpgts4(w4[w], thr4) & 0x80808080u;
      }
#pragma unroll
      for (int w = 0; w < 4; ++w)
        qbits |= (((gt[w] >> 7) & 1u) | ((gt[w] >> 14) & 2u) | ((gt[w] >> 21) & 4u) | ((gt[w] >> 28) & 8u)) << (w * 4);
      const int mine = __popc(qbits);
      int pre = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, pre, o);
        if (lane >= o) pre += t;
      }
      const int total = __shfl_sync(0xffffffffu, pre, 31);
      int pos = n_buf + pre - mine;
      unsigned bits = qbits;
      while (bits) {
        const int bpos = __ffs(bits) - 1;
        bits &= bits - 1;
        const int q = (int)(int8_t)((w4[bpos >> 2] >> ((bpos & 3) * 8)) & 0xff);
        buf[pos++] = topk_key(q, off + bpos);
      }
      n_buf += total;
      __syncwarp();
      if (n_buf > 32) {
        thr = max(thr, topk_flush(buf, n_buf, K, lane, &n_buf));
        add7 = 0x01010101u * (unsigned)(127 - max(thr, 0));
        // published one lower: another warp may hold an equal value at a lower token id, which wins the tie
        if (lane == 0) atomicMax(&s_thr, thr - 1);
      }
    }
  }
  __syncwarp();
  topk_flush(buf, n_buf, K, lane, &n_buf);
  double sum = ((double)ps01.x + (double)ps01.y) + ((double)ps23.x + (double)ps23.y);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) {
    s_sum[warp] = sum;
    s_kept[warp] = n_buf;
  }
  __syncthreads();
  if (warp != 0) return;
  // merge: the K best of the warps' K best (keys order by value, then lower token), sums in warp order
  int n_all = n_buf;  // warp 0's own list already sits at buf[0 .. n_buf)
  for (int w = 1; w < TOPK_WARPS; ++w) {
    const int nk = s_kept[w];
    if (lane < nk) buf[n_all + lane] = s_buf[w][lane];
    n_all += nk;
  }
  __syncwarp();
  topk_flush(buf, n_all, K, lane, &n_buf);
  double tot = 0.0;
  for (int w = 0; w < TOPK_WARPS; ++w) tot += s_sum[w];
  if (lane < K) {
    // log-sum-exp relative to 127*s:  lse = log(sum) + 127*s;  base = prefix - lse
    const float ref = __fmul_rn(127.f, a.s_logits);
    const float lse = __fadd_rn(logf((float)tot), ref);
    const float base = __fsub_rn(a.seq_probs[row], lse);
    const float ln = a.length_norm[step];
    if (lane >= n_buf) {
      cs[lane] = -FLT_MAX;
      ct[lane] = a.end_id;
    } else {
      const unsigned key = buf[lane];
      const int val = (int)(key >> 22) - 128;
      const float lg = __fmul_rn((float)val, a.s_logits);
      cs[lane] = __fsub_rn(fmaxf(__fmul_rn(__fadd_rn(lg, base), ln), MIN_LOG_PROB + 1.f),
                           __fmul_rn(a.diverse_lambda, (float)(lane + 1)));  // lane = rank of the candidate in its row
      ct[lane] = 0x3fffff - (int)(key & 0x3fffff);
    }
  }
}

// The same candidates as beam_topk_kernel, from the statistics the logits GEMM kept per (row, 64-column group) -
// the group's largest value and its sum of exponentials - so that the [rows, vocab] matrix is not read again:
//   1. lane = row: every warp walks a share of the row's groups (coalesced: the 128 rows of a row block are
//      contiguous), adds the sums and keeps the K largest group maxima; the eight warps' partial results meet in
//      shared memory. The K-th largest group maximum T of a row is a lower bound of its K-th best logit: at least K
//      groups hold a value >= T.
//   2. lane = row again: the groups whose maximum reaches T (a handful) are listed per row.
//   3. warp = row: only those groups' 64 bytes are read; values >= the running bound enter the candidate buffer of
//      beam_topk_kernel and the same selection picks the exact top K by (value desc, token asc).
// A CTA serves 32 rows. The scores are formed exactly as in beam_topk_kernel.
constexpr int SEL_ROWS = 32;
constexpr int SEL_WARPS = 8;
constexpr int SEL_LIST = 32;   // candidate groups listed per row (one per lane); a row with more reads every group, serially
constexpr int SEL_HITS = 128;  // candidate values buffered per row on the lane-parallel path

__global__ void __launch_bounds__(32 * SEL_WARPS) beam_select_kernel(const ls100_beam_select_args s) {
  const ls100_beam_topk_args& a = s.topk;
  __shared__ double s_sum[SEL_WARPS][SEL_ROWS];
  __shared__ signed char s_top[SEL_WARPS][SEL_ROWS][MAX_BEAM];
  __shared__ double s_total[SEL_ROWS];
  __shared__ int s_T[SEL_ROWS];
  __shared__ int s_cnt[SEL_ROWS];
  __shared__ unsigned short s_list[SEL_ROWS][SEL_LIST];
  __shared__ unsigned s_hits[SEL_ROWS][SEL_HITS];
  __shared__ int s_nhit[SEL_ROWS];
  __shared__ unsigned s_buf[SEL_WARPS][TOPK_BUF];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();
  const int rows = a.batch * a.beam;
  const int K = a.beam;
  const int G = s.n_groups;
  const int step = *a.step_ptr;
  const int row0 = blockIdx.x * SEL_ROWS;
  const int row = row0 + lane;
  const bool row_ok = row < rows;
  // statistics of row r live at ((r / 128) * G + g) * 128 + r % 128
  const long long base = row_ok ? ((long long)(row >> 7) * G) * 128 + (row & 127) : 0;
  {
    double sum = 0.0;
    int top[MAX_BEAM];
#pragma unroll
    for (int j = 0; j < MAX_BEAM; ++j) top[j] = -128;
    if (row_ok) {
      // eight groups per round, their loads issued together (one after the other they would each cost an L2 round trip)
      for (int g0 = warp; g0 < G; g0 += 8 * SEL_WARPS) {
        float sm[8];
        int mx[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int g = g0 + u * SEL_WARPS;
          const long long o = base + (long long)(g < G ? g : g0) * 128;
          sm[u] = s.stat_sum[o];
          mx[u] = (int)s.stat_max[o];
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (g0 + u * SEL_WARPS >= G) break;
          sum += (double)sm[u];
          int v = mx[u];
#pragma unroll
          for (int j = 0; j < MAX_BEAM; ++j) {  // sorted insertion, largest first
            const int hi = max(top[j], v);
            v = min(top[j], v);
            top[j] = hi;
          }
        }
      }
    }
    s_sum[warp][lane] = sum;
#pragma unroll
    for (int j = 0; j < MAX_BEAM; ++j) s_top[warp][lane][j] = (signed char)top[j];
    if (warp == 0) {
      s_cnt[lane] = 0;
      s_nhit[lane] = 0;
    }
  }
  __syncthreads();
  if (warp == 0) {
    double tot = 0.0;
    int top[MAX_BEAM];
#pragma unroll
    for (int j = 0; j < MAX_BEAM; ++j) top[j] = -128;
    for (int w = 0; w < SEL_WARPS; ++w) {
      tot += s_sum[w][lane];
      for (int i = 0; i < MAX_BEAM; ++i) {
        int v = (int)s_top[w][lane][i];
#pragma unroll
        for (int j = 0; j < MAX_BEAM; ++j) {
          const int hi = max(top[j], v);
          v = min(top[j], v);
          top[j] = hi;
        }
      }
    }
    s_total[lane] = tot;
    int T = -128;  // fewer than K groups: every group is a candidate
#pragma unroll
    for (int j = 0; j < MAX_BEAM; ++j)
      if (j == K - 1 && G >= K) T = top[j];
    s_T[lane] = T;
  }
  __syncthreads();
  if (row_ok) {
    const int T = s_T[lane];
    for (int g0 = warp; g0 < G; g0 += 8 * SEL_WARPS) {
      int mx[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int g = g0 + u * SEL_WARPS;
        mx[u] = g < G ? (int)s.stat_max[base + (long long)g * 128] : -129;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (mx[u] >= T) {
          const int pos = atomicAdd(&s_cnt[lane], 1);
          if (pos < SEL_LIST) s_list[lane][pos] = (unsigned short)(g0 + u * SEL_WARPS);
        }
      }
    }
  }
  __syncthreads();
  unsigned* buf = s_buf[warp];
  for (int rl = warp; rl < SEL_ROWS; rl += SEL_WARPS) {
    const int r = row0 + rl;
    if (r >= rows) break;
    float* cs = a.cand_score + (long long)r * K;
    int32_t* ct = a.cand_token + (long long)r * K;
    if (step != 0 && a.alive[(long long)r * a.max_step + step] == a.end_id) {  // a finished beam: EOS, its frozen score
      if (lane < K) {
        cs[lane] = (lane == 0) ? __fsub_rn(a.seq_score[r], a.diverse_lambda) : -FLT_MAX;
        ct[lane] = a.end_id;
      }
      continue;
    }
    const int8_t* lp = a.logits + (long long)r * a.ld_logits;
    const int n_list = s_cnt[rl];
    int thr = s_T[rl];  // values >= thr are candidates (ties included: the selection orders them by token)
    int n_buf = 0;
    bool serial = n_list > SEL_LIST;
    if (!serial) {
      // lane-parallel: every lane reads one candidate group (64 bytes, one round trip for the whole row) and appends its
      // values >= thr to the row's list; a list that would overflow sends the row down the serial path instead
      if (lane < n_list) {
        const int g = (int)s_list[rl][lane];
        const int off0 = g * 64;
        unsigned w[16];
        if (off0 + 64 <= a.vocab && ((a.ld_logits & 15) == 0)) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 v4 = *reinterpret_cast<const uint4*>(lp + off0 + c * 16);
            w[c * 4] = v4.x;
            w[c * 4 + 1] = v4.y;
            w[c * 4 + 2] = v4.z;
            w[c * 4 + 3] = v4.w;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            unsigned word = 0x80808080u;
            for (int e = 0; e < 4; ++e) {
              const int o = off0 + c * 4 + e;
              if (o < a.vocab) word = (word & ~(0xffu << (8 * e))) | ((unsigned)(uint8_t)lp[o] << (8 * e));
            }
            w[c] = word;
          }
        }
        const unsigned thr4 = (unsigned)(thr & 0xff) * 0x01010101u;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          unsigned ge = __vcmpges4(w[c], thr4) & 0x80808080u;
          while (ge) {
            const int e = (__ffs(ge) - 1) >> 3;
            ge &= ge - 1;
            const int o = off0 + c * 4 + e;
            if (o < a.vocab) {
              const int pos = atomicAdd(&s_nhit[rl], 1);
              if (pos < SEL_HITS) s_hits[rl][pos] = topk_key((int)(int8_t)((w[c] >> (8 * e)) & 0xff), o);
            }
          }
        }
      }
      __syncwarp();
      const int nh = s_nhit[rl];
      if (nh <= SEL_HITS) {
        for (int i = lane; i < nh; i += 32) buf[i] = s_hits[rl][i];
        n_buf = nh;
        __syncwarp();
      } else {
        serial = true;
      }
    }
    if (serial) {
      const bool all_groups = n_list > SEL_LIST;
      const int n_scan = all_groups ? G : n_list;
      for (int i = 0; i < n_scan; ++i) {
        const int g = all_groups ? i : (int)s_list[rl][i];
        const int off = g * 64 + lane * 2;
        int q0 = -128, q1 = -128;
        if (off + 1 < a.vocab) {
          const short two = *reinterpret_cast<const short*>(lp + off);
          q0 = (int)(int8_t)(two & 0xff);
          q1 = (int)(int8_t)((two >> 8) & 0xff);
        } else if (off < a.vocab) {
          q0 = (int)lp[off];
        }
        const bool h0 = q0 >= thr && off < a.vocab, h1 = q1 >= thr && off + 1 < a.vocab;
        const int mine = (h0 ? 1 : 0) + (h1 ? 1 : 0);
        int pre = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, pre, o);
          if (lane >= o) pre += t;
        }
        const int total = __shfl_sync(0xffffffffu, pre, 31);
        if (total == 0) continue;
        int pos = n_buf + pre - mine;
        if (h0) buf[pos++] = topk_key(q0, off);
        if (h1) buf[pos++] = topk_key(q1, off + 1);
        n_buf += total;
        __syncwarp();
        if (n_buf > TOPK_BUF - 64) {  // at most 64 entries per group: the buffer never overflows
          const int t2 = topk_flush(buf, n_buf, K, lane, &n_buf);
          thr = max(thr, t2);
        }
      }
    }
    __syncwarp();
    topk_flush(buf, n_buf, K, lane, &n_buf);
    if (lane < K) {
      const float ref = __fmul_rn(127.f, a.s_logits);
      const float lse = __fadd_rn(logf((float)s_total[rl]), ref);
      const float base_lp = __fsub_rn(a.seq_probs[r], lse);
      const float ln = a.length_norm[step];
      if (lane >= n_buf) {
        cs[lane] = -FLT_MAX;
        ct[lane] = a.end_id;
      } else {
        const unsigned key = buf[lane];
        const int val = (int)(key >> 22) - 128;
        const float lg = __fmul_rn((float)val, a.s_logits);
        cs[lane] = __fsub_rn(fmaxf(__fmul_rn(__fadd_rn(lg, base_lp), ln), MIN_LOG_PROB + 1.f),
                             __fmul_rn(a.diverse_lambda, (float)(lane + 1)));
        ct[lane] = 0x3fffff - (int)(key & 0x3fffff);
      }
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(128) beam_update_kernel(const ls100_beam_update_args a) {
  extern __shared__ int stage[];  // [2][K][max_step]
  __shared__ int s_parent[MAX_BEAM], s_token[MAX_BEAM];
  __shared__ float s_score[MAX_BEAM];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, t = threadIdx.x;
  const int K = a.beam;
  const int step = *a.step_ptr;
  const int ms = a.max_step;
  int* st_alive = stage;
  int* st_anc = stage + K * ms;
  if (t < 32) {
    // best K of K*K candidates by (score desc, beam asc, token asc). Candidate c = beam * K + rank is already in
    // (beam asc, then logit desc / token asc) order, so "lower c" is the tie-break. Lane t holds c = t and t + 32.
    const float* cs = a.cand_score + (long long)b * K * K;
    const int32_t* ct = a.cand_token + (long long)b * K * K;
    const int n = K * K;
    float sc0 = (t < n) ? cs[t] : -INFINITY, sc1 = (t + 32 < n) ? cs[t + 32] : -INFINITY;
    const int tk0 = (t < n) ? ct[t] : 0, tk1 = (t + 32 < n) ? ct[t + 32] : 0;
    bool used0 = !(t < n), used1 = !(t + 32 < n);
    for (int j = 0; j < K; ++j) {
      float my = -INFINITY;
      int myc = 0x7fffffff;
      if (!used0) {
        my = sc0;
        myc = t;
      }
      if (!used1 && (sc1 > my || myc == 0x7fffffff)) {
        my = sc1;
        myc = t + 32;
      }
      float best = my;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
      int bc = (myc != 0x7fffffff && my == best) ? myc : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) bc = min(bc, __shfl_xor_sync(0xffffffffu, bc, o));
      if (bc == t) used0 = true;
      if (bc == t + 32) used1 = true;
      const int owner = bc & 31;
      const int tok = __shfl_sync(0xffffffffu, bc < 32 ? tk0 : tk1, owner);
      if (t == 0) {
        s_parent[j] = bc / K;
        s_token[j] = tok;
        // candidates competed with the diversity penalty of their rank in their row; what is stored is the score itself
        s_score[j] = __fadd_rn(best, __fmul_rn(a.diverse_lambda, (float)(bc % K + 1)));
      }
    }
  }
  int* alive_b = a.alive + (long long)b * K * ms;
  int* anc_b = a.anc ? a.anc + (long long)b * K * ms : nullptr;
  for (int i = t; i < K * ms; i += 128) {
    const int p = i % ms;
    if (p <= step) {
      st_alive[i] = alive_b[i];
      if (anc_b) st_anc[i] = anc_b[i];
    }
  }
  __syncthreads();
  for (int i = t; i < K * ms; i += 128) {
    const int j = i / ms, p = i % ms;
    const int par = s_parent[j];
    if (p <= step) {
      alive_b[i] = st_alive[par * ms + p];
      if (anc_b) anc_b[i] = (p < step) ? st_anc[par * ms + p] : (b * K + par);
    } else if (p == step + 1) {
      alive_b[i] = s_token[j];
    }
  }
  if (t == 0) {
    const float ln = a.length_norm[step];
    int fin = 0;
    for (int j = 0; j < K; ++j) {
      a.seq_score[b * K + j] = s_score[j];
      if (s_token[j] != a.end_id) a.seq_probs[b * K + j] = __fdiv_rn(s_score[j], ln);
      else ++fin;
    }
    atomicAdd(a.fin_count + step, fin);
    __threadfence();
    const int ticket = atomicAdd(a.ticket + step, 1);
    if (ticket == (int)gridDim.x - 1) {
      const int total = atomicAdd(a.fin_count + step, 0);
      if (total == (int)gridDim.x * K) {
        if (atomicCAS(a.stop_step, -1, step) == -1 && a.stop_host) *((volatile int*)a.stop_host) = step;
      }
      *a.step_ptr = step + 1;
    }
  }
}

// Writes the result of a finished generation from the beam state (one CTA per output row):
//   mode 0  beam 0 of every sentence, tokens at positions 1 .. n_out, its score
//           (ker_write_trg_tokenid_pos_penalty, lightseq/inference/kernels/transformerKernels.cc.cu:1722-1733)
//   mode 1  the beam with the best score / (number of non-EOS tokens + 1e-12), for a negative length penalty when
//           the generation stopped early (ker_write_trg_tokenid_neg_penalty, :1752-1784); ties keep the lower beam
//   mode 2  every beam, the last position forced to EOS (ker_write_topk_result, :1803-1813)
__global__ void __launch_bounds__(128) beam_write_result_kernel(const ls100_beam_result_args a) {
  __shared__ int s_pick;
  __shared__ float s_best;
  pdl_launch_dependents();
  pdl_wait();
  const int K = a.beam, ms = a.max_step, n = a.n_out;
  const int row_out = blockIdx.x;
  int src_row;
  if (a.mode == 2) {
    src_row = row_out;
  } else if (a.mode == 0) {
    src_row = row_out * K;
  } else {
    if (threadIdx.x < 32) {
      int pick = 0;
      float best = -INFINITY;
      for (int j = 0; j < K; ++j) {  // beams in order: an equal later score does not replace an earlier one
        const int32_t* seq = a.alive + ((long long)row_out * K + j) * ms + 1;
        int len = 0;
        for (int p = threadIdx.x; p < n; p += 32) len += (seq[p] != a.end_id) ? 1 : 0;
        len = warp_sum_i(len);
        const float sc = __fdiv_rn(a.seq_score[row_out * K + j], __fadd_rn((float)len, 1e-12f));
        if (sc > best) {
          best = sc;
          pick = j;
        }
      }
      if (threadIdx.x == 0) {
        s_pick = pick;
        s_best = best;
      }
    }
    __syncthreads();
    src_row = row_out * K + s_pick;
  }
  const int32_t* seq = a.alive + (long long)src_row * ms + 1;
  int32_t* out = a.out_tokens + (long long)row_out * n;
  for (int p = threadIdx.x; p < n; p += blockDim.x) out[p] = (a.mode == 2 && p == n - 1) ? a.end_id : seq[p];
  if (threadIdx.x == 0) a.out_scores[row_out] = (a.mode == 1) ? s_best : a.seq_score[src_row];
}

}  // namespace ls100

using namespace ls100;

extern "C" int ls100_beam_write_result(ls100_ctx* ctx, const ls100_beam_result_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->alive || !a->seq_score || !a->out_tokens || !a->out_scores) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->max_step <= 1 || a->n_out <= 0 || a->n_out >= a->max_step) return LS100_ERR_BAD_ARG;
  if (a->mode < 0 || a->mode > 2) return LS100_ERR_BAD_ARG;
  if (a->beam > MAX_BEAM) return LS100_ERR_UNSUPPORTED;
  const int rows = a->mode == 2 ? a->batch * a->beam : a->batch;
  return ls100_launch(beam_write_result_kernel, dim3(rows), dim3(128), 0, (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_beam_topk(ls100_ctx* ctx, const ls100_beam_topk_args* a, ls100_stream_t stream_) {
  if (!ctx || !a || !a->logits || !a->step_ptr || !a->length_norm || !a->alive || !a->seq_probs || !a->seq_score ||
      !a->cand_score || !a->cand_token)
    return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->vocab <= 0 || a->max_step <= 0 || !(a->s_logits > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->beam > MAX_BEAM || a->vocab < a->beam || a->vocab > (1 << 22)) return LS100_ERR_UNSUPPORTED;
  if (254.f * a->s_logits > 64.f) return LS100_ERR_UNSUPPORTED;  // the -64 clamp of the reference would matter
  if ((((uintptr_t)a->logits) & 15) || (a->ld_logits & 15)) return LS100_ERR_ALIGN;
  const int rows = a->batch * a->beam;
  return ls100_launch(beam_topk_kernel, dim3(rows), dim3(32 * TOPK_WARPS), 0,
                      (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

// Argument checks of the beam update; `need_scratch` is false when the caller's fin_count / ticket pointers are
// going to be replaced by the library's own scratch. Nothing is enqueued before these pass.
static int beam_update_check(const ls100_ctx* ctx, const ls100_beam_update_args* a, bool need_scratch) {
  if (!ctx || !a || !a->cand_score || !a->cand_token || !a->step_ptr || !a->length_norm || !a->alive || !a->seq_probs ||
      !a->seq_score || !a->stop_step)
    return LS100_ERR_BAD_ARG;
  if (need_scratch && (!a->fin_count || !a->ticket)) return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->max_step <= 0) return LS100_ERR_BAD_ARG;
  if (a->beam > MAX_BEAM) return LS100_ERR_UNSUPPORTED;
  if ((size_t)2 * a->beam * a->max_step * sizeof(int) > 48 * 1024) return LS100_ERR_UNSUPPORTED;
  return LS100_OK;
}

extern "C" int ls100_beam_select(ls100_ctx* ctx, const ls100_beam_select_args* s, ls100_stream_t stream_) {
  if (!ctx || !s || !s->stat_max || !s->stat_sum) return LS100_ERR_BAD_ARG;
  const ls100_beam_topk_args* a = &s->topk;
  if (!a->logits || !a->step_ptr || !a->length_norm || !a->alive || !a->seq_probs || !a->seq_score || !a->cand_score ||
      !a->cand_token)
    return LS100_ERR_BAD_ARG;
  if (a->batch <= 0 || a->beam <= 0 || a->vocab <= 0 || a->max_step <= 0 || !(a->s_logits > 0.f)) return LS100_ERR_BAD_ARG;
  if (a->beam > MAX_BEAM || a->vocab < a->beam || a->vocab > (1 << 22)) return LS100_ERR_UNSUPPORTED;
  if (254.f * a->s_logits > 64.f) return LS100_ERR_UNSUPPORTED;
  if (s->n_groups != (a->vocab + 63) / 64 || s->n_groups > 65535) return LS100_ERR_BAD_ARG;
  if ((((uintptr_t)a->logits) & 1) || (a->ld_logits & 1)) return LS100_ERR_ALIGN;
  const int rows = a->batch * a->beam;
  return ls100_launch(beam_select_kernel, dim3((rows + SEL_ROWS - 1) / SEL_ROWS), dim3(32 * SEL_WARPS), 0,
                      (cudaStream_t)stream_, *s) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

extern "C" int ls100_beam_update(ls100_ctx* ctx, const ls100_beam_update_args* a, ls100_stream_t stream_) {
  const int rc = beam_update_check(ctx, a, true);
  if (rc != LS100_OK) return rc;
  const size_t smem = (size_t)2 * a->beam * a->max_step * sizeof(int);
  return ls100_launch(beam_update_kernel, dim3(a->batch), dim3(128), smem, (cudaStream_t)stream_, *a) == cudaSuccess
             ? LS100_OK
             : LS100_ERR_CUDA;
}

// ------------------------------------------------------------------ allocation-free variant
// Scratch of ls100_beam_update_noalloc: the per-step finished counters and CTA tickets that
// ls100_beam_update takes from the caller. Lives in the library image: every GPU that loads
// libls100.so holds these 8 KB until the process exits.
static __device__ __align__(256) int32_t g_noalloc_scratch[2 * LS100_BEAM_UPDATE_NOALLOC_MAX_STEP];

namespace {
std::mutex g_noalloc_mu;
int32_t* g_noalloc_ptr[64] = {nullptr};  // device address of g_noalloc_scratch, per device ordinal
}  // namespace

extern "C" int ls100_beam_update_noalloc(ls100_ctx* ctx, const ls100_beam_update_args* a, ls100_stream_t stream_) {
  if (!ctx || !a) return LS100_ERR_BAD_ARG;
  if (a->max_step > LS100_BEAM_UPDATE_NOALLOC_MAX_STEP) {
    fprintf(stderr, "ls100_beam_update_noalloc: max_step %d exceeds the built-in scratch (limit %d); use ls100_beam_update "
                    "with caller-provided fin_count/ticket arrays\n", a->max_step, LS100_BEAM_UPDATE_NOALLOC_MAX_STEP);
    return LS100_ERR_UNSUPPORTED;
  }
  {  // every other argument is checked before anything is enqueued: a rejected call leaves the stream and the scratch alone
    const int rc = beam_update_check(ctx, a, false);
    if (rc != LS100_OK) return rc;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) return LS100_ERR_CUDA;
  if (dev != ctx->device || dev < 0 || dev >= 64) return LS100_ERR_BAD_ARG;  // the context's device must be current
  int32_t* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      // In host code the array's name is only a handle for the runtime, not a device address:
      // ask the runtime for the address on the current device, once per device.
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || !p) return LS100_ERR_CUDA;
      g_noalloc_ptr[dev] = static_cast<int32_t*>(p);
    }
    scratch = g_noalloc_ptr[dev];
  }
  cudaStream_t stream = (cudaStream_t)stream_;
  // The array keeps whatever the previous call left in it; the counters must start at zero.
  if (cudaMemsetAsync(scratch, 0, sizeof(int32_t) * 2 * LS100_BEAM_UPDATE_NOALLOC_MAX_STEP, stream) != cudaSuccess)
    return LS100_ERR_CUDA;
  ls100_beam_update_args b = *a;
  b.fin_count = scratch;
  b.ticket = scratch + LS100_BEAM_UPDATE_NOALLOC_MAX_STEP;
  return ls100_beam_update(ctx, &b, stream_);
}

