// Pieces of the decode scorer that other kernels reuse (the sampled-threshold kernel, the exact
// re-scoring of a row inside the selector): parameters, query quantisation, the plain per-token score.
#pragma once
#include "common.cuh"

namespace kvb {

constexpr int SC_THREADS = 128;                  // generic kernel
constexpr int SC_HIST_BITS = 12;
constexpr int SC_HIST_BINS = 1 << SC_HIST_BITS;
constexpr int SC_MAX_C = 128;
constexpr int SC_MAX_G = 16;
constexpr int SC_COUNT_STRIDE = 32;              // words between per-row counters (one 128-byte line each)
constexpr int SC_EMIT_WARP_BUF = 512;            // composites a warp buffers per row segment before one global reservation
constexpr int SC_EMIT_BUF = 8 * SC_EMIT_WARP_BUF; // per CTA (8 warps)
// SAMPLE: the plain mode over the sample tiles of every row only (see fs_sample_geometry); the group maxima go,
// compacted, to the start of the row's gmax workspace.
enum { SC_MODE_PLAIN = 0, SC_MODE_HIST = 1, SC_MODE_EMIT = 2, SC_MODE_SAMPLE = 3 };

// ---- the sample that sets a row's candidate threshold ----------------------------------------
constexpr int FS_THREADS = 512;
constexpr int FS_RUNS = 32;                    // evenly spaced runs of sampled tokens per row
constexpr int FS_PER_THREAD = 8;                // sampled tokens per thread for rows up to FS_LONG_ROW (4096 per row) ...
constexpr int FS_PER_THREAD_LONG = 16;          // ... beyond it (8192 per row) ...
constexpr int FS_PER_THREAD_MAX = 32;           // ... and beyond twice that (16384 per row); loaded four at a time
constexpr int FS_LONG_ROW = 262144;
// (the sample stays at least 1/64 of the row up to a million tokens, so the rank that sets the threshold stays
// near 1.75 k / 64 and its relative spread near 10 %)
__host__ __device__ inline int fs_per_thread(int T) {
  return T > 2 * FS_LONG_ROW ? FS_PER_THREAD_MAX : (T > FS_LONG_ROW ? FS_PER_THREAD_LONG : FS_PER_THREAD);
}

// The sample as tiles of the streaming scorer (tile = TW tokens): FS_RUNS runs of `grp` consecutive tiles whose
// starts are `stride` tiles apart; n_sample = FS_RUNS * grp * TW tokens (<= T whenever T >= FS_RUNS * run tokens,
// which the fast path requires).
__host__ __device__ inline void fs_sample_geometry(int T, int TW, int& grp, int& stride, int& n_sample) {
  int run_tokens = fs_per_thread(T) * (FS_THREADS / FS_RUNS);     // 128, 256 or 512
  if (run_tokens < TW) run_tokens = TW;
  grp = run_tokens / TW;
  stride = (T / FS_RUNS) / TW;
  if (stride < grp) stride = grp;
  n_sample = FS_RUNS * grp * TW;
}


struct ScoreParams {
  const __nv_bfloat16* query;
  int64_t q_sb, q_sh;
  const uint8_t* packed;
  int64_t packed_sb, packed_sh;
  const float* scale;
  int64_t scale_sb, scale_sh;
  const int32_t* channel_idx;
  int B, Hq, Hkv, T, D, C, G;      // T: history length, or its upper bound (= row pitch of gmax) when T_dev is set
  const int32_t* T_dev;            // optional: the history length lives on the device (graph replays with a growing cache)
  float* gmax_out;
  int32_t* acc_out;
  float* deq_out;
  uint32_t* hist_out;
  // candidate emission (fused decode step): tokens whose group max reaches tau[row] are appended
  // to cand[row] as composites; cand_count[row * SC_COUNT_STRIDE] counts them (may exceed cand_cap)
  const float* tau;
  uint64_t* cand;
  uint32_t* cand_count;
  int cand_cap;
  int units_per_row;     // full tiles per row + 1 if the row has a ragged tail
  int full_tiles;        // T / tile tokens
  int64_t total_units;   // rows * units_per_row
};

// Quantise the G query heads of one KV head to int8 codes (shared memory) and per-head scales.
// All threads of the CTA take part; ends with a __syncthreads().
template <int NTHREADS>
__device__ __forceinline__ void quantize_query_group(const ScoreParams& p, int b, int g, int G, float* s_qv /*[G*C]*/,
                                                     int8_t* s_qcode /*[G*C]*/, float* s_qscale /*[G]*/) {
  const int tid = threadIdx.x;
  const int C = p.C;
  const int32_t* ch = p.channel_idx + (int64_t)g * C;
  for (int i = tid; i < G * C; i += NTHREADS) {
    const int hd = i / C, c = i - hd * C;
    const __nv_bfloat16* qrow = p.query + (int64_t)b * p.q_sb + (int64_t)(g * G + hd) * p.q_sh;
    s_qv[i] = __bfloat162float(qrow[ch[c]]);
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  for (int hd = warp; hd < G; hd += NTHREADS / 32) {
    float amax = 0.0f;
    for (int c = lane; c < C; c += 32) amax = fmaxf(amax, fabsf(s_qv[hd * C + c]));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float qs = __fdiv_rn(fmaxf(amax, 5.9604644775390625e-08f /* 2^-24 */), 127.0f);
    if (lane == 0) s_qscale[hd] = qs;
    for (int c = lane; c < C; c += 32) {
      float r = rintf(__fdiv_rn(s_qv[hd * C + c], qs));
      r = fminf(fmaxf(r, -127.0f), 127.0f);
      s_qcode[hd * C + c] = (int8_t)(int)r;
    }
  }
  __syncthreads();
}

// One token scored the plain way (byte loads): the ragged tail of a row and the generic kernel.
// Returns the group maximum (with -0 folded into +0); writes acc/deq when asked.
template <int GMAX>
__device__ __forceinline__ float score_token_plain(const ScoreParams& p, int G, int b, int g, int64_t t,
                                                   const int8_t* s_qcode, const float* s_qscale) {
  const int C = p.C;
  const uint8_t* src = p.packed + (int64_t)b * p.packed_sb + (int64_t)g * p.packed_sh + t * (C >> 1);
  int acc[GMAX];
#pragma unroll
  for (int hd = 0; hd < GMAX; ++hd) acc[hd] = 0;
  for (int j = 0; j < (C >> 1); ++j) {
    const int byte = src[j];
    const int lo = (int)((int8_t)(byte << 4)) >> 4;
    const int hi = (int)((int8_t)(byte & 0xF0)) >> 4;
#pragma unroll
    for (int hd = 0; hd < GMAX; ++hd) {
      if (hd < G) acc[hd] += lo * (int)s_qcode[hd * C + 2 * j] + hi * (int)s_qcode[hd * C + 2 * j + 1];
    }
  }
  const float ks = p.scale[(int64_t)b * p.scale_sb + (int64_t)g * p.scale_sh + t];
  float best = -INFINITY;
#pragma unroll
  for (int hd = 0; hd < GMAX; ++hd) {
    if (hd < G) {
      const float d = __fmul_rn(__fmul_rn((float)acc[hd], ks), s_qscale[hd]);
      best = fmaxf(best, d);
      const int64_t o = ((int64_t)b * p.Hq + (int64_t)g * G + hd) * p.T + t;
      if (p.acc_out) p.acc_out[o] = acc[hd];
      if (p.deq_out) p.deq_out[o] = d;
    }
  }
  if (best == 0.0f) best = 0.0f;   // -0 -> +0
  return best;
}


}  // namespace kvb
