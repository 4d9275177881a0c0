// Fused per-layer decode step: threshold from a sample, candidate-emitting score, exact select, attend over
// the implicit final list (with the quantize-append of the new row), chunk merge — five stream-ordered
// launches sharing one caller-provided workspace (the score + histogram + select chain where the sampled
// front end does not apply). Candidates, selected ids and attention partials never leave the workspace.
#include "common.cuh"
#include "score_common.cuh"

namespace kvb {

// ---- fast path of the fused step ---------------------------------------------------------
// The scorer can hand the selector its candidates directly (no group-max row in memory, no
// histogram, no collect pass) if it knows, per row, a threshold tau with
//     k  <=  #{t : gmax[t] >= tau}  <=  candidate capacity.
// tau comes from a SAMPLE of the row: 32 evenly spaced runs of tokens (1/32 of the row, at most
// 4096 tokens) are scored first and tau is set to the sample value whose rank predicts about
// 1.75 k tokens above it in the whole row (rank ~ 112: the prediction is good to about +-10 %, so
// both bounds hold by many standard deviations). The bounds are CHECKED, not assumed: a row whose
// count misses them (heavy ties, adversarial layouts) is re-scored into the group-max workspace by
// the select kernel itself and selected by the exact refinement path, so the result is always the
// exact top-k.
struct SampleParams {
  ScoreParams sp;             // query / packed / scale / channels / shapes (outputs unused)
  float* tau;                 // [R]
  int top_k;
  int cap;                    // candidate capacity per row
  // optional: per-row words this kernel clears for the kernels after it (the candidate counter line and the
  // failed flag), which spares the step a separate memset node
  uint32_t* zero_count;       // [R * SC_COUNT_STRIDE] (word 0 of every row's line is the counter) or NULL
  uint32_t* zero_failed;      // [R] or NULL
  // optional: the decoded token's K and V rows (bf16 [R,128] dense), stored by this kernel as row T of the caches
  const uint4* new_k; const uint4* new_v;
  __nv_bfloat16* key; int64_t k_sb, k_sh, k_st;
  __nv_bfloat16* value; int64_t v_sb, v_sh, v_st;
  uint32_t* step_counter = nullptr;   // optional: CTA 0 adds one (the step number of the sequence-sharded exchange)
  KvPages pages;                      // optional: key / value are page pools
};

// The rank-th largest of the sample values a CTA holds in registers (v[e], e < per, of every thread; NaN =
// absent), as an order-preserving key — without a histogram: scores cluster in a few dozen exponent bins, and
// the 8192 or 16384 shared-memory atomics of a long row's sample on those few words took 20 us.
//   1. a lower bound L of the answer from the threads' largest keys: every warp sorts its 32 maxima and offers
//      its ceil(rank / warps)-th largest; L is the smallest offer (at least rank sample values are >= L);
//   2. the values >= L (about rank of them for well-spread scores) are compacted into a list with one
//      ballot per step;
//   3. the rank-th largest of the list, by counting: the entry that exactly rank - 1 others beat (ties by
//      position) is the answer.
// Returns false (and no key) when rank > NT or the list outgrows its room (heavy ties): the caller then takes
// the histogram route. `s_work` needs NT + LIST + 4 words. Ends with a barrier.
template <int NT, int VMAX, int LIST>
__device__ __forceinline__ bool block_rank_select(const float (&v)[VMAX], int per, int rank, uint32_t* s_work,
                                                  uint32_t& key_out) {
  const int tid = threadIdx.x, lane = tid & 31;
  uint32_t* s_keys = s_work;
  uint32_t* s_list = s_work + NT;
  uint32_t* s_misc = s_list + LIST;             // [0] L, [1] list length, [2] answer, [3] found flag
  if (rank > NT) return false;                  // (uniform)
  uint32_t key[VMAX];
  uint32_t kmax = 0;
#pragma unroll
  for (int e = 0; e < VMAX; ++e) {
    key[e] = (e < per && v[e] == v[e]) ? float_to_key(v[e]) : 0u;
    kmax = key[e] > kmax ? key[e] : kmax;
  }
  // every warp sorts its 32 maxima (bitonic network of shuffles, descending) and offers its r-th largest,
  // r = ceil(rank / warps): the smallest offer L has at least warps * r >= rank sample values at or above it
  {
    uint32_t x = kmax;
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
      for (int j = k >> 1; j > 0; j >>= 1) {
        const uint32_t y = __shfl_xor_sync(0xffffffffu, x, j);
        const bool keep_max = ((lane & j) == 0) == ((lane & k) == 0);
        x = keep_max ? (x > y ? x : y) : (x < y ? x : y);
      }
    }
    constexpr int NW = NT / 32;
    const int r = (rank + NW - 1) / NW;          // <= 32 because rank <= NT
    const uint32_t offer = __shfl_sync(0xffffffffu, x, r - 1);
    if (lane == 0) s_keys[tid >> 5] = offer;
    if (tid == 0) { s_misc[1] = 0; s_misc[3] = 0; }
    __syncthreads();
    uint32_t lo = 0xFFFFFFFFu;
#pragma unroll
    for (int j = 0; j < NW; ++j) { const uint32_t o = s_keys[j]; lo = o < lo ? o : lo; }
    if (tid == 0) s_misc[0] = lo;
  }
  __syncthreads();
  const uint32_t L = s_misc[0];
  if (L == 0) return false;                     // fewer than rank threads hold a value (uniform)
#pragma unroll
  for (int e = 0; e < VMAX; ++e) {
    if (e >= per) break;
    const bool take = key[e] >= L;
    const uint32_t mask = __ballot_sync(0xffffffffu, take);
    if (mask) {
      uint32_t base = 0;
      if (lane == 0) base = atomicAdd(&s_misc[1], (uint32_t)__popc(mask));
      base = __shfl_sync(0xffffffffu, base, 0);
      const uint32_t pos = base + (uint32_t)__popc(mask & ((1u << lane) - 1u));
      if (take && pos < (uint32_t)LIST) s_list[pos] = key[e];
    }
  }
  __syncthreads();
  const uint32_t n = s_misc[1];
  if (n > (uint32_t)LIST) { __syncthreads(); return false; }
  for (uint32_t i = tid; i < n; i += NT) {
    const uint32_t ki = s_list[i];
    int beat = 0;
    for (uint32_t j = 0; j < n; ++j) {
      const uint32_t kj = s_list[j];
      beat += (kj > ki || (kj == ki && j < i)) ? 1 : 0;
    }
    if (beat == rank - 1) { s_misc[2] = ki; s_misc[3] = 1; }
  }
  __syncthreads();
  const bool found = s_misc[3] != 0;
  key_out = s_misc[2];
  __syncthreads();
  return found;
}

constexpr int FS_LIST = 2048;                   // room of block_rank_select's list

// tau of a row from the key of the rank-th largest sample value
__device__ __forceinline__ float fs_tau_from_key(uint32_t key) {
  float t = key_to_float(key);
  if (key <= 0x007FFFFFu || t != t) t = -INFINITY;            // NaN patterns: take everything
  return t;
}

// The threshold of every row from sample values that the streaming scorer left at the start of the row's
// workspace (score_sample_stream_run). Also does score_sample_kernel's side jobs (per-row counters, the
// decoded token's K/V rows, the step number).
__global__ void __launch_bounds__(FS_THREADS) sample_threshold_kernel(SampleParams q, const float* sample, int tile_tokens) {
  __shared__ uint32_t s_hist[SEL_HIST_BINS];    // also the work area of block_rank_select (FS_THREADS + FS_LIST + 4 words)
  __shared__ uint32_t s_tmp[80];
  static_assert(FS_THREADS + FS_LIST + 4 <= SEL_HIST_BINS, "work area");
  const ScoreParams& p = q.sp;
  const int row = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();                      // the scorer may become resident and prepare its query codes
  pdl_wait();
  if (q.step_counter && row == 0 && tid == 33) *q.step_counter += 1;
  if (q.zero_count && tid == 0) q.zero_count[(int64_t)row * SC_COUNT_STRIDE] = 0;
  if (q.zero_failed && tid == 32) q.zero_failed[row] = 0;
  const int T = p.T_dev ? min(*p.T_dev, p.T) : p.T;
  if (q.new_k && tid >= 64 && tid < 96) {          // one warp: 16 lanes per row, 16 bytes per lane
    const int l = tid - 64, rb = row / p.Hkv, rh = row - rb * p.Hkv;
    int64_t ko = (int64_t)rb * q.k_sb + (int64_t)rh * q.k_sh + (int64_t)T * q.k_st;
    int64_t vo = (int64_t)rb * q.v_sb + (int64_t)rh * q.v_sh + (int64_t)T * q.v_st;
    if (q.pages.table) ko = vo = kv_paged_row(q.pages, p.Hkv, rb, rh, T) * 128;      // rows of D = 128 elements
    if (l < 16) *reinterpret_cast<uint4*>(q.key + ko + l * 8) = q.new_k[row * 16 + l];
    else *reinterpret_cast<uint4*>(q.value + vo + (l - 16) * 8) = q.new_v[row * 16 + l - 16];
  }
  if (T <= q.cap) {                             // short rows: every token is a candidate
    if (tid == 0) q.tau[row] = -INFINITY;
    return;
  }
  int grp, stride, n_sample;
  fs_sample_geometry(T, tile_tokens, grp, stride, n_sample);
  const float frac = (float)n_sample / (float)T;
  const int kk = q.top_k < T ? q.top_k : T;
  float expect = 1.75f * (float)kk;
  if (expect * frac < 96.0f) expect = 96.0f / frac;
  int rank = (int)(expect * frac + 0.999f);
  if (rank < 1) rank = 1;
  if (rank > n_sample) rank = n_sample;
  // thread t holds the values t, t + NT, ... of the row's sample (scalar loads: the row pitch T need not be a
  // multiple of four floats)
  constexpr int VMAX = FS_PER_THREAD_MAX;       // n_sample <= FS_THREADS * VMAX
  const int per = n_sample / FS_THREADS;        // 8, 16 or 32
  const float* mine = sample + (int64_t)row * p.T;
  float v[VMAX];
#pragma unroll
  for (int e = 0; e < VMAX; ++e) v[e] = e < per ? __ldcg(mine + tid + e * FS_THREADS) : __int_as_float(0x7fc00000);
  uint32_t key;
  if (block_rank_select<FS_THREADS, VMAX, FS_LIST>(v, per, rank, s_hist, key)) {
    if (tid == 0) q.tau[row] = fs_tau_from_key(key);
    return;
  }
  // heavy ties: two-level histogram of the keys
  for (int i = tid; i < SEL_HIST_BINS; i += FS_THREADS) s_hist[i] = 0;
  __syncthreads();
#pragma unroll
  for (int e = 0; e < VMAX; ++e) {
    if (e >= per) break;
    if (v[e] == v[e]) atomicAdd(&s_hist[float_to_key(v[e]) >> (32 - SEL_HIST_BITS)], 1u);
  }
  __syncthreads();
  uint32_t bin, above, inb;
  find_threshold<FS_THREADS>(s_hist, SEL_HIST_BINS, (uint32_t)rank, s_tmp, bin, above, inb);
  for (int i = tid; i < 2048; i += FS_THREADS) s_hist[i] = 0;
  __syncthreads();
#pragma unroll
  for (int e = 0; e < VMAX; ++e) {
    if (e >= per) break;
    if (v[e] == v[e]) {
      const uint32_t k2 = float_to_key(v[e]);
      if ((k2 >> (32 - SEL_HIST_BITS)) == bin) atomicAdd(&s_hist[(k2 >> 9) & 2047u], 1u);
    }
  }
  __syncthreads();
  uint32_t d, ab2, in2;
  find_threshold<FS_THREADS>(s_hist, 2048, (uint32_t)rank - above, s_tmp, d, ab2, in2);
  if (tid == 0) q.tau[row] = fs_tau_from_key((bin << (32 - SEL_HIST_BITS)) | (d << 9));
}

template <int C, int G>
__global__ void __launch_bounds__(FS_THREADS) score_sample_kernel(SampleParams q) {
  __shared__ float s_qv[G * C];
  __shared__ float s_qscale[SC_MAX_G];
  __shared__ int8_t s_qcode[G * C];
  __shared__ uint32_t s_hist[SEL_HIST_BINS];
  __shared__ uint32_t s_tmp[80];
  const ScoreParams& p = q.sp;
  const int row = blockIdx.x, tid = threadIdx.x;
  pdl_launch_dependents();                      // the scorer may become resident and prepare its query codes
  pdl_wait();
  if (q.step_counter && row == 0 && tid == 33) *q.step_counter += 1;
  if (q.zero_count && tid == 0) q.zero_count[(int64_t)row * SC_COUNT_STRIDE] = 0;
  if (q.zero_failed && tid == 32) q.zero_failed[row] = 0;
  const int T = p.T_dev ? min(*p.T_dev, p.T) : p.T;
  if (q.new_k && tid >= 64 && tid < 96) {          // one warp: 16 lanes per row, 16 bytes per lane
    const int l = tid - 64, rb = row / p.Hkv, rh = row - rb * p.Hkv;
    int64_t ko = (int64_t)rb * q.k_sb + (int64_t)rh * q.k_sh + (int64_t)T * q.k_st;
    int64_t vo = (int64_t)rb * q.v_sb + (int64_t)rh * q.v_sh + (int64_t)T * q.v_st;
    if (q.pages.table) ko = vo = kv_paged_row(q.pages, p.Hkv, rb, rh, T) * 128;      // rows of D = 128 elements
    if (l < 16) *reinterpret_cast<uint4*>(q.key + ko + l * 8) = q.new_k[row * 16 + l];
    else *reinterpret_cast<uint4*>(q.value + vo + (l - 16) * 8) = q.new_v[row * 16 + l - 16];
  }
  if (T <= q.cap) {                             // short rows: every token is a candidate
    if (tid == 0) q.tau[row] = -INFINITY;
    return;
  }
  // sample geometry: FS_RUNS runs of run_len tokens; rank = the sample rank that predicts about
  // 1.75 k (at least 96 / fraction) tokens above tau in the whole row
  const int per_thread = fs_per_thread(T);
  int run_len = (T / FS_RUNS) / per_thread * per_thread;
  if (run_len > per_thread * FS_THREADS / FS_RUNS) run_len = per_thread * FS_THREADS / FS_RUNS;
  const float frac = (float)(run_len * FS_RUNS) / (float)T;
  const int kk = q.top_k < T ? q.top_k : T;
  float expect = 1.75f * (float)kk;
  if (expect * frac < 96.0f) expect = 96.0f / frac;
  int rank = (int)(expect * frac + 0.999f);
  if (rank < 1) rank = 1;
  if (rank > run_len * FS_RUNS) rank = run_len * FS_RUNS;
  const int b = row / p.Hkv, g = row - b * p.Hkv;
  for (int i = tid; i < SEL_HIST_BINS; i += FS_THREADS) s_hist[i] = 0;
  // thread -> run (tid / threads_per_run), per_thread consecutive tokens inside the run
  constexpr int W = C / 8;
  const int threads_per_run = run_len / per_thread;
  const int run = tid / threads_per_run;
  const int64_t t0 = (int64_t)run * (T / FS_RUNS) + (int64_t)(tid - run * threads_per_run) * per_thread;
  const bool live = run < FS_RUNS;
  const uint8_t* packed_row = p.packed + (int64_t)b * p.packed_sb + (int64_t)g * p.packed_sh;
  const float* scale_row = p.scale + (int64_t)b * p.scale_sb + (int64_t)g * p.scale_sh;
  // four tokens at a time: all their loads are issued before the first use
  auto load_batch = [&](int e0, uint32_t (&wv)[4][W], float (&ks)[4]) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const bool ok = live && t0 + e0 + e < T;
      const uint4* src = reinterpret_cast<const uint4*>(packed_row + (t0 + e0 + e) * (C / 2));
#pragma unroll
      for (int x = 0; x < C / 32; ++x) {
        const uint4 u = ok ? __ldg(src + x) : make_uint4(0, 0, 0, 0);
        wv[e][4 * x] = u.x; wv[e][4 * x + 1] = u.y; wv[e][4 * x + 2] = u.z; wv[e][4 * x + 3] = u.w;
      }
      ks[e] = ok ? scale_row[t0 + e0 + e] : 0.0f;
    }
  };
  uint32_t wv[4][W];
  float ks[4];
  quantize_query_group<FS_THREADS>(p, b, g, G, s_qv, s_qcode, s_qscale);
  // query words in shared memory (every thread reads the same word: a broadcast): word w of a token
  // holds channels 8w + {0,2,4,6} in its low nibbles and 8w + {1,3,5,7} in its high nibbles
  __shared__ int s_qlo[G][W], s_qhi[G][W];
  for (int i = tid; i < G * W; i += FS_THREADS) {
    const int hd = i / W, w = i - hd * W;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= (uint32_t)(uint8_t)s_qcode[hd * C + 8 * w + 2 * j] << (8 * j);
      hi |= (uint32_t)(uint8_t)s_qcode[hd * C + 8 * w + 2 * j + 1] << (8 * j);
    }
    s_qlo[hd][w] = (int)lo;
    s_qhi[hd][w] = (int)hi;
  }
  __syncthreads();
  float v[FS_PER_THREAD_MAX];
#pragma unroll 1
  for (int e0 = 0; e0 < per_thread; e0 += 4) {
    load_batch(e0, wv, ks);
    int acc[4][G];
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
      for (int hd = 0; hd < G; ++hd) acc[e][hd] = 0;
#pragma unroll
    for (int w = 0; w < W; ++w) {
#pragma unroll
      for (int hd = 0; hd < G; ++hd) {
        const int ql = s_qlo[hd][w], qh = s_qhi[hd][w];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[e][hd] = __dp4a((int)((wv[e][w] << 4) & 0xF0F0F0F0u), ql, acc[e][hd]);
          acc[e][hd] = __dp4a((int)(wv[e][w] & 0xF0F0F0F0u), qh, acc[e][hd]);
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float m = -INFINITY;
#pragma unroll
      for (int hd = 0; hd < G; ++hd) {
        const float f = __int_as_float(acc[e][hd] + 0x4B400000) - 12582912.0f;     // 16 * dot, exact
        m = fmaxf(m, __fmul_rn(__fmul_rn(f, ks[e]), s_qscale[hd] * 0.0625f));
      }
      if (m == 0.0f) m = 0.0f;
      const bool ok = live && t0 + e0 + e < T;
      v[e0 + e] = ok ? m : __int_as_float(0x7fc00000);
      if (ok) atomicAdd(&s_hist[float_to_key(m) >> (32 - SEL_HIST_BITS)], 1u);
    }
  }
  __syncthreads();
  uint32_t bin, above, inb;
  find_threshold<FS_THREADS>(s_hist, SEL_HIST_BINS, (uint32_t)rank, s_tmp, bin, above, inb);
  // second level: 11 more key bits inside the bin
  for (int i = tid; i < 2048; i += FS_THREADS) s_hist[i] = 0;
  __syncthreads();
  for (int e = 0; e < per_thread; ++e) {
    if (v[e] == v[e]) {
      const uint32_t key = float_to_key(v[e]);
      if ((key >> (32 - SEL_HIST_BITS)) == bin) atomicAdd(&s_hist[(key >> 9) & 2047u], 1u);
    }
  }
  __syncthreads();
  uint32_t d, ab2, in2;
  find_threshold<FS_THREADS>(s_hist, 2048, (uint32_t)rank - above, s_tmp, d, ab2, in2);
  if (tid == 0) {
    const uint32_t key_lo = (bin << (32 - SEL_HIST_BITS)) | (d << 9);
    float t = key_to_float(key_lo);
    if (key_lo <= 0x007FFFFFu || t != t) t = -INFINITY;       // NaN patterns: take everything
    q.tau[row] = t;
  }
}

template <int C>
static int sample_launch_g(const SampleParams& q, int R, cudaStream_t st) {
  switch (q.sp.G) {
    case 1: KVB_CHECK_CUDA(launch_kernel(score_sample_kernel<C, 1>, dim3(R), dim3(FS_THREADS), 0, st, q)); break;
    case 2: KVB_CHECK_CUDA(launch_kernel(score_sample_kernel<C, 2>, dim3(R), dim3(FS_THREADS), 0, st, q)); break;
    case 4: KVB_CHECK_CUDA(launch_kernel(score_sample_kernel<C, 4>, dim3(R), dim3(FS_THREADS), 0, st, q)); break;
    default: KVB_CHECK_CUDA(launch_kernel(score_sample_kernel<C, 8>, dim3(R), dim3(FS_THREADS), 0, st, q)); break;
  }
  return KVB_OK;
}

// Stores the decoded token's K and V rows (bf16 [B*Hkv, 128] dense) as row T of the caches: one warp per
// (batch, KV head), 16 lanes per row, 16 bytes per lane.
__global__ void __launch_bounds__(32) store_new_rows_kernel(const uint4* new_k, const uint4* new_v, __nv_bfloat16* key,
                                                            int64_t k_sb, int64_t k_sh, int64_t k_st,
                                                            __nv_bfloat16* value, int64_t v_sb, int64_t v_sh,
                                                            int64_t v_st, int Hkv, int T, const int32_t* T_dev,
                                                            KvPages pages) {
  const int row = blockIdx.x, lane = threadIdx.x;
  const int b = row / Hkv, h = row - b * Hkv;
  const int t = T_dev ? min(*T_dev, T) : T;
  pdl_launch_dependents();
  int64_t ko = (int64_t)b * k_sb + (int64_t)h * k_sh + (int64_t)t * k_st;
  int64_t vo = (int64_t)b * v_sb + (int64_t)h * v_sh + (int64_t)t * v_st;
  if (pages.table) ko = vo = kv_paged_row(pages, Hkv, b, h, t) * 128;
  if (lane < 16) {
    *reinterpret_cast<uint4*>(key + ko + lane * 8) = new_k[row * 16 + lane];
  } else {
    *reinterpret_cast<uint4*>(value + vo + (lane - 16) * 8) = new_v[row * 16 + lane - 16];
  }
}

// Candidate capacity of the fast path: room for ~1.75 k expected candidates plus a wide margin.
static int fast_cap(int kk) {
  int c = 8192;
  while (c < 3 * kk && c < SEL_MAX_K) c <<= 1;
  return c;
}

static void fill_score_params(ScoreParams& sp, const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed,
                              int64_t packed_sb, int64_t packed_sh, const float* scale, int64_t scale_sb,
                              int64_t scale_sh, const int32_t* channel_idx, int B, int Hq, int Hkv, int T, int D, int C,
                              const int32_t* T_dev) {
  sp.query = reinterpret_cast<const __nv_bfloat16*>(query); sp.q_sb = q_sb; sp.q_sh = q_sh;
  sp.packed = packed; sp.packed_sb = packed_sb; sp.packed_sh = packed_sh;
  sp.scale = scale; sp.scale_sb = scale_sb; sp.scale_sh = scale_sh;
  sp.channel_idx = channel_idx;
  sp.B = B; sp.Hq = Hq; sp.Hkv = Hkv; sp.T = T; sp.D = D; sp.C = C; sp.G = Hq / Hkv;
  sp.T_dev = T_dev;
  sp.gmax_out = nullptr; sp.acc_out = nullptr; sp.deq_out = nullptr; sp.hist_out = nullptr;
  sp.tau = nullptr; sp.cand = nullptr; sp.cand_count = nullptr; sp.cand_cap = 0;
  sp.units_per_row = 0; sp.full_tiles = 0; sp.total_units = 0;
}

// `sample_ws`: optional fp32 workspace [R, sp.T] (the group-max workspace of the caller). With it, long rows have
// their sample scored by the streaming int8-MMA scorer and a small kernel derives the thresholds; otherwise one
// kernel does both with dp4a.
// The page table of a step's parameters (table == nullptr: contiguous caches); false if the fields are inconsistent.
static bool step_kv_pages(const kvb_decode_step_params* p, KvPages& pg) {
  pg = KvPages();
  if (!p->kv_page_table) return true;
  const int P = p->kv_page_tokens;
  if (P < 1 || (P & (P - 1)) || p->D != 128) return false;                       // a power of two; rows of 128 elements
  if (p->kv_page_table_stride * (int64_t)P < (int64_t)p->history_count + 1) return false;   // the table must cover row T
  int shift = 0;
  while ((1 << shift) < P) ++shift;
  pg.table = p->kv_page_table; pg.table_stride = p->kv_page_table_stride; pg.shift = shift;
  return true;
}

static int sample_run(const ScoreParams& sp, float* tau, int top_k, int cap, cudaStream_t st,
                      uint32_t* zero_count = nullptr, uint32_t* zero_failed = nullptr,
                      const kvb_decode_step_params* rows = nullptr, uint32_t* step_counter = nullptr,
                      float* sample_ws = nullptr, int device = -1) {
  SampleParams sq;
  sq.sp = sp; sq.tau = tau; sq.top_k = top_k; sq.cap = cap;
  sq.zero_count = zero_count; sq.zero_failed = zero_failed;
  sq.step_counter = step_counter;
  sq.new_k = nullptr; sq.new_v = nullptr; sq.key = nullptr; sq.value = nullptr;
  sq.k_sb = sq.k_sh = sq.k_st = sq.v_sb = sq.v_sh = sq.v_st = 0;
  if (rows && rows->new_key_row) {
    sq.new_k = reinterpret_cast<const uint4*>(rows->new_key_row);
    sq.new_v = reinterpret_cast<const uint4*>(rows->new_value_row);
    sq.key = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(rows->key));
    sq.value = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(rows->value));
    sq.k_sb = rows->k_sb; sq.k_sh = rows->k_sh; sq.k_st = rows->k_st;
    sq.v_sb = rows->v_sb; sq.v_sh = rows->v_sh; sq.v_st = rows->v_st;
    step_kv_pages(rows, sq.pages);                 // (validated by the caller)
  }
  const int R = sp.B * sp.Hkv;
  const int tile_tokens = score_stream_tile_tokens(sp.C, sp.G);
  if (sample_ws && device >= 0 && tile_tokens > 0 && sp.T > FS_LONG_ROW) {
    // (the single dp4a kernel is instruction-bound on the 8192- and 16384-token samples of long rows)
    int grp, stride, n_sample;
    fs_sample_geometry(sp.T, tile_tokens, grp, stride, n_sample);
    if (n_sample <= FS_THREADS * FS_PER_THREAD_MAX && n_sample <= sp.T && (n_sample % FS_THREADS) == 0) {
      const int rc = score_sample_stream_run(sp, sample_ws, cap, device, st);
      if (rc != KVB_OK) return rc;
      ChainLaunchScope early;                   // the threshold kernel starts early and waits inside
      early.on();
      KVB_CHECK_CUDA(launch_kernel(sample_threshold_kernel, dim3(R), dim3(FS_THREADS), 0, st, sq, (const float*)sample_ws, tile_tokens));
      return KVB_OK;
    }
  }
  if (sp.C == 32) return sample_launch_g<32>(sq, R, st);
  if (sp.C == 64) return sample_launch_g<64>(sq, R, st);
  return sample_launch_g<128>(sq, R, st);
}

// Workspace of the fused step. The regions that must start at zero (attention split counters,
// select candidate counters, histogram) are adjacent so ONE memset per step clears them.
struct StepLayout {
  int R, kk, S;
  size_t off_attcnt, off_selws, off_attpart, off_gmax, off_sel;
  size_t zero_bytes, selws_bytes, bytes;
  // fast path (scorer emits candidates): counters + failed flags are zeroed per step
  size_t off_fcount, off_ffailed, off_ftau, off_fcand, fzero_bytes;
  int fcap;
};

static StepLayout step_layout(int B, int Hq, int Hkv, int T, int k, int sink, int recent, int keep_self) {
  StepLayout L;
  L.R = B * Hkv;
  L.kk = k < T ? k : T;
  L.S = kvb_final_index_count(L.kk, T, sink, recent, keep_self);
  const SelectWorkspace sw = select_carve(nullptr, L.R, L.kk > 0 ? L.kk : 1);
  const AttendPlan ap = attend_plan(B, Hq, Hkv, L.S > 0 ? L.S : 1);
  size_t off = 0;
  L.off_attcnt = off;  off += ap.counter_bytes;
  L.off_selws = off;   off += round_up(sw.bytes, 256);
  L.selws_bytes = sw.bytes;
  L.zero_bytes = ap.counter_bytes + sw.zero_bytes;       // attention counters + select counters + histogram
  L.off_attpart = off; off += ap.partial_bytes;
  L.off_gmax = off;    off += round_up(sizeof(float) * (size_t)L.R * (size_t)T, 256);
  L.off_sel = off;     off += round_up(sizeof(int32_t) * (size_t)L.R * (size_t)(L.kk > 0 ? L.kk : 1), 256);
  L.fcap = fast_cap(L.kk > 0 ? L.kk : 1);
  L.off_fcount = off;  off += round_up(sizeof(uint32_t) * (size_t)L.R * SC_COUNT_STRIDE, 256);
  L.off_ffailed = off; off += round_up(sizeof(uint32_t) * (size_t)L.R, 256);
  L.fzero_bytes = off - L.off_fcount;
  L.off_ftau = off;    off += round_up(sizeof(float) * (size_t)L.R, 256);
  L.off_fcand = off;   off += round_up(sizeof(uint64_t) * (size_t)L.R * L.fcap, 256);
  L.bytes = off;
  return L;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_decode_step_workspace_bytes(
    int B, int Hq, int Hkv, int history_count, int top_k, int protect_sink, int protect_recent, int keep_self) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || history_count < 0 || top_k <= 0 || (Hq % Hkv)) return 0;
  return kvb::step_layout(B, Hq, Hkv, history_count, top_k, protect_sink, protect_recent, keep_self).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_decode_step(const kvb_decode_step_params* p, int device,
                                                                      void* stream) {
  using namespace kvb;
  if (!p || !p->query || !p->key || !p->value || !p->packed || !p->scale || !p->channel_idx || !p->out ||
      !p->workspace)
    return KVB_BAD_ARG;
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || (p->Hq % p->Hkv) || p->history_count <= 0 || p->top_k <= 0)
    return KVB_BAD_SHAPE;
  if (p->top_k > SEL_MAX_K && p->history_count > SEL_MAX_K) return KVB_BAD_SHAPE;
  if (!aligned_to(p->workspace, 256)) return KVB_BAD_ALIGN;
  const int T = p->history_count;
  const StepLayout L = step_layout(p->B, p->Hq, p->Hkv, T, p->top_k, p->protect_sink, p->protect_recent,
                                   p->keep_self);
  if (p->workspace_bytes < L.bytes) return KVB_WORKSPACE_TOO_SMALL;
  if (L.S <= 0) return KVB_BAD_SHAPE;
  uint8_t* ws = reinterpret_cast<uint8_t*>(p->workspace);
  uint32_t* attcnt = reinterpret_cast<uint32_t*>(ws + L.off_attcnt);
  void* selws = ws + L.off_selws;
  const SelectWorkspace sw = select_carve(selws, L.R, L.kk);
  float* attpart = reinterpret_cast<float*>(ws + L.off_attpart);
  float* gmax = reinterpret_cast<float*>(ws + L.off_gmax);
  int32_t* sel = p->sel_idx_out ? p->sel_idx_out : reinterpret_cast<int32_t*>(ws + L.off_sel);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  ChainLaunchScope chain;

  // Fast path: sample -> tau, scorer emits candidates, rescue check, exact finish. Needs the
  // streaming scorer, a row longer than the candidate capacity but short enough for the 4096-token
  // sample to be a 1/32 fraction, and k small enough for the capacity.
  const int G = p->Hq / p->Hkv;
  const int fcap = L.fcap;
  const bool stream_ok = score_stream_supported(p->C, G, p->packed, p->packed_sb, p->packed_sh, p->scale,
                                                p->scale_sb, p->scale_sh);
  // the sample kernel aims at max(1.75 k, 96 / sampled fraction) candidates: that, with margin, must
  // fit the capacity at the (largest) history length this call can see
  const int per_thread = fs_per_thread(T);
  int run_len = (T / FS_RUNS) / per_thread * per_thread;
  if (run_len > per_thread * FS_THREADS / FS_RUNS) run_len = per_thread * FS_THREADS / FS_RUNS;
  const double frac = run_len > 0 ? (double)(run_len * FS_RUNS) / (double)T : 0.0;
  double expect = 1.75 * L.kk;
  if (frac > 0.0 && expect * frac < 96.0) expect = 96.0 / frac;
  const bool all_candidates = T <= fcap;                    // short rows: tau = -inf, every token is a candidate
  const bool fast = stream_ok && 3 * L.kk <= fcap &&
                    (all_candidates || (run_len >= per_thread && 1.7 * expect <= (double)fcap));
  const int32_t* T_dev = p->history_count_dev;
  if (T_dev && !fast) return KVB_BAD_SHAPE;
  KvPages pages;
  if (!step_kv_pages(p, pages)) return KVB_BAD_SHAPE;
  if ((p->new_key_row == nullptr) != (p->new_value_row == nullptr)) return KVB_BAD_ARG;
  if (p->new_key_row && (p->D != 128 || !aligned_to(p->new_key_row, 16) || !aligned_to(p->new_value_row, 16)))
    return KVB_BAD_ALIGN;
  if (p->new_key_row && !fast) {                   // (the fast path's first kernel stores the rows itself)
    DeviceGuard guard(device);
    if (!guard.ok) return KVB_BAD_DEVICE;
    store_new_rows_kernel<<<p->B * p->Hkv, 32, 0, st>>>(
        reinterpret_cast<const uint4*>(p->new_key_row), reinterpret_cast<const uint4*>(p->new_value_row),
        reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p->key)), p->k_sb, p->k_sh, p->k_st,
        reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(p->value)), p->v_sb, p->v_sh, p->v_st, p->Hkv, T, T_dev, pages);
    KVB_CHECK_CUDA(cudaGetLastError());
  }
  if (fast) {
    {
      DeviceGuard guard(device);
      if (!guard.ok) return KVB_BAD_DEVICE;
      uint32_t* fcount = reinterpret_cast<uint32_t*>(ws + L.off_fcount);      // cleared by the sample kernel
      float* ftau = reinterpret_cast<float*>(ws + L.off_ftau);
      uint64_t* fcand = reinterpret_cast<uint64_t*>(ws + L.off_fcand);

      ScoreParams base;
      fill_score_params(base, p->query, p->q_sb, p->q_sh, p->packed, p->packed_sb, p->packed_sh, p->scale, p->scale_sb,
                        p->scale_sh, p->channel_idx, p->B, p->Hq, p->Hkv, T, p->D, p->C, T_dev);
      rc = sample_run(base, ftau, p->top_k, fcap, st, fcount, reinterpret_cast<uint32_t*>(ws + L.off_ffailed), p, nullptr,
                      gmax, device);
      if (rc != KVB_OK) return rc;
      chain.on();                             // every later kernel of the step starts early and waits inside

      ScoreEmit emit{ftau, fcand, fcount, fcap};
      rc = score_run(p->query, p->q_sb, p->q_sh, p->packed, p->packed_sb, p->packed_sh, p->scale, p->scale_sb,
                     p->scale_sh, p->channel_idx, p->B, p->Hq, p->Hkv, T, p->D, p->C, nullptr, nullptr, nullptr,
                     nullptr, &emit, T_dev, device, st);
      if (rc != KVB_OK) return rc;

      SelectParams sp;
      sp.scores = gmax; sp.row_stride = T; sp.payload = nullptr;
      sp.R = L.R; sp.T = T; sp.k = p->top_k; sp.kk = L.kk; sp.idx_offset = 0;
      sp.out_idx32 = sel; sp.out_idx64 = nullptr; sp.out_scores = nullptr;
      sp.hist = nullptr; sp.cand = fcand; sp.cand_count = fcount; sp.cap = fcap;
      sp.tokens_per_cta = 0; sp.thresholds = nullptr;
      sp.order_by_index = 1;
      sp.from_candidates = 1; sp.row_failed = nullptr; sp.T_dev = T_dev;
      sp.out_comp = nullptr; sp.gather = nullptr; sp.gather_n = 0; sp.gather_len = 0; sp.gather_stride = 0;
      sp.rescue = 1; sp.rescue_sp = base;          // rows that miss [kk, cap] are re-scored inside the kernel
      const size_t bitmap_bytes = sizeof(uint32_t) * (size_t)((T + 31) / 32);
      size_t smem = (size_t)fcap * 8 + SEL_FINAL_FIXED_SMEM;
      sp.use_bitmap = (smem + bitmap_bytes <= SEL_SMEM_LIMIT) ? 1 : 0;
      if (sp.use_bitmap) smem += bitmap_bytes;
      if (p->selected_any_order) {                                                 // skip the ordering bitmap
        if (sp.use_bitmap) smem -= bitmap_bytes;
        sp.order_by_index = 2; sp.use_bitmap = 0;
        if (smem + select_stage_bytes(L.kk) <= SEL_SMEM_LIMIT) { sp.stage = 1; smem += select_stage_bytes(L.kk); }
      }
      { const int prc = select_final_prepare(device); if (prc != KVB_OK) return prc; }
      KVB_CHECK_CUDA(launch_kernel(select_final_kernel, dim3(L.R), dim3(SEL_FINAL_THREADS), smem, st, sp));
    }
  } else {
    {
      DeviceGuard guard(device);
      if (!guard.ok) return KVB_BAD_DEVICE;
      KVB_CHECK_CUDA(cudaMemsetAsync(ws + L.off_attcnt, 0, L.zero_bytes, st));
    }
    rc = kvb_score_decode(p->query, p->q_sb, p->q_sh, p->packed, p->packed_sb, p->packed_sh, p->scale, p->scale_sb,
                          p->scale_sh, p->channel_idx, p->B, p->Hq, p->Hkv, T, p->D, p->C, gmax, nullptr, nullptr,
                          sw.hist, device, stream);
    if (rc != KVB_OK) return rc;
    // ascending-index order: the set is what matters to the attention, and it is the cheapest to emit
    rc = select_run(gmax, T, nullptr, L.R, T, p->top_k, 0, /*order=*/1, sel, nullptr, nullptr, nullptr,
                    /*hist_in_workspace=*/true, /*zeroed=*/true, selws, L.selws_bytes, device, st);
    if (rc != KVB_OK) return rc;
  }
  // The attention kernel reads the list  selected || sink || recent || self  implicitly (no list is
  // materialised) and its chunk-0 warps append the decoded token's K row to the int4 cache.
  const FinalLayout f = final_layout(L.kk, T, p->protect_sink, p->protect_recent, p->keep_self);
  AttendList list{};
  list.implicit = 1;
  list.selected = sel; list.kk = L.kk; list.sel_pitch = L.kk;
  list.sel_base = 0; list.sel_limit = T;
  list.sink_end = f.sink_end; list.n_recent = f.n_recent; list.recent_from = f.recent_from;
  list.recent_start = f.recent_start; list.recent_on = f.recent_on; list.history = T;
  list.append_protected = p->append_protected;
  AttendAppend ap{};
  ap.enabled = p->append_self ? 1 : 0;
  ap.channel_idx = p->channel_idx; ap.C = p->C;
  ap.packed = p->packed; ap.packed_sb = p->packed_sb; ap.packed_sh = p->packed_sh;
  ap.scale = p->scale; ap.scale_sb = p->scale_sb; ap.scale_sh = p->scale_sh;
  ap.t_src = T; ap.t_dst = T;
  AttendDeviceLength adl{T_dev, p->top_k, p->protect_sink, p->protect_recent, p->keep_self, p->advance_history};
  rc = attend_run(p->query, p->q_sb, p->q_sh, p->key, p->k_sb, p->k_sh, p->k_st, p->value, p->v_sb, p->v_sh, p->v_st,
                  list, &ap, T_dev ? &adl : nullptr, p->mask, p->mask_sb, p->B, p->Hq, p->Hkv, p->Hkv, T + 1, p->D, L.S, p->scaling,
                  p->out, nullptr, attcnt, attpart, /*counters_zeroed=*/true, device, st, nullptr, nullptr, nullptr,
                  &pages);
  if (rc != KVB_OK) return rc;
  return KVB_OK;
}

namespace kvb {

// Workspace of kvb_shard_candidates: [counters | failed flags] (zeroed per call) | tau | candidates | gmax rows (rescue only)
struct ShardLayout {
  int R, kk, cap;
  size_t off_count, off_failed, zero_bytes, off_tau, off_cand, off_gmax, bytes;
};

static ShardLayout shard_layout(int B, int Hkv, int T, int top_k) {
  ShardLayout L;
  L.R = B * Hkv;
  L.kk = top_k < T ? top_k : T;
  L.cap = fast_cap(L.kk > 0 ? L.kk : 1);
  size_t off = 0;
  L.off_count = off;  off += round_up(sizeof(uint32_t) * (size_t)L.R * SC_COUNT_STRIDE, 256);
  L.off_failed = off; off += round_up(sizeof(uint32_t) * (size_t)L.R, 256);
  L.zero_bytes = off;
  L.off_tau = off;    off += round_up(sizeof(float) * (size_t)L.R, 256);
  L.off_cand = off;   off += round_up(sizeof(uint64_t) * (size_t)L.R * L.cap, 256);
  L.off_gmax = off;   off += round_up(sizeof(float) * (size_t)L.R * (size_t)T, 256);
  L.bytes = off;
  return L;
}

// The conditions under which the sampled-threshold front end applies to rows of length T.
static bool fast_front_ok(int C, int G, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                          const float* scale, int64_t scale_sb, int64_t scale_sh, int T, int kk, int cap) {
  if (!score_stream_supported(C, G, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh)) return false;
  if (3 * kk > cap) return false;
  if (T <= cap) return true;
  const int per_thread = fs_per_thread(T);
  int run_len = (T / FS_RUNS) / per_thread * per_thread;
  if (run_len > per_thread * FS_THREADS / FS_RUNS) run_len = per_thread * FS_THREADS / FS_RUNS;
  if (run_len < per_thread) return false;
  const double frac = (double)(run_len * FS_RUNS) / (double)T;
  double expect = 1.75 * kk;
  if (expect * frac < 96.0) expect = 96.0 / frac;
  return 1.7 * expect <= (double)cap;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_shard_candidates_workspace_bytes(int B, int Hkv, int T,
                                                                                              int top_k) {
  if (B <= 0 || Hkv <= 0 || T <= 0 || top_k <= 0) return 0;
  return kvb::shard_layout(B, Hkv, T, top_k).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_merge_candidates(
    const uint64_t* gathered, int N, int R, int kk, int top_k, int64_t id_range, int prefix_k, int32_t* out_idx,
    int64_t own_base, int64_t own_limit, int32_t* out_owned, int32_t* out_owned_count, int device, void* stream) {
  using namespace kvb;
  if (!gathered || !out_idx) return KVB_BAD_ARG;
  if (N <= 0 || R <= 0 || kk <= 0 || top_k <= 0 || id_range <= 0 || id_range > 0x7fffffffLL || prefix_k < 0)
    return KVB_BAD_SHAPE;
  if (out_owned && (!out_owned_count || own_limit <= own_base)) return KVB_BAD_ARG;
  if (kk < top_k && N > 1) return KVB_BAD_SHAPE;            // every shard must bring top_k entries (see header)
  const int64_t total = (int64_t)N * kk;
  const int kout = (int)(top_k < total ? top_k : total);
  if (kout > SEL_MAX_K) return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  SelectParams sp;
  sp.scores = nullptr; sp.row_stride = 0; sp.payload = nullptr;
  sp.R = R; sp.T = (int)id_range; sp.k = top_k; sp.kk = kout; sp.idx_offset = 0;
  sp.out_idx32 = out_idx; sp.out_idx64 = nullptr; sp.out_scores = nullptr; sp.out_comp = nullptr;
  sp.hist = nullptr; sp.cand = nullptr; sp.cand_count = nullptr; sp.cap = select_cap(kout);
  sp.tokens_per_cta = 0; sp.thresholds = nullptr;
  sp.from_candidates = 0; sp.row_failed = nullptr; sp.T_dev = nullptr;
  sp.gather = gathered; sp.gather_n = N; sp.gather_len = kk; sp.gather_stride = (int64_t)R * kk;
  sp.rescue = 0;
  sp.gather_prefix = prefix_k;
  sp.out_owned = out_owned; sp.out_owned_count = out_owned_count; sp.own_base = own_base; sp.own_limit = own_limit;
  const size_t bitmap_bytes = sizeof(uint32_t) * (size_t)((id_range + 31) / 32);
  size_t smem = (size_t)sp.cap * 8 + SEL_FINAL_FIXED_SMEM;
  if (!out_owned && id_range <= 262144 && smem + bitmap_bytes <= SEL_SMEM_LIMIT) {
    sp.order_by_index = 1; sp.use_bitmap = 1; smem += bitmap_bytes;      // ascending global ids (cheap bitmap only)
  } else {
    sp.order_by_index = 2; sp.use_bitmap = 0;                              // exact set, arbitrary order
    if (smem + select_stage_bytes(sp.kk) <= SEL_SMEM_LIMIT) { sp.stage = 1; smem += select_stage_bytes(sp.kk); }
  }
  { const int prc = select_final_prepare(device); if (prc != KVB_OK) return prc; }
  select_final_kernel<<<R, SEL_FINAL_THREADS, smem, reinterpret_cast<cudaStream_t>(stream)>>>(sp);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

extern "C" __attribute__((visibility("default"))) int kvb_candidate_capacity(int top_k) {
  if (top_k <= 0 || 3 * top_k > kvb::SEL_MAX_K) return 0;
  return kvb::fast_cap(top_k);
}

extern "C" __attribute__((visibility("default"))) int kvb_sample_thresholds(
    const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, const int32_t* channel_idx, int B, int Hq, int Hkv, int T,
    int D, int C, int top_k, float* tau, int device, void* stream) {
  using namespace kvb;
  if (!query || !packed || !scale || !channel_idx || !tau) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || T <= 0 || (Hq % Hkv) || top_k <= 0) return KVB_BAD_SHAPE;
  if (!score_stream_supported(C, Hq / Hkv, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh)) return KVB_BAD_SHAPE;
  const int cap = kvb_candidate_capacity(top_k < T ? top_k : T);
  if (cap == 0) return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  ScoreParams sp;
  fill_score_params(sp, query, q_sb, q_sh, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, channel_idx, B, Hq,
                    Hkv, T, D, C, nullptr);
  return sample_run(sp, tau, top_k, cap, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int kvb_score_candidates(
    const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, const int32_t* channel_idx, int B, int Hq, int Hkv, int T,
    int D, int C, const float* tau, uint64_t* cand, uint32_t* cand_count, int cand_cap, int device, void* stream) {
  using namespace kvb;
  if (!tau || !cand || !cand_count || cand_cap <= 0) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv)) return KVB_BAD_SHAPE;
  if (!score_stream_supported(C, Hq / Hkv, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh)) return KVB_BAD_SHAPE;
  ScoreEmit emit{tau, cand, cand_count, cand_cap};
  return score_run(query, q_sb, q_sh, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, channel_idx, B, Hq, Hkv,
                   T, D, C, nullptr, nullptr, nullptr, nullptr, &emit, nullptr, device,
                   reinterpret_cast<cudaStream_t>(stream));
}
