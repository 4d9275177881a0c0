// Stage 3: exact top-k per row; ties between equal scores go to the lower index.
//
// Every element becomes a unique 64-bit composite  (order-preserving key of the score) << 32 |
// (0xFFFFFFFF - index), so "larger composite" is exactly "better score, then lower index" and
// ties need no special case. Selection is an MSB-first radix select on the composite:
//   1. a 4096-bin histogram of the top 12 bits (taken from the scorer when it already made one),
//   2. one small CTA per row finds the bin b* that holds the k-th element,
//   3. a streaming pass appends all elements of bins >= b* to a per-row candidate list (a few
//      thousand entries for Gaussian-like scores; one atomic per CTA),
//   4. one CTA per row loads the candidates into shared memory, finishes the radix select there
//      (11 bits per pass) to get the exact k-th composite, and writes the k winners either
//      ordered by (score desc, index asc) — bitonic sort — or by ascending index — a bitmap in
//      shared memory read out in order, which is what the gather of the attention stage likes.
// When a row has more than CAP candidates after step 2 (heavy ties, e.g. constant scores) the
// last kernel first refines the prefix with 11-bit passes over the row itself until the
// candidate set fits; that path is slower but exact for any input.
#include "common.cuh"
#include "score_common.cuh"

namespace kvb {

constexpr int SEL_HIST_BITS = 12;
constexpr int SEL_HIST_BINS = 1 << SEL_HIST_BITS;
constexpr int SEL_SCAN_THREADS = 256;
constexpr int SEL_FINAL_THREADS = 512;            // measured best for ~3.5k on-chip candidates (barriers get cheaper, work per thread stays small)
constexpr int SEL_MAX_K = 16384;
constexpr int SEL_COUNT_STRIDE = 32;        // words between per-row candidate counters: one 128-byte line each,
                                            // so the atomics of different rows do not queue on one L2 line

constexpr int SEL_MAX_SEGMENTS = 64;          // shard lists a prefix merge can take

struct SelectParams {
  const float* scores;
  int64_t row_stride;
  const int32_t* payload;
  int R, T, k, kk;
  int64_t idx_offset;
  int32_t* out_idx32;
  int64_t* out_idx64;
  float* out_scores;
  const uint32_t* hist;       // [R, 4096]
  uint64_t* cand;             // [R, cap]
  uint32_t* cand_count;       // [R * SEL_COUNT_STRIDE]
  int cap;
  int tokens_per_cta;         // scan kernels: tokens per CTA along a row
  uint4* thresholds;          // [R] (bin, above, in-bin, unused)
  int order_by_index;         // 0: (score desc, index asc); 1: ascending index
  int use_bitmap;             // order_by_index served by the shared-memory bitmap
  int from_candidates;        // the candidate lists were filled by the scorer: no histogram / thresholds
  const uint32_t* row_failed; // [R] with from_candidates: rows whose list is unusable; `scores` holds their full row
  const int32_t* T_dev;       // optional (fused step): the row length lives on the device; T is then its upper bound
  uint64_t* out_comp;         // optional output: the winners' composites, re-based to the returned (global) index
  // gathered source (merge of sequence shards): the row's elements are gather_n segments of gather_len
  // ready-made composites (global ids), segment s of row r at gather + s*gather_stride + r*gather_len;
  // T is then the global id range (for the bitmap), and every segment must hold at least k real entries
  const uint64_t* gather;
  int gather_n, gather_len;
  int64_t gather_stride;
  // with from_candidates: a row whose candidate count misses [kk, cap] is re-scored, whole, by this
  // kernel into `scores` (the group-max workspace) and then selected by the refinement path
  int rescue;
  ScoreParams rescue_sp;
  // unordered output only: the split_k best winners are written first (positions [0, split_k)), the
  // others after them, so that a reader may take a prefix of the list as "the split_k best"
  int split_k = 0;
  // gathered source only: every segment has its gather_prefix best entries first (see split_k). The
  // kernel then selects from the prefixes alone and accepts the result iff no segment can hold a
  // better entry behind its prefix; otherwise it falls back to the whole segments
  int gather_prefix = 0;
  // optional second output: the winners whose id lies in [own_base, own_limit), compacted, and how many
  int32_t* out_owned = nullptr;
  int32_t* out_owned_count = nullptr;
  int64_t own_base = 0, own_limit = 0;
  int common_start = 1;       // start the on-chip select below the common key prefix of the candidates
  // Sequence-sharded step without a collective: the local top-k kernel PUSHES its best entries into every
  // rank's inbox (push.n > 0, unordered output with split_k == push.prefix or push.prefix >= kk); the merge
  // kernel WAITS for all ranks' flags (wait.n > 0) and then selects from its local inbox (`gather`, rows
  // gather_pitch apart), falling back to the ranks' whole lists (wait.full) for a row its prefixes cannot decide.
  int stage = 0;              // unordered output: 12 * kk bytes of staging follow the fixed shared-memory areas
  int out_pitch = 0;          // row pitch of the outputs; 0 = kk
  int gather_pitch = 0;       // row pitch of a segment in `gather`; 0 = gather_len
  PeerPush push;
  PeerWait wait;
};

__device__ __forceinline__ uint32_t element_index(const SelectParams& p, int row, int64_t t) {
  return p.payload ? (uint32_t)p.payload[(int64_t)row * p.row_stride + t] : (uint32_t)(t + p.idx_offset);
}

// Exclusive prefix sum of one value per thread over the CTA; also returns the total.
// s_warp needs NT/32 + 1 words. Ends with a barrier.
template <int NT>
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* s_warp, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = lane < NT / 32 ? s_warp[lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, wi, off);
      if (lane >= off) wi += n;
    }
    if (lane < NT / 32) s_warp[lane] = wi - w;
    if (lane == 31) s_warp[NT / 32] = wi;
  }
  __syncthreads();
  const uint32_t res = s_warp[warp] + incl - v;
  total = s_warp[NT / 32];
  __syncthreads();
  return res;
}

// Whole-CTA search of a histogram from its TOP bin downwards: finds the bin d whose cumulative
// count (bins > d, then bin d) first reaches `need` (1 <= need <= total). Results, identical in
// every thread: bin d, count of elements in bins above d, count in bin d.
// `hist` may live in global or shared memory. s_tmp needs 80 words. Ends with a barrier.
template <int NT>
__device__ __forceinline__ void find_threshold(const uint32_t* hist, int nbins, uint32_t need, uint32_t* s_tmp,
                                               uint32_t& bin_out, uint32_t& above_out, uint32_t& in_out) {
  constexpr int MAXPER = SEL_HIST_BINS / 256;         // largest bins-per-thread ever asked for (NT >= 256)
  const int tid = threadIdx.x;
  const int per = (nbins + NT - 1) / NT;              // bins per thread, taken from the top
  // thread i owns reversed bins [i*per, (i+1)*per): reversed bin r <-> bin nbins-1-r
  uint32_t local[MAXPER];
  uint32_t sum = 0;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    const int r = tid * per + j;
    local[j] = (j < per && r < nbins) ? hist[nbins - 1 - r] : 0u;
    sum += local[j];
  }
  uint32_t total;
  const uint32_t excl = block_exclusive_scan<NT>(sum, s_tmp, total);
  uint32_t* s_res = s_tmp + 64;
  if (excl < need && need <= excl + sum) {
    uint32_t cum = excl, bin = 0, inb = 0;
    bool found = false;
#pragma unroll
    for (int j = 0; j < MAXPER; ++j) {
      if (!found) {
        if (cum + local[j] >= need) {
          bin = (uint32_t)(nbins - 1 - (tid * per + j));
          inb = local[j];
          found = true;
        } else {
          cum += local[j];
        }
      }
    }
    s_res[0] = bin;
    s_res[1] = cum;
    s_res[2] = inb;
  }
  __syncthreads();
  bin_out = s_res[0];
  above_out = s_res[1];
  in_out = s_res[2];
  __syncthreads();
}

// Histogram of the top 12 key bits of every row (only when the scorer did not produce one).
__global__ void __launch_bounds__(SEL_SCAN_THREADS) select_hist_kernel(SelectParams p, uint32_t* hist_out) {
  __shared__ uint32_t s_hist[SEL_HIST_BINS];
  const int row = blockIdx.y;
  for (int i = threadIdx.x; i < SEL_HIST_BINS; i += SEL_SCAN_THREADS) s_hist[i] = 0;
  __syncthreads();
  const float* src = p.scores + (int64_t)row * p.row_stride;
  const int64_t t0 = (int64_t)blockIdx.x * p.tokens_per_cta;
  int64_t t1 = t0 + p.tokens_per_cta;
  if (t1 > p.T) t1 = p.T;
  for (int64_t t = t0 + threadIdx.x; t < t1; t += SEL_SCAN_THREADS)
    atomicAdd(&s_hist[float_to_key(src[t]) >> (32 - SEL_HIST_BITS)], 1u);
  __syncthreads();
  uint32_t* gh = hist_out + (int64_t)row * SEL_HIST_BINS;
  for (int i = threadIdx.x; i < SEL_HIST_BINS; i += SEL_SCAN_THREADS) {
    const uint32_t c = s_hist[i];
    if (c) atomicAdd(&gh[i], c);
  }
}

// One CTA per row: the bin that holds the k-th element, the count above it and inside it.
__global__ void __launch_bounds__(SEL_SCAN_THREADS) select_threshold_kernel(SelectParams p) {
  __shared__ uint32_t s_tmp[80];
  const int row = blockIdx.x;
  uint32_t bin, above, inb;
  find_threshold<SEL_SCAN_THREADS>(p.hist + (int64_t)row * SEL_HIST_BINS, SEL_HIST_BINS, (uint32_t)p.kk, s_tmp, bin,
                                   above, inb);
  if (threadIdx.x == 0) p.thresholds[row] = make_uint4(bin, above, inb, 0u);
}

// Appends every element whose top-12-bit bin is >= the threshold bin to the row's candidate list
// (skipped for rows whose candidate set would not fit; the final kernel handles those).
// Warps work alone: a warp holds 512 elements in registers (16 per lane, loads issued before the
// threshold is read), ranks its candidates with a shuffle scan and reserves its output range with
// ONE atomic; there is no block barrier.
constexpr int SEL_TOK_PER_THREAD = 16;
constexpr int SEL_TOK_PER_WARP = SEL_TOK_PER_THREAD * 32;                 // 512
constexpr int SEL_TOK_PER_CTA = SEL_TOK_PER_THREAD * SEL_SCAN_THREADS;   // 4096

// One 512-element chunk per warp, 16 elements per lane held in registers (loads issued before the
// threshold is read). Winners are first queued in shared memory (a few predicated stores per
// element), then the lanes copy the queue out together: the 64-bit composites are built and
// stored once per winner, coalesced, instead of once per element slot.
template <bool VEC>
__global__ void __launch_bounds__(SEL_SCAN_THREADS, 6) select_collect_kernel(SelectParams p) {
  __shared__ uint2 s_queue[SEL_SCAN_THREADS / 32][SEL_TOK_PER_WARP];
  __shared__ uint32_t s_wtotal[SEL_SCAN_THREADS / 32 + 1];
  const int row = blockIdx.y;
  const float* src = p.scores + (int64_t)row * p.row_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = blockIdx.x * SEL_TOK_PER_CTA + warp * SEL_TOK_PER_WARP;     // T < 2^31; may lie past the row end

  float v[SEL_TOK_PER_THREAD];
  const float qnan = __int_as_float(0x7fc00000);           // padding compares false against anything
#pragma unroll
  for (int j = 0; j < SEL_TOK_PER_THREAD / 4; ++j) {
    const int t = t0 + j * 128 + lane * 4;
    float4 x = make_float4(qnan, qnan, qnan, qnan);
    if (VEC && t + 3 < p.T) {
      x = __ldcg(reinterpret_cast<const float4*>(src + t));
    } else {
      if (t < p.T) x.x = __ldcg(src + t);
      if (t + 1 < p.T) x.y = __ldcg(src + t + 1);
      if (t + 2 < p.T) x.z = __ldcg(src + t + 2);
      if (t + 3 < p.T) x.w = __ldcg(src + t + 3);
    }
    v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
  }
  // the row's threshold is read after the element loads were issued, so both latencies overlap
  const uint4 thr = __ldcg(p.thresholds + row);
  if (thr.y + thr.z > (uint32_t)p.cap) return;             // (CTA-uniform) this row is refined by the final kernel instead
  // key(v) >= bin << 20  <=>  v >= the float whose key is bin << 20 (keys are order preserving;
  // bins that only NaN patterns can reach are clamped to -inf / "nothing").
  const uint32_t key_lo = thr.x << (32 - SEL_HIST_BITS);
  float f_lo = key_to_float(key_lo);
  if (key_lo <= 0x007FFFFFu) f_lo = -INFINITY;
  uint32_t takemask = 0;
#pragma unroll
  for (int e = 0; e < SEL_TOK_PER_THREAD; ++e)
    if (v[e] >= f_lo) takemask |= 1u << e;
  const uint32_t cnt = (uint32_t)__popc(takemask);
  uint32_t incl = cnt;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += n;
  }
  const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
  // One global atomic per CTA (same-address atomics of a row queue up in L2): warp totals meet in
  // shared memory, thread 0 reserves the CTA's range, every warp takes its slice.
  if (lane == 0) s_wtotal[warp] = total;
  uint2* q = s_queue[warp];
  uint32_t qpos = incl - cnt;
#pragma unroll
  for (int e = 0; e < SEL_TOK_PER_THREAD; ++e) {
    if (takemask & (1u << e)) {
      q[qpos] = make_uint2(__float_as_uint(v[e]), (uint32_t)((e >> 2) * 128 + lane * 4 + (e & 3)));
      ++qpos;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t sum = 0;
#pragma unroll
    for (int w = 0; w < SEL_SCAN_THREADS / 32; ++w) {
      const uint32_t c = s_wtotal[w];
      s_wtotal[w] = sum;
      sum += c;
    }
    s_wtotal[SEL_SCAN_THREADS / 32] = sum ? atomicAdd(p.cand_count + (int64_t)row * SEL_COUNT_STRIDE, sum) : 0u;
  }
  __syncthreads();
  if (total == 0) return;
  const uint32_t base = s_wtotal[SEL_SCAN_THREADS / 32] + s_wtotal[warp];
  uint64_t* cand = p.cand + (int64_t)row * p.cap;
  for (uint32_t i = lane; i < total; i += 32) {
    const uint2 e = q[i];
    const int t = t0 + (int)e.y;
    if (base + i < (uint32_t)p.cap) cand[base + i] = make_composite(__uint_as_float(e.x), element_index(p, row, t));
  }
}

// Descending bitonic sort of n (a power of two) 64-bit keys in shared memory by the whole CTA.
// find_threshold for a shared-memory histogram that is re-used pass after pass: every thread clears the
// bins it has read (the next pass needs no clearing loop and no barrier for it), and the barriers that only
// protect s_tmp against the next call are dropped: the next call writes s_tmp[0..NT/32] after a barrier of
// its own caller (the one behind the histogram atomics) and s_tmp[64..66] after two more barriers.
template <int NT>
__device__ __forceinline__ void find_threshold_clear(uint32_t* hist, int nbins, uint32_t need, uint32_t* s_tmp,
                                                     uint32_t& bin_out, uint32_t& above_out, uint32_t& in_out) {
  constexpr int MAXPER = 2048 / NT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int per = (nbins + NT - 1) / NT;              // bins per thread, taken from the top
  uint32_t local[MAXPER];
  uint32_t sum = 0;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    const int r = tid * per + j;                      // reversed bin r <-> bin nbins-1-r
    const bool live = j < per && r < nbins;
    local[j] = live ? hist[nbins - 1 - r] : 0u;
    if (live) hist[nbins - 1 - r] = 0u;
    sum += local[j];
  }
  uint32_t incl = sum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += nb;
  }
  if (lane == 31) s_tmp[warp] = incl;
  __syncthreads();
  // every warp scans the (at most 32) warp totals itself: no second hand-over through shared memory
  uint32_t w = lane < NT / 32 ? s_tmp[lane] : 0u;
  uint32_t wi = w;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, wi, off);
    if (lane >= off) wi += nb;
  }
  const uint32_t warp_excl = __shfl_sync(0xffffffffu, wi - w, warp);
  const uint32_t excl = warp_excl + incl - sum;
  uint32_t* s_res = s_tmp + 64;
  if (excl < need && need <= excl + sum) {
    uint32_t cum = excl, bin = 0, inb = 0;
    bool found = false;
#pragma unroll
    for (int j = 0; j < MAXPER; ++j) {
      if (!found) {
        if (cum + local[j] >= need) {
          bin = (uint32_t)(nbins - 1 - (tid * per + j));
          inb = local[j];
          found = true;
        } else {
          cum += local[j];
        }
      }
    }
    s_res[0] = bin;
    s_res[1] = cum;
    s_res[2] = inb;
  }
  __syncthreads();
  bin_out = s_res[0];
  above_out = s_res[1];
  in_out = s_res[2];
}
template <int NT>
__device__ __forceinline__ void bitonic_sort_desc(uint64_t* s, int n) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < (n >> 1); i += NT) {
        const int lo = 2 * i - (i & (stride - 1));     // index with the `stride` bit clear
        const int hi = lo + stride;
        const bool desc = ((lo & size) == 0);          // first half of each 2*size block descends
        const uint64_t a = s[lo], b = s[hi];
        if ((a < b) == desc) { s[lo] = b; s[hi] = a; }
      }
      __syncthreads();
    }
  }
}

// Copies n 64-bit entries from global to shared memory with eight loads of every thread in flight at once
// (a plain strided loop leaves one dependent L2 round trip per iteration on the critical path of the CTA).
template <int NT>
__device__ __forceinline__ void load_list_to_smem(uint64_t* dst, const uint64_t* src, int n) {
  for (int i0 = 0; i0 < n; i0 += NT * 8) {
    uint64_t v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * NT + (int)threadIdx.x;
      v[u] = i < n ? __ldcg(src + i) : 0ull;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * NT + (int)threadIdx.x;
      if (i < n) dst[i] = v[u];
    }
  }
}

// Exclusive prefix sums of TWO values per thread over the CTA with the barriers of one scan; also the totals.
// s_warp needs 2 * (NT/32 + 1) words. Ends with a barrier.
template <int NT>
__device__ __forceinline__ void block_exclusive_scan2(uint32_t va, uint32_t vb, uint32_t* s_warp, uint32_t& ea,
                                                      uint32_t& eb, uint32_t& ta, uint32_t& tb) {
  constexpr int NW = NT / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t ia = va, ib = vb;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t na = __shfl_up_sync(0xffffffffu, ia, off), nb = __shfl_up_sync(0xffffffffu, ib, off);
    if (lane >= off) { ia += na; ib += nb; }
  }
  if (lane == 31) { s_warp[warp] = ia; s_warp[NW + 1 + warp] = ib; }
  __syncthreads();
  // every warp scans the (at most 32) warp totals itself
  uint32_t wa = lane < NW ? s_warp[lane] : 0u, wb = lane < NW ? s_warp[NW + 1 + lane] : 0u;
  uint32_t sa = wa, sb = wb;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t na = __shfl_up_sync(0xffffffffu, sa, off), nb = __shfl_up_sync(0xffffffffu, sb, off);
    if (lane >= off) { sa += na; sb += nb; }
  }
  ea = __shfl_sync(0xffffffffu, sa - wa, warp) + ia - va;
  eb = __shfl_sync(0xffffffffu, sb - wb, warp) + ib - vb;
  ta = __shfl_sync(0xffffffffu, sa, 31);
  tb = __shfl_sync(0xffffffffu, sb, 31);
  __syncthreads();
}

// One CTA per row: candidates -> exact k-th composite -> the k winners in the requested order.
__global__ void __launch_bounds__(SEL_FINAL_THREADS) select_final_kernel(SelectParams pin) {
  // the row length (and with it the count to select) may live on the device
  // (the parameters stay in constant memory: a modifiable copy would live on the thread's stack because
  // the rank tables are indexed at run time; only the two values that can change are held in registers)
  const SelectParams& p = pin;
  const int out_pitch = pin.out_pitch > 0 ? pin.out_pitch : pin.kk;     // rows of the outputs stay kk_max apart
  int rT = pin.T, rkk = pin.kk;
  // A kernel that pushes its winners to the ranks is followed by a merge that reads the step number WITHOUT
  // waiting for its predecessors: that merge may become resident only after this kernel's own wait has
  // returned, i.e. after the first kernel of the step — which increments the step number — has completed.
  if (pin.push.n == 0) pdl_launch_dependents();
  // The merge of the ranks' prefixes takes nothing from the kernel before it in the stream except what that
  // kernel stores into the inbox as tagged pairs (and, for a row the prefixes cannot decide, lists guarded by
  // flags): it does not wait for that kernel to end — its blocks poll the pairs while the local select still
  // runs, so neither that kernel's tail (the release of its flags) nor a launch gap lies on the step's path.
  if (pin.wait.n == 0) pdl_wait();
  if (pin.push.n > 0) pdl_launch_dependents();
  if (p.T_dev) {
    const int t = *p.T_dev;
    rT = t < pin.T ? t : pin.T;
    rkk = p.k < rT ? p.k : rT;
  }
  extern __shared__ __align__(16) uint8_t sel_smem[];
  uint64_t* s_cand = reinterpret_cast<uint64_t*>(sel_smem);                     // [cap]
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(sel_smem + (size_t)p.cap * 8);  // [2048]
  uint32_t* s_tmp = s_hist + 2048;                                              // [NT + 40] (80 used)
  uint32_t* s_count = s_tmp + SEL_FINAL_THREADS + 40;                           // [8]
  unsigned long long* s_segmin = reinterpret_cast<unsigned long long*>(s_count + 8);   // [SEL_MAX_SEGMENTS]
  uint32_t* s_bitmap = reinterpret_cast<uint32_t*>(s_segmin + SEL_MAX_SEGMENTS); // [ceil(T/32)] when use_bitmap

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const bool peer = p.wait.n > 0;
  uint32_t epoch = 0;
  if (p.push.n > 0) epoch = *p.push.epoch;
  // (the arrival word lives in the dynamic area: this kernel may ask for all the shared memory there is, which
  // leaves no room for a static variable)
  volatile uint32_t* s_arrived = s_count + 7;
  if (peer) {
    epoch = *p.wait.epoch;
    if (tid == 0) *s_arrived = 1;
    __syncthreads();
  }
  // Every rank's flag for this row (its whole list may be read): bounded; false when one never came.
  auto wait_for_lists = [&]() -> bool {
    if (tid < p.wait.n && !wait_flag_bounded(p.wait.flags + (int64_t)tid * p.R + row, epoch, p.wait.limit)) *s_arrived = 0;
    __syncthreads();
    const bool arrived = *s_arrived != 0;
    __syncthreads();
    return arrived;
  };
  auto give_up = [&]() {                                  // (status word set): this row selects nothing
    if (tid == 0 && p.out_owned_count) p.out_owned_count[row] = 0;
  };
  const float* src = p.scores ? p.scores + (int64_t)row * p.row_stride : nullptr;
  const bool gathered = p.gather_n > 0;
  const int gpitch = p.gather_pitch > 0 ? p.gather_pitch : p.gather_len;
  const int64_t n_src = gathered ? (int64_t)p.gather_n * p.gather_len : (int64_t)rT;     // elements of the row
  // composite of element t of this row, whatever the source
  auto load_comp = [&](int64_t t) -> uint64_t {
    if (gathered) {
      const int64_t seg = t / p.gather_len;
      const int64_t off = (int64_t)row * p.gather_len + (t - seg * p.gather_len);
      // whole lists: a slice of the all-gathered buffer, or (peer exchange) the list in rank seg's own memory
      return peer ? __ldcg(p.wait.full[seg] + off) : __ldcg(p.gather + seg * p.gather_stride + off);
    }
    return make_composite(src[t], element_index(p, row, t));
  };

  uint64_t prefix;                                      // top `fixed` bits of the k-th composite so far
  int fixed;
  uint32_t need;                                        // still to take from inside the prefix
  uint32_t in_prefix;
  int n = 0;                                            // candidates in s_cand: all with composite >= prefix
  bool have_candidates;
  uint64_t kth;
  const uint64_t* cand = p.cand ? p.cand + (int64_t)row * p.cap : nullptr;
  bool prefix_mode = gathered && p.gather_prefix > 0 && (peer || p.gather_prefix < p.gather_len) &&
                     p.gather_n <= SEL_MAX_SEGMENTS && (int64_t)p.gather_n * p.gather_prefix <= (int64_t)p.cap &&
                     (int64_t)p.gather_n * p.gather_prefix >= (int64_t)rkk;
again:
  if (prefix_mode) {
    // The best gather_prefix entries of every segment, all on chip; the smallest of each prefix is kept
    // for the acceptance test after the select.
    for (int i = tid; i < p.gather_n; i += SEL_FINAL_THREADS) s_segmin[i] = ~0ull;
    __syncthreads();
    n = p.gather_n * p.gather_prefix;
    for (int i0 = 0; i0 < n; i0 += SEL_FINAL_THREADS * 8) {          // eight loads of every thread in flight
      uint64_t v[8];
      if (peer) {
        // tagged pairs stored by the ranks' select kernels: all eight loads first, then whatever has not arrived
        uint4 w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * SEL_FINAL_THREADS + tid;
          const int seg = i / p.gather_prefix, j = i - seg * p.gather_prefix;
          w[u] = i < n ? ld_pair2(p.wait.inbox + ((int64_t)seg * p.R + row) * p.gather_prefix + j) : make_uint4(0, epoch, 0, epoch);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * SEL_FINAL_THREADS + tid;
          const int seg = i / p.gather_prefix, j = i - seg * p.gather_prefix;
          v[u] = 0ull;
          if (i < n && !wait_pair2(p.wait.inbox + ((int64_t)seg * p.R + row) * p.gather_prefix + j, w[u], epoch, p.wait.limit, v[u]))
            *s_arrived = 0;
        }
      } else {
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * SEL_FINAL_THREADS + tid;
          const int seg = i / p.gather_prefix, j = i - seg * p.gather_prefix;
          v[u] = i < n ? __ldcg(p.gather + (int64_t)seg * p.gather_stride + (int64_t)row * gpitch + j) : 0ull;
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * SEL_FINAL_THREADS + tid;
        if (i < n) {
          s_cand[i] = v[u];
          if (p.gather_prefix < p.gather_len) atomicMin(&s_segmin[i / p.gather_prefix], (unsigned long long)v[u]);
        }
      }
    }
    __syncthreads();
    if (peer && *s_arrived == 0) { give_up(); return; }  // a rank's entries never came (uniform: read after the barrier)
    prefix = 0; fixed = 0; need = (uint32_t)rkk; in_prefix = (uint32_t)n;
    have_candidates = true;
  } else if (gathered) {
    if (peer && !wait_for_lists()) { give_up(); return; }  // the whole lists live in the ranks' memory
    // All-gathered shard lists: up to gather_n * gather_len composites, far more than fit on chip. The
    // refinement below narrows them with 11-bit histogram passes over global memory (two passes bring
    // i.i.d. shard lists under the capacity) and then collects the survivors.
    // (Dropping everything below "max over segments of the segment minimum" is exact but useless here:
    // each shard's worst entry lies far below the global k-th one.)
    prefix = 0; fixed = 0; need = (uint32_t)rkk; in_prefix = (uint32_t)n_src;
    have_candidates = false;
  } else if (p.from_candidates) {
    prefix = 0; fixed = 0; need = (uint32_t)rkk;
    bool failed = p.row_failed != nullptr && p.row_failed[row] != 0;
    if (p.rescue && !failed) {
      const uint32_t have = p.cand_count[(int64_t)row * SEL_COUNT_STRIDE];
      if (have < (uint32_t)rkk || have > (uint32_t)p.cap) {
        // the sampled threshold missed its bounds for this row: score the whole row again, exactly
        const ScoreParams& sp = p.rescue_sp;
        float* r_qv = reinterpret_cast<float*>(s_cand);                    // scratch inside the (still unused) candidate area
        float* r_qscale = r_qv + SC_MAX_G * SC_MAX_C;
        int8_t* r_qcode = reinterpret_cast<int8_t*>(r_qscale + SC_MAX_G);
        const int rb = row / sp.Hkv, rg = row - rb * sp.Hkv;
        quantize_query_group<SEL_FINAL_THREADS>(sp, rb, rg, sp.G, r_qv, r_qcode, r_qscale);
        float* dst = const_cast<float*>(src);
        for (int64_t t = tid; t < rT; t += SEL_FINAL_THREADS)
          dst[t] = score_token_plain<SC_MAX_G>(sp, sp.G, rb, rg, t, r_qcode, r_qscale);
        __syncthreads();
        failed = true;
      }
    }
    have_candidates = !failed;
    if (failed) {
      in_prefix = (uint32_t)rT;
    } else {
      const uint32_t have = p.cand_count[(int64_t)row * SEL_COUNT_STRIDE];
      n = (int)(have < (uint32_t)p.cap ? have : (uint32_t)p.cap);
      in_prefix = (uint32_t)n;
      load_list_to_smem<SEL_FINAL_THREADS>(s_cand, cand, n);
      __syncthreads();
    }
  } else {
    const uint4 thr = p.thresholds[row];
    prefix = thr.x; fixed = SEL_HIST_BITS; need = (uint32_t)rkk - thr.y; in_prefix = thr.z;
    have_candidates = thr.y + thr.z <= (uint32_t)p.cap;
    if (have_candidates) {
      n = (int)(thr.y + thr.z);
      const uint32_t have = p.cand_count[(int64_t)row * SEL_COUNT_STRIDE];
      if ((uint32_t)n > have) n = (int)have;            // cannot happen; keeps reads in bounds
      load_list_to_smem<SEL_FINAL_THREADS>(s_cand, cand, n);
      __syncthreads();
    }
  }
  if (!have_candidates) {
    // Too many candidates share the prefix (or none were prepared): refine over the row itself.
    while ((uint32_t)rkk - need + in_prefix > (uint32_t)p.cap && fixed < 64) {
      const int width = (64 - fixed) >= 11 ? 11 : (64 - fixed);
      const int shift = 64 - fixed - width;
      const int nb = 1 << width;
      for (int i = tid; i < nb; i += SEL_FINAL_THREADS) s_hist[i] = 0;
      __syncthreads();
      for (int64_t t = tid; t < n_src; t += SEL_FINAL_THREADS) {
        const uint64_t c = load_comp(t);
        if (fixed == 0 || (c >> (64 - fixed)) == prefix)
          atomicAdd(&s_hist[(uint32_t)(c >> shift) & (uint32_t)(nb - 1)], 1u);
      }
      __syncthreads();
      uint32_t d, ab, in;
      find_threshold<SEL_FINAL_THREADS>(s_hist, nb, need, s_tmp, d, ab, in);
      need -= ab;
      in_prefix = in;
      prefix = (prefix << width) | d;
      fixed += width;
    }
    if (tid == 0) *s_count = 0;
    __syncthreads();
    const int sh = 64 - fixed;
    for (int64_t t = tid; t < n_src; t += SEL_FINAL_THREADS) {
      const uint64_t c = load_comp(t);
      const bool take = (sh == 0) ? (c >= prefix) : (sh >= 64 ? true : ((c >> sh) >= prefix));
      if (take) {
        const uint32_t pos = atomicAdd(s_count, 1u);
        if (pos < (uint32_t)p.cap) s_cand[pos] = c;
      }
    }
    __syncthreads();
    n = (int)*s_count;
    if (n > p.cap) n = p.cap;
  }

  // When the select starts from scratch on a prepared list, the entries usually share many leading key
  // bits (all of them passed the same threshold): a digit taken there would send everything to one or two
  // histogram bins, i.e. thousands of shared-memory atomics on the same word. Start below the common
  // prefix of the smallest and the largest entry instead.
  uint64_t common_prefix = 0;
  int common_bits = 0;
  if (p.common_start && fixed == 0 && have_candidates && n > 1 && in_prefix > need) {
    unsigned long long lo = ~0ull, hi = 0ull;
    for (int i = tid; i < n; i += SEL_FINAL_THREADS) {
      const unsigned long long c = s_cand[i];
      lo = c < lo ? c : lo;
      hi = c > hi ? c : hi;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const unsigned long long ol = __shfl_xor_sync(0xffffffffu, lo, off), oh = __shfl_xor_sync(0xffffffffu, hi, off);
      lo = ol < lo ? ol : lo;
      hi = oh > hi ? oh : hi;
    }
    unsigned long long* s_mm = reinterpret_cast<unsigned long long*>(s_tmp);      // [2], 8-byte aligned
    if (tid == 0) { s_mm[0] = ~0ull; s_mm[1] = 0ull; }
    __syncthreads();
    if ((tid & 31) == 0) { atomicMin(&s_mm[0], lo); atomicMax(&s_mm[1], hi); }
    __syncthreads();
    lo = s_mm[0]; hi = s_mm[1];
    __syncthreads();                                  // s_tmp is reused by find_threshold
    const unsigned long long diff = lo ^ hi;
    common_bits = diff ? __clzll((long long)diff) : 63;
    if (common_bits > 0) {
      common_prefix = hi >> (64 - common_bits);
      prefix = common_prefix;
      fixed = common_bits;
    }
  }
  // Finish the radix select inside shared memory: stop when exactly `need` elements carry the prefix.
  if (in_prefix > need && fixed < 64) {               // the passes below clear the bins they read: zero once
    for (int i = tid; i < 2048; i += SEL_FINAL_THREADS) s_hist[i] = 0;
    __syncthreads();
  }
  while (in_prefix > need && fixed < 64) {
    const int width = (64 - fixed) >= 11 ? 11 : (64 - fixed);
    const int shift = 64 - fixed - width;
    const int nb = 1 << width;
    for (int i = tid; i < n; i += SEL_FINAL_THREADS) {
      const uint64_t c = s_cand[i];
      if (fixed == 0 || (c >> (64 - fixed)) == prefix)
        atomicAdd(&s_hist[(uint32_t)(c >> shift) & (uint32_t)(nb - 1)], 1u);
    }
    __syncthreads();
    uint32_t d, ab, in;
    find_threshold_clear<SEL_FINAL_THREADS>(s_hist, nb, need, s_tmp, d, ab, in);
    need -= ab;
    in_prefix = in;
    prefix = (prefix << width) | d;
    fixed += width;
  }
  kth = fixed >= 64 ? prefix : (fixed == 0 ? 0ull : (prefix << (64 - fixed)));   // winners: composite >= kth
  if (prefix_mode) {
    // Everything behind a segment's prefix is smaller than the prefix's smallest entry: if that entry is
    // itself no winner-beating value (<= kth), nothing behind it can be a winner. Otherwise start over
    // on the whole segments.
    bool ok = true;
    if (p.gather_prefix < p.gather_len)                 // (a prefix that is the whole list hides nothing)
      for (int sgm = 0; sgm < p.gather_n; ++sgm) ok = ok && (s_segmin[sgm] <= kth);
    if (!ok) {
      prefix_mode = false;
      n = 0;
      __syncthreads();
      goto again;
    }
  }

  // Composites built from scores carry index + idx_offset; scorer-made lists carry row-local ids and
  // gathered ones global ids: id_sub maps a composite's id to the bitmap position, id_add to the output.
  const uint32_t id_sub = (p.from_candidates || gathered) ? 0u : (uint32_t)p.idx_offset;
  const uint32_t id_add = gathered ? 0u : (uint32_t)p.idx_offset;
  if (p.order_by_index == 2) {
    // Unordered output: the winners in whatever order the threads meet them (the SET is exact); with
    // split_k the split_k best of them come first.
    uint64_t kth_split = ~0ull;
    const bool split = p.split_k > 0 && p.split_k < rkk;
    if (split) {
      // a second radix select over the same on-chip candidates, for rank split_k
      uint64_t pf = common_prefix;                    // (0 bits when the first select did not start from scratch)
      int fx = common_bits;
      uint32_t nd = (uint32_t)p.split_k, inp = (uint32_t)n;
      for (int i = tid; i < 2048; i += SEL_FINAL_THREADS) s_hist[i] = 0;
      __syncthreads();
      while (inp > nd && fx < 64) {
        const int width = (64 - fx) >= 11 ? 11 : (64 - fx);
        const int shift = 64 - fx - width;
        const int nb = 1 << width;
        for (int i = tid; i < n; i += SEL_FINAL_THREADS) {
          const uint64_t c = s_cand[i];
          if (fx == 0 || (c >> (64 - fx)) == pf) atomicAdd(&s_hist[(uint32_t)(c >> shift) & (uint32_t)(nb - 1)], 1u);
        }
        __syncthreads();
        uint32_t d, ab, in;
        find_threshold_clear<SEL_FINAL_THREADS>(s_hist, nb, nd, s_tmp, d, ab, in);
        nd -= ab;
        inp = in;
        pf = (pf << width) | d;
        fx += width;
      }
      kth_split = fx >= 64 ? pf : (fx == 0 ? 0ull : (pf << (64 - fx)));
    }
    const bool own = p.out_owned != nullptr;
    // Output positions come from prefix sums, not from atomics: a thread owns the entries tid, tid + NT, ...
    // (at most cap / NT <= 32 of them), notes in three bit masks which of them win, win among the split_k
    // best, and win inside the owned id range; two block scans then give every thread the start of its run
    // in each of the (up to) three output lists, and a second walk over the same entries writes them.
    uint32_t m_first = 0, m_second = 0, m_mine = 0;
    {
      int j = 0;
      for (int i = tid; i < n; i += SEL_FINAL_THREADS, ++j) {
        const uint64_t c = s_cand[i];
        const bool win = c >= kth;
        const bool first = win && !(split && c < kth_split);
        const uint32_t idx = (0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull)) - id_sub + id_add;
        const bool mine = own && win && (int64_t)idx >= p.own_base && (int64_t)idx < p.own_limit;
        m_first |= (first ? 1u : 0u) << j;
        m_second |= ((win && !first) ? 1u : 0u) << j;
        m_mine |= (mine ? 1u : 0u) << j;
      }
    }
    uint32_t pa, pb, pq = 0, ta, tb, tq = 0, unused_e, unused_t;
    block_exclusive_scan2<SEL_FINAL_THREADS>((uint32_t)__popc(m_first), (uint32_t)__popc(m_second), s_tmp, pa, pb, ta, tb);
    if (own) block_exclusive_scan2<SEL_FINAL_THREADS>((uint32_t)__popc(m_mine), 0u, s_tmp, pq, unused_e, tq, unused_t);
    (void)unused_e; (void)unused_t;
    if (tid == 0) s_count[2] = tq;
    // With a staging area the winners are first compacted in shared memory (a scatter there costs nothing) and
    // then written out by consecutive threads to consecutive addresses — the lists, and the prefix that goes to
    // the ranks' inboxes over NVLink, leave as full lines. Written straight from the walk, a warp's stores land
    // in 32 different sectors (a thread's winners are neighbours, the lanes' runs are not).
    const bool staged = p.stage != 0 && (!split || ta == (uint32_t)p.split_k);
    if (staged) {
      uint64_t* s_stage = reinterpret_cast<uint64_t*>(s_bitmap);                 // [rkk] (no bitmap in this mode)
      int32_t* s_own = reinterpret_cast<int32_t*>(s_stage + rkk);               // [rkk]
      int j = 0;
      for (int i = tid; i < n; i += SEL_FINAL_THREADS, ++j) {
        const bool first = (m_first >> j) & 1u, second = (m_second >> j) & 1u, mine = (m_mine >> j) & 1u;
        if (!(first || second)) continue;
        const uint64_t c = s_cand[i];
        const uint32_t idx = (0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull)) - id_sub + id_add;
        const uint32_t pos = first ? pa++ : (uint32_t)p.split_k + pb++;
        if (pos < (uint32_t)rkk) s_stage[pos] = (c & 0xFFFFFFFF00000000ull) | (uint64_t)(0xFFFFFFFFu - idx);
        if (mine) {
          if (pq < (uint32_t)rkk) s_own[pq] = (int32_t)idx;
          ++pq;
        }
      }
      __syncthreads();
      uint32_t filled = split ? (uint32_t)p.split_k + tb : ta;
      if (filled > (uint32_t)rkk) filled = (uint32_t)rkk;
      const uint32_t npush = p.push.n > 0 ? ((uint32_t)p.push.prefix < filled ? (uint32_t)p.push.prefix : filled) : 0u;
      const int64_t slot0 = ((int64_t)p.push.rank * p.R + row) * p.push.prefix;
      for (uint32_t t = tid; t < filled; t += SEL_FINAL_THREADS) {
        const uint64_t cg = s_stage[t];
        const uint32_t idx = 0xFFFFFFFFu - (uint32_t)(cg & 0xFFFFFFFFull);
        const int64_t o = (int64_t)row * out_pitch + t;
        if (p.out_idx32) p.out_idx32[o] = (int32_t)idx;
        if (p.out_idx64) p.out_idx64[o] = (int64_t)idx;
        if (p.out_scores) p.out_scores[o] = key_to_float((uint32_t)(cg >> 32));
        if (p.out_comp) p.out_comp[o] = cg;
        if (t < npush)
          for (int q = 0; q < p.push.n; ++q) st_pair2(p.push.inbox[q] + slot0 + t, cg, epoch);
      }
      if (own) {
        const uint32_t nown = tq < (uint32_t)rkk ? tq : (uint32_t)rkk;
        for (uint32_t t = tid; t < nown; t += SEL_FINAL_THREADS) p.out_owned[(int64_t)row * out_pitch + t] = s_own[t];
      }
    } else {
      int j = 0;
      for (int i = tid; i < n; i += SEL_FINAL_THREADS, ++j) {
        const bool first = (m_first >> j) & 1u, second = (m_second >> j) & 1u, mine = (m_mine >> j) & 1u;
        if (!(first || second)) continue;
        const uint64_t c = s_cand[i];
        const uint32_t idx = (0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull)) - id_sub + id_add;
        const uint32_t pos = first ? pa++ : (uint32_t)p.split_k + pb++;
        if (pos < (uint32_t)rkk) {
          const int64_t o = (int64_t)row * out_pitch + pos;
          if (p.out_idx32) p.out_idx32[o] = (int32_t)idx;
          if (p.out_idx64) p.out_idx64[o] = (int64_t)idx;
          if (p.out_scores) p.out_scores[o] = key_to_float((uint32_t)(c >> 32));
          const uint64_t cg = (c & 0xFFFFFFFF00000000ull) | (uint64_t)(0xFFFFFFFFu - idx);
          if (p.out_comp) p.out_comp[o] = cg;
          if (p.push.n > 0 && !p.out_comp && pos < (uint32_t)p.push.prefix) {      // (no local list to copy from)
            const int64_t slot = ((int64_t)p.push.rank * p.R + row) * p.push.prefix + pos;
            for (int q = 0; q < p.push.n; ++q) st_pair2(p.push.inbox[q] + slot, cg, epoch);
          }
        }
        if (mine) {
          if (pq < (uint32_t)rkk) p.out_owned[(int64_t)row * out_pitch + pq] = (int32_t)idx;
          ++pq;
        }
      }
    }
    if (own && p.out_owned_count) {
      __syncthreads();
      if (tid == 0) p.out_owned_count[row] = (int32_t)(s_count[2] < (uint32_t)rkk ? s_count[2] : (uint32_t)rkk);
    }
    if (p.push.n > 0 && p.out_comp && !staged) {
      // (no staging area) The prefix goes to the ranks' inboxes from the row's finished local list, not entry by
      // entry from the walk above: consecutive threads store consecutive entries, so a rank receives full lines
      // over NVLink instead of scattered stores.
      __syncthreads();                                   // the list of this row is complete (written by this CTA)
      int npush = p.push.prefix < rkk ? p.push.prefix : rkk;
      const uint64_t* mine = p.out_comp + (int64_t)row * out_pitch;
      const int64_t slot0 = ((int64_t)p.push.rank * p.R + row) * p.push.prefix;
      for (int j = tid; j < npush; j += SEL_FINAL_THREADS) {
        const uint64_t v = __ldcg(mine + j);
        for (int q = 0; q < p.push.n; ++q) st_pair2(p.push.inbox[q] + slot0 + j, v, epoch);
      }
    }
    if (p.push.n > 0) {
      // The prefix entries are tagged pairs and need nothing more. The flag tells a rank that this row's WHOLE
      // local list may be read (the merge does that only when the prefixes cannot decide the row): every
      // thread's stores precede the barrier, one thread per rank then releases the flag there
      // (the release is cumulative over the barrier: it orders every thread's stores before the flag, at system
      // scope, without a separate fence)
      __syncthreads();
      if (tid < p.push.n) st_release_sys_u32(p.push.flags[tid] + (int64_t)p.push.rank * p.R + row, epoch);
    }
    return;
  }
  if (p.use_bitmap) {
    // Ascending-index output: one bit per token of the row, read out in order.
    const int words = (rT + 31) >> 5;
    for (int i = tid; i < words; i += SEL_FINAL_THREADS) s_bitmap[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += SEL_FINAL_THREADS) {
      const uint64_t c = s_cand[i];
      if (c >= kth) {
        const uint32_t local = (0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull)) - id_sub;
        atomicOr(&s_bitmap[local >> 5], 1u << (local & 31));
      }
    }
    __syncthreads();
    const int per = (words + SEL_FINAL_THREADS - 1) / SEL_FINAL_THREADS;
    const int w0 = tid * per;
    uint32_t cnt = 0;
    for (int j = 0; j < per; ++j)
      if (w0 + j < words) cnt += (uint32_t)__popc(s_bitmap[w0 + j]);
    uint32_t total;
    uint32_t pos = block_exclusive_scan<SEL_FINAL_THREADS>(cnt, s_tmp, total);
    // a row with fewer candidates than kk: report how many it got and mark the unused tail
    if (p.out_owned_count && !p.out_owned) {
      const uint32_t got = total < (uint32_t)rkk ? total : (uint32_t)rkk;
      if (tid == 0) p.out_owned_count[row] = (int32_t)got;
      if (p.out_idx32)
        for (uint32_t i = got + tid; i < (uint32_t)out_pitch; i += SEL_FINAL_THREADS) p.out_idx32[(int64_t)row * out_pitch + i] = -1;
    }
    for (int j = 0; j < per; ++j) {
      if (w0 + j >= words) break;
      uint32_t bits = s_bitmap[w0 + j];
      while (bits) {
        const int bit = __ffs(bits) - 1;
        bits &= bits - 1;
        const uint32_t local = (uint32_t)(w0 + j) * 32u + (uint32_t)bit;
        if (pos < (uint32_t)rkk) {
          const int64_t o = (int64_t)row * out_pitch + pos;
          const uint32_t idx = local + id_add;
          if (p.out_idx32) p.out_idx32[o] = (int32_t)idx;
          if (p.out_idx64) p.out_idx64[o] = (int64_t)idx;
          if (p.out_scores && src) {
            float sv = src[local];
            if (sv == 0.0f) sv = 0.0f;
            p.out_scores[o] = sv;
          }
        }
        ++pos;
      }
    }
    return;
  }

  // Sorted output: losers become 0 (below every real composite); with order_by_index the key is
  // re-built so that a descending sort yields ascending indices.
  for (int i = tid; i < n; i += SEL_FINAL_THREADS) {
    const uint64_t c = s_cand[i];
    if (c < kth) s_cand[i] = 0;
    else if (p.order_by_index) s_cand[i] = ((c & 0xFFFFFFFFull) << 32) | (c >> 32);
  }
  int n2 = 2;
  while (n2 < n) n2 <<= 1;
  for (int i = n + tid; i < n2; i += SEL_FINAL_THREADS) s_cand[i] = 0;
  __syncthreads();
  bitonic_sort_desc<SEL_FINAL_THREADS>(s_cand, n2);
  for (int i = tid; i < rkk; i += SEL_FINAL_THREADS) {
    uint64_t c = s_cand[i];
    if (p.order_by_index) c = ((c & 0xFFFFFFFFull) << 32) | (c >> 32);
    const uint32_t idx = (0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull)) - id_sub + id_add;
    const int64_t o = (int64_t)row * out_pitch + i;
    if (p.out_idx32) p.out_idx32[o] = (int32_t)idx;
    if (p.out_idx64) p.out_idx64[o] = (int64_t)idx;
    if (p.out_scores) p.out_scores[o] = key_to_float((uint32_t)(c >> 32));
  }
}

static int select_cap(int k) {
  int c = 8192;
  while (c < 2 * k && c < SEL_MAX_K) c <<= 1;
  if (c < k) c = SEL_MAX_K;
  return c;
}

constexpr size_t SEL_FINAL_FIXED_SMEM = sizeof(uint32_t) * (2048 + SEL_FINAL_THREADS + 40 + 8) + 8 * SEL_MAX_SEGMENTS;
constexpr size_t SEL_SMEM_LIMIT = 227 * 1024;
// staging of the unordered output: kk composites + kk owned ids
static inline size_t select_stage_bytes(int kk) { return (size_t)kk * 12; }

// Opts select_final_kernel into its large dynamic shared memory once per device (the device must be
// current). Safe to call from several host threads: the flag is atomic and the attribute call is idempotent.
static int select_final_prepare(int device) {
  static std::atomic<bool> done[KVB_MAX_DEVICES];
  return ensure_dynamic_smem(select_final_kernel, done, device, SEL_SMEM_LIMIT);
}

struct SelectWorkspace {
  uint32_t* count;     // [R]      } zeroed per call, contiguous
  uint32_t* hist;      // [R,4096] }
  uint4* thresholds;   // [R]
  uint64_t* cand;      // [R,cap]
  size_t zero_bytes;   // count + hist
  size_t bytes;
};

static SelectWorkspace select_carve(void* base, int R, int k) {
  SelectWorkspace w;
  uint8_t* ptr = reinterpret_cast<uint8_t*>(base);
  size_t off = 0;
  w.count = reinterpret_cast<uint32_t*>(ptr + off);
  off += round_up(sizeof(uint32_t) * (size_t)R * SEL_COUNT_STRIDE, 256);
  w.hist = reinterpret_cast<uint32_t*>(ptr + off);
  off += round_up(sizeof(uint32_t) * (size_t)R * SEL_HIST_BINS, 256);
  w.zero_bytes = off;
  w.thresholds = reinterpret_cast<uint4*>(ptr + off);
  off += round_up(sizeof(uint4) * (size_t)R, 256);
  w.cand = reinterpret_cast<uint64_t*>(ptr + off);
  off += round_up(sizeof(uint64_t) * (size_t)R * select_cap(k), 256);
  w.bytes = off;
  return w;
}

// Shared by kvb_select_topk and the fused step. `zeroed` tells that the caller already cleared
// the first zero_bytes of the workspace (count + histogram) on this stream.
static int select_run(const float* scores, int64_t row_stride, const int32_t* payload, int R, int T, int k,
                      int64_t idx_offset, int order, int32_t* out_idx32, int64_t* out_idx64, float* out_scores,
                      const uint32_t* hist_in, bool hist_in_workspace, bool zeroed, void* workspace,
                      size_t workspace_bytes, int device, cudaStream_t st) {
  if (!scores || !workspace) return KVB_BAD_ARG;
  if (!out_idx32 && !out_idx64 && !out_scores) return KVB_BAD_ARG;
  if (R <= 0 || T <= 0 || k <= 0 || R > 65535) return KVB_BAD_SHAPE;
  if (order != 0 && order != 1) return KVB_BAD_ARG;
  const int kk = k < T ? k : T;
  if (kk > SEL_MAX_K) return KVB_BAD_SHAPE;
  if (row_stride < T) return KVB_BAD_SHAPE;
  if (!payload && (idx_offset < 0 || idx_offset + T > 0x7fffffffLL)) return KVB_BAD_SHAPE;
  if (!aligned_to(workspace, 256) || !aligned_to(scores, 4)) return KVB_BAD_ALIGN;
  SelectWorkspace w = select_carve(workspace, R, kk);
  if (workspace_bytes < w.bytes) return KVB_WORKSPACE_TOO_SMALL;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;

  SelectParams p;
  p.scores = scores; p.row_stride = row_stride; p.payload = payload;
  p.R = R; p.T = T; p.k = k; p.kk = kk; p.idx_offset = idx_offset;
  p.out_idx32 = out_idx32; p.out_idx64 = out_idx64; p.out_scores = out_scores;
  p.cand = w.cand; p.cand_count = w.count; p.cap = select_cap(kk);
  p.thresholds = w.thresholds;
  p.order_by_index = order;
  p.from_candidates = 0;
  p.row_failed = nullptr;
  p.T_dev = nullptr;
  p.out_comp = nullptr;
  p.gather = nullptr; p.gather_n = 0; p.gather_len = 0; p.gather_stride = 0;
  p.rescue = 0;
  const size_t bitmap_bytes = sizeof(uint32_t) * (size_t)((T + 31) / 32);
  size_t smem = (size_t)p.cap * 8 + SEL_FINAL_FIXED_SMEM;
  p.use_bitmap = (order == 1 && !payload && smem + bitmap_bytes <= SEL_SMEM_LIMIT) ? 1 : 0;
  if (p.use_bitmap) smem += bitmap_bytes;

  if (hist_in_workspace) {
    p.hist = w.hist;
    if (!zeroed) KVB_CHECK_CUDA(cudaMemsetAsync(w.count, 0, sizeof(uint32_t) * (size_t)R * SEL_COUNT_STRIDE, st));
  } else if (hist_in) {
    p.hist = hist_in;
    if (!zeroed) KVB_CHECK_CUDA(cudaMemsetAsync(w.count, 0, sizeof(uint32_t) * (size_t)R * SEL_COUNT_STRIDE, st));
  } else {
    if (!zeroed) KVB_CHECK_CUDA(cudaMemsetAsync(workspace, 0, w.zero_bytes, st));
    p.hist = w.hist;
    int splits = ceil_div(sm_count(device) * 8, R);
    const int max_splits = ceil_div(T, 2048);
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    int tokens_per_cta = ceil_div(ceil_div(T, splits), 32) * 32;
    splits = ceil_div(T, tokens_per_cta);
    p.tokens_per_cta = tokens_per_cta;
    select_hist_kernel<<<dim3(splits, R), SEL_SCAN_THREADS, 0, st>>>(p, w.hist);
    KVB_CHECK_CUDA(cudaGetLastError());
  }
  p.tokens_per_cta = SEL_TOK_PER_CTA;
  select_threshold_kernel<<<R, SEL_SCAN_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  const dim3 cgrid(ceil_div(T, SEL_TOK_PER_CTA), R);
  const bool vec = aligned_to(scores, 16) && (row_stride % 4) == 0;
  if (vec) select_collect_kernel<true><<<cgrid, SEL_SCAN_THREADS, 0, st>>>(p);
  else select_collect_kernel<false><<<cgrid, SEL_SCAN_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());

  { const int prc = select_final_prepare(device); if (prc != KVB_OK) return prc; }
  select_final_kernel<<<R, SEL_FINAL_THREADS, smem, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

// ---- built-in scratch for callers that cannot allocate ------------------------------------
// A fixed device array that lives in the library image: every GPU that loads the library holds
// these bytes until the process exits. Host code must not pass the array's name to a kernel (on
// the host it is only a stand-in symbol); the device address is looked up once per device.
constexpr size_t SEL_STATIC_SCRATCH_BYTES = 4u << 20;    // 4 MiB
static __device__ __align__(256) unsigned char g_select_static_scratch[SEL_STATIC_SCRATCH_BYTES];

// Device address of the built-in scratch on `device` (which must be current); looked up on the
// first call per device and remembered. The lookup is a runtime call that is not allowed while
// `st` is being captured into a graph: in that case nothing is called and KVB_BAD_ARG comes back,
// so the capture stays valid (make one call outside capture first).
static int select_static_scratch(int device, cudaStream_t st, void** out) {
  static std::atomic<void*> cached[KVB_MAX_DEVICES];
  if (device < 0 || device >= KVB_MAX_DEVICES) return KVB_BAD_DEVICE;
  void* ptr = cached[device].load(std::memory_order_acquire);
  if (!ptr) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) return KVB_CUDA_ERROR;
    if (cap != cudaStreamCaptureStatusNone) return KVB_BAD_ARG;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_select_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) return KVB_CUDA_ERROR;
    cached[device].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return KVB_OK;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_select_topk_static_limit_bytes(void) {
  return kvb::SEL_STATIC_SCRATCH_BYTES;
}

extern "C" __attribute__((visibility("default"))) int kvb_select_topk_static(
    const float* scores, int64_t row_stride, int R, int T, int k, int64_t idx_offset, int order, int32_t* out_idx32,
    int64_t* out_idx64, float* out_scores, int device, void* stream) {
  using namespace kvb;
  if (R <= 0 || T <= 0 || k <= 0) return KVB_BAD_SHAPE;
  const int kk = k < T ? k : T;
  if (kk > SEL_MAX_K) return KVB_BAD_SHAPE;
  if (select_carve(nullptr, R, kk).bytes > SEL_STATIC_SCRATCH_BYTES) return KVB_SCRATCH_LIMIT;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  void* scratch = nullptr;
  const int rc = select_static_scratch(device, reinterpret_cast<cudaStream_t>(stream), &scratch);
  if (rc != KVB_OK) return rc;
  // select_run clears the counters and the histogram itself (memset nodes, no allocation); the
  // candidate area needs no clearing because only the counted prefix is ever read.
  return select_run(scores, row_stride, nullptr, R, T, k, idx_offset, order, out_idx32, out_idx64, out_scores,
                    nullptr, /*hist_in_workspace=*/false, /*zeroed=*/false, scratch, SEL_STATIC_SCRATCH_BYTES, device,
                    reinterpret_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) size_t kvb_select_topk_workspace_bytes(int R, int T, int k) {
  (void)T;
  if (R <= 0 || k <= 0) return 0;
  if (k > kvb::SEL_MAX_K) k = kvb::SEL_MAX_K;
  return kvb::select_carve(nullptr, R, k).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_select_topk(
    const float* scores, int64_t row_stride, const int32_t* payload, int R, int T, int k, int64_t idx_offset,
    int order, int32_t* out_idx32, int64_t* out_idx64, float* out_scores, const uint32_t* hist_in, void* workspace,
    size_t workspace_bytes, int device, void* stream) {
  return kvb::select_run(scores, row_stride, payload, R, T, k, idx_offset, order, out_idx32, out_idx64, out_scores,
                         hist_in, /*hist_in_workspace=*/false, /*zeroed=*/false, workspace, workspace_bytes, device,
                         reinterpret_cast<cudaStream_t>(stream));
}

