// Stage 3: exact top-k per row with the order (score descending, index ascending).
//
// Every element becomes a unique 64-bit composite  (order-preserving key of the score) << 32 |
// (0xFFFFFFFF - index), so "larger composite" is exactly "better score, then lower index" and
// ties need no special case. Selection is an MSB-first radix select on the composite:
//   1. a 4096-bin histogram of the top 12 bits (taken from the scorer when it already made one),
//   2. every CTA finds the bin b* holding the k-th element and appends all elements of bins
//      >= b* to a per-row candidate list (a few thousand entries for Gaussian-like scores),
//   3. one CTA per row sorts the candidates in shared memory (bitonic, descending) and writes
//      the first k.
// When a row has more than CAP candidates after step 1 (heavy ties, e.g. constant scores) the
// last kernel refines the prefix with further 11-bit passes over the row itself until the
// candidate set fits; that path is slower but exact for any input.
#include "common.cuh"

namespace kvb {

constexpr int SEL_HIST_BITS = 12;
constexpr int SEL_HIST_BINS = 1 << SEL_HIST_BITS;
constexpr int SEL_SCAN_THREADS = 256;
constexpr int SEL_FINAL_THREADS = 1024;
constexpr int SEL_MAX_K = 16384;

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
  uint32_t* cand_count;       // [R]
  int cap;
  int tokens_per_cta;         // scan kernels: tokens per CTA along a row
};

__device__ __forceinline__ uint64_t make_composite(float score, uint32_t idx) {
  return ((uint64_t)float_to_key(score) << 32) | (uint64_t)(0xFFFFFFFFu - idx);
}

__device__ __forceinline__ uint32_t element_index(const SelectParams& p, int row, int64_t t) {
  return p.payload ? (uint32_t)p.payload[(int64_t)row * p.row_stride + t] : (uint32_t)(t + p.idx_offset);
}

// Whole-CTA search of a histogram from its TOP bin downwards: finds the bin d whose cumulative
// count (bins > d, then bin d) first reaches `need` (1 <= need <= total). Results, identical in
// every thread: bin d, count of elements in bins above d, count in bin d.
// `hist` may live in global or shared memory. s_tmp needs NT + 40 words. Ends with a barrier.
template <int NT>
__device__ __forceinline__ void find_threshold(const uint32_t* hist, int nbins, uint32_t need, uint32_t* s_tmp,
                                               uint32_t& bin_out, uint32_t& above_out, uint32_t& in_out) {
  const int tid = threadIdx.x;
  const int per = (nbins + NT - 1) / NT;              // bins per thread, taken from the top
  // thread i owns reversed bins [i*per, (i+1)*per): reversed bin r <-> bin nbins-1-r
  uint32_t sum = 0;
  for (int j = 0; j < per; ++j) {
    const int r = tid * per + j;
    if (r < nbins) sum += hist[nbins - 1 - r];
  }
  s_tmp[tid] = sum;
  __syncthreads();
  uint32_t* s_res = s_tmp + NT + 32;
  if (tid < 32) {
    constexpr int CH = NT / 32;                       // chunk sums per lane
    uint32_t lane_sum = 0;
    for (int j = 0; j < CH; ++j) lane_sum += s_tmp[tid * CH + j];
    uint32_t incl = lane_sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
      if (tid >= off) incl += v;
    }
    const uint32_t excl = incl - lane_sum;
    if (excl < need && need <= incl) {
      // the crossing lies inside this lane's chunks
      uint32_t cum = excl;
      int chunk = tid * CH;
      for (int j = 0; j < CH; ++j) {
        const uint32_t c = s_tmp[tid * CH + j];
        if (cum + c >= need) { chunk = tid * CH + j; break; }
        cum += c;
      }
      uint32_t bin = 0, inb = 0;
      for (int j = 0; j < per; ++j) {
        const int r = chunk * per + j;
        if (r >= nbins) break;
        const uint32_t c = hist[nbins - 1 - r];
        if (cum + c >= need) { bin = (uint32_t)(nbins - 1 - r); inb = c; break; }
        cum += c;
      }
      s_res[0] = bin;
      s_res[1] = cum;
      s_res[2] = inb;
    }
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

// Appends every element whose top-12-bit bin is >= the threshold bin to the row's candidate list
// (skipped for rows whose candidate set would not fit; the final kernel handles those).
__global__ void __launch_bounds__(SEL_SCAN_THREADS) select_collect_kernel(SelectParams p) {
  __shared__ uint32_t s_tmp[SEL_SCAN_THREADS + 40];
  const int row = blockIdx.y;
  uint32_t bin, above, inb;
  find_threshold<SEL_SCAN_THREADS>(p.hist + (int64_t)row * SEL_HIST_BINS, SEL_HIST_BINS, (uint32_t)p.kk, s_tmp, bin,
                                   above, inb);
  if (above + inb > (uint32_t)p.cap) return;
  const float* src = p.scores + (int64_t)row * p.row_stride;
  uint64_t* cand = p.cand + (int64_t)row * p.cap;
  uint32_t* count = p.cand_count + row;
  const int lane = threadIdx.x & 31;
  const int64_t t0 = (int64_t)blockIdx.x * p.tokens_per_cta;
  int64_t t1 = t0 + p.tokens_per_cta;
  if (t1 > p.T) t1 = p.T;
  // warp-uniform trip count so the ballots below see the whole warp
  for (int64_t tb = t0 + (threadIdx.x & ~31); tb < t1; tb += SEL_SCAN_THREADS) {
    const int64_t t = tb + lane;
    bool take = false;
    uint32_t key = 0;
    if (t < t1) {
      key = float_to_key(src[t]);
      take = (key >> (32 - SEL_HIST_BITS)) >= bin;
    }
    const uint32_t m = __ballot_sync(0xffffffffu, take);
    if (m) {
      uint32_t base = 0;
      const int leader = __ffs(m) - 1;
      if (lane == leader) base = atomicAdd(count, (uint32_t)__popc(m));
      base = __shfl_sync(0xffffffffu, base, leader);
      if (take) {
        const uint32_t pos = base + (uint32_t)__popc(m & ((1u << lane) - 1u));
        if (pos < (uint32_t)p.cap)
          cand[pos] = ((uint64_t)key << 32) | (uint64_t)(0xFFFFFFFFu - element_index(p, row, t));
      }
    }
  }
}

// Descending bitonic sort of n (a power of two) 64-bit keys in shared memory by the whole CTA.
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

// One CTA per row: take the prepared candidates (or refine the prefix over the row itself when
// they did not fit), sort, write the first kk.
__global__ void __launch_bounds__(SEL_FINAL_THREADS) select_final_kernel(SelectParams p) {
  extern __shared__ __align__(16) uint8_t sel_smem[];
  uint64_t* s_cand = reinterpret_cast<uint64_t*>(sel_smem);                     // [cap]
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(sel_smem + (size_t)p.cap * 8);  // [2048]
  uint32_t* s_tmp = s_hist + 2048;                                              // [NT + 40]
  uint32_t* s_count = s_tmp + SEL_FINAL_THREADS + 40;                           // [1]

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const float* src = p.scores + (int64_t)row * p.row_stride;

  uint32_t bin, above, inb;
  find_threshold<SEL_FINAL_THREADS>(p.hist + (int64_t)row * SEL_HIST_BINS, SEL_HIST_BINS, (uint32_t)p.kk, s_tmp, bin,
                                    above, inb);
  int n;   // number of candidates placed in s_cand
  if (above + inb <= (uint32_t)p.cap) {
    n = (int)(above + inb);
    const uint32_t have = p.cand_count[row];
    if ((uint32_t)n > have) n = (int)have;             // cannot happen; keeps reads in bounds
    const uint64_t* cand = p.cand + (int64_t)row * p.cap;
    for (int i = tid; i < n; i += SEL_FINAL_THREADS) s_cand[i] = cand[i];
  } else {
    // Refinement: prefix = the bits fixed so far (top `fixed` bits of the composite).
    uint64_t prefix = bin;
    int fixed = SEL_HIST_BITS;
    uint32_t need = (uint32_t)p.kk - above;            // still to take from inside the prefix
    uint32_t in_prefix = inb;
    while ((uint32_t)p.kk - need + in_prefix > (uint32_t)p.cap && fixed < 64) {
      const int width = (64 - fixed) >= 11 ? 11 : (64 - fixed);
      const int shift = 64 - fixed - width;
      const int nb = 1 << width;
      for (int i = tid; i < nb; i += SEL_FINAL_THREADS) s_hist[i] = 0;
      __syncthreads();
      for (int64_t t = tid; t < p.T; t += SEL_FINAL_THREADS) {
        const uint64_t c = make_composite(src[t], element_index(p, row, t));
        if ((c >> (64 - fixed)) == prefix) atomicAdd(&s_hist[(uint32_t)(c >> shift) & (uint32_t)(nb - 1)], 1u);
      }
      __syncthreads();
      uint32_t d, ab, in;
      find_threshold<SEL_FINAL_THREADS>(s_hist, nb, need, s_tmp, d, ab, in);
      need -= ab;
      in_prefix = in;
      prefix = (prefix << width) | d;
      fixed += width;
    }
    // Collect everything at or above the prefix: (kk - need) sure ones + in_prefix <= cap.
    if (tid == 0) *s_count = 0;
    __syncthreads();
    const int sh = 64 - fixed;
    for (int64_t t = tid; t < p.T; t += SEL_FINAL_THREADS) {
      const uint64_t c = make_composite(src[t], element_index(p, row, t));
      const bool take = (sh >= 64) ? true : ((c >> sh) >= prefix);
      if (take) {
        const uint32_t pos = atomicAdd(s_count, 1u);
        if (pos < (uint32_t)p.cap) s_cand[pos] = c;
      }
    }
    __syncthreads();
    n = (int)*s_count;
    if (n > p.cap) n = p.cap;
  }
  int n2 = 1;
  while (n2 < n) n2 <<= 1;
  if (n2 < 2) n2 = 2;
  for (int i = n + tid; i < n2; i += SEL_FINAL_THREADS) s_cand[i] = 0;   // below every real composite
  __syncthreads();
  bitonic_sort_desc<SEL_FINAL_THREADS>(s_cand, n2);
  for (int i = tid; i < p.kk; i += SEL_FINAL_THREADS) {
    const uint64_t c = s_cand[i];
    const uint32_t idx = 0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull);
    const int64_t o = (int64_t)row * p.kk + i;
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

struct SelectWorkspace {
  uint32_t* hist;
  uint64_t* cand;
  uint32_t* count;
  size_t bytes;
};

static SelectWorkspace select_carve(void* base, int R, int k) {
  SelectWorkspace w;
  uint8_t* ptr = reinterpret_cast<uint8_t*>(base);
  size_t off = 0;
  w.count = reinterpret_cast<uint32_t*>(ptr + off);
  off += round_up(sizeof(uint32_t) * (size_t)R, 256);
  w.hist = reinterpret_cast<uint32_t*>(ptr + off);
  off += round_up(sizeof(uint32_t) * (size_t)R * SEL_HIST_BINS, 256);
  w.cand = reinterpret_cast<uint64_t*>(ptr + off);
  off += round_up(sizeof(uint64_t) * (size_t)R * select_cap(k), 256);
  w.bytes = off;
  return w;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_select_topk_workspace_bytes(int R, int T, int k) {
  (void)T;
  if (R <= 0 || k <= 0) return 0;
  if (k > kvb::SEL_MAX_K) k = kvb::SEL_MAX_K;
  return kvb::select_carve(nullptr, R, k).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_select_topk(const float* scores, int64_t row_stride, const int32_t* payload, int R, int T, int k,
                               int64_t idx_offset, int32_t* out_idx32, int64_t* out_idx64, float* out_scores,
                               const uint32_t* hist_in, void* workspace, size_t workspace_bytes, int device,
                               void* stream) {
  using namespace kvb;
  if (!scores || !workspace) return KVB_BAD_ARG;
  if (!out_idx32 && !out_idx64 && !out_scores) return KVB_BAD_ARG;
  if (R <= 0 || T <= 0 || k <= 0 || R > 65535) return KVB_BAD_SHAPE;
  const int kk = k < T ? k : T;
  if (kk > SEL_MAX_K) return KVB_BAD_SHAPE;
  if (row_stride < T) return KVB_BAD_SHAPE;
  if (!payload && (idx_offset < 0 || idx_offset + T > 0x7fffffffLL)) return KVB_BAD_SHAPE;
  if (!aligned_to(workspace, 256) || !aligned_to(scores, 4)) return KVB_BAD_ALIGN;
  SelectWorkspace w = select_carve(workspace, R, kk);
  if (workspace_bytes < w.bytes) return KVB_WORKSPACE_TOO_SMALL;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  SelectParams p;
  p.scores = scores; p.row_stride = row_stride; p.payload = payload;
  p.R = R; p.T = T; p.k = k; p.kk = kk; p.idx_offset = idx_offset;
  p.out_idx32 = out_idx32; p.out_idx64 = out_idx64; p.out_scores = out_scores;
  p.cand = w.cand; p.cand_count = w.count; p.cap = select_cap(kk);

  // CTAs along a row: aim at ~8 CTAs per SM in total, at least 2048 tokens each.
  int splits = ceil_div(sm_count(device) * 8, R);
  const int max_splits = ceil_div(T, 2048);
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  int tokens_per_cta = ceil_div(T, splits);
  tokens_per_cta = ceil_div(tokens_per_cta, 32) * 32;
  splits = ceil_div(T, tokens_per_cta);
  p.tokens_per_cta = tokens_per_cta;

  KVB_CHECK_CUDA(cudaMemsetAsync(w.count, 0, sizeof(uint32_t) * (size_t)R, st));
  if (hist_in) {
    p.hist = hist_in;
  } else {
    KVB_CHECK_CUDA(cudaMemsetAsync(w.hist, 0, sizeof(uint32_t) * (size_t)R * SEL_HIST_BINS, st));
    p.hist = w.hist;
    select_hist_kernel<<<dim3(splits, R), SEL_SCAN_THREADS, 0, st>>>(p, w.hist);
    KVB_CHECK_CUDA(cudaGetLastError());
  }
  select_collect_kernel<<<dim3(splits, R), SEL_SCAN_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());

  const size_t smem = (size_t)p.cap * 8 + sizeof(uint32_t) * (2048 + SEL_FINAL_THREADS + 40 + 4);
  static bool attr_done[64] = {false};
  if (device < 64 && !attr_done[device]) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(select_final_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)((size_t)SEL_MAX_K * 8 + sizeof(uint32_t) * (2048 + SEL_FINAL_THREADS + 44))));
    attr_done[device] = true;
  }
  select_final_kernel<<<R, SEL_FINAL_THREADS, smem, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}
