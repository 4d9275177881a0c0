// Exact rerank of a candidate union, as LISTS (the reference's best-quality modes).
//
// The reference (littlexi001/kv_cache) builds, per decode step and head, the union of the current
// candidates with the previous step's candidates and previous final set, computes the exact q.k on
// that union and keeps the best ceil(top_fraction * T) tokens
// (ymluo/projects/qwen3_top2_head_limit3_ppl/src/evaluate_qwen3_top2_head_limit3_ppl.py:4147-4311;
// its CUDA scoring kernel qabs_cuda_kernels.py:160-216 takes three dense bool masks [B,H,T] and writes
// a dense [B,H,T] score row, which its authors name as the cost of that mode). Here the three sets are
// id lists and nothing of size T is touched in global memory:
//   1. rerank_union_kernel   one CTA per list row: a bitmap of T bits in shared memory takes the ids of the
//                            (up to) three lists, protected ranges optionally forced in; its set bits are
//                            read out in ascending order as the de-duplicated union;
//   2. rerank_score_kernel   8 lanes per union entry gather its 256-byte K row and form the fp32 dot
//                            products with the query heads that share the list; the maximum over those
//                            heads, times the softmax scale, plus the additive mask, becomes a 64-bit
//                            composite (score key, ~id);
//   3. select_final_kernel   the exact top-r of the composites on chip, (score desc, id asc), written in
//                            ascending id order with the row's count.
#include "common.cuh"

namespace kvb {

constexpr int RR_THREADS = 512;
constexpr int RR_MAX_UNION = SEL_MAX_K;               // the final select holds the union on chip
constexpr int RR_SCORE_THREADS = 256;
constexpr int RR_IDS_PER_CTA = 256;                   // union entries per scoring CTA

struct RerankParams {
  const int32_t* list[3]; int n[3]; const int32_t* count[3];     // id lists [R, n[i]] (NULL = absent), optional per-row counts
  int R, T;                                                       // list rows, history length
  int force_sink, force_recent;                                   // ranges forced into the union (0 = none)
  int block;                                                      // > 1: a token brings in its whole aligned block of this many tokens
  int32_t* uni; int cap;                                          // out: union ids [R, cap] ascending
  uint32_t* ucount; int ucount_stride;                            // out: count of row r at ucount[r * ucount_stride]
};

// One bit per token (per aligned block when block > 1) in shared memory; the set bits are read out in
// ascending order. Entries beyond `cap` are dropped (the count saturates at cap).
__global__ void __launch_bounds__(RR_THREADS) rerank_union_kernel(RerankParams p) {
  extern __shared__ __align__(16) uint32_t rr_bitmap[];            // [words] then scan scratch
  const int row = blockIdx.x, tid = threadIdx.x;
  const int blk = p.block > 1 ? p.block : 1;
  const int nbits = (p.T + blk - 1) / blk;
  const int words = (nbits + 31) >> 5;
  uint32_t* s_scan = rr_bitmap + words;                            // [RR_THREADS / 32 + 1]
  pdl_launch_dependents();
  pdl_wait();
  for (int i = tid; i < words; i += RR_THREADS) rr_bitmap[i] = 0u;
  __syncthreads();
  auto mark = [&](int id) {
    const int bit = id / blk;
    atomicOr(&rr_bitmap[bit >> 5], 1u << (bit & 31));
  };
#pragma unroll
  for (int l = 0; l < 3; ++l) {
    if (!p.list[l]) continue;
    int n = p.n[l];
    if (p.count[l]) { const int c = p.count[l][row]; n = c < n ? (c < 0 ? 0 : c) : n; }
    const int32_t* src = p.list[l] + (int64_t)row * p.n[l];
    for (int i = tid; i < n; i += RR_THREADS) {
      const int id = src[i];
      if (id >= 0 && id < p.T) mark(id);                           // ids past the history (stale) and -1 padding are dropped
    }
  }
  if (p.force_sink > 0) {
    const int e = p.force_sink < p.T ? p.force_sink : p.T;
    for (int id = tid; id < e; id += RR_THREADS) mark(id);
  }
  if (p.force_recent > 0) {
    const int b = p.T - p.force_recent > 0 ? p.T - p.force_recent : 0;
    for (int id = b + tid; id < p.T; id += RR_THREADS) mark(id);
  }
  __syncthreads();
  // ascending read-out: every thread owns a contiguous run of words; a set bit stands for blk tokens
  // (fewer for the last, partial block)
  const int per = (words + RR_THREADS - 1) / RR_THREADS;
  const int w0 = tid * per;
  const int last_bit = nbits - 1;
  const int last_len = p.T - last_bit * blk;
  uint32_t cnt = 0;
  for (int j = 0; j < per; ++j) {
    if (w0 + j >= words) break;
    const uint32_t bits = rr_bitmap[w0 + j];
    cnt += (uint32_t)__popc(bits) * (uint32_t)blk;
    if ((last_bit >> 5) == w0 + j && (bits >> (last_bit & 31)) & 1u) cnt -= (uint32_t)(blk - last_len);
  }
  uint32_t total;
  uint32_t pos = block_exclusive_scan<RR_THREADS>(cnt, s_scan, total);
  int32_t* dst = p.uni + (int64_t)row * p.cap;
  for (int j = 0; j < per; ++j) {
    if (w0 + j >= words) break;
    uint32_t bits = rr_bitmap[w0 + j];
    while (bits) {
      const int bit = (w0 + j) * 32 + (__ffs(bits) - 1);
      bits &= bits - 1;
      const int t0 = bit * blk;
      const int len = bit == last_bit ? last_len : blk;
      for (int e = 0; e < len; ++e, ++pos)
        if (pos < (uint32_t)p.cap) dst[pos] = t0 + e;
    }
  }
  const uint32_t got = total < (uint32_t)p.cap ? total : (uint32_t)p.cap;
  // the tail of the row is marked unused so that a reader without the count sees no stale ids
  for (uint32_t i = got + tid; i < (uint32_t)p.cap; i += RR_THREADS) dst[i] = -1;
  if (tid == 0) p.ucount[(int64_t)row * p.ucount_stride] = got;
}

struct RerankScoreParams {
  const __nv_bfloat16* query; int64_t q_sb, q_sh;
  const __nv_bfloat16* key;   int64_t k_sb, k_sh, k_st;
  const float* mask; int64_t mask_sb;
  const int32_t* uni; const uint32_t* ucount; int cap;
  uint64_t* cand;                                                  // out: composites [R, cap]
  int B, Hq, Hkv, Hi;                                              // Hi list rows per batch row (Hkv or Hq)
  float scaling;
};

// GG = query heads that share one list.
template <int GG>
__global__ void __launch_bounds__(RR_SCORE_THREADS) rerank_score_kernel(RerankScoreParams p) {
  __shared__ __align__(16) float s_q[GG][AT_D];
  const int row = blockIdx.y, tid = threadIdx.x;
  const int b = row / p.Hi, hi = row - b * p.Hi;
  const int head0 = hi * GG;
  const int kvh = head0 / (p.Hq / p.Hkv);
  pdl_launch_dependents();
  for (int i = tid; i < GG * AT_D; i += RR_SCORE_THREADS) {
    const int h = i / AT_D, d = i - h * AT_D;
    s_q[h][d] = __bfloat162float(p.query[(int64_t)b * p.q_sb + (int64_t)(head0 + h) * p.q_sh + d]);
  }
  pdl_wait();
  const int n = (int)p.ucount[(int64_t)row * SEL_COUNT_STRIDE];
  const int base = blockIdx.x * RR_IDS_PER_CTA;
  if (base >= n) return;
  __syncthreads();
  const __nv_bfloat16* kbase = p.key + (int64_t)b * p.k_sb + (int64_t)kvh * p.k_sh;
  const int32_t* ids = p.uni + (int64_t)row * p.cap;
  uint64_t* out = p.cand + (int64_t)row * p.cap;
  const int sub = tid & 7;                                          // lane inside the 8-lane team: dims [16*sub, 16*sub+16)
  // query slice of this lane, all heads, in registers
  float qv[GG][16];
#pragma unroll
  for (int h = 0; h < GG; ++h)
#pragma unroll
    for (int j = 0; j < 16; ++j) qv[h][j] = s_q[h][16 * sub + j];
  for (int e = base + (tid >> 3); e < base + RR_IDS_PER_CTA; e += RR_SCORE_THREADS / 8) {
    const bool live = e < n;                                        // (whole teams agree; shuffles stay inside the team)
    const int id = live ? ids[e] : 0;
    const uint4* src = reinterpret_cast<const uint4*>(kbase + (int64_t)id * p.k_st + 16 * sub);
    const uint4 x0 = live ? __ldg(src) : make_uint4(0, 0, 0, 0);
    const uint4 x1 = live ? __ldg(src + 1) : make_uint4(0, 0, 0, 0);
    const uint32_t w[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    float kf[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      kf[2 * j] = __uint_as_float(w[j] << 16);
      kf[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
    float best = -INFINITY;
#pragma unroll
    for (int h = 0; h < GG; ++h) {
      float acc = 0.0f;
#pragma unroll
      for (int j = 0; j < 16; ++j) acc = fmaf(qv[h][j], kf[j], acc);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      best = fmaxf(best, acc);
    }
    if (live && sub == 0) {
      float s = best * p.scaling;
      if (p.mask) s += p.mask[(int64_t)b * p.mask_sb + id];
      if (s == 0.0f) s = 0.0f;
      out[e] = make_composite(s, (uint32_t)id);
    }
  }
}

struct RerankLayout {
  int cap;
  size_t off_uni, off_count, off_cand, bytes;
};

static RerankLayout rerank_layout(int R, int max_union) {
  RerankLayout L;
  L.cap = (int)round_up((size_t)(max_union > 0 ? max_union : 1), 1024);
  size_t off = 0;
  L.off_uni = off;   off += round_up(sizeof(int32_t) * (size_t)R * L.cap, 256);
  L.off_count = off; off += round_up(sizeof(uint32_t) * (size_t)R * SEL_COUNT_STRIDE, 256);
  L.off_cand = off;  off += round_up(sizeof(uint64_t) * (size_t)R * L.cap, 256);
  L.bytes = off;
  return L;
}

template <int GG>
static int rerank_score_launch(const RerankScoreParams& p, int R, int cap, cudaStream_t st) {
  KVB_CHECK_CUDA(launch_kernel(rerank_score_kernel<GG>, dim3(ceil_div(cap, RR_IDS_PER_CTA), R), dim3(RR_SCORE_THREADS), 0, st, p));
  return KVB_OK;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_rerank_union_workspace_bytes(int R, int max_union) {
  if (R <= 0 || max_union <= 0 || max_union > kvb::RR_MAX_UNION) return 0;
  return kvb::rerank_layout(R, max_union).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_rerank_union(
    const void* query, int64_t q_sb, int64_t q_sh, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
    const int32_t* list0, int n0, const int32_t* count0, const int32_t* list1, int n1, const int32_t* count1,
    const int32_t* list2, int n2, const int32_t* count2, int force_sink, int force_recent, const float* mask,
    int64_t mask_sb, int B, int Hq, int Hkv, int Hi, int history_count, int D, float scaling, int keep,
    int32_t* out_idx, int32_t* out_count, void* workspace, size_t workspace_bytes, int device, void* stream) {
  using namespace kvb;
  if (!query || !key || !list0 || !out_idx || !out_count || !workspace) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv) || (Hi != Hkv && Hi != Hq) || D != AT_D || history_count <= 0 ||
      keep <= 0 || n0 <= 0 || n1 < 0 || n2 < 0 || force_sink < 0 || force_recent < 0)
    return KVB_BAD_SHAPE;
  const int GG = Hq / Hi;
  if (GG != 1 && GG != 2 && GG != 4 && GG != 8) return KVB_BAD_SHAPE;
  const int R = B * Hi;
  if (R > 65535) return KVB_BAD_SHAPE;
  int64_t max_union = (int64_t)n0 + (list1 ? n1 : 0) + (list2 ? n2 : 0) + force_sink + force_recent;
  if (max_union > history_count) max_union = history_count;
  if (max_union > RR_MAX_UNION) return KVB_BAD_SHAPE;
  if (keep > SEL_MAX_K) return KVB_BAD_SHAPE;
  if (!aligned_to(query, 2) || !aligned_to(key, 16) || (k_sb % 8) || (k_sh % 8) || (k_st % 8)) return KVB_BAD_ALIGN;
  if (!aligned_to(workspace, 256)) return KVB_BAD_ALIGN;
  const RerankLayout L = rerank_layout(R, (int)max_union);
  if (workspace_bytes < L.bytes) return KVB_WORKSPACE_TOO_SMALL;
  const size_t union_smem = sizeof(uint32_t) * ((size_t)((history_count + 31) / 32) + RR_THREADS / 32 + 1);
  const int kk = keep < (int)max_union ? keep : (int)max_union;
  const size_t bitmap_bytes = sizeof(uint32_t) * (size_t)((history_count + 31) / 32);
  const size_t sel_smem = (size_t)L.cap * 8 + SEL_FINAL_FIXED_SMEM + bitmap_bytes;
  if (union_smem > SEL_SMEM_LIMIT || sel_smem > SEL_SMEM_LIMIT) return KVB_BAD_SHAPE;      // history too long for the on-chip bitmaps
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  int32_t* uni = reinterpret_cast<int32_t*>(ws + L.off_uni);
  uint32_t* ucount = reinterpret_cast<uint32_t*>(ws + L.off_count);
  uint64_t* cand = reinterpret_cast<uint64_t*>(ws + L.off_cand);

  RerankParams up;
  up.list[0] = list0; up.n[0] = n0; up.count[0] = count0;
  up.list[1] = list1; up.n[1] = list1 ? n1 : 0; up.count[1] = count1;
  up.list[2] = list2; up.n[2] = list2 ? n2 : 0; up.count[2] = count2;
  up.R = R; up.T = history_count; up.force_sink = force_sink; up.force_recent = force_recent;
  up.block = 1;
  up.uni = uni; up.cap = L.cap; up.ucount = ucount; up.ucount_stride = SEL_COUNT_STRIDE;
  static std::atomic<bool> union_attr[KVB_MAX_DEVICES];
  { const int arc = ensure_dynamic_smem(rerank_union_kernel, union_attr, device, SEL_SMEM_LIMIT); if (arc != KVB_OK) return arc; }
  KVB_CHECK_CUDA(launch_kernel(rerank_union_kernel, dim3(R), dim3(RR_THREADS), union_smem, st, up));
  ChainLaunchScope chain;
  chain.on();

  RerankScoreParams sp;
  sp.query = reinterpret_cast<const __nv_bfloat16*>(query); sp.q_sb = q_sb; sp.q_sh = q_sh;
  sp.key = reinterpret_cast<const __nv_bfloat16*>(key); sp.k_sb = k_sb; sp.k_sh = k_sh; sp.k_st = k_st;
  sp.mask = mask; sp.mask_sb = mask_sb;
  sp.uni = uni; sp.ucount = ucount; sp.cap = L.cap; sp.cand = cand;
  sp.B = B; sp.Hq = Hq; sp.Hkv = Hkv; sp.Hi = Hi; sp.scaling = scaling;
  int rc;
  switch (GG) {
    case 1: rc = rerank_score_launch<1>(sp, R, L.cap, st); break;
    case 2: rc = rerank_score_launch<2>(sp, R, L.cap, st); break;
    case 4: rc = rerank_score_launch<4>(sp, R, L.cap, st); break;
    default: rc = rerank_score_launch<8>(sp, R, L.cap, st); break;
  }
  if (rc != KVB_OK) return rc;

  SelectParams fp;
  fp.scores = nullptr; fp.row_stride = 0; fp.payload = nullptr;
  fp.R = R; fp.T = history_count; fp.k = keep; fp.kk = kk; fp.idx_offset = 0;
  fp.out_idx32 = out_idx; fp.out_idx64 = nullptr; fp.out_scores = nullptr; fp.out_comp = nullptr;
  fp.hist = nullptr; fp.cand = cand; fp.cand_count = ucount; fp.cap = L.cap;
  fp.tokens_per_cta = 0; fp.thresholds = nullptr;
  fp.order_by_index = 1; fp.use_bitmap = 1;
  fp.from_candidates = 1; fp.row_failed = nullptr; fp.T_dev = nullptr;
  fp.gather = nullptr; fp.gather_n = 0; fp.gather_len = 0; fp.gather_stride = 0;
  fp.rescue = 0;
  fp.out_owned_count = out_count;                      // the bitmap read-out reports how many entries the row got
  fp.out_pitch = keep;
  { const int prc = select_final_prepare(device); if (prc != KVB_OK) return prc; }
  KVB_CHECK_CUDA(launch_kernel(select_final_kernel, dim3(R), dim3(SEL_FINAL_THREADS), sel_smem, st, fp));
  return KVB_OK;
}

extern "C" __attribute__((visibility("default"))) int kvb_expand_final(
    const int32_t* list, int n, const int32_t* count, int R, int history_count, int force_sink, int force_recent,
    int block_size, int32_t* out_idx, int out_cap, int32_t* out_count, int device, void* stream) {
  using namespace kvb;
  if (!list || !out_idx || !out_count) return KVB_BAD_ARG;
  if (n <= 0 || R <= 0 || R > 65535 || history_count <= 0 || force_sink < 0 || force_recent < 0 || block_size < 1 ||
      out_cap <= 0)
    return KVB_BAD_SHAPE;
  const int nbits = (history_count + block_size - 1) / block_size;
  const size_t smem = sizeof(uint32_t) * ((size_t)((nbits + 31) / 32) + RR_THREADS / 32 + 1);
  if (smem > SEL_SMEM_LIMIT) return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  RerankParams up;
  up.list[0] = list; up.n[0] = n; up.count[0] = count;
  up.list[1] = nullptr; up.n[1] = 0; up.count[1] = nullptr;
  up.list[2] = nullptr; up.n[2] = 0; up.count[2] = nullptr;
  up.R = R; up.T = history_count; up.force_sink = force_sink; up.force_recent = force_recent;
  up.block = block_size;
  up.uni = out_idx; up.cap = out_cap;
  up.ucount = reinterpret_cast<uint32_t*>(out_count); up.ucount_stride = 1;
  static std::atomic<bool> union_attr[KVB_MAX_DEVICES];
  { const int arc = ensure_dynamic_smem(rerank_union_kernel, union_attr, device, SEL_SMEM_LIMIT); if (arc != KVB_OK) return arc; }
  KVB_CHECK_CUDA(launch_kernel(rerank_union_kernel, dim3(R), dim3(RR_THREADS), smem, reinterpret_cast<cudaStream_t>(stream), up));
  return KVB_OK;
}
