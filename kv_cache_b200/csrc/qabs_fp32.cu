// The reference's own fp32 "QABS" front-end operators on un-quantised bf16 K, for call sites that
// still use them (littlexi001/kv_cache, ymluo/projects/qwen3_top2_head_limit3_ppl/src/
// qabs_cuda_kernels.py = QCK):
//   partial scores over the dim_count channels with the largest |q| per (batch, head)   QCK:98-158
//   the same with the channel list given and K stored dim-major                          QCK:63-96
//   full q.k * scaling on a candidate union, -inf elsewhere                              QCK:160-216
// Semantics follow those kernels (greedy channel choice with strict '>', so ties go to the lower
// channel; fp32 accumulation in selection order). K may be given per KV head (not repeated):
// head h then reads KV head h / (H / Hk). Query and keys may be bf16, fp16 or fp32 (the reference dispatches
// over the same three types, QCK:430-458); every product is formed in fp32.
#include <cuda_fp16.h>

#include "common.cuh"

namespace kvb {

constexpr int QF_THREADS = 128;
constexpr int QF_TILE = 128;                 // tokens per CTA
constexpr int QF_MAX_D = 256;

__device__ __forceinline__ float qf_load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float qf_load(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ float qf_load(const float* p) { return *p; }

template <typename E>
struct QabsParams {
  const E* query;                            // [B,H,D] dense
  const E* key;                              // token-major [B,Hk,T,D] or dim-major [B,Hk,D,T], element strides below
  int64_t k_sb, k_sh, k_st, k_sd;
  const int64_t* dim_indices;                // [B,H,S] or NULL (choose by |q|)
  float* out;                                // [B,H,T]
  int B, H, Hk, T, D, S;
};

// Greedy top-S |q| (strict '>' => lower channel wins ties), done by warp 0; results in shared memory.
template <typename E>
__device__ __forceinline__ void qabs_choose(const E* qrow, int D, int S, int* s_idx, float* s_q, float* s_abs) {
  const int tid = threadIdx.x;
  for (int d = tid; d < D; d += QF_THREADS) s_abs[d] = fabsf(qf_load(qrow + d));
  __syncthreads();
  if (tid < 32) {
    for (int s = 0; s < S; ++s) {
      float best = -1.0f;
      int bi = 0;
      for (int d = tid; d < D; d += 32) {
        const float a = s_abs[d];
        if (a > best) { best = a; bi = d; }            // ascending d inside the lane: lower index kept on ties
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (tid == 0) {
        s_idx[s] = bi;
        s_q[s] = qf_load(qrow + bi);
        s_abs[bi] = -2.0f;                              // used
      }
      __syncwarp();
    }
  }
  __syncthreads();
}

template <typename E>
__global__ void __launch_bounds__(QF_THREADS) qabs_partial_scores_kernel(QabsParams<E> p) {
  __shared__ int s_idx[QF_MAX_D];
  __shared__ float s_q[QF_MAX_D];
  __shared__ float s_abs[QF_MAX_D];
  const int row = blockIdx.y;
  const int b = row / p.H, h = row - b * p.H;
  const int hk = h / (p.H / p.Hk);
  const E* qrow = p.query + (int64_t)row * p.D;
  if (p.dim_indices) {
    for (int s = threadIdx.x; s < p.S; s += QF_THREADS) {
      const int d = (int)p.dim_indices[(int64_t)row * p.S + s];
      s_idx[s] = d;
      s_q[s] = qf_load(qrow + d);
    }
    __syncthreads();
  } else {
    qabs_choose(qrow, p.D, p.S, s_idx, s_q, s_abs);
  }
  const int64_t t = (int64_t)blockIdx.x * QF_TILE + threadIdx.x;
  if (t >= p.T) return;
  const E* kb = p.key + (int64_t)b * p.k_sb + (int64_t)hk * p.k_sh + t * p.k_st;
  float acc = 0.0f;
  for (int s = 0; s < p.S; ++s) acc = fmaf(s_q[s], qf_load(kb + (int64_t)s_idx[s] * p.k_sd), acc);
  p.out[(int64_t)row * p.T + t] = acc;
}

template <typename E>
struct FullScoreParams {
  const E* query;                            // [B,H,D]
  const E* key; int64_t k_sb, k_sh, k_st;    // [B,Hk,T,D], D contiguous
  const uint8_t* current; const uint8_t* prev_cand; const uint8_t* prev_final;   // bool [B,H,T] (prev_* may be NULL)
  float* out;
  int B, H, Hk, T, D, sink, recent;
  float scaling;
};

// One warp per 32 tokens: lanes test their token, then the warp walks the selected ones together
// (each lane 4 channels of the 128, shuffle reduction).
template <typename E>
__global__ void __launch_bounds__(QF_THREADS) qabs_candidate_full_scores_kernel(FullScoreParams<E> p) {
  const int row = blockIdx.y;
  const int b = row / p.H, h = row - b * p.H;
  const int hk = h / (p.H / p.Hk);
  const int lane = threadIdx.x & 31;
  const int64_t t0 = ((int64_t)blockIdx.x * (QF_THREADS / 32) + (threadIdx.x >> 5)) * 32;
  if (t0 >= p.T) return;
  const int64_t t = t0 + lane;
  bool sel = false;
  if (t < p.T) {
    const int64_t o = (int64_t)row * p.T + t;
    sel = p.current[o] != 0;
    if (p.prev_cand) sel = sel || p.prev_cand[o] != 0;
    if (p.prev_final) sel = sel || p.prev_final[o] != 0;
    if (p.sink > 0 && t < p.sink) sel = true;
    if (p.recent > 0 && t >= (p.T - p.recent > 0 ? p.T - p.recent : 0)) sel = true;
  }
  const E* qrow = p.query + (int64_t)row * p.D;
  const E* kb = p.key + (int64_t)b * p.k_sb + (int64_t)hk * p.k_sh;
  uint32_t m = __ballot_sync(0xffffffffu, sel);
  float mine = -INFINITY;
  while (m) {
    const int src = __ffs(m) - 1;
    m &= m - 1;
    const E* krow = kb + (t0 + src) * p.k_st;
    float acc = 0.0f;
    for (int d = lane; d < p.D; d += 32) acc = fmaf(qf_load(qrow + d), qf_load(krow + d), acc);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == src) mine = acc * p.scaling;
  }
  if (t < p.T) p.out[(int64_t)row * p.T + t] = mine;
}

template <typename E>
static int qabs_partial_launch(const void* query, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st, int64_t k_sd,
                               const int64_t* dim_indices, int S, float* out, int B, int H, int Hk, int T, int D,
                               cudaStream_t st) {
  QabsParams<E> p;
  p.query = reinterpret_cast<const E*>(query);
  p.key = reinterpret_cast<const E*>(key);
  p.k_sb = k_sb; p.k_sh = k_sh; p.k_st = k_st; p.k_sd = k_sd;
  p.dim_indices = dim_indices; p.out = out;
  p.B = B; p.H = H; p.Hk = Hk; p.T = T; p.D = D; p.S = S;
  dim3 grid(ceil_div(T, QF_TILE), B * H);
  qabs_partial_scores_kernel<E><<<grid, QF_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

template <typename E>
static int qabs_full_launch(const void* query, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
                            const uint8_t* current, const uint8_t* previous_candidate, const uint8_t* previous_final,
                            int protect_sink, int protect_recent, float scaling, float* out, int B, int H, int Hk, int T,
                            int D, cudaStream_t st) {
  FullScoreParams<E> p;
  p.query = reinterpret_cast<const E*>(query);
  p.key = reinterpret_cast<const E*>(key);
  p.k_sb = k_sb; p.k_sh = k_sh; p.k_st = k_st;
  p.current = current; p.prev_cand = previous_candidate; p.prev_final = previous_final;
  p.out = out; p.B = B; p.H = H; p.Hk = Hk; p.T = T; p.D = D;
  p.sink = protect_sink; p.recent = protect_recent; p.scaling = scaling;
  dim3 grid(ceil_div(T, QF_THREADS), B * H);
  qabs_candidate_full_scores_kernel<E><<<grid, QF_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_qabs_partial_scores(
    const void* query, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st, int64_t k_sd,
    const int64_t* dim_indices, int dim_count, float* out, int B, int H, int Hk, int T, int D, int elem_type, int device,
    void* stream) {
  using namespace kvb;
  if (!query || !key || !out) return KVB_BAD_ARG;
  if (elem_type < 0 || elem_type > 2) return KVB_BAD_ARG;
  if (B <= 0 || H <= 0 || Hk <= 0 || T < 0 || D <= 0 || D > QF_MAX_D || (H % Hk)) return KVB_BAD_SHAPE;
  if ((int64_t)B * H > 65535) return KVB_BAD_SHAPE;
  int S = dim_count < 1 ? 1 : dim_count;
  if (S > D) S = D;
  if (T == 0) return KVB_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (elem_type == 0) return qabs_partial_launch<__nv_bfloat16>(query, key, k_sb, k_sh, k_st, k_sd, dim_indices, S, out, B, H, Hk, T, D, st);
  if (elem_type == 1) return qabs_partial_launch<__half>(query, key, k_sb, k_sh, k_st, k_sd, dim_indices, S, out, B, H, Hk, T, D, st);
  return qabs_partial_launch<float>(query, key, k_sb, k_sh, k_st, k_sd, dim_indices, S, out, B, H, Hk, T, D, st);
}

extern "C" __attribute__((visibility("default"))) int kvb_qabs_candidate_full_scores(
    const void* query, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st, const uint8_t* current,
    const uint8_t* previous_candidate, const uint8_t* previous_final, int protect_sink, int protect_recent,
    float scaling, float* out, int B, int H, int Hk, int T, int D, int elem_type, int device, void* stream) {
  using namespace kvb;
  if (!query || !key || !current || !out) return KVB_BAD_ARG;
  if (elem_type < 0 || elem_type > 2) return KVB_BAD_ARG;
  if (B <= 0 || H <= 0 || Hk <= 0 || T < 0 || D <= 0 || (H % Hk)) return KVB_BAD_SHAPE;
  if ((int64_t)B * H > 65535) return KVB_BAD_SHAPE;
  if (T == 0) return KVB_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (elem_type == 0) return qabs_full_launch<__nv_bfloat16>(query, key, k_sb, k_sh, k_st, current, previous_candidate, previous_final, protect_sink, protect_recent, scaling, out, B, H, Hk, T, D, st);
  if (elem_type == 1) return qabs_full_launch<__half>(query, key, k_sb, k_sh, k_st, current, previous_candidate, previous_final, protect_sink, protect_recent, scaling, out, B, H, Hk, T, D, st);
  return qabs_full_launch<float>(query, key, k_sb, k_sh, k_st, current, previous_candidate, previous_final, protect_sink, protect_recent, scaling, out, B, H, Hk, T, D, st);
}
