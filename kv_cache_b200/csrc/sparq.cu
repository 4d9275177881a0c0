// SparQ-style mean-value correction on the int4 path.
//
// The reference's "sparqfast" mode (littlexi001/kv_cache, ymluo/projects/qwen3_top2_head_limit3_ppl/src/
// evaluate_qwen3_top2_head_limit3_ppl.py:2646-2722) approximates every attention logit from a subset of the
// head-dim channels, s[t] = q_sel . k_sel[t] / sqrt(D * |q_sel|_1 / |q|_1), takes the softmax of s over ALL keys,
// runs exact attention over the top candidates only and blends the result with the mean of V by the softmax
// mass alpha the candidates carry:  out = lerp(mean(V), exact_out, alpha).
// Here the approximate logits are the dequantised int4 partial scores of the side cache (same integer
// arithmetic as the decode scorer). Two small kernels produce alpha; the blend itself rides on the chunk
// merge of the attention kernel.
//   sparq_lse_kernel    per (batch, query head): running maximum and sum of exp over all T cached tokens of the
//                       scaled partial score (one streaming pass over the int4 cache, per-chunk partials);
//   sparq_alpha_kernel  merges the partials and adds up exp(s[t] - max) over the SELECTED tokens (re-scored
//                       from the packed rows): alpha = that sum / the total.
#include "common.cuh"
#include "score_common.cuh"

namespace kvb {

constexpr int SQ_THREADS = 256;
constexpr int SQ_CHUNK = 8192;                 // tokens per CTA of the streaming pass
constexpr float SQ_LOG2E = 1.4426950408889634f;

struct SparqParams {
  ScoreParams sp;                              // query / packed / scale / channels / shapes
  const float* mask; int64_t mask_sb;          // additive mask fp32 [B, >= T] or NULL
  float2* partial;                             // [R, nchunk, G] (max, sum) in base-2 units
  int nchunk;
  const int32_t* selected; int kk; const int32_t* sel_count;      // [R, kk] token ids, optional per-row count
  float* alpha;                                // [B*Hq]
};

// 1 / sqrt(D * |q_sel|_1 / |q|_1) * log2(e) for head `head` (both sums clamped at 1e-6 as the reference does),
// computed by one warp.
__device__ __forceinline__ float sparq_inv_divscale_log2e(const ScoreParams& p, int b, int head, int kvh, int lane) {
  const __nv_bfloat16* qrow = p.query + (int64_t)b * p.q_sb + (int64_t)head * p.q_sh;
  const int32_t* ch = p.channel_idx + (int64_t)kvh * p.C;
  float all = 0.0f, sel = 0.0f;
  for (int d = lane; d < p.D; d += 32) all += fabsf(__bfloat162float(qrow[d]));
  for (int c = lane; c < p.C; c += 32) sel += fabsf(__bfloat162float(qrow[ch[c]]));
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    all += __shfl_xor_sync(0xffffffffu, all, off);
    sel += __shfl_xor_sync(0xffffffffu, sel, off);
  }
  all = fmaxf(all, 1.0e-6f);
  sel = fmaxf(sel, 1.0e-6f);
  return SQ_LOG2E / sqrtf((float)p.D * sel / all);
}

// Scaled base-2 logits of one token for the G heads of a KV head (plain byte arithmetic; exact integers).
template <int GMAX>
__device__ __forceinline__ void sparq_token_logits(const ScoreParams& p, int G, int b, int g, int64_t t,
                                                   const int8_t* s_qcode, const float* s_qscale, const float* s_inv,
                                                   float mask_add, float (&x)[GMAX]) {
  const int C = p.C;
  const uint8_t* src = p.packed + (int64_t)b * p.packed_sb + (int64_t)g * p.packed_sh + t * (C >> 1);
  int acc[GMAX];
#pragma unroll
  for (int hd = 0; hd < GMAX; ++hd) acc[hd] = 0;
  for (int j = 0; j < (C >> 1); j += 4) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(src + j);      // rows are 16-byte aligned, C/2 a multiple of 4
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int byte = (int)((w >> (8 * i)) & 0xFFu);
      const int lo = (int)((int8_t)(byte << 4)) >> 4;
      const int hi = (int)((int8_t)(byte & 0xF0)) >> 4;
#pragma unroll
      for (int hd = 0; hd < GMAX; ++hd)
        if (hd < G) acc[hd] += lo * (int)s_qcode[hd * C + 2 * (j + i)] + hi * (int)s_qcode[hd * C + 2 * (j + i) + 1];
    }
  }
  const float ks = p.scale[(int64_t)b * p.scale_sb + (int64_t)g * p.scale_sh + t];
#pragma unroll
  for (int hd = 0; hd < GMAX; ++hd)
    if (hd < G) x[hd] = fmaf(__fmul_rn(__fmul_rn((float)acc[hd], ks), s_qscale[hd]), s_inv[hd], mask_add);
}

__global__ void __launch_bounds__(SQ_THREADS) sparq_lse_kernel(SparqParams q) {
  __shared__ float s_qv[SC_MAX_G * SC_MAX_C];
  __shared__ float s_qscale[SC_MAX_G];
  __shared__ int8_t s_qcode[SC_MAX_G * SC_MAX_C];
  __shared__ float s_inv[SC_MAX_G];
  __shared__ float s_red[SQ_THREADS / 32][8][2];
  const ScoreParams& p = q.sp;
  const int row = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = row / p.Hkv, g = row - b * p.Hkv, G = p.G;
  quantize_query_group<SQ_THREADS>(p, b, g, G, s_qv, s_qcode, s_qscale);
  if (warp < G) {
    const float v = sparq_inv_divscale_log2e(p, b, g * G + warp, g, lane);
    if (lane == 0) s_inv[warp] = v;
  }
  __syncthreads();
  float m[8], l[8];
#pragma unroll
  for (int hd = 0; hd < 8; ++hd) { m[hd] = -INFINITY; l[hd] = 0.0f; }
  const int64_t t0 = (int64_t)chunk * SQ_CHUNK;
  const int64_t t1 = t0 + SQ_CHUNK < p.T ? t0 + SQ_CHUNK : p.T;
  for (int64_t t = t0 + tid; t < t1; t += SQ_THREADS) {
    float x[8];
    const float madd = q.mask ? q.mask[(int64_t)b * q.mask_sb + t] * SQ_LOG2E : 0.0f;
    sparq_token_logits<8>(p, G, b, g, t, s_qcode, s_qscale, s_inv, madd, x);
#pragma unroll
    for (int hd = 0; hd < 8; ++hd) {
      if (hd < G) {
        if (x[hd] > m[hd]) { l[hd] *= exp2f(m[hd] - x[hd]); m[hd] = x[hd]; }      // exp2f(-inf) = 0 on the first token
        l[hd] += exp2f(x[hd] - m[hd]);
      }
    }
  }
  // merge the (max, sum) pairs of the CTA's threads, head by head
#pragma unroll
  for (int hd = 0; hd < 8; ++hd) {
    if (hd < G) {
      float mm = m[hd], ll = l[hd];
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mm, off), ol = __shfl_xor_sync(0xffffffffu, ll, off);
        const float nm = fmaxf(mm, om);
        ll = (nm == -INFINITY) ? 0.0f : ll * exp2f(mm - nm) + ol * exp2f(om - nm);
        mm = nm;
      }
      if (lane == 0) { s_red[warp][hd][0] = mm; s_red[warp][hd][1] = ll; }
    }
  }
  __syncthreads();
  if (tid < G) {
    float mm = -INFINITY, ll = 0.0f;
    for (int w = 0; w < SQ_THREADS / 32; ++w) {
      const float om = s_red[w][tid][0], ol = s_red[w][tid][1];
      const float nm = fmaxf(mm, om);
      ll = (nm == -INFINITY) ? 0.0f : ll * exp2f(mm - nm) + ol * exp2f(om - nm);
      mm = nm;
    }
    q.partial[((int64_t)row * q.nchunk + chunk) * G + tid] = make_float2(mm, ll);
  }
}

__global__ void __launch_bounds__(SQ_THREADS) sparq_alpha_kernel(SparqParams q) {
  __shared__ float s_qv[SC_MAX_G * SC_MAX_C];
  __shared__ float s_qscale[SC_MAX_G];
  __shared__ int8_t s_qcode[SC_MAX_G * SC_MAX_C];
  __shared__ float s_inv[SC_MAX_G];
  __shared__ float s_ml[8][2];
  __shared__ float s_red[SQ_THREADS / 32][8];
  const ScoreParams& p = q.sp;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = row / p.Hkv, g = row - b * p.Hkv, G = p.G;
  quantize_query_group<SQ_THREADS>(p, b, g, G, s_qv, s_qcode, s_qscale);
  if (warp < G) {
    const float v = sparq_inv_divscale_log2e(p, b, g * G + warp, g, lane);
    if (lane == 0) s_inv[warp] = v;
    // the totals of head `warp`: merge of the chunk partials
    float mm = -INFINITY, ll = 0.0f;
    for (int c = lane; c < q.nchunk; c += 32) {
      const float2 pr = q.partial[((int64_t)row * q.nchunk + c) * G + warp];
      const float nm = fmaxf(mm, pr.x);
      ll = (nm == -INFINITY) ? 0.0f : ll * exp2f(mm - nm) + pr.y * exp2f(pr.x - nm);
      mm = nm;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mm, off), ol = __shfl_xor_sync(0xffffffffu, ll, off);
      const float nm = fmaxf(mm, om);
      ll = (nm == -INFINITY) ? 0.0f : ll * exp2f(mm - nm) + ol * exp2f(om - nm);
      mm = nm;
    }
    if (lane == 0) { s_ml[warp][0] = mm; s_ml[warp][1] = ll; }
  }
  __syncthreads();
  int n = q.kk;
  if (q.sel_count) { const int c = q.sel_count[row]; n = c < n ? (c < 0 ? 0 : c) : n; }
  float acc[8];
#pragma unroll
  for (int hd = 0; hd < 8; ++hd) acc[hd] = 0.0f;
  for (int i = tid; i < n; i += SQ_THREADS) {
    const int t = q.selected[(int64_t)row * q.kk + i];
    if (t < 0 || t >= p.T) continue;
    float x[8];
    const float madd = q.mask ? q.mask[(int64_t)b * q.mask_sb + t] * SQ_LOG2E : 0.0f;
    sparq_token_logits<8>(p, G, b, g, t, s_qcode, s_qscale, s_inv, madd, x);
#pragma unroll
    for (int hd = 0; hd < 8; ++hd)
      if (hd < G) acc[hd] += exp2f(x[hd] - s_ml[hd][0]);
  }
#pragma unroll
  for (int hd = 0; hd < 8; ++hd) {
    if (hd < G) {
      float a = acc[hd];
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      if (lane == 0) s_red[warp][hd] = a;
    }
  }
  __syncthreads();
  if (tid < G) {
    float a = 0.0f;
    for (int w = 0; w < SQ_THREADS / 32; ++w) a += s_red[w][tid];
    const float tot = s_ml[tid][1];
    float al = tot > 0.0f ? a / tot : 0.0f;
    q.alpha[(int64_t)b * p.Hq + g * G + tid] = fminf(fmaxf(al, 0.0f), 1.0f);
  }
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_sparq_alpha_workspace_bytes(int B, int Hq, int T) {
  if (B <= 0 || Hq <= 0 || T <= 0) return 0;
  return kvb::round_up(sizeof(float2) * (size_t)B * Hq * kvb::ceil_div(T, kvb::SQ_CHUNK), 256);
}

extern "C" __attribute__((visibility("default"))) int kvb_sparq_alpha(
    const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, const int32_t* channel_idx, const float* mask,
    int64_t mask_sb, const int32_t* selected, int kk, const int32_t* sel_count, int B, int Hq, int Hkv, int T, int D,
    int C, float* alpha, void* workspace, size_t workspace_bytes, int device, void* stream) {
  using namespace kvb;
  if (!query || !packed || !scale || !channel_idx || !selected || !alpha || !workspace) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || (Hq % Hkv) || T <= 0 || kk <= 0 || D <= 0) return KVB_BAD_SHAPE;
  const int G = Hq / Hkv;
  if (G > 8 || C <= 0 || C > SC_MAX_C || (C % 8) || C > D) return KVB_BAD_SHAPE;
  if ((int64_t)B * Hkv > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(packed, 4) || (packed_sb % 4) || (packed_sh % 4) || !aligned_to(workspace, 256)) return KVB_BAD_ALIGN;
  if (workspace_bytes < kvb_sparq_alpha_workspace_bytes(B, Hq, T)) return KVB_WORKSPACE_TOO_SMALL;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  SparqParams q;
  q.sp.query = reinterpret_cast<const __nv_bfloat16*>(query); q.sp.q_sb = q_sb; q.sp.q_sh = q_sh;
  q.sp.packed = packed; q.sp.packed_sb = packed_sb; q.sp.packed_sh = packed_sh;
  q.sp.scale = scale; q.sp.scale_sb = scale_sb; q.sp.scale_sh = scale_sh;
  q.sp.channel_idx = channel_idx;
  q.sp.B = B; q.sp.Hq = Hq; q.sp.Hkv = Hkv; q.sp.T = T; q.sp.D = D; q.sp.C = C; q.sp.G = G;
  q.sp.T_dev = nullptr; q.sp.gmax_out = nullptr; q.sp.acc_out = nullptr; q.sp.deq_out = nullptr; q.sp.hist_out = nullptr;
  q.sp.tau = nullptr; q.sp.cand = nullptr; q.sp.cand_count = nullptr; q.sp.cand_cap = 0;
  q.sp.units_per_row = 0; q.sp.full_tiles = 0; q.sp.total_units = 0;
  q.mask = mask; q.mask_sb = mask_sb;
  q.partial = reinterpret_cast<float2*>(workspace);
  q.nchunk = ceil_div(T, SQ_CHUNK);
  q.selected = selected; q.kk = kk; q.sel_count = sel_count;
  q.alpha = alpha;
  sparq_lse_kernel<<<dim3(q.nchunk, B * Hkv), SQ_THREADS, 0, st>>>(q);
  KVB_CHECK_CUDA(cudaGetLastError());
  sparq_alpha_kernel<<<B * Hkv, SQ_THREADS, 0, st>>>(q);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}
