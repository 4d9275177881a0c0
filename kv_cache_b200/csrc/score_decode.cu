// Stage 2: decode scoring. One query token per sequence against all T int4-packed keys.
//
// HBM-bound: every packed token (C/2 bytes) and its fp32 scale is read exactly once. The stream
// is staged through shared memory by the TMA engine (1-D cp.async.bulk + mbarrier), one private
// stage ring per warp so no CTA-wide barrier sits in the loop. Nibbles are widened to int8*16 with
// one shift and two masks per 32-bit word, accumulated exactly in int32 with dp4a against the
// int8 query codes of all G heads of the KV head, combined across the C/32 lanes that share a
// token with warp shuffles, dequantised with two rounded fp32 products and reduced to the
// group maximum in registers. Only the group maximum (4 bytes per token per KV head) is written.
#include "common.cuh"

namespace kvb {

constexpr int SC_WARPS = 4;
constexpr int SC_THREADS = SC_WARPS * 32;
constexpr int SC_TILE_PACKED_BYTES = 4096;       // packed bytes per warp tile, whatever C is
constexpr int SC_HIST_BITS = 12;
constexpr int SC_HIST_BINS = 1 << SC_HIST_BITS;
constexpr int SC_MAX_C = 128;
constexpr int SC_MAX_G = 16;

struct ScoreParams {
  const __nv_bfloat16* query;
  int64_t q_sb, q_sh;
  const uint8_t* packed;
  int64_t packed_sb, packed_sh;
  const float* scale;
  int64_t scale_sb, scale_sh;
  const int32_t* channel_idx;
  int B, Hq, Hkv, T, D, C, G;
  float* gmax_out;
  int32_t* acc_out;
  float* deq_out;
  uint32_t* hist_out;
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
template <int GMAX>
__device__ __forceinline__ void score_token_plain(const ScoreParams& p, int G, int row, int b, int g, int64_t t,
                                                  const int8_t* s_qcode, const float* s_qscale,
                                                  uint32_t* s_hist /* or nullptr */) {
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
  if (p.gmax_out) p.gmax_out[(int64_t)row * p.T + t] = best;
  if (s_hist) atomicAdd(&s_hist[float_to_key(best) >> (32 - SC_HIST_BITS)], 1u);
}

// Streaming kernel. C in {32,64,128}; LPT = C/32 lanes share one token (16 bytes each).
// NS = stages of each warp's ring. Persistent: CTA c owns the contiguous unit range
// [c*U/grid, (c+1)*U/grid) of the flattened (row, tile) space.
template <int C, int G, int NS, bool HIST>
__global__ void __launch_bounds__(SC_THREADS) score_decode_stream_kernel(ScoreParams p) {
  constexpr int LPT = C / 32;
  constexpr int TW = SC_TILE_PACKED_BYTES / (C / 2);    // tokens per warp tile: 256 / 128 / 64
  constexpr int IT = TW / 32;                           // 32-token iterations per tile
  constexpr int STAGE_BYTES = SC_TILE_PACKED_BYTES + TW * 4;
  constexpr int TOK_PER_LOAD = 32 / LPT;

  extern __shared__ __align__(128) uint8_t smem_raw[];
  // layout: [warps][NS][STAGE_BYTES] | bars [warps][NS] | qv | qscale | qcode | hist
  uint8_t* s_stage = smem_raw;
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_stage + SC_WARPS * NS * STAGE_BYTES);
  float* s_qv = reinterpret_cast<float*>(s_bar + SC_WARPS * NS);
  float* s_qscale = s_qv + G * C;
  int8_t* s_qcode = reinterpret_cast<int8_t*>(s_qscale + SC_MAX_G);
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_qcode + G * C);   // G*C is a multiple of 32

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hq = lane % LPT;                 // which 16-byte quarter/half of a token this lane reads
  uint8_t* my_stage = s_stage + warp * NS * STAGE_BYTES;
  uint64_t* my_bar = s_bar + warp * NS;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) mbar_init(&my_bar[s], 1);
    fence_mbar_init();
  }
  if (HIST) {
    for (int i = tid; i < SC_HIST_BINS; i += SC_THREADS) s_hist[i] = 0;
  }
  fence_proxy_async_smem();
  __syncthreads();

  const uint64_t policy = l2_policy_evict_first();
  const int64_t u_begin = (int64_t)blockIdx.x * p.total_units / gridDim.x;
  const int64_t u_end = (int64_t)(blockIdx.x + 1) * p.total_units / gridDim.x;

  uint32_t ring = 0;        // tiles this warp has consumed so far (stage = ring % NS, parity = ring / NS & 1)
  bool dead = false;        // a bounded wait gave up: skip all further streaming work

  int64_t u = u_begin;
  while (u < u_end) {
    const int row = (int)(u / p.units_per_row);
    const int ua = (int)(u - (int64_t)row * p.units_per_row);
    int64_t row_end_u = (int64_t)(row + 1) * p.units_per_row;
    const int ub = (int)((row_end_u < u_end ? row_end_u : u_end) - (int64_t)row * p.units_per_row);
    u += (ub - ua);
    const int b = row / p.Hkv, g = row - b * p.Hkv;

    quantize_query_group<SC_THREADS>(p, b, g, G, s_qv, s_qcode, s_qscale);

    // Per-lane query words: word w of this lane's 16-byte piece holds channels
    // 32*hq + 8*w + {0,2,4,6} in its low nibbles and + {1,3,5,7} in its high nibbles.
    int qlo[G][4], qhi[G][4];
    float qs[G];
#pragma unroll
    for (int hd = 0; hd < G; ++hd) {
      qs[hd] = s_qscale[hd];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = 32 * hq + 8 * w + 2 * i;
          lo |= (uint32_t)(uint8_t)s_qcode[hd * C + c] << (8 * i);
          hi |= (uint32_t)(uint8_t)s_qcode[hd * C + c + 1] << (8 * i);
        }
        qlo[hd][w] = (int)lo;
        qhi[hd][w] = (int)hi;
      }
    }

    const uint8_t* packed_row = p.packed + (int64_t)b * p.packed_sb + (int64_t)g * p.packed_sh;
    const float* scale_row = p.scale + (int64_t)b * p.scale_sb + (int64_t)g * p.scale_sh;
    float* gmax_row = p.gmax_out ? p.gmax_out + (int64_t)row * p.T : nullptr;

    // Full tiles of this segment: [ta, tb); warp w takes ta + w, ta + w + SC_WARPS, ...
    const int ta = ua;
    const int tb = ub < p.full_tiles ? ub : p.full_tiles;
    const int nmy = (tb - ta - warp + SC_WARPS - 1) / SC_WARPS;   // <= 0 when none

    auto issue = [&](int j, uint32_t slot) {
      // lane 0 only: tile j of this warp into ring slot `slot`
      const int64_t t0 = (int64_t)(ta + warp + j * SC_WARPS) * TW;
      uint8_t* dst = my_stage + (slot % NS) * STAGE_BYTES;
      mbar_arrive_expect_tx(&my_bar[slot % NS], STAGE_BYTES);
      bulk_g2s_evict_first(dst, packed_row + t0 * (C / 2), SC_TILE_PACKED_BYTES, &my_bar[slot % NS], policy);
      bulk_g2s_evict_first(dst + SC_TILE_PACKED_BYTES, scale_row + t0, TW * 4, &my_bar[slot % NS], policy);
    };

    if (!dead && nmy > 0) {
      if (lane == 0) {
        const int pre = nmy < NS ? nmy : NS;
        for (int j = 0; j < pre; ++j) issue(j, ring + j);
      }
      for (int j = 0; j < nmy; ++j) {
        const uint32_t slot = ring + j;
        bool ok = mbar_wait_bounded(&my_bar[slot % NS], (slot / NS) & 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { dead = true; break; }
        const uint8_t* st = my_stage + (slot % NS) * STAGE_BYTES;
        const uint4* sp = reinterpret_cast<const uint4*>(st);
        const float* ssc = reinterpret_cast<const float*>(st + SC_TILE_PACKED_BYTES);
        const int64_t t0 = (int64_t)(ta + warp + j * SC_WARPS) * TW;

#pragma unroll 1
        for (int it = 0; it < IT; ++it) {
          int part[LPT][G];
#pragma unroll
          for (int ld = 0; ld < LPT; ++ld) {
            const uint4 v = sp[it * 32 * LPT + ld * 32 + lane];
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int hd = 0; hd < G; ++hd) part[ld][hd] = 0;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              const int lo = (int)((wv[w] << 4) & 0xF0F0F0F0u);   // int8 lanes = 16 * low-nibble code
              const int hi = (int)(wv[w] & 0xF0F0F0F0u);          // int8 lanes = 16 * high-nibble code
#pragma unroll
              for (int hd = 0; hd < G; ++hd) {
                part[ld][hd] = __dp4a(lo, qlo[hd][w], part[ld][hd]);
                part[ld][hd] = __dp4a(hi, qhi[hd][w], part[ld][hd]);
              }
            }
          }
          // Transposing reduction over the LPT lanes of a token: afterwards lane with
          // hq == ld owns the complete sum of the token read by load ld.
          int mine[G];
          if constexpr (LPT == 1) {
#pragma unroll
            for (int hd = 0; hd < G; ++hd) mine[hd] = part[0][hd];
          } else if constexpr (LPT == 2) {
#pragma unroll
            for (int hd = 0; hd < G; ++hd) {
              const int send = hq ? part[0][hd] : part[LPT - 1][hd];
              const int keep = hq ? part[LPT - 1][hd] : part[0][hd];
              mine[hd] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
            }
          } else {
            const int hb = (hq >> 1) & 1, lb = hq & 1;
#pragma unroll
            for (int hd = 0; hd < G; ++hd) {
              // step 1 (partner lane ^ 2): keep loads {0,1} when hb == 0, {2,3} when hb == 1
              const int s0 = hb ? part[0][hd] : part[LPT - 2][hd];
              const int s1 = hb ? part[1][hd] : part[LPT - 1][hd];
              const int k0 = hb ? part[LPT - 2][hd] : part[0][hd];
              const int k1 = hb ? part[LPT - 1][hd] : part[1][hd];
              const int r0 = k0 + __shfl_xor_sync(0xffffffffu, s0, 2);
              const int r1 = k1 + __shfl_xor_sync(0xffffffffu, s1, 2);
              // step 2 (partner lane ^ 1): keep r0 when lb == 0, r1 when lb == 1
              const int send = lb ? r0 : r1;
              const int keep = lb ? r1 : r0;
              mine[hd] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
            }
          }
          const int tl = it * 32 + hq * TOK_PER_LOAD + lane / LPT;    // token inside the tile
          const float ks = ssc[tl];
          const int64_t t = t0 + tl;
          float best = -INFINITY;
#pragma unroll
          for (int hd = 0; hd < G; ++hd) {
            const int a = mine[hd] >> 4;                               // exact: the sum is 16 * acc
            const float d = __fmul_rn(__fmul_rn((float)a, ks), qs[hd]);
            best = fmaxf(best, d);
            if (p.acc_out || p.deq_out) {
              const int64_t o = ((int64_t)b * p.Hq + (int64_t)g * G + hd) * p.T + t;
              if (p.acc_out) p.acc_out[o] = a;
              if (p.deq_out) p.deq_out[o] = d;
            }
          }
          if (best == 0.0f) best = 0.0f;                               // -0 -> +0
          if (gmax_row) gmax_row[t] = best;
          if (HIST) atomicAdd(&s_hist[float_to_key(best) >> (32 - SC_HIST_BITS)], 1u);
        }

        __syncwarp();
        if (lane == 0 && j + NS < nmy) {
          fence_proxy_async_smem();
          issue(j + NS, slot + NS);
        }
      }
      if (!dead) ring += (uint32_t)nmy;
    }

    // Ragged tail of the row (fewer than TW tokens), owned by the segment that holds the tail unit.
    if (ub > p.full_tiles) {
      const int64_t tail0 = (int64_t)p.full_tiles * TW;
      for (int64_t t = tail0 + tid; t < p.T; t += SC_THREADS)
        score_token_plain<G>(p, G, row, b, g, t, s_qcode, s_qscale, HIST ? s_hist : nullptr);
    }

    if (HIST) {
      __syncthreads();
      uint32_t* gh = p.hist_out + (int64_t)row * SC_HIST_BINS;
      for (int i = tid; i < SC_HIST_BINS; i += SC_THREADS) {
        const uint32_t c = s_hist[i];
        if (c) {
          atomicAdd(&gh[i], c);
          s_hist[i] = 0;
        }
      }
    }
    __syncthreads();   // s_qcode / s_hist are rewritten by the next segment
  }
}

// Generic kernel: any even C <= 128, any G <= 16; one thread per token, byte loads.
__global__ void __launch_bounds__(SC_THREADS) score_decode_generic_kernel(ScoreParams p) {
  __shared__ float s_qv[SC_MAX_G * SC_MAX_C];
  __shared__ float s_qscale[SC_MAX_G];
  __shared__ int8_t s_qcode[SC_MAX_G * SC_MAX_C];
  __shared__ uint32_t s_hist[SC_HIST_BINS];
  const int row = blockIdx.y;
  const int b = row / p.Hkv, g = row - b * p.Hkv;
  const bool hist = p.hist_out != nullptr;
  if (hist) {
    for (int i = threadIdx.x; i < SC_HIST_BINS; i += SC_THREADS) s_hist[i] = 0;
  }
  quantize_query_group<SC_THREADS>(p, b, g, p.G, s_qv, s_qcode, s_qscale);
  for (int64_t t = (int64_t)blockIdx.x * SC_THREADS + threadIdx.x; t < p.T; t += (int64_t)gridDim.x * SC_THREADS)
    score_token_plain<SC_MAX_G>(p, p.G, row, b, g, t, s_qcode, s_qscale, hist ? s_hist : nullptr);
  if (hist) {
    __syncthreads();
    uint32_t* gh = p.hist_out + (int64_t)row * SC_HIST_BINS;
    for (int i = threadIdx.x; i < SC_HIST_BINS; i += SC_THREADS) {
      const uint32_t c = s_hist[i];
      if (c) atomicAdd(&gh[i], c);
    }
  }
}

template <int C, int G, int NS, bool HIST>
static size_t score_stream_smem_bytes() {
  constexpr int TW = SC_TILE_PACKED_BYTES / (C / 2);
  constexpr int STAGE_BYTES = SC_TILE_PACKED_BYTES + TW * 4;
  size_t s = (size_t)SC_WARPS * NS * STAGE_BYTES + sizeof(uint64_t) * SC_WARPS * NS + sizeof(float) * G * C +
             sizeof(float) * SC_MAX_G + (size_t)G * C;
  if (HIST) s += sizeof(uint32_t) * SC_HIST_BINS;
  return s;
}

template <int C, int G, int NS, bool HIST>
static int score_stream_launch(const ScoreParams& p0, int device, cudaStream_t st) {
  ScoreParams p = p0;
  constexpr int TW = SC_TILE_PACKED_BYTES / (C / 2);
  p.full_tiles = p.T / TW;
  p.units_per_row = p.full_tiles + ((p.T % TW) ? 1 : 0);
  p.total_units = (int64_t)p.B * p.Hkv * p.units_per_row;
  const size_t smem = score_stream_smem_bytes<C, G, NS, HIST>();
  auto kern = score_decode_stream_kernel<C, G, NS, HIST>;
  static bool attr_done[64] = {false};
  if (device < 64 && !attr_done[device]) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[device] = true;
  }
  int per_sm = (int)((227 * 1024) / (smem + 1024));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 4) per_sm = 4;
  int64_t grid = (int64_t)sm_count(device) * per_sm;
  if (grid > p.total_units) grid = p.total_units;
  if (grid < 1) grid = 1;
  kern<<<(unsigned)grid, SC_THREADS, smem, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

template <int C, bool HIST>
static int score_stream_dispatch_g(const ScoreParams& p, int device, cudaStream_t st) {
  // 3 stages when the histogram shares the CTA's shared memory, else 4.
  constexpr int NS = HIST ? 3 : 4;
  switch (p.G) {
    case 1: return score_stream_launch<C, 1, NS, HIST>(p, device, st);
    case 2: return score_stream_launch<C, 2, NS, HIST>(p, device, st);
    case 4: return score_stream_launch<C, 4, NS, HIST>(p, device, st);
    case 8: return score_stream_launch<C, 8, NS, HIST>(p, device, st);
    default: return -1;
  }
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_score_decode(const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed,
                                int64_t packed_sb, int64_t packed_sh, const float* scale, int64_t scale_sb,
                                int64_t scale_sh, const int32_t* channel_idx, int B, int Hq, int Hkv, int T, int D,
                                int C, float* gmax_out, int32_t* acc_out, float* deq_out, uint32_t* hist_out,
                                int device, void* stream) {
  using namespace kvb;
  if (!query || !packed || !scale || !channel_idx) return KVB_BAD_ARG;
  if (!gmax_out && !acc_out && !deq_out) return KVB_BAD_ARG;
  if (hist_out && !gmax_out) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || T < 0 || D <= 0) return KVB_BAD_SHAPE;
  if (Hq % Hkv) return KVB_BAD_SHAPE;
  const int G = Hq / Hkv;
  if (G > SC_MAX_G || C <= 0 || C > SC_MAX_C || (C & 1) || C > D) return KVB_BAD_SHAPE;
  if ((int64_t)B * Hkv > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(query, 2) || !aligned_to(scale, 4)) return KVB_BAD_ALIGN;
  if (T == 0) return KVB_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  ScoreParams p;
  p.query = reinterpret_cast<const __nv_bfloat16*>(query);
  p.q_sb = q_sb; p.q_sh = q_sh;
  p.packed = packed; p.packed_sb = packed_sb; p.packed_sh = packed_sh;
  p.scale = scale; p.scale_sb = scale_sb; p.scale_sh = scale_sh;
  p.channel_idx = channel_idx;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.T = T; p.D = D; p.C = C; p.G = G;
  p.gmax_out = gmax_out; p.acc_out = acc_out; p.deq_out = deq_out; p.hist_out = hist_out;
  p.units_per_row = 0; p.full_tiles = 0; p.total_units = 0;

  const bool stream_ok = (C == 32 || C == 64 || C == 128) && (G == 1 || G == 2 || G == 4 || G == 8) &&
                         aligned_to(packed, 16) && (packed_sb % 16) == 0 && (packed_sh % 16) == 0 &&
                         aligned_to(scale, 16) && (scale_sb % 4) == 0 && (scale_sh % 4) == 0;
  if (stream_ok) {
    int rc = -1;
    if (hist_out) {
      if (C == 32) rc = score_stream_dispatch_g<32, true>(p, device, st);
      else if (C == 64) rc = score_stream_dispatch_g<64, true>(p, device, st);
      else rc = score_stream_dispatch_g<128, true>(p, device, st);
    } else {
      if (C == 32) rc = score_stream_dispatch_g<32, false>(p, device, st);
      else if (C == 64) rc = score_stream_dispatch_g<64, false>(p, device, st);
      else rc = score_stream_dispatch_g<128, false>(p, device, st);
    }
    if (rc >= 0) return rc;
  }
  int gx = ceil_div(T, SC_THREADS);
  const int cap = ceil_div(sm_count(device) * 16, B * Hkv);
  if (gx > cap) gx = cap < 1 ? 1 : cap;
  dim3 grid(gx, B * Hkv);
  score_decode_generic_kernel<<<grid, SC_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}
