// Stage 2: decode scoring. One query token per sequence against all T int4-packed keys.
//
// HBM-bound: every packed token (C/2 bytes) and its fp32 scale is read exactly once. The stream
// is staged through shared memory by the TMA engine (1-D cp.async.bulk + mbarrier), one private
// stage ring per warp so no CTA-wide barrier sits in the loop. Nibbles are widened to int8*16 with
// one shift and two masks per 32-bit word and multiplied exactly in int32 against the int8 query
// codes of all G heads of the KV head (int8 tensor-core tiles in the streaming kernel, plain
// integer arithmetic in the generic one), dequantised with two rounded fp32 products and reduced
// to the group maximum in registers. Only the group maximum (4 bytes per token per KV head) is
// written, plus an optional histogram of its sort keys for the selector.
#include "common.cuh"
#include "score_common.cuh"

namespace kvb {

// int8 tensor-core tile: D[16x8] (int32) += A[16x32] (int8, row) * B[32x8] (int8, col).
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// First MMA of an accumulation: D = A*B + c with the same register c in all four accumulator slots. With
// c = 0x4B400000 (the bits of 1.5 * 2^23) the finished accumulator, read as a float, is 1.5 * 2^23 + dot
// exactly (|dot| < 2^22): the integer add of the int -> float conversion rides on the MMA for free.
__device__ __forceinline__ void mma_s8_16832_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1, int c) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}
constexpr int SC_FLOAT_MAGIC = 0x4B400000;

// Streaming kernel. C in {32,64,128}, G in {1,2,4,8}.
//
// A warp owns a ring of NS stages; each stage holds TW tokens (packed bytes + scales) brought in
// by two bulk copies. The integer dot products of 16 tokens x 32 channels x 8 columns run as one
// m16n8k32 int8 MMA: a lane (g = lane/4, t = lane%4) reads C/8 contiguous bytes of the tokens in
// rows g and g+8, widens each packed word into "low nibbles * 16" and "high nibbles * 16" (three
// integer ops) and uses them directly as A fragments; the query codes sit in the B fragment in
// the matching channel order. With G < 8 heads the 8 columns are shared by 8/G token tiles
// (tile j's heads go to columns [jG, jG+G)), so one accumulator covers 128/G tokens densely and
// every lane dequantises exactly four (token, head) values.
// Persistent: CTA c owns the contiguous unit range [c*U/grid, (c+1)*U/grid) of the flattened
// (row, tile) space.
constexpr int SC_STAGE_PACKED_BYTES = 4096;

template <int C, int G>
struct ScoreCfg {
  static constexpr int WARPS = 8;
  static constexpr int THREADS = WARPS * 32;
  static constexpr int KS = C / 32;                     // k-steps of 32 channels; also packed words per lane-token
  static constexpr int TPA = 8 / G;                     // 16-token tiles that share one accumulator
  static constexpr int ITER_TOKENS = 16 * TPA;          // tokens per accumulator
  // tokens per stage: about 4 KiB of packed codes per bulk copy (copies of 2 KiB reach only ~93 % of the
  // streaming bandwidth that 4 KiB copies reach with the same bytes in flight)
  static constexpr int STAGE_TOKENS = SC_STAGE_PACKED_BYTES / (C / 2);
  static constexpr int TW = ITER_TOKENS > STAGE_TOKENS ? ITER_TOKENS : STAGE_TOKENS;
  static constexpr int IT = TW / ITER_TOKENS;
  static constexpr int TOKEN_BYTES = C / 2;
  static constexpr int PACKED_BYTES = TW * TOKEN_BYTES;
  static constexpr int STAGE_BYTES = PACKED_BYTES + TW * 4;
};

template <int C, int G, int NS, int MODE>
__global__ void __launch_bounds__(ScoreCfg<C, G>::THREADS, 2) score_decode_stream_kernel(ScoreParams p) {
  constexpr bool HIST = MODE == SC_MODE_HIST;
  constexpr bool EMIT = MODE == SC_MODE_EMIT;
  constexpr bool SAMPLE = MODE == SC_MODE_SAMPLE;
  using Cfg = ScoreCfg<C, G>;
  constexpr int KS = Cfg::KS, TPA = Cfg::TPA, TW = Cfg::TW, IT = Cfg::IT;
  constexpr int WARPS = Cfg::WARPS, THREADS = Cfg::THREADS;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES, PACKED_BYTES = Cfg::PACKED_BYTES, TOKEN_BYTES = Cfg::TOKEN_BYTES;

  extern __shared__ __align__(128) uint8_t smem_raw[];
  // layout: [warps][NS][STAGE_BYTES] | bars [warps][NS] | qv | qscale | qcode | hist
  uint8_t* s_stage = smem_raw;
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_stage + WARPS * NS * STAGE_BYTES);
  float* s_qv = reinterpret_cast<float*>(s_bar + WARPS * NS);
  float* s_qscale = s_qv + G * C;
  int8_t* s_qcode = reinterpret_cast<int8_t*>(s_qscale + SC_MAX_G);
  uint32_t* s_hist = reinterpret_cast<uint32_t*>(s_qcode + G * C);   // G*C is a multiple of 32 (HIST)
  uint64_t* s_cbuf = reinterpret_cast<uint64_t*>(s_qcode + G * C);   // same place, EMIT: [warps][SC_EMIT_WARP_BUF]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  pdl_launch_dependents();
  uint8_t* my_stage = s_stage + warp * NS * STAGE_BYTES;
  uint64_t* my_bar = s_bar + warp * NS;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) mbar_init(&my_bar[s], 1);
    fence_mbar_init();
  }
  if (HIST) {
    for (int i = tid; i < SC_HIST_BINS; i += THREADS) s_hist[i] = 0;
  }
  fence_proxy_async_smem();
  __syncthreads();

  const uint64_t policy = l2_policy_evict_first();
  // The group-max row is re-read by the selector right away and overwritten by the next step:
  // ask L2 to keep it so that it need not travel to HBM and back.
  const uint64_t keep = l2_policy_evict_last();
  // work geometry from the history length (read from the device when it lives there)
  const int T = p.T_dev ? min(*p.T_dev, p.T) : p.T;
  int full_tiles = T / TW;
  int units_per_row = full_tiles + ((T % TW) ? 1 : 0);
  // SAMPLE: logical tile lt of a row is physical tile (lt / grp) * grp_stride + lt % grp; outputs are compact
  int grp = 1, grp_stride = 1;
  if constexpr (SAMPLE) {
    int n_sample;
    fs_sample_geometry(T, TW, grp, grp_stride, n_sample);
    full_tiles = units_per_row = (T > p.cand_cap) ? FS_RUNS * grp : 0;      // short rows need no threshold
  }
  const int64_t total_units = (int64_t)p.B * p.Hkv * units_per_row;
  const int64_t u_begin = (int64_t)blockIdx.x * total_units / gridDim.x;
  const int64_t u_end = (int64_t)(blockIdx.x + 1) * total_units / gridDim.x;

  uint32_t ring = 0;        // tiles this warp has consumed so far (stage = ring % NS, parity = ring / NS & 1)
  bool dead = false;        // a bounded wait gave up: skip all further streaming work

  // Which accumulator column pair this lane reads back: columns 2*t4, 2*t4+1.
  //   G >= 2: both columns belong to tile jt = 2*t4 / G, heads h0 = 2*t4 % G and h0 + 1.
  //   G == 1: column c is tile c, head 0.
  constexpr int HV = G >= 2 ? 2 : 1;                     // distinct heads among the lane's two columns
  const int jt = (2 * t4) / G;
  const int h0 = (2 * t4) % G;

  int64_t u = u_begin;
  while (u < u_end) {
    const int row = (int)(u / units_per_row);
    const int ua = (int)(u - (int64_t)row * units_per_row);
    int64_t row_end_u = (int64_t)(row + 1) * units_per_row;
    const int ub = (int)((row_end_u < u_end ? row_end_u : u_end) - (int64_t)row * units_per_row);
    u += (ub - ua);
    const int b = row / p.Hkv, kvh = row - b * p.Hkv;

    const uint8_t* packed_row = p.packed + (int64_t)b * p.packed_sb + (int64_t)kvh * p.packed_sh;
    const float* scale_row = p.scale + (int64_t)b * p.scale_sb + (int64_t)kvh * p.scale_sh;

    // Full tiles of this segment: [ta, tb); warp w takes ta + w, ta + w + WARPS, ...
    const int ta = ua;
    const int tb = ub < full_tiles ? ub : full_tiles;
    const int nmy = (tb - ta - warp + WARPS - 1) / WARPS;   // <= 0 when none

    auto issue = [&](int j, uint32_t slot) {
      // lane 0 only: tile j of this warp into ring slot `slot`
      const int lt = ta + warp + j * WARPS;
      const int64_t t0 = (int64_t)(SAMPLE ? (lt / grp) * grp_stride + lt % grp : lt) * TW;
      uint8_t* dst = my_stage + (slot % NS) * STAGE_BYTES;
      mbar_arrive_expect_tx(&my_bar[slot % NS], STAGE_BYTES);
      bulk_g2s_evict_first(dst, packed_row + t0 * TOKEN_BYTES, PACKED_BYTES, &my_bar[slot % NS], policy);
      bulk_g2s_evict_first(dst + PACKED_BYTES, scale_row + t0, TW * 4, &my_bar[slot % NS], policy);
    };
    // The first copies of the segment go out before the query is quantised (and before the wait for the
    // kernel that produces the thresholds): the ring fills while the prologue runs.
    if (!dead && nmy > 0 && lane == 0) {
      fence_proxy_async_smem();                      // the slots were last read with ordinary loads
      const int pre = nmy < NS ? nmy : NS;
      for (int j = 0; j < pre; ++j) issue(j, ring + j);
    }

    quantize_query_group<THREADS>(p, b, kvh, G, s_qv, s_qcode, s_qscale);

    // B fragments. Lane t4 owns packed bytes [KS*4*t4, KS*4*(t4+1)) of every token; k-step s uses
    // packed word s: its low nibbles are channels 2*(KS*4*t4 + 4*s + i), its high nibbles the odd
    // neighbours. Column n = g carries head g - j*G in the variant for tile j, zero elsewhere.
    uint32_t bq[TPA][KS][2];
#pragma unroll
    for (int j = 0; j < TPA; ++j) {
      const bool mine = (g / G) == j;
      const int hd = g % G;
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = 2 * (KS * 4 * t4 + 4 * s + i);
          lo |= (uint32_t)(uint8_t)s_qcode[hd * C + c] << (8 * i);
          hi |= (uint32_t)(uint8_t)s_qcode[hd * C + c + 1] << (8 * i);
        }
        bq[j][s][0] = mine ? lo : 0u;
        bq[j][s][1] = mine ? hi : 0u;
      }
    }
    // The accumulator holds 16 * dot; fold the 1/16 into the (power-of-two exact) query scale.
    float qs16[HV];
#pragma unroll
    for (int v = 0; v < HV; ++v) qs16[v] = s_qscale[(h0 + v) % G] * 0.0625f;

    float* gmax_row = p.gmax_out ? p.gmax_out + (int64_t)row * p.T : nullptr;
    // Everything above reads only the caller's inputs; the thresholds (and the zeroed counters) come
    // from the kernels before this one.
    pdl_wait();
    const float tau = EMIT ? p.tau[row] : 0.0f;
    uint64_t* cand_row = EMIT ? p.cand + (int64_t)row * p.cand_cap : nullptr;
    uint32_t* count_row = EMIT ? p.cand_count + (int64_t)row * SC_COUNT_STRIDE : nullptr;

    // What happens to a finished token: group max m (already +0-normalised) of token t of this row.
    // Called by ALL lanes of the warp together; `active` says whether this lane really has a token.
    // Candidate emission keeps a warp-private buffer whose fill count lives in a register (the
    // ballot gives every taker its slot), so the hot loop has no atomics at all.
    uint64_t* wbuf = s_cbuf + warp * SC_EMIT_WARP_BUF;
    uint32_t wcount = 0;
    bool wdead = false;          // the row's list is already over capacity: it will be re-scored, stop feeding it
    auto finish = [&](float m, int64_t t, bool active) {
      if (gmax_row && active) st_global_hint_f32(gmax_row + t, m, keep);
      if (HIST && active) atomicAdd(&s_hist[float_to_key(m) >> (32 - SC_HIST_BITS)], 1u);
      if (EMIT) {
        const bool take = active && !wdead && (m >= tau);
        const uint32_t mask = __ballot_sync(0xffffffffu, take);
        if (mask) {
          const uint32_t filled = wcount + (uint32_t)__popc(mask);
          bool over = false;
          if (take) {
            const uint64_t c = make_composite(m, (uint32_t)t);
            const uint32_t pos = wcount + (uint32_t)__popc(mask & ((1u << lane) - 1u));
            if (pos < (uint32_t)SC_EMIT_WARP_BUF) {
              wbuf[pos] = c;
            } else {                                           // buffer full: straight to the row's list
              const uint32_t gp = atomicAdd(count_row, 1u);
              if (gp < (uint32_t)p.cand_cap) cand_row[gp] = c;
              else over = true;                                // count > capacity already marks the row as failed
            }
          }
          // (warp-uniform test: only a warp that ran past its buffer can have met the capacity)
          if (filled > (uint32_t)SC_EMIT_WARP_BUF && __any_sync(0xffffffffu, over)) wdead = true;
          wcount = filled;
        }
      }
    };

    if (!dead && nmy > 0) {
      for (int j = 0; j < nmy; ++j) {
        const uint32_t slot = ring + j;
        bool ok = mbar_wait_bounded(&my_bar[slot % NS], (slot / NS) & 1u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { dead = true; break; }
        const uint8_t* st = my_stage + (slot % NS) * STAGE_BYTES;
        const float* ssc = reinterpret_cast<const float*>(st + PACKED_BYTES);
        const int64_t t0 = (int64_t)(ta + warp + j * WARPS) * TW;

#pragma unroll
        for (int it = 0; it < IT; ++it) {
          int acc[4];                                       // starts at SC_FLOAT_MAGIC (see mma_s8_16832_first)
#pragma unroll
          for (int tj = 0; tj < TPA; ++tj) {
            // rows g and g+8 of token tile tj: KS packed words each, from this lane's byte range
            const uint8_t* r0 = st + (size_t)(it * Cfg::ITER_TOKENS + tj * 16 + g) * TOKEN_BYTES + KS * 4 * t4;
            const uint8_t* r1 = r0 + 8 * TOKEN_BYTES;
            uint32_t w0[KS], w1[KS];
            if constexpr (KS == 1) {
              w0[0] = *reinterpret_cast<const uint32_t*>(r0);
              w1[0] = *reinterpret_cast<const uint32_t*>(r1);
            } else if constexpr (KS == 2) {
              const uint2 x0 = *reinterpret_cast<const uint2*>(r0);
              const uint2 x1 = *reinterpret_cast<const uint2*>(r1);
              w0[0] = x0.x; w0[1] = x0.y; w1[0] = x1.x; w1[1] = x1.y;
            } else {
              const uint4 x0 = *reinterpret_cast<const uint4*>(r0);
              const uint4 x1 = *reinterpret_cast<const uint4*>(r1);
              w0[0] = x0.x; w0[1] = x0.y; w0[2] = x0.z; w0[3] = x0.w;
              w1[0] = x1.x; w1[1] = x1.y; w1[2] = x1.z; w1[3] = x1.w;
            }
#pragma unroll
            for (int s = 0; s < KS; ++s) {
              const uint32_t a0 = (w0[s] << 4) & 0xF0F0F0F0u;   // int8 lanes = 16 * low-nibble codes, row g
              const uint32_t a1 = (w1[s] << 4) & 0xF0F0F0F0u;   // row g+8
              const uint32_t a2 = w0[s] & 0xF0F0F0F0u;          // 16 * high-nibble codes, row g
              const uint32_t a3 = w1[s] & 0xF0F0F0F0u;
              if (tj == 0 && s == 0) mma_s8_16832_first(acc, a0, a1, a2, a3, bq[tj][s][0], bq[tj][s][1], SC_FLOAT_MAGIC);
              else mma_s8_16832(acc, a0, a1, a2, a3, bq[tj][s][0], bq[tj][s][1]);
            }
          }
          // acc[0], acc[1]: row g, columns 2*t4, 2*t4+1; acc[2], acc[3]: row g+8, same columns.
          // value v of the lane: row (v>>1 ? g+8 : g), column 2*t4 + (v&1).
          float d[4];
          int tl[4];                                        // token (inside the stage) of each value
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = v & 1;
            const int tile = G >= 2 ? jt : (2 * t4 + col);
            tl[v] = it * Cfg::ITER_TOKENS + tile * 16 + g + ((v >> 1) ? 8 : 0);
            const float f = __int_as_float(acc[v]) - 12582912.0f;   // exact: acc = bits(1.5 * 2^23) + 16 * dot, |16 * dot| < 2^22
            d[v] = __fmul_rn(__fmul_rn(f, ssc[tl[v]]), qs16[G >= 2 ? col : 0]);
          }
          if (p.acc_out || p.deq_out) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int hd = G >= 2 ? (h0 + (v & 1)) : 0;
              const int64_t o = ((int64_t)b * p.Hq + (int64_t)kvh * G + hd) * p.T + t0 + tl[v];
              if (p.acc_out) p.acc_out[o] = (acc[v] - SC_FLOAT_MAGIC) >> 4;
              if (p.deq_out) p.deq_out[o] = d[v];
            }
          }
          // Group maximum per token, then every lane finishes NOUT tokens of its own.
          if constexpr (G >= 2) {
            float m0 = fmaxf(d[0], d[1]);                   // row g
            float m1 = fmaxf(d[2], d[3]);                   // row g+8
            if constexpr (G >= 4) {
              m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
              m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
            }
            if constexpr (G >= 8) {
              m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
              m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
            }
            if constexpr (G == 2) {
              // the lane alone holds both heads of its two tokens
              if (m0 == 0.0f) m0 = 0.0f;
              if (m1 == 0.0f) m1 = 0.0f;
              finish(m0, t0 + tl[0], true);
              finish(m1, t0 + tl[2], true);
            } else {
              // G == 4: lanes (t4, t4^1) share two tokens -> even lane finishes row g, odd lane row g+8.
              // G == 8: the quad shares two tokens -> lane t4 == 0 finishes row g, t4 == 1 row g+8.
              const bool second = (t4 & 1) != 0;
              float m = second ? m1 : m0;
              const int tok = second ? tl[2] : tl[0];
              const bool writer = (G == 4) ? true : (t4 < 2);
              if (m == 0.0f) m = 0.0f;
              finish(m, t0 + tok, writer);
            }
          } else {
            // G == 1: four tokens per lane, no reduction
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float m = d[v];
              if (m == 0.0f) m = 0.0f;
              finish(m, t0 + tl[v], true);
            }
          }
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
    if (ub > full_tiles) {
      const int64_t tail0 = (int64_t)full_tiles * TW;
      for (int64_t tb = tail0 + warp * 32; tb < T; tb += THREADS) {        // warp-uniform trips (ballot in finish)
        const int64_t t = tb + lane;
        const bool live = t < T;
        const float m = live ? score_token_plain<G>(p, G, b, kvh, t, s_qcode, s_qscale) : 0.0f;
        finish(m, t, live);
      }
    }
    if (EMIT) {
      // hand the warp's buffered candidates of this row over with ONE reservation
      __syncwarp();
      const uint32_t n = wcount < (uint32_t)SC_EMIT_WARP_BUF ? wcount : (uint32_t)SC_EMIT_WARP_BUF;
      uint32_t base = 0;
      if (lane == 0 && n) base = atomicAdd(count_row, n);
      base = __shfl_sync(0xffffffffu, base, 0);
      for (uint32_t i = lane; i < n; i += 32)
        if (base + i < (uint32_t)p.cand_cap) cand_row[base + i] = wbuf[i];
      __syncwarp();
    }
    if (HIST) {
      __syncthreads();
      uint32_t* gh = p.hist_out + (int64_t)row * SC_HIST_BINS;
      for (int i = tid; i < SC_HIST_BINS; i += THREADS) {
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
  for (int64_t t = (int64_t)blockIdx.x * SC_THREADS + threadIdx.x; t < p.T; t += (int64_t)gridDim.x * SC_THREADS) {
    const float m = score_token_plain<SC_MAX_G>(p, p.G, b, g, t, s_qcode, s_qscale);
    if (p.gmax_out) p.gmax_out[(int64_t)row * p.T + t] = m;
    if (hist) atomicAdd(&s_hist[float_to_key(m) >> (32 - SC_HIST_BITS)], 1u);
  }
  if (hist) {
    __syncthreads();
    uint32_t* gh = p.hist_out + (int64_t)row * SC_HIST_BINS;
    for (int i = threadIdx.x; i < SC_HIST_BINS; i += SC_THREADS) {
      const uint32_t c = s_hist[i];
      if (c) atomicAdd(&gh[i], c);
    }
  }
}

template <int C, int G, int NS, int MODE>
static size_t score_stream_smem_bytes() {
  using Cfg = ScoreCfg<C, G>;
  size_t s = (size_t)Cfg::WARPS * NS * Cfg::STAGE_BYTES + sizeof(uint64_t) * Cfg::WARPS * NS +
             sizeof(float) * G * C + sizeof(float) * SC_MAX_G + (size_t)G * C;
  if (MODE == SC_MODE_HIST) s += sizeof(uint32_t) * SC_HIST_BINS;
  if (MODE == SC_MODE_EMIT) s += sizeof(uint64_t) * SC_EMIT_BUF;
  return s;
}

template <int C, int G, int NS, int MODE>
static int score_stream_launch(const ScoreParams& p0, int device, cudaStream_t st) {
  using Cfg = ScoreCfg<C, G>;
  ScoreParams p = p0;
  p.full_tiles = p.T / Cfg::TW;
  p.units_per_row = p.full_tiles + ((p.T % Cfg::TW) ? 1 : 0);
  if (MODE == SC_MODE_SAMPLE) {
    int grp, stride, n_sample;
    fs_sample_geometry(p.T, Cfg::TW, grp, stride, n_sample);
    p.full_tiles = p.units_per_row = FS_RUNS * grp;
  }
  p.total_units = (int64_t)p.B * p.Hkv * p.units_per_row;
  const size_t smem = score_stream_smem_bytes<C, G, NS, MODE>();
  auto kern = score_decode_stream_kernel<C, G, NS, MODE>;
  static std::atomic<bool> attr_done[KVB_MAX_DEVICES];
  { const int arc = ensure_dynamic_smem(kern, attr_done, device, (size_t)smem); if (arc != KVB_OK) return arc; }
  int per_sm = (int)((227 * 1024) / (smem + 1024));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 2) per_sm = 2;
  int64_t grid = (int64_t)sm_count(device) * per_sm;
  const int64_t max_ctas = (p.total_units + 1) / 2;        // at least two units per CTA
  if (grid > max_ctas) grid = max_ctas;
  if (grid < 1) grid = 1;
  KVB_CHECK_CUDA(launch_kernel(kern, dim3((unsigned)grid), dim3(Cfg::THREADS), smem, st, p));
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

// Stages per warp ring so that two 8-warp CTAs (plus the histogram) fit one SM's shared memory.
template <int C, int G>
constexpr int score_stages() {
  constexpr int budget = 96 * 1024 - 20 * 1024;
  constexpr int per_stage = ScoreCfg<C, G>::WARPS * ScoreCfg<C, G>::STAGE_BYTES;
  return budget / per_stage >= 4 ? 4 : (budget / per_stage >= 2 ? budget / per_stage : 2);
}

template <int C, int MODE>
static int score_stream_dispatch_g(const ScoreParams& p, int device, cudaStream_t st) {
  switch (p.G) {
    case 1: return score_stream_launch<C, 1, score_stages<C, 1>(), MODE>(p, device, st);
    case 2: return score_stream_launch<C, 2, score_stages<C, 2>(), MODE>(p, device, st);
    case 4: return score_stream_launch<C, 4, score_stages<C, 4>(), MODE>(p, device, st);
    case 8: return score_stream_launch<C, 8, score_stages<C, 8>(), MODE>(p, device, st);
    default: return -1;
  }
}

// Tokens per tile of the streaming kernel for (C, G) (the unit of the sample geometry); 0 if unsupported.
static int score_stream_tile_tokens(int C, int G) {
  if (C != 32 && C != 64 && C != 128) return 0;
  switch (G) {
    case 1: return C == 32 ? ScoreCfg<32, 1>::TW : (C == 64 ? ScoreCfg<64, 1>::TW : ScoreCfg<128, 1>::TW);
    case 2: return C == 32 ? ScoreCfg<32, 2>::TW : (C == 64 ? ScoreCfg<64, 2>::TW : ScoreCfg<128, 2>::TW);
    case 4: return C == 32 ? ScoreCfg<32, 4>::TW : (C == 64 ? ScoreCfg<64, 4>::TW : ScoreCfg<128, 4>::TW);
    case 8: return C == 32 ? ScoreCfg<32, 8>::TW : (C == 64 ? ScoreCfg<64, 8>::TW : ScoreCfg<128, 8>::TW);
    default: return 0;
  }
}

// The sample of every row scored by the streaming kernel: group maxima of the sample tiles, compacted, at
// the start of row r of `sample` (row pitch base.T floats). Rows of at most `cap` tokens are skipped.
static int score_sample_stream_run(const ScoreParams& base, float* sample, int cap, int device, cudaStream_t st) {
  ScoreParams p = base;
  p.gmax_out = sample; p.acc_out = nullptr; p.deq_out = nullptr; p.hist_out = nullptr;
  p.tau = nullptr; p.cand = nullptr; p.cand_count = nullptr; p.cand_cap = cap;
  int rc = -1;
  if (p.C == 32) rc = score_stream_dispatch_g<32, SC_MODE_SAMPLE>(p, device, st);
  else if (p.C == 64) rc = score_stream_dispatch_g<64, SC_MODE_SAMPLE>(p, device, st);
  else if (p.C == 128) rc = score_stream_dispatch_g<128, SC_MODE_SAMPLE>(p, device, st);
  return rc < 0 ? KVB_BAD_SHAPE : rc;
}

struct ScoreEmit {
  const float* tau;        // [B*Hkv] emission thresholds
  uint64_t* cand;          // [B*Hkv, cand_cap]
  uint32_t* cand_count;    // [B*Hkv * SC_COUNT_STRIDE], zeroed by the caller
  int cand_cap;
};

// The streaming kernel's preconditions (everything else takes the generic kernel).
static bool score_stream_supported(int C, int G, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                                   const float* scale, int64_t scale_sb, int64_t scale_sh) {
  return (C == 32 || C == 64 || C == 128) && (G == 1 || G == 2 || G == 4 || G == 8) && aligned_to(packed, 16) &&
         (packed_sb % 16) == 0 && (packed_sh % 16) == 0 && aligned_to(scale, 16) && (scale_sb % 4) == 0 &&
         (scale_sh % 4) == 0;
}

// Shared by kvb_score_decode and the fused step. With `emit` the kernel appends candidates instead
// of (or besides) writing gmax; that mode exists only in the streaming kernel.
static int score_run(const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb,
                     int64_t packed_sh, const float* scale, int64_t scale_sb, int64_t scale_sh,
                     const int32_t* channel_idx, int B, int Hq, int Hkv, int T, int D, int C, float* gmax_out,
                     int32_t* acc_out, float* deq_out, uint32_t* hist_out, const ScoreEmit* emit,
                     const int32_t* T_dev, int device, cudaStream_t st) {
  if (!query || !packed || !scale || !channel_idx) return KVB_BAD_ARG;
  if (!gmax_out && !acc_out && !deq_out && !emit) return KVB_BAD_ARG;
  if (hist_out && !gmax_out) return KVB_BAD_ARG;
  if (emit && hist_out) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || T < 0 || D <= 0) return KVB_BAD_SHAPE;
  if (Hq % Hkv) return KVB_BAD_SHAPE;
  const int G = Hq / Hkv;
  if (G > SC_MAX_G || C <= 0 || C > SC_MAX_C || (C & 1) || C > D) return KVB_BAD_SHAPE;
  if ((int64_t)B * Hkv > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(query, 2) || !aligned_to(scale, 4)) return KVB_BAD_ALIGN;
  if (T == 0) return KVB_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;

  ScoreParams p;
  p.query = reinterpret_cast<const __nv_bfloat16*>(query);
  p.q_sb = q_sb; p.q_sh = q_sh;
  p.packed = packed; p.packed_sb = packed_sb; p.packed_sh = packed_sh;
  p.scale = scale; p.scale_sb = scale_sb; p.scale_sh = scale_sh;
  p.channel_idx = channel_idx;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.T = T; p.D = D; p.C = C; p.G = G;
  p.gmax_out = gmax_out; p.acc_out = acc_out; p.deq_out = deq_out; p.hist_out = hist_out;
  p.T_dev = T_dev;
  p.tau = emit ? emit->tau : nullptr;
  p.cand = emit ? emit->cand : nullptr;
  p.cand_count = emit ? emit->cand_count : nullptr;
  p.cand_cap = emit ? emit->cand_cap : 0;
  p.units_per_row = 0; p.full_tiles = 0; p.total_units = 0;

  if (score_stream_supported(C, G, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh)) {
    int rc = -1;
    if (emit) {
      if (C == 32) rc = score_stream_dispatch_g<32, SC_MODE_EMIT>(p, device, st);
      else if (C == 64) rc = score_stream_dispatch_g<64, SC_MODE_EMIT>(p, device, st);
      else rc = score_stream_dispatch_g<128, SC_MODE_EMIT>(p, device, st);
    } else if (hist_out) {
      if (C == 32) rc = score_stream_dispatch_g<32, SC_MODE_HIST>(p, device, st);
      else if (C == 64) rc = score_stream_dispatch_g<64, SC_MODE_HIST>(p, device, st);
      else rc = score_stream_dispatch_g<128, SC_MODE_HIST>(p, device, st);
    } else {
      if (C == 32) rc = score_stream_dispatch_g<32, SC_MODE_PLAIN>(p, device, st);
      else if (C == 64) rc = score_stream_dispatch_g<64, SC_MODE_PLAIN>(p, device, st);
      else rc = score_stream_dispatch_g<128, SC_MODE_PLAIN>(p, device, st);
    }
    if (rc >= 0) return rc;
  }
  if (emit || T_dev) return KVB_BAD_SHAPE;     // callers check score_stream_supported() first
  int gx = ceil_div(T, SC_THREADS);
  const int cap = ceil_div(sm_count(device) * 16, B * Hkv);
  if (gx > cap) gx = cap < 1 ? 1 : cap;
  dim3 grid(gx, B * Hkv);
  score_decode_generic_kernel<<<grid, SC_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_score_decode(
    const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, const int32_t* channel_idx, int B, int Hq, int Hkv, int T,
    int D, int C, float* gmax_out, int32_t* acc_out, float* deq_out, uint32_t* hist_out, int device, void* stream) {
  return kvb::score_run(query, q_sb, q_sh, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, channel_idx, B, Hq,
                        Hkv, T, D, C, gmax_out, acc_out, deq_out, hist_out, nullptr, nullptr, device,
                        reinterpret_cast<cudaStream_t>(stream));
}
