// Chunked-prefill block scoring: a chunk of Tq query tokens against all Tk cached int4 keys.
//
//   acc[b,h,i,t]  = sum_c qcode[b,h,i,c] * code[b,h/G,t,c]                  (int32, exact)
//   deq           = (float(acc) * kscale[b,h/G,t]) * qscale[b,h,i]           (two rounded products)
//   blk[b,g,i,j]  = max over the G heads of group g and the 64 tokens of block j of deq
//   then the top blocks per (b, g, i) by (blk desc, j asc).
//
// This is a genuine dense contraction (M = G*Tq rows, N = Tk, K = C), so it runs on the tensor
// cores: int4 codes are widened to int8 in registers and multiplied with mma.sync m16n8k32 s8.
// A warp owns 16 queries x G heads (one 16-row tile per head, so the group max never leaves the
// lane) and walks the key blocks staged in shared memory by the CTA. With K = C <= 128 the
// kernel is bound by the per-element epilogue (int->float, scale, max), not by the MMAs; the
// monotonicity of x -> fl(x * qscale) for qscale > 0 lets the query scale be applied once per
// block maximum instead of once per element without changing a single bit.
#include "common.cuh"

#include <string.h>

namespace kvb {

constexpr int PF_WARPS = 8;
constexpr int PF_THREADS = PF_WARPS * 32;
constexpr int PF_QTILE = PF_WARPS * 16;          // queries per CTA
constexpr int PF_BLOCK = 64;                     // tokens per key block
constexpr int PF_OUT_BLOCKS = 8;                 // block maxima buffered before a coalesced flush

struct PrefillParams {
  const int8_t* qcode;      // [B,Hq,Tq,C]
  const float* qscale;      // [B,Hq,Tq]
  const uint8_t* packed; int64_t packed_sb, packed_sh;
  const float* scale; int64_t scale_sb, scale_sh;
  float* out;               // [B,Hkv,Tq,nblk]
  int B, Hq, Hkv, Tq, Tk, C, G, nblk;
  int blocks_per_cta;
};

__device__ __forceinline__ void pf_mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int C, int G>
__global__ void __launch_bounds__(PF_THREADS, 2) score_prefill_kernel(PrefillParams p) {
  constexpr int KS = C / 32;                      // k-steps of 32 channels = packed words per lane per token
  constexpr int TOKEN_BYTES = C / 2;
  constexpr int STAGE_BYTES = PF_BLOCK * TOKEN_BYTES + PF_BLOCK * 4;
  __shared__ __align__(16) uint8_t s_stage[2][STAGE_BYTES];
  __shared__ __align__(16) float s_out[PF_QTILE][PF_OUT_BLOCKS];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int bh = blockIdx.z;
  const int b = bh / p.Hkv, kvh = bh - b * p.Hkv;
  const int q0 = blockIdx.x * PF_QTILE;            // first query of the CTA
  const int qw = q0 + warp * 16;                   // first query of the warp
  const int blk0 = blockIdx.y * p.blocks_per_cta;
  int blk1 = blk0 + p.blocks_per_cta;
  if (blk1 > p.nblk) blk1 = p.nblk;

  // A fragments: head hd is the 16-row tile hd; rows g and g+8 are queries qw+g and qw+g+8.
  // k-step s, lane t4 covers channels 8*(4s+t4) .. +7: even ones in a0/a1, odd ones in a2/a3,
  // the same order in which the widened K words deliver them.
  uint32_t qa[G][KS][4];
  float qs[G][2];
#pragma unroll
  for (int hd = 0; hd < G; ++hd) {
    const int head = kvh * G + hd;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      int qi = qw + g + 8 * r;
      const bool live = qi < p.Tq;
      if (!live) qi = p.Tq - 1;
      const int64_t rowoff = ((int64_t)b * p.Hq + head) * p.Tq + qi;
      qs[hd][r] = p.qscale[rowoff];
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        const uint2 x = *reinterpret_cast<const uint2*>(p.qcode + rowoff * C + 8 * (4 * s + t4));
        qa[hd][s][r] = __byte_perm(x.x, x.y, 0x6420);          // channels +0,+2,+4,+6
        qa[hd][s][2 + r] = __byte_perm(x.x, x.y, 0x7531);      // channels +1,+3,+5,+7
      }
    }
  }

  const uint8_t* packed_row = p.packed + (int64_t)b * p.packed_sb + (int64_t)kvh * p.packed_sh;
  const float* scale_row = p.scale + (int64_t)b * p.scale_sb + (int64_t)kvh * p.scale_sh;

  // CTA-wide staging of one 64-token block: packed bytes then scales (pre-multiplied by 1/16 on read).
  auto stage_block = [&](int blk, int buf) {
    const int64_t t0 = (int64_t)blk * PF_BLOCK;
    uint8_t* dst = s_stage[buf];
    constexpr int VECS = PF_BLOCK * TOKEN_BYTES / 16;
    for (int v = tid; v < VECS + PF_BLOCK / 4; v += PF_THREADS) {
      if (v < VECS) {
        const int64_t tok = t0 + (v * 16) / TOKEN_BYTES;
        if (tok < p.Tk) cp_async_16(dst + v * 16, packed_row + t0 * TOKEN_BYTES + (int64_t)v * 16);
        else *reinterpret_cast<uint4*>(dst + v * 16) = make_uint4(0, 0, 0, 0);
      } else {
        const int sv = v - VECS;
        const int64_t tok = t0 + sv * 4;
        float* sd = reinterpret_cast<float*>(dst + PF_BLOCK * TOKEN_BYTES) + sv * 4;
        if (tok + 3 < p.Tk) {
          cp_async_16(sd, scale_row + tok);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) sd[e] = (tok + e < p.Tk) ? scale_row[tok + e] : 0.0f;
        }
      }
    }
  };

  if (blk0 < blk1) stage_block(blk0, 0);
  cp_async_commit();

  for (int blk = blk0; blk < blk1; ++blk) {
    const int buf = (blk - blk0) & 1;
    if (blk + 1 < blk1) stage_block(blk + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const uint8_t* st = s_stage[buf];
    const float* ssc = reinterpret_cast<const float*>(st + PF_BLOCK * TOKEN_BYTES);
    const int64_t t0 = (int64_t)blk * PF_BLOCK;

    float rm[G][2];                                 // running max over the block of fl(acc * kscale)
#pragma unroll
    for (int hd = 0; hd < G; ++hd) rm[hd][0] = rm[hd][1] = -INFINITY;

#pragma unroll 2
    for (int nt = 0; nt < PF_BLOCK / 8; ++nt) {
      // B fragments: token 8*nt + g, packed word 4*s + t4 -> low nibbles (b0) and high nibbles (b1), times 16
      uint32_t bk[KS][2];
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(st + (8 * nt + g) * TOKEN_BYTES + 4 * (4 * s + t4));
        bk[s][0] = (w << 4) & 0xF0F0F0F0u;
        bk[s][1] = w & 0xF0F0F0F0u;
      }
      // scales of the accumulator's two token columns (2*t4, 2*t4+1), with the exact 1/16 folded in
      const float2 ks2 = *reinterpret_cast<const float2*>(ssc + 8 * nt + 2 * t4);
      const float k0 = ks2.x * 0.0625f, k1 = ks2.y * 0.0625f;
      const bool live0 = t0 + 8 * nt + 2 * t4 < p.Tk, live1 = t0 + 8 * nt + 2 * t4 + 1 < p.Tk;
#pragma unroll
      for (int hd = 0; hd < G; ++hd) {
        int acc[4] = {0, 0, 0, 0};
#pragma unroll
        for (int s = 0; s < KS; ++s) pf_mma_s8(acc, qa[hd][s][0], qa[hd][s][1], qa[hd][s][2], qa[hd][s][3], bk[s][0], bk[s][1]);
        // acc[0], acc[1]: query row g, tokens 2*t4, 2*t4+1; acc[2], acc[3]: query row g+8
        const float f0 = __int_as_float(acc[0] + 0x4B400000) - 12582912.0f;
        const float f1 = __int_as_float(acc[1] + 0x4B400000) - 12582912.0f;
        const float f2 = __int_as_float(acc[2] + 0x4B400000) - 12582912.0f;
        const float f3 = __int_as_float(acc[3] + 0x4B400000) - 12582912.0f;
        const float x0 = live0 ? __fmul_rn(f0, k0) : -INFINITY;
        const float x1 = live1 ? __fmul_rn(f1, k1) : -INFINITY;
        const float x2 = live0 ? __fmul_rn(f2, k0) : -INFINITY;
        const float x3 = live1 ? __fmul_rn(f3, k1) : -INFINITY;
        rm[hd][0] = fmaxf(rm[hd][0], fmaxf(x0, x1));
        rm[hd][1] = fmaxf(rm[hd][1], fmaxf(x2, x3));
      }
    }
    // block maximum per (head, query): across the quad, then the query scale, then across heads
    float best[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int hd = 0; hd < G; ++hd)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float m = rm[hd][r];
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
        best[r] = fmaxf(best[r], __fmul_rn(m, qs[hd][r]));
      }
    if (t4 == 0) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float m = best[r];
        if (m == 0.0f) m = 0.0f;                      // -0 -> +0
        s_out[warp * 16 + g + 8 * r][(blk - blk0) & (PF_OUT_BLOCKS - 1)] = m;
      }
    }
    __syncthreads();                                  // stage buffer free for the next prefetch; s_out visible
    // flush every PF_OUT_BLOCKS blocks (and at the end): rows of consecutive block maxima
    const int done = blk - blk0 + 1;
    if ((done & (PF_OUT_BLOCKS - 1)) == 0 || blk + 1 == blk1) {
      const int nb = ((done - 1) & (PF_OUT_BLOCKS - 1)) + 1;      // valid columns in s_out
      const int jb = blk + 1 - nb;                                 // first block of the batch
      for (int e = tid; e < PF_QTILE * PF_OUT_BLOCKS; e += PF_THREADS) {
        const int r = e / PF_OUT_BLOCKS, c = e - r * PF_OUT_BLOCKS;
        const int qi = q0 + r;
        if (c < nb && qi < p.Tq) p.out[(((int64_t)b * p.Hkv + kvh) * p.Tq + qi) * p.nblk + jb + c] = s_out[r][c];
      }
      __syncthreads();
    }
  }
}

// Per-token int8 quantisation of a chunk of queries over the channels of their KV head:
// one warp per (b, head, token).
__global__ void __launch_bounds__(256) quantize_query_tokens_kernel(const __nv_bfloat16* q, int64_t q_sb, int64_t q_sh,
                                                                    int64_t q_st, const int32_t* channel_idx, int8_t* qcode,
                                                                    float* qscale, int B, int Hq, int Hkv, int Tq, int C) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= (int64_t)B * Hq * Tq) return;
  const int i = (int)(row % Tq);
  const int h = (int)((row / Tq) % Hq);
  const int b = (int)(row / ((int64_t)Tq * Hq));
  const int G = Hq / Hkv;
  const int32_t* ch = channel_idx + (int64_t)(h / G) * C;
  const __nv_bfloat16* src = q + (int64_t)b * q_sb + (int64_t)h * q_sh + (int64_t)i * q_st;
  float x[4];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane + 32 * j;
    x[j] = c < C ? __bfloat162float(src[ch[c]]) : 0.0f;
    amax = fmaxf(amax, fabsf(x[j]));
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float s = __fdiv_rn(fmaxf(amax, 5.9604644775390625e-08f /* 2^-24 */), 127.0f);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = lane + 32 * j;
    if (c < C) {
      float r = rintf(__fdiv_rn(x[j], s));
      r = fminf(fmaxf(r, -127.0f), 127.0f);
      qcode[row * C + c] = (int8_t)(int)r;
    }
  }
  if (lane == 0) qscale[row] = s;
}

// Top-k blocks of every row of block scores, ordered (score desc, block asc): one warp per row.
// The row sits in shared memory; lanes own the strided elements lane, lane+32, ...; each round the
// warp takes the best composite and only the lane that owned it rescans its elements.
constexpr int BT_WARPS = 4;
constexpr int BT_MAX_T = 4096;

__global__ void __launch_bounds__(BT_WARPS * 32) block_topk_kernel(const float* scores, int64_t row_stride, int64_t R,
                                                                   int T, int k, int32_t* out_idx, float* out_scores) {
  extern __shared__ float bt_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * BT_WARPS + warp;
  if (row >= R) return;
  float* s = bt_smem + (size_t)warp * T;
  const float* src = scores + row * row_stride;
  for (int j = lane; j < T; j += 32) s[j] = src[j];
  __syncwarp();
  auto local_best = [&]() {
    uint64_t best = 0;                                  // below every real composite
    for (int j = lane; j < T; j += 32) {
      const float v = s[j];
      if (!(v != v)) {                                  // NaN marks a taken element
        const uint64_t c = ((uint64_t)float_to_key(v) << 32) | (uint64_t)(0xFFFFFFFFu - (uint32_t)j);
        best = c > best ? c : best;
      }
    }
    return best;
  };
  uint64_t mine = local_best();
  const int kk = k < T ? k : T;
  for (int r = 0; r < kk; ++r) {
    uint64_t top = mine;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      const uint64_t o = __shfl_xor_sync(0xffffffffu, top, off);
      top = o > top ? o : top;
    }
    const uint32_t j = 0xFFFFFFFFu - (uint32_t)(top & 0xFFFFFFFFull);
    if (lane == 0) {
      out_idx[row * kk + r] = (int32_t)j;
      if (out_scores) out_scores[row * kk + r] = key_to_float((uint32_t)(top >> 32));
    }
    if (mine == top) {                                  // exactly one lane: composites are unique
      s[j] = __int_as_float(0x7fc00000);
      mine = local_best();
    }
  }
}

// The same selection for k <= 32 and rows of at most 32 * NPL elements, with the row in registers: one warp per
// row, lane l holds elements l, l + 32, ... as order-preserving keys. The k-th largest key is found by a
// bitwise binary search (32 steps of NPL compares and one warp sum), ties at that key are taken in index
// order, and the winners (one per lane) are put into (score desc, index asc) order by a warp bitonic sort.
template <int NPL>
__global__ void __launch_bounds__(BT_WARPS * 32) block_topk_reg_kernel(const float* scores, int64_t row_stride, int64_t R,
                                                                       int T, int k, int32_t* out_idx, float* out_scores) {
  __shared__ uint64_t s_win[BT_WARPS][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * BT_WARPS + warp;
  if (row >= R) return;
  const float* src = scores + row * row_stride;
  uint32_t key[NPL];
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const int e = j * 32 + lane;
    float v = e < T ? src[e] : 0.0f;
    key[j] = (e < T && v == v) ? float_to_key(v) : 0u;          // absent and NaN: below every real score
  }
  const int kk = k < T ? k : T;
  // largest K with #{key >= K} >= kk
  uint32_t K = 0;
#pragma unroll 1
  for (int bit = 31; bit >= 0; --bit) {
    const uint32_t cand = K | (1u << bit);
    int c = 0;
#pragma unroll
    for (int j = 0; j < NPL; ++j) c += key[j] >= cand ? 1 : 0;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) c += __shfl_xor_sync(0xffffffffu, c, off);
    if (c >= kk) K = cand;
  }
  // winners: every key above K, and the first (kk - that many) keys equal to K in index order
  int above = 0;
#pragma unroll
  for (int j = 0; j < NPL; ++j) above += key[j] > K ? 1 : 0;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) above += __shfl_xor_sync(0xffffffffu, above, off);
  int ties_left = kk - above;
  const uint32_t lt = (1u << lane) - 1u;
  int slot_base = 0;
#pragma unroll
  for (int j = 0; j < NPL; ++j) {
    const bool gt = key[j] > K;
    const bool eq = key[j] == K;
    const uint32_t meq = __ballot_sync(0xffffffffu, eq);
    const bool take_eq = eq && (int)__popc(meq & lt) < ties_left;
    ties_left -= min(ties_left, (int)__popc(meq));
    const bool take = gt || take_eq;
    const uint32_t mt = __ballot_sync(0xffffffffu, take);
    if (take) {
      const int slot = slot_base + (int)__popc(mt & lt);
      if (slot < 32) s_win[warp][slot] = ((uint64_t)key[j] << 32) | (uint64_t)(0xFFFFFFFFu - (uint32_t)(j * 32 + lane));
    }
    slot_base += (int)__popc(mt);
  }
  __syncwarp();
  uint64_t c = lane < kk ? s_win[warp][lane] : 0ull;
  // warp bitonic sort, descending
#pragma unroll
  for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const uint64_t o = __shfl_xor_sync(0xffffffffu, c, stride);
      const bool upper = (lane & stride) != 0;                   // this lane holds the higher index of the pair
      const bool desc = (lane & size) == 0;                      // the pair's block sorts descending
      const bool keep_max = (upper != desc);                     // lower index of a descending pair keeps the max
      c = keep_max ? (c > o ? c : o) : (c < o ? c : o);
    }
  }
  if (lane < kk) {
    out_idx[row * kk + lane] = (int32_t)(0xFFFFFFFFu - (uint32_t)(c & 0xFFFFFFFFull));
    if (out_scores) out_scores[row * kk + lane] = key_to_float((uint32_t)(c >> 32));
  }
}

template <int C, int G>
static int prefill_launch(const PrefillParams& p0, int device, cudaStream_t st) {
  PrefillParams p = p0;
  const int qtiles = ceil_div(p.Tq, PF_QTILE);
  // split the key blocks so that the grid fills the machine a few times over
  const int64_t base_ctas = (int64_t)qtiles * p.B * p.Hkv;
  int splits = (int)(((int64_t)sm_count(device) * 2 * 3 + base_ctas - 1) / base_ctas);
  if (splits < 1) splits = 1;
  int bpc = ceil_div(p.nblk, splits);
  bpc = ceil_div(bpc, PF_OUT_BLOCKS) * PF_OUT_BLOCKS;            // flush batches stay aligned
  splits = ceil_div(p.nblk, bpc);
  p.blocks_per_cta = bpc;
  dim3 grid(qtiles, splits, p.B * p.Hkv);
  score_prefill_kernel<C, G><<<grid, PF_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

template <int C>
static int prefill_dispatch_g(const PrefillParams& p, int device, cudaStream_t st) {
  switch (p.G) {
    case 1: return prefill_launch<C, 1>(p, device, st);
    case 2: return prefill_launch<C, 2>(p, device, st);
    case 4: return prefill_launch<C, 4>(p, device, st);
    case 8: return prefill_launch<C, 8>(p, device, st);
    default: return KVB_BAD_SHAPE;
  }
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_quantize_query_tokens(
    const void* query, int64_t q_sb, int64_t q_sh, int64_t q_st, const int32_t* channel_idx, int8_t* qcode,
    float* qscale, int B, int Hq, int Hkv, int Tq, int D, int C, int device, void* stream) {
  using namespace kvb;
  if (!query || !channel_idx || !qcode || !qscale) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Tq <= 0 || (Hq % Hkv) || C <= 0 || C > 128 || C > D) return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  const int64_t rows = (int64_t)B * Hq * Tq;
  quantize_query_tokens_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(query), q_sb, q_sh, q_st, channel_idx, qcode, qscale, B, Hq, Hkv, Tq, C);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

namespace kvb {

// engine: 0 = automatic, 1 = mma.sync int8 (score_prefill_kernel), 2 = tcgen05 kind::i8, 3 = tcgen05 kind::f16.
static int prefill_blocks_run(const int8_t* qcode, const float* qscale, const uint8_t* packed, int64_t packed_sb,
                              int64_t packed_sh, const float* scale, int64_t scale_sb, int64_t scale_sh, int B, int Hq,
                              int Hkv, int Tq, int Tk, int C, int block_size, float* block_scores, int engine,
                              int device, void* stream) {
  if (!qcode || !qscale || !packed || !scale || !block_scores) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Tq <= 0 || Tk <= 0 || (Hq % Hkv)) return KVB_BAD_SHAPE;
  if (block_size != PF_BLOCK) return KVB_BAD_SHAPE;
  if (C != 32 && C != 64 && C != 128) return KVB_BAD_SHAPE;
  if (engine < 0 || engine > 3) return KVB_BAD_ARG;
  if ((int64_t)B * Hkv > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(qcode, 8) || !aligned_to(packed, 16) || (packed_sb % 16) || (packed_sh % 16) ||
      !aligned_to(scale, 16) || (scale_sb % 4) || (scale_sh % 4))
    return KVB_BAD_ALIGN;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int G = Hq / Hkv;
  if (engine == 0) engine = 3;                      // tensor-memory path, fp16 encoding of the integer codes
  if (engine >= 2) {
    PrefillTcParams t;
    t.qcode = qcode; t.qscale = qscale;
    t.packed = packed; t.packed_sb = packed_sb; t.packed_sh = packed_sh;
    t.scale = scale; t.scale_sb = scale_sb; t.scale_sh = scale_sh;
    t.out = block_scores;
    t.B = B; t.Hq = Hq; t.Hkv = Hkv; t.Tq = Tq; t.Tk = Tk; t.nblk = ceil_div(Tk, PF_BLOCK);
    return prefill_tc_run(t, C, G, engine == 2 ? 0 : 1, device, st);
  }
  PrefillParams p;
  p.qcode = qcode; p.qscale = qscale;
  p.packed = packed; p.packed_sb = packed_sb; p.packed_sh = packed_sh;
  p.scale = scale; p.scale_sb = scale_sb; p.scale_sh = scale_sh;
  p.out = block_scores;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Tq = Tq; p.Tk = Tk; p.C = C; p.G = G;
  p.nblk = ceil_div(Tk, PF_BLOCK);
  p.blocks_per_cta = p.nblk;
  if (C == 32) return prefill_dispatch_g<32>(p, device, st);
  if (C == 64) return prefill_dispatch_g<64>(p, device, st);
  return prefill_dispatch_g<128>(p, device, st);
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_score_prefill_blocks(
    const int8_t* qcode, const float* qscale, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, int B, int Hq, int Hkv, int Tq, int Tk, int C,
    int block_size, float* block_scores, int device, void* stream) {
  return kvb::prefill_blocks_run(qcode, qscale, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, B, Hq, Hkv, Tq,
                                 Tk, C, block_size, block_scores, 0, device, stream);
}

extern "C" __attribute__((visibility("default"))) int kvb_score_prefill_blocks_engine(
    const int8_t* qcode, const float* qscale, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, int B, int Hq, int Hkv, int Tq, int Tk, int C,
    int block_size, float* block_scores, int engine, int device, void* stream) {
  return kvb::prefill_blocks_run(qcode, qscale, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, B, Hq, Hkv, Tq,
                                 Tk, C, block_size, block_scores, engine, device, stream);
}

extern "C" __attribute__((visibility("default"))) size_t kvb_prefill_operand_bytes(int B, int Hkv, int key_capacity,
                                                                                    int C, int engine) {
  if (B <= 0 || Hkv <= 0 || key_capacity <= 0 || (C != 32 && C != 64 && C != 128)) return 0;
  if (engine != 0 && engine != 2 && engine != 3) return 0;
  return (size_t)B * Hkv * kvb::ceil_div(key_capacity, kvb::TC_NTILE) * kvb::prefill_operand_tile_bytes(C, engine == 2 ? 0 : 1);
}

extern "C" __attribute__((visibility("default"))) int kvb_widen_keys(
    const uint8_t* packed, int64_t packed_sb, int64_t packed_sh, int B, int Hkv, int Tk, int key_capacity, int C,
    int engine, int first_token, void* operands, size_t operand_bytes, int device, void* stream) {
  using namespace kvb;
  if (!packed || !operands) return KVB_BAD_ARG;
  if (B <= 0 || Hkv <= 0 || Tk <= 0 || key_capacity < Tk || first_token < 0) return KVB_BAD_SHAPE;
  if (C != 32 && C != 64 && C != 128) return KVB_BAD_SHAPE;
  if (engine != 0 && engine != 2 && engine != 3) return KVB_BAD_ARG;
  if ((int64_t)B * Hkv > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(packed, 16) || (packed_sb % 16) || (packed_sh % 16) || !aligned_to(operands, 128)) return KVB_BAD_ALIGN;
  if (operand_bytes < kvb_prefill_operand_bytes(B, Hkv, key_capacity, C, engine)) return KVB_WORKSPACE_TOO_SMALL;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  return prefill_widen_run(packed, packed_sb, packed_sh, B, Hkv, Tk, C, engine == 2 ? 0 : 1,
                           ceil_div(key_capacity, TC_NTILE), first_token / TC_NTILE,
                           reinterpret_cast<uint8_t*>(operands), reinterpret_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int kvb_score_prefill_blocks_widened(
    const int8_t* qcode, const float* qscale, const void* operands, size_t operand_bytes, int key_capacity,
    const float* scale, int64_t scale_sb, int64_t scale_sh, int B, int Hq, int Hkv, int Tq, int Tk, int C,
    int block_size, float* block_scores, int engine, int device, void* stream) {
  using namespace kvb;
  if (!qcode || !qscale || !operands || !scale || !block_scores) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Tq <= 0 || Tk <= 0 || (Hq % Hkv) || key_capacity < Tk) return KVB_BAD_SHAPE;
  if (block_size != PF_BLOCK) return KVB_BAD_SHAPE;
  if (C != 32 && C != 64 && C != 128) return KVB_BAD_SHAPE;
  if (engine != 0 && engine != 2 && engine != 3) return KVB_BAD_ARG;
  if ((int64_t)B * Hkv > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(qcode, 8) || !aligned_to(operands, 128) || !aligned_to(scale, 16) || (scale_sb % 4) || (scale_sh % 4))
    return KVB_BAD_ALIGN;
  if (operand_bytes < kvb_prefill_operand_bytes(B, Hkv, key_capacity, C, engine)) return KVB_WORKSPACE_TOO_SMALL;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  PrefillTwParams pw;
  pw.base.qcode = qcode; pw.base.qscale = qscale;
  pw.base.packed = nullptr; pw.base.packed_sb = 0; pw.base.packed_sh = 0;
  pw.base.scale = scale; pw.base.scale_sb = scale_sb; pw.base.scale_sh = scale_sh;
  pw.base.out = block_scores;
  pw.base.B = B; pw.base.Hq = Hq; pw.base.Hkv = Hkv; pw.base.Tq = Tq; pw.base.Tk = Tk;
  pw.base.nblk = ceil_div(Tk, PF_BLOCK);
  pw.operands = reinterpret_cast<const uint8_t*>(operands);
  pw.cap_tiles = ceil_div(key_capacity, TC_NTILE);
  return prefill_tw_run(pw, C, Hq / Hkv, engine == 2 ? 0 : 1, device, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int kvb_block_topk(const float* block_scores, int64_t row_stride,
                                                                      int64_t R, int nblk, int k, int32_t* out_idx,
                                                                      float* out_scores, int device, void* stream) {
  using namespace kvb;
  if (!block_scores || !out_idx) return KVB_BAD_ARG;
  if (R <= 0 || nblk <= 0 || k <= 0 || nblk > BT_MAX_T || row_stride < nblk) return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (k <= 32 && nblk <= 2048) {
    const unsigned grid = (unsigned)((R + BT_WARPS - 1) / BT_WARPS);
    if (nblk <= 512) block_topk_reg_kernel<16><<<grid, BT_WARPS * 32, 0, st>>>(block_scores, row_stride, R, nblk, k, out_idx, out_scores);
    else if (nblk <= 1024) block_topk_reg_kernel<32><<<grid, BT_WARPS * 32, 0, st>>>(block_scores, row_stride, R, nblk, k, out_idx, out_scores);
    else block_topk_reg_kernel<64><<<grid, BT_WARPS * 32, 0, st>>>(block_scores, row_stride, R, nblk, k, out_idx, out_scores);
    KVB_CHECK_CUDA(cudaGetLastError());
    return KVB_OK;
  }
  const size_t smem = sizeof(float) * (size_t)BT_WARPS * nblk;
  static std::atomic<bool> attr_done[KVB_MAX_DEVICES];
  { const int arc = ensure_dynamic_smem(block_topk_kernel, attr_done, device, (size_t)(sizeof(float) * BT_WARPS * BT_MAX_T)); if (arc != KVB_OK) return arc; }
  block_topk_kernel<<<(unsigned)((R + BT_WARPS - 1) / BT_WARPS), BT_WARPS * 32, smem,
                      reinterpret_cast<cudaStream_t>(stream)>>>(block_scores, row_stride, R, nblk, k, out_idx, out_scores);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}
