// Stage 1: gather C channels of each bf16 K row, per-token symmetric absmax scale, int4 codes,
// two codes per byte. Reads the 2*D-byte K rows with 128-bit asynchronous copies into a per-token ring in
// shared memory; four lanes share a token.
#include "common.cuh"

namespace kvb {

constexpr int QZ_THREADS = 256;            // 8 warps; four lanes per token => 64 tokens per pass
constexpr int QZ_LPT = 4;                  // lanes per token
constexpr int QZ_TOKENS_PER_PASS = QZ_THREADS / QZ_LPT;
constexpr int QZ_MAX_D = 256;
constexpr int QZ_STAGES = 3;               // ring stages of one token row per token slot
constexpr int QZ_PAD = 8;                  // elements between rows in shared memory beyond D: neighbouring token slots
                                           // then start four banks apart, so the teams of a warp, which read the same
                                           // channel of different rows, do not collide
constexpr int QZ_MAX_C = 128;

struct QuantizeParams {
  const __nv_bfloat16* key;
  int64_t key_sb, key_sh, key_st;
  const int32_t* channel_idx;
  uint8_t* packed;
  int64_t packed_sb, packed_sh;
  float* scale;
  int64_t scale_sb, scale_sh;
  int T, D, C;
  int64_t t_dst;
  int wide_store;   // rows and strides allow one VPL/2-byte store per lane
};

__device__ __forceinline__ int quantize_code(float x, float s) {
  // IEEE division, round half to even, clamp to the symmetric int4 range.
  float r = rintf(__fdiv_rn(x, s));
  r = fminf(fmaxf(r, -7.0f), 7.0f);
  return (int)r;
}

// ---- small PTX helpers of the quantizer -----------------------------------------------------------
__device__ __forceinline__ float qz_lds_bf16(uint32_t addr) {           // bf16 at a shared-memory byte address -> fp32
  uint16_t h;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(addr));
  return __uint_as_float((uint32_t)h << 16);
}
__device__ __forceinline__ uint64_t qz_pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void qz_unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t qz_mul2(uint64_t a, uint64_t b) {   // two rounded fp32 products
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t qz_add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t qz_fma2(uint64_t a, uint64_t b, uint64_t c) {   // two fused multiply-adds
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t qz_sub2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// amax / 7 correctly rounded without the division routine: q = amax * fl(1/7), one residual step with two
// fused multiply-adds (the classic division by a constant; exact for every bf16 magnitude, which a test checks
// exhaustively against the IEEE quotient).
__device__ __forceinline__ float qz_div7(float a) {
  const float c = 0.14285714924335479736328125f;                 // fl(1/7)
  const float q = a * c;
  const float r = fmaf(-7.0f, q, a);
  return fmaf(r, c, q);
}

// VPL = values (channels) per lane: 8 (C <= 32), 16 (C <= 64), 32 (C <= 128); a lane stores VPL / 2 bytes.
// FULL: C == 4 * VPL, every lane value is a real channel.
//
// Which entries of the channel list a lane reads: entry e belongs to lane e % 4 of the token's team. The
// list is ascending, so neighbouring entries are neighbouring channels (about two apart when half of the
// channels are chosen): the four lanes of a team then read four neighbouring 32-bit words of the staged row,
// and the eight teams of a warp, whose rows start four banks apart, cover all 32 banks — the gather runs
// without bank conflicts for the typical list, where a blocked assignment (lane = e / VPL) put lanes 0 and 2,
// and teams r and r + 4, on the same banks. The price is that the codes of one output byte now sit in two
// lanes; they are brought together by a 4 x 4 exchange inside the team (below).
//
// The codes are formed without the division routine, exactly: with y = RN(1 / s) (the correctly rounded
// reciprocal, computed once per token), q = RN(x y), the exact residual r = x - s q (one fused multiply-add)
// and q' = RN(q + r y), q' is the correctly rounded quotient x / s (Markstein's theorem; it needs y
// correctly rounded and no underflow, and tokens whose scale is outside [2^-100, 2^100] take the plain IEEE
// division instead). rint(q') + 8 then comes from adding 1.5 * 2^23 + 8 and taking 1.5 * 2^23 off again —
// the addition rounds half to even exactly like rint, and |x / s| <= 7 needs no clamp. Exact ties at k + 0.5
// are COMMON for bf16 inputs (7 x / amax is a ratio of two 8-bit mantissas), which is why an approximate
// quotient with a recheck near the boundaries was slow: most warps had a lane in the recheck. Products, sums
// and fused multiply-adds run two at a time (f32x2). A test compares the codes of every (amax, x) pair of
// bf16 values against IEEE division.
//
// The exchange: lane l' stores the entries [VPL l', VPL l' + VPL); of those, lane l holds e = 4 i + l for
// VPL / 4 consecutive i, i.e. the nibbles 4 j + l (j = 0 .. VPL/4 - 1) of the destination's VPL / 8 words.
// Lane l therefore builds, per destination, words that hold its offset codes (1..15) already at their final
// bit positions 16 (j % 2) + 4 l of word j / 2 — two codes per word, placed by one exact fp32 multiply-add
// with the lane's constants 2^(4 l) and 2^(16 + 4 l) and one conversion — and the destination ORs the four
// contributions. Each lane orders its values by (destination XOR own lane), so that in exchange round r
// every lane sends its r-th group with one xor-shuffle per word; flipping bit 3 of every nibble at the end
// turns offset codes into two's complement.
template <int VPL, bool FULL>
__global__ void __launch_bounds__(QZ_THREADS) quantize_pack_kernel(QuantizeParams p) {
  extern __shared__ __align__(16) uint16_t qz_rows[];            // [QZ_STAGES][QZ_TOKENS_PER_PASS][D + QZ_PAD]
  constexpr int GPL = VPL / 4;   // codes per (source lane, destination lane)
  constexpr int NW = VPL / 8;    // packed words per lane
  const int tid = threadIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int slot = tid >> 2;     // token slot inside the CTA
  const int l = tid & 3;         // lane inside the token's team
  const int nb = p.C >> 1;       // packed bytes per token
  const int byte0 = l * (VPL / 2);
  // byte offsets, inside a staged row, of this lane's channels: value r * GPL + j is list entry
  // 4 * ((l ^ r) * GPL + j) + l, destined to lane l ^ r
  uint32_t choff[VPL];
  uint32_t live_mask = 0;        // (!FULL) values that are real channels
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int r = i / GPL, j = i - r * GPL;
    const int e = 4 * (((l ^ r) * GPL) + j) + l;
    const bool real = FULL || e < p.C;
    choff[i] = real ? 2u * (uint32_t)p.channel_idx[(int64_t)h * p.C + e] : 0u;
    live_mask |= (real ? 1u : 0u) << i;
  }
  const __nv_bfloat16* key_row0 = p.key + (int64_t)b * p.key_sb + (int64_t)h * p.key_sh;
  uint8_t* packed_row0 = p.packed + (int64_t)b * p.packed_sb + (int64_t)h * p.packed_sh + (int64_t)p.t_dst * nb + byte0;
  float* scale_row0 = p.scale + (int64_t)b * p.scale_sb + (int64_t)h * p.scale_sh + p.t_dst;
  const int vec_per_row = p.D >> 3;
  const uint32_t pitch_b = 2u * (uint32_t)(p.D + QZ_PAD);
  const uint32_t my_rows = smem_u32(qz_rows) + (uint32_t)slot * pitch_b;
  const uint32_t stage_b = (uint32_t)QZ_TOKENS_PER_PASS * pitch_b;

  const int step = (int)gridDim.x * QZ_TOKENS_PER_PASS;
  auto issue = [&](int t0, int stage) {
    const int t = t0 + slot;
    if (t < p.T) {
      const uint4* src = reinterpret_cast<const uint4*>(key_row0 + (int64_t)t * p.key_st);
      const uint32_t dst = my_rows + (uint32_t)stage * stage_b;
      for (int j = l; j < vec_per_row; j += QZ_LPT)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * (uint32_t)j), "l"(src + j) : "memory");
    }
    cp_async_commit();
  };
  const uint64_t magic2 = qz_pack2(12582920.0f, 12582920.0f);      // 1.5 * 2^23 + 8
  const uint64_t base2 = qz_pack2(12582912.0f, 12582912.0f);       // 1.5 * 2^23
  const float w_lo = (float)(1u << (4 * l));                         // the lane's nibble inside a 16-bit half
  const float w_hi = w_lo * 65536.0f;
  // All teams of a warp run the same number of iterations (full-mask shuffles below). T < 2^31.
  int t0 = (int)blockIdx.x * QZ_TOKENS_PER_PASS;
  issue(t0, 0);
  issue(t0 + step, 1);
  int stage = 0;
  for (; t0 < p.T; t0 += step, stage = stage == QZ_STAGES - 1 ? 0 : stage + 1) {
    issue(t0 + 2 * step, stage >= 1 ? stage - 1 : QZ_STAGES - 1);   // (an empty group past the end keeps the count regular)
    cp_async_wait<QZ_STAGES - 1>();
    __syncwarp();
    const int t = t0 + slot;
    const bool active = t < p.T;                                    // (an inactive slot computes on stale bytes and stores nothing)
    const uint32_t row = my_rows + (uint32_t)stage * stage_b;
    float x[VPL];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      x[i] = qz_lds_bf16(row + choff[i]);
      if (!FULL && !((live_mask >> i) & 1u)) x[i] = 0.0f;
      amax = fmaxf(amax, fabsf(x[i]));
    }
    if (!active) amax = 0.0f;                                       // stale bytes may hold NaN patterns: keep the shuffles clean
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float sc = qz_div7(fmaxf(amax, 5.9604644775390625e-08f /* 2^-24 */));
    const bool plain = !(sc > 7.8886090522101181e-31f && sc < 1.2676506002282294e30f);   // 2^-100 .. 2^100 (NaN: plain)
    const float rcp = __frcp_rn(sc);
    const uint64_t rcp2 = qz_pack2(rcp, rcp);
    const uint64_t nsc2 = qz_pack2(-sc, -sc);

    uint32_t grp[4][NW];                                            // grp[r]: this lane's contribution to lane l ^ r
    if (!plain) {
#pragma unroll
      for (int i = 0; i < VPL; i += 2) {
        const uint64_t x2 = qz_pack2(x[i], x[i + 1]);
        const uint64_t q2 = qz_mul2(x2, rcp2);
        const uint64_t r2 = qz_fma2(nsc2, q2, x2);                  // x - s q, exact
        const uint64_t y2 = qz_fma2(r2, rcp2, q2);                  // RN(x / s)
        const uint64_t c2 = qz_sub2(qz_add2(y2, magic2), base2);    // rint(x / s) + 8: the offset code, 1..15
        float c0, c1;
        qz_unpack2(c2, c0, c1);
        // values i, i + 1 are codes j, j + 1 (j even) of group r: nibbles 4 j + l and 4 (j + 1) + l of the destination
        grp[i / GPL][(i % GPL) >> 1] = __float2uint_rn(fmaf(c1, w_hi, c0 * w_lo));
      }
    } else {                                                        // scales near the ends of the fp32 range: IEEE division
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int w = 0; w < NW; ++w) grp[r][w] = 0;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const uint32_t u = (uint32_t)(quantize_code(x[i], sc) + 8);
        grp[i / GPL][(i % GPL) >> 1] |= u << (4 * l + 16 * (i & 1));
      }
    }
    uint32_t words[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      uint32_t v = grp[0][w];
      v |= __shfl_xor_sync(0xffffffffu, grp[1][w], 1);
      v |= __shfl_xor_sync(0xffffffffu, grp[2][w], 2);
      v |= __shfl_xor_sync(0xffffffffu, grp[3][w], 3);
      words[w] = v ^ 0x88888888u;
    }
    if (active) {
      uint8_t* dst = packed_row0 + (int64_t)t * nb;
      if (p.wide_store && byte0 + VPL / 2 <= nb) {
        if constexpr (VPL == 8) *reinterpret_cast<uint32_t*>(dst) = words[0];
        else if constexpr (VPL == 16) *reinterpret_cast<uint2*>(dst) = make_uint2(words[0], words[1]);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
      } else {
#pragma unroll
        for (int j = 0; j < VPL / 2; ++j)
          if (byte0 + j < nb) dst[j] = (uint8_t)(words[j >> 2] >> (8 * (j & 3)));
      }
      if (l == 0) scale_row0[t] = sc;
    }
    __syncwarp();
  }
  cp_async_wait<0>();
}

template <int VPL, bool FULL>
static int quantize_launch_t(const QuantizeParams& p, dim3 grid, size_t smem, size_t smem_max, int device, cudaStream_t st) {
  static std::atomic<bool> attr[KVB_MAX_DEVICES];
  const int arc = ensure_dynamic_smem(quantize_pack_kernel<VPL, FULL>, attr, device, smem_max);
  if (arc != KVB_OK) return arc;
  quantize_pack_kernel<VPL, FULL><<<grid, QZ_THREADS, smem, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

static int quantize_launch(const void* key, int64_t key_sb, int64_t key_sh, int64_t key_st,
                           const int32_t* channel_idx, uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                           float* scale, int64_t scale_sb, int64_t scale_sh, int B, int Hkv, int T, int D, int C,
                           int64_t t_dst, int device, void* stream) {
  if (!key || !channel_idx || !packed || !scale) return KVB_BAD_ARG;
  if (B <= 0 || Hkv <= 0 || T < 0 || D <= 0 || D > QZ_MAX_D || (D % 8) != 0) return KVB_BAD_SHAPE;
  if (C <= 0 || C > QZ_MAX_C || (C & 1) || C > D || t_dst < 0) return KVB_BAD_SHAPE;
  if (Hkv > 65535 || B > 65535 || (int64_t)T > 0x7fffffffLL - (1 << 22)) return KVB_BAD_SHAPE;
  if (!aligned_to(key, 16) || (key_sb % 8) || (key_sh % 8) || (key_st % 8)) return KVB_BAD_ALIGN;
  if (!aligned_to(scale, 4)) return KVB_BAD_ALIGN;
  // One VPL/2-byte packed store per lane is used when every token row starts on such a boundary.
  const int nb = C / 2;
  const int vpl = (C <= 32) ? 8 : (C <= 64 ? 16 : 32);
  const int bpl = vpl / 2;
  const int wide = (nb % bpl) == 0 && aligned_to(packed, bpl) && (packed_sb % bpl) == 0 && (packed_sh % bpl) == 0;
  if (T == 0) return KVB_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;

  QuantizeParams p;
  p.key = reinterpret_cast<const __nv_bfloat16*>(key);
  p.key_sb = key_sb; p.key_sh = key_sh; p.key_st = key_st;
  p.channel_idx = channel_idx;
  p.packed = packed; p.packed_sb = packed_sb; p.packed_sh = packed_sh;
  p.scale = scale; p.scale_sb = scale_sb; p.scale_sh = scale_sh;
  p.T = T; p.D = D; p.C = C; p.t_dst = t_dst; p.wide_store = wide;

  const int passes = ceil_div(T, QZ_TOKENS_PER_PASS);
  // Enough CTAs to fill the machine several times over, each looping over a few passes.
  int64_t want = (int64_t)sm_count(device) * 8 * 4;
  int per_row = (int)((want + (int64_t)B * Hkv - 1) / ((int64_t)B * Hkv));
  if (per_row < 1) per_row = 1;
  int gx = passes < per_row ? passes : per_row;
  dim3 grid(gx, Hkv, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(uint16_t) * (size_t)QZ_TOKENS_PER_PASS * QZ_STAGES * (D + QZ_PAD);      // 51 KiB at D = 128
  const size_t smem_max = sizeof(uint16_t) * (size_t)QZ_TOKENS_PER_PASS * QZ_STAGES * (QZ_MAX_D + QZ_PAD);
  const bool full = C == 4 * vpl;
  if (vpl == 8) return full ? quantize_launch_t<8, true>(p, grid, smem, smem_max, device, st) : quantize_launch_t<8, false>(p, grid, smem, smem_max, device, st);
  if (vpl == 16) return full ? quantize_launch_t<16, true>(p, grid, smem, smem_max, device, st) : quantize_launch_t<16, false>(p, grid, smem, smem_max, device, st);
  return full ? quantize_launch_t<32, true>(p, grid, smem, smem_max, device, st) : quantize_launch_t<32, false>(p, grid, smem, smem_max, device, st);
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_quantize_pack(const void* key, int64_t key_sb, int64_t key_sh, int64_t key_st,
                                 const int32_t* channel_idx, uint8_t* packed, int64_t packed_sb,
                                 int64_t packed_sh, float* scale, int64_t scale_sb, int64_t scale_sh, int B,
                                 int Hkv, int T, int D, int C, int64_t t_dst, int device, void* stream) {
  return kvb::quantize_launch(key, key_sb, key_sh, key_st, channel_idx, packed, packed_sb, packed_sh, scale,
                              scale_sb, scale_sh, B, Hkv, T, D, C, t_dst, device, stream);
}

extern "C" __attribute__((visibility("default"))) int kvb_quantize_append(const void* key_row, int64_t key_sb, int64_t key_sh,
                                   const int32_t* channel_idx, uint8_t* packed, int64_t packed_sb,
                                   int64_t packed_sh, float* scale, int64_t scale_sb, int64_t scale_sh, int B,
                                   int Hkv, int D, int C, int64_t t_dst, int device, void* stream) {
  return kvb::quantize_launch(key_row, key_sb, key_sh, /*key_st=*/(int64_t)D, channel_idx, packed, packed_sb,
                              packed_sh, scale, scale_sb, scale_sh, B, Hkv, /*T=*/1, D, C, t_dst, device, stream);
}
