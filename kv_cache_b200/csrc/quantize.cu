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

// VPL = values (channels) per lane: 8 (C <= 32), 16 (C <= 64), 32 (C <= 128); a lane packs VPL / 2 bytes.
// FULL: C == 4 * VPL, every lane value is a real channel.
//
// The kernel is bound by instruction issue, not by memory, unless the per-code work is a handful of
// operations, so the codes are formed without a division: y = x * (1 / s) differs from the correctly rounded
// quotient by less than 2e-6 (|x / s| <= 7; the roundings of the product and of the reciprocal), hence
// rint(y) can differ from rint(x / s) only when y lies within that distance of a rounding boundary k + 0.5.
// rint(y) + 8 comes from adding 1.5 * 2^23 + 8 and taking it off again (|x / s| <= 7 needs no clamp); the
// offset codes 1..15 of four neighbours are summed as c0 + 16 c1 + 256 c2 + 4096 c3 in one exact fp32
// accumulator, converted once, and flipping bit 3 of every nibble turns offset codes into two's complement.
// A lane that meets a value within 1e-5 of a boundary (about one value in 10^5) redoes its codes with the
// IEEE division. Products, sums and differences run two at a time (f32x2).
template <int VPL, bool FULL>
__global__ void __launch_bounds__(QZ_THREADS) quantize_pack_kernel(QuantizeParams p) {
  extern __shared__ __align__(16) uint16_t qz_rows[];            // [QZ_STAGES][QZ_TOKENS_PER_PASS][D + QZ_PAD]
  const int tid = threadIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int slot = tid >> 2;     // token slot inside the CTA
  const int l = tid & 3;         // lane inside the token's team
  const int nb = p.C >> 1;       // packed bytes per token
  const int byte0 = l * (VPL / 2);
  // byte offsets, inside a staged row, of this lane's channels (VPL consecutive entries of the channel list)
  uint32_t choff[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = l * VPL + i;
    choff[i] = (FULL || c < p.C) ? 2u * (uint32_t)p.channel_idx[(int64_t)h * p.C + c] : 0u;
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
  const uint64_t eight2 = qz_pack2(8.0f, 8.0f);
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
      if (!FULL && l * VPL + i >= p.C) x[i] = 0.0f;
      amax = fmaxf(amax, fabsf(x[i]));
    }
    if (!active) amax = 0.0f;                                       // stale bytes may hold NaN patterns: keep the shuffles clean
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float sc = qz_div7(fmaxf(amax, 5.9604644775390625e-08f /* 2^-24 */));
    float rcp;
    asm("rcp.approx.f32 %0, %1;" : "=f"(rcp) : "f"(sc));
    const uint64_t rcp2 = qz_pack2(rcp, rcp);

    uint32_t words[VPL / 8];
    float emax = 0.0f;
#pragma unroll
    for (int w = 0; w < VPL / 8; ++w) {
      float acc[2] = {0.0f, 0.0f};
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const uint64_t y2 = qz_mul2(qz_pack2(x[8 * w + j], x[8 * w + j + 1]), rcp2);
        const uint64_t m2 = qz_add2(y2, magic2);                    // 1.5 * 2^23 + 8 + rint(y)
        const uint64_t c2 = qz_sub2(m2, base2);                     // rint(y) + 8: the offset code, 1..15
        const uint64_t e2 = qz_sub2(y2, qz_sub2(c2, eight2));       // y - rint(y)
        float c0, c1, e0, e1;
        qz_unpack2(c2, c0, c1);
        qz_unpack2(e2, e0, e1);
        emax = fmaxf(emax, fmaxf(fabsf(e0), fabsf(e1)));
        const float sh = (j & 2) ? 256.0f : 1.0f;                   // nibble position inside the 16-bit half
        acc[j >> 2] = fmaf(c0, sh, acc[j >> 2]);
        acc[j >> 2] = fmaf(c1, 16.0f * sh, acc[j >> 2]);
      }
      words[w] = (((uint32_t)__float2int_rn(acc[0])) | ((uint32_t)__float2int_rn(acc[1]) << 16)) ^ 0x88888888u;
    }
    if (emax > 0.49999f) {                                          // rare: exact codes for this lane's values
#pragma unroll
      for (int w = 0; w < VPL / 8; ++w) {
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) word |= (uint32_t)(quantize_code(x[8 * w + j], sc) & 0xF) << (4 * j);
        words[w] = word;
      }
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
