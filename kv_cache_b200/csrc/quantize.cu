// Stage 1: gather C channels of each bf16 K row, per-token symmetric absmax scale, int4 codes,
// two codes per byte. HBM-bound on reading the 2*D-byte K rows (one 128-bit load per lane).
#include "common.cuh"

namespace kvb {

constexpr int QZ_THREADS = 256;            // 8 warps, one half-warp per token => 16 tokens per pass
constexpr int QZ_TOKENS_PER_PASS = QZ_THREADS / 16;
constexpr int QZ_MAX_D = 256;
constexpr int QZ_UNROLL = 4;               // tokens per half-warp per iteration, all their rows in flight at once
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
  int wide_store;   // rows and strides allow BPL-byte stores
};

__device__ __forceinline__ int quantize_code(float x, float s) {
  // IEEE division, round half to even, clamp to the symmetric int4 range.
  float r = rintf(__fdiv_rn(x, s));
  r = fminf(fmaxf(r, -7.0f), 7.0f);
  return (int)r;
}

// BPL = packed bytes handled by one of the 16 lanes of a token: 1 (C <= 32), 2 (C <= 64), 4 (C <= 128).
template <int BPL>
__global__ void __launch_bounds__(QZ_THREADS) quantize_pack_kernel(QuantizeParams p) {
  __shared__ int s_ch[QZ_MAX_C];
  __shared__ __align__(16) uint16_t s_rows[QZ_TOKENS_PER_PASS][QZ_UNROLL][QZ_MAX_D];

  const int tid = threadIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  for (int i = tid; i < p.C; i += QZ_THREADS) s_ch[i] = p.channel_idx[(int64_t)h * p.C + i];
  __syncthreads();

  const int hw = tid >> 4;       // half-warp index inside the CTA = token slot
  const int l = tid & 15;        // lane inside the half-warp
  const int nb = p.C >> 1;       // packed bytes per token
  const int byte0 = l * BPL;
  const __nv_bfloat16* key_row0 = p.key + (int64_t)b * p.key_sb + (int64_t)h * p.key_sh;
  uint8_t* packed_row0 = p.packed + (int64_t)b * p.packed_sb + (int64_t)h * p.packed_sh;
  float* scale_row0 = p.scale + (int64_t)b * p.scale_sb + (int64_t)h * p.scale_sh;
  const int vec_per_row = p.D >> 3;

  // Both half-warps of a warp run the same number of iterations (full-mask shuffles below). A half-warp
  // takes QZ_UNROLL tokens per iteration and copies all their rows to shared memory asynchronously before it
  // touches the first one: several 16-byte requests per lane are in flight without costing registers.
  constexpr int U = QZ_UNROLL;
  for (int64_t t0 = (int64_t)blockIdx.x * QZ_TOKENS_PER_PASS * U; t0 < p.T;
       t0 += (int64_t)gridDim.x * QZ_TOKENS_PER_PASS * U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t t = t0 + (int64_t)u * QZ_TOKENS_PER_PASS + hw;
      if (t < p.T) {
        const uint4* src = reinterpret_cast<const uint4*>(key_row0 + t * p.key_st);
        for (int j = l; j < vec_per_row; j += 16) cp_async_16(reinterpret_cast<uint4*>(s_rows[hw][u]) + j, src + j);
      }
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t t = t0 + (int64_t)u * QZ_TOKENS_PER_PASS + hw;
      const bool active = t < p.T;
      const uint16_t* row = s_rows[hw][u];
      float x[2 * BPL];
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 2 * BPL; ++i) {
        const int c = 2 * byte0 + i;
        x[i] = (active && c < p.C) ? bf16_bits_to_float(row[s_ch[c]]) : 0.0f;
        amax = fmaxf(amax, fabsf(x[i]));
      }
#pragma unroll
      for (int off = 8; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
      const float sc = __fdiv_rn(fmaxf(amax, 5.9604644775390625e-08f /* 2^-24 */), 7.0f);

      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < BPL; ++j) {
        const int lo = quantize_code(x[2 * j], sc);
        const int hi = quantize_code(x[2 * j + 1], sc);
        word |= (uint32_t)((lo & 0xF) | ((hi & 0xF) << 4)) << (8 * j);
      }
      if (active) {
        uint8_t* dst = packed_row0 + (p.t_dst + t) * nb + byte0;
        if (BPL > 1 && p.wide_store && byte0 + BPL <= nb) {
          if (BPL == 2) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)word;
          else *reinterpret_cast<uint32_t*>(dst) = word;
        } else {
#pragma unroll
          for (int j = 0; j < BPL; ++j)
            if (byte0 + j < nb) dst[j] = (uint8_t)(word >> (8 * j));
        }
        if (l == 0) scale_row0[p.t_dst + t] = sc;
      }
    }
    __syncwarp();
  }
}

static int quantize_launch(const void* key, int64_t key_sb, int64_t key_sh, int64_t key_st,
                           const int32_t* channel_idx, uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
                           float* scale, int64_t scale_sb, int64_t scale_sh, int B, int Hkv, int T, int D, int C,
                           int64_t t_dst, int device, void* stream) {
  if (!key || !channel_idx || !packed || !scale) return KVB_BAD_ARG;
  if (B <= 0 || Hkv <= 0 || T < 0 || D <= 0 || D > QZ_MAX_D || (D % 8) != 0) return KVB_BAD_SHAPE;
  if (C <= 0 || C > QZ_MAX_C || (C & 1) || C > D || t_dst < 0) return KVB_BAD_SHAPE;
  if (Hkv > 65535 || B > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(key, 16) || (key_sb % 8) || (key_sh % 8) || (key_st % 8)) return KVB_BAD_ALIGN;
  if (!aligned_to(scale, 4)) return KVB_BAD_ALIGN;
  // 2-/4-byte packed stores are used when every token row starts on such a boundary.
  const int nb = C / 2;
  const int bpl = (C <= 32) ? 1 : (C <= 64 ? 2 : 4);
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

  const int passes = ceil_div(T, QZ_TOKENS_PER_PASS * QZ_UNROLL);
  // Enough CTAs to fill the machine several times over, each looping over a few passes.
  int64_t want = (int64_t)sm_count(device) * 8 * 4;
  int per_row = (int)((want + (int64_t)B * Hkv - 1) / ((int64_t)B * Hkv));
  if (per_row < 1) per_row = 1;
  int gx = passes < per_row ? passes : per_row;
  dim3 grid(gx, Hkv, B);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (C <= 32) quantize_pack_kernel<1><<<grid, QZ_THREADS, 0, st>>>(p);
  else if (C <= 64) quantize_pack_kernel<2><<<grid, QZ_THREADS, 0, st>>>(p);
  else quantize_pack_kernel<4><<<grid, QZ_THREADS, 0, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
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
