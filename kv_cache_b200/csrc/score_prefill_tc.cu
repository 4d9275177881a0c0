// Chunked-prefill block scoring on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// Same result, bit for bit, as score_prefill_kernel (score_prefill.cu):
//   blk[b,g,i,j] = max over the G heads of KV head g and the 64 tokens of key block j of
//                  fl(fl(float(acc) * kscale[t]) * qscale[h,i]),  acc = sum_c qcode * kcode  (exact)
//
// One CTA owns QT tiles of 128 accumulator rows (a tile = 128/G queries x the G heads of one KV head)
// and walks the whole key range in tiles of 128 tokens (two blocks):
//   * 4 producer warps read the packed int4 codes, widen them and store them as the K-major,
//     un-swizzled core-matrix layout the tensor core reads from shared memory (4-stage ring);
//   * 1 thread issues tcgen05.mma (M=128, N=128) into a double-buffered accumulator in tensor memory
//     and signals completion with tcgen05.commit -> mbarrier;
//   * 16 epilogue warps, four per TMEM lane quadrant: one per (accumulator tile, accumulator stage).
//     The warps of a stage drain it while the tensor core fills the other one. Each warp pulls its 128
//     columns with tcgen05.ld in 16-column chunks, the next chunk in flight while the current one is
//     scaled (packed fp32 multiply) and reduced (3-input maximum); the G heads of a query sit in
//     neighbouring rows = lanes, so the group maximum is a few shuffles, and the warp writes its two
//     block maxima per query straight to memory. Epilogue warps never synchronise with each other.
// The contraction is only C (32..128) deep, so the kernel is bound by the instructions of the
// per-element epilogue, not by the MMA; that is why most warps are epilogue warps.
//
// Two operand encodings give the same integers:
//   KIND 0: kind::i8  — int8 codes (K codes as 16*code, the exact 1/16 folded into the key scale),
//                       int32 accumulators, int -> float in the epilogue (2 extra instructions/element);
//   KIND 1: kind::f16 — the same integers as fp16 values with fp32 accumulation. |acc| <= 127*7*C
//                       < 2^17, every partial sum is an integer far below 2^24, so the fp32
//                       accumulator holds exactly the int32 result and the epilogue needs no conversion.
// Every wait on an mbarrier is bounded; a wait that gives up records KVB_TIMEOUT, and all roles leave
// their loops, meet at the final barrier and free the tensor memory.
#include "common.cuh"

#include <cuda_fp16.h>

namespace kvb {

constexpr int TC_EPI_WARPS = 16;                   // four per TMEM lane quadrant: one (tile, block) unit each
constexpr int TC_PROD_WARPS = 4;                   // 1, 2 or 4 (128 tokens per tile are split over them)
constexpr int TC_WARPS = TC_EPI_WARPS + TC_PROD_WARPS + 1;
constexpr int TC_THREADS = TC_WARPS * 32;
constexpr int TC_NTILE = 128;                      // key tokens per MMA tile (two 64-token blocks)
constexpr int TC_QT = 2;                           // 128-row accumulator tiles per CTA
constexpr int TC_ASTAGES = 2;                      // accumulator stages in tensor memory
constexpr int TC_TMEM_COLS = TC_ASTAGES * TC_QT * TC_NTILE;   // 512: all of it
constexpr int TC_CHW = 16;                         // accumulator columns per tensor-memory load
constexpr bool TC_DOUBLE_BUFFER = TC_CHW <= 32;    // two loads alternate in registers when they fit
constexpr bool TC_PACKED_MUL = true;               // fp32 accumulators: scale two columns per instruction (mul.rn.f32x2)
constexpr int TC_LBO = 128;                        // bytes between core matrices along K

struct PrefillTcParams {
  const int8_t* qcode;      // [B,Hq,Tq,C]
  const float* qscale;      // [B,Hq,Tq]
  const uint8_t* packed; int64_t packed_sb, packed_sh;
  const float* scale; int64_t scale_sb, scale_sh;
  float* out;               // [B,Hkv,Tq,nblk]
  int B, Hq, Hkv, Tq, Tk, nblk;
};

// ---- PTX wrappers --------------------------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_alloc(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (KIND == 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// TcLd<N>::ld reads N consecutive accumulator columns of this thread's TMEM lane; TcLd<N>::wait waits for
// every tcgen05.ld of this thread. The registers of the load are passed through the wait statement so that
// no use of them can be scheduled ahead of it.
template <int N>
struct TcLd;
template <>
struct TcLd<16> {
  static __device__ __forceinline__ void ld(uint32_t taddr, uint32_t* v) {
    asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {"
      "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15"
      "}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  }
  static __device__ __forceinline__ void wait(uint32_t* v) {
    asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
        "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
      :
      : "memory");
  }
};
template <>
struct TcLd<32> {
  static __device__ __forceinline__ void ld(uint32_t taddr, uint32_t* v) {
    asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {"
      "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
      "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31"
      "}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
        "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
        "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  }
  static __device__ __forceinline__ void wait(uint32_t* v) {
    asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
        "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
        "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]),
        "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]),
        "+r"(v[30]), "+r"(v[31])
      :
      : "memory");
  }
};
template <>
struct TcLd<64> {
  static __device__ __forceinline__ void ld(uint32_t taddr, uint32_t* v) {
    asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {"
      "%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
      "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, "
      "%42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, "
      "%62, %63"
      "}, [%64];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
        "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
        "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]),
        "=r"(v[37]), "=r"(v[38]), "=r"(v[39]), "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]),
        "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]), "=r"(v[50]),
        "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]),
        "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
      : "r"(taddr)
      : "memory");
  }
  static __device__ __forceinline__ void wait(uint32_t* v) {
    asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
        "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
        "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]),
        "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]),
        "+r"(v[30]), "+r"(v[31]), "+r"(v[32]), "+r"(v[33]), "+r"(v[34]), "+r"(v[35]), "+r"(v[36]),
        "+r"(v[37]), "+r"(v[38]), "+r"(v[39]), "+r"(v[40]), "+r"(v[41]), "+r"(v[42]), "+r"(v[43]),
        "+r"(v[44]), "+r"(v[45]), "+r"(v[46]), "+r"(v[47]), "+r"(v[48]), "+r"(v[49]), "+r"(v[50]),
        "+r"(v[51]), "+r"(v[52]), "+r"(v[53]), "+r"(v[54]), "+r"(v[55]), "+r"(v[56]), "+r"(v[57]),
        "+r"(v[58]), "+r"(v[59]), "+r"(v[60]), "+r"(v[61]), "+r"(v[62]), "+r"(v[63])
      :
      : "memory");
  }
};
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Shared-memory matrix descriptor: K-major, no swizzle. A core matrix is 8 rows x 16 bytes stored
// contiguously (128 bytes); `lbo` is the distance between core matrices that follow each other along
// K, `sbo` between groups of 8 rows. Bits [46,48) carry the descriptor version of this architecture.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) |
         (1ull << 46);
}
// Instruction descriptor: dense, no negation, both operands K-major, M x N accumulator tile.
//   KIND 0: int8 x int8 -> int32;  KIND 1: fp16 x fp16 -> fp32.
template <int KIND>
__host__ __device__ constexpr uint32_t tc_instr_desc(int M, int N) {
  const uint32_t cfmt = KIND == 0 ? 2u : 1u;      // S32 : F32
  const uint32_t abfmt = KIND == 0 ? 1u : 0u;     // signed 8-bit : F16
  return (cfmt << 4) | (abfmt << 7) | (abfmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

template <int C, int KIND>
struct TcCfg {
  static constexpr int ES = KIND == 0 ? 1 : 2;                 // operand element bytes
  static constexpr int ROWB = C * ES;                          // bytes of one operand row (all of K)
  static constexpr int CHUNKS = ROWB / 16;                     // 16-byte K chunks per row
  static constexpr int SBO = CHUNKS * TC_LBO;                  // bytes between 8-row groups
  static constexpr int KSTEPS = ROWB / 32;                     // MMAs per tile: 32 bytes of K each
  static constexpr int A_TILE = 128 * ROWB;
  static constexpr int B_STAGE = TC_NTILE * ROWB;
  static constexpr int BSTAGES = ROWB >= 256 ? 3 : 4;
  // shared memory carve-up
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + TC_QT * A_TILE;
  static constexpr int OFF_KS = OFF_B + BSTAGES * B_STAGE;                 // [epilogue warps][2][128] key scales, warp-private
  static constexpr int OFF_BAR = OFF_KS + TC_EPI_WARPS * 2 * TC_NTILE * 4;
  static constexpr int NBAR = 2 * BSTAGES + 2 * TC_ASTAGES + 1;
  static constexpr int OFF_MISC = OFF_BAR + NBAR * 8;                      // tmem base, dead flag
  static constexpr int BYTES = OFF_MISC + 16;
};

// The packed int4 codes of one token (W = C/8 words, two's complement nibbles) as one operand row in the
// core-matrix layout: 16-byte chunk c of the row goes to dst + c * TC_LBO. `dst` may be shared or global.
//   KIND 0: chunk c = words 2c, 2c+1 -> bytes 16*code in the order (even, odd, even, odd channels);
//   KIND 1: chunk c = word c -> 8 halves (4 even channels, 4 odd), built as 1024 + (code + 8) by byte
//           permutation and brought to the signed code by one exact half2 subtraction.
template <int C, int KIND>
__device__ __forceinline__ void tc_widen_token(const uint32_t* words, uint8_t* dst) {
  constexpr int W = C / 8;
  if constexpr (KIND == 0) {
#pragma unroll
    for (int c = 0; c < W / 2; ++c) {
      const uint32_t w0 = words[2 * c], w1 = words[2 * c + 1];
      *reinterpret_cast<uint4*>(dst + c * TC_LBO) =
          make_uint4((w0 << 4) & 0xF0F0F0F0u, w0 & 0xF0F0F0F0u, (w1 << 4) & 0xF0F0F0F0u, w1 & 0xF0F0F0F0u);
    }
  } else {
    const __half2 bias = __floats2half2_rn(1032.0f, 1032.0f);
#pragma unroll
    for (int c = 0; c < W; ++c) {
      const uint32_t x = words[c] ^ 0x88888888u;    // two's complement nibble -> code + 8
      const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu;
      uint32_t hh[4];
      hh[0] = __byte_perm(lo, 0x64u, 0x4140);       // halves 1024 + (code + 8) of bytes 0, 1
      hh[1] = __byte_perm(lo, 0x64u, 0x4342);
      hh[2] = __byte_perm(hi, 0x64u, 0x4140);
      hh[3] = __byte_perm(hi, 0x64u, 0x4342);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 r = __hsub2(*reinterpret_cast<const __half2*>(&hh[j]), bias);
        hh[j] = *reinterpret_cast<const uint32_t*>(&r);
      }
      *reinterpret_cast<uint4*>(dst + c * TC_LBO) = make_uint4(hh[0], hh[1], hh[2], hh[3]);
    }
  }
}

// Maximum of N accumulator columns against their key scales, continued from m: one rounded fp32 multiply per
// column (two per instruction for fp32 accumulators; the scales come from shared memory four at a time, the
// same address for every lane) and one 3-input maximum per two columns, on two independent chains. The accumulator registers of the
// tensor-memory load are used as they are; int32 accumulators are converted exactly (|acc| < 2^22) through
// the bits of 1.5 * 2^23 + acc.
template <int KIND, int N>
__device__ __forceinline__ float tc_chunk_max(const uint32_t* v, const float* ks, float m) {
  float ma = m, mb = -INFINITY;
#pragma unroll
  for (int c = 0; c < N; c += 4) {
    const float4 kk = *reinterpret_cast<const float4*>(ks + c);
    float x0, x1, x2, x3;
    if constexpr (KIND == 0) {
      x0 = __uint_as_float(v[c] + 0x4B400000u) - 12582912.0f;
      x1 = __uint_as_float(v[c + 1] + 0x4B400000u) - 12582912.0f;
      x2 = __uint_as_float(v[c + 2] + 0x4B400000u) - 12582912.0f;
      x3 = __uint_as_float(v[c + 3] + 0x4B400000u) - 12582912.0f;
    } else {
      x0 = __uint_as_float(v[c]); x1 = __uint_as_float(v[c + 1]);
      x2 = __uint_as_float(v[c + 2]); x3 = __uint_as_float(v[c + 3]);
    }
    float a0, a1, a2, a3;
    if constexpr (KIND == 1 && TC_PACKED_MUL) {
      // two rounded products per instruction; the accumulator registers of a tensor-memory load and the
      // halves of a 16-byte shared load are neighbouring registers, so the pairs need no moves
      uint64_t p01, p23, k01, k23, r01, r23;
      asm("mov.b64 %0, {%1, %2};" : "=l"(p01) : "f"(x0), "f"(x1));
      asm("mov.b64 %0, {%1, %2};" : "=l"(p23) : "f"(x2), "f"(x3));
      asm("mov.b64 %0, {%1, %2};" : "=l"(k01) : "f"(kk.x), "f"(kk.y));
      asm("mov.b64 %0, {%1, %2};" : "=l"(k23) : "f"(kk.z), "f"(kk.w));
      asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r01) : "l"(p01), "l"(k01));
      asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r23) : "l"(p23), "l"(k23));
      asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(r01));
      asm("mov.b64 {%0, %1}, %2;" : "=f"(a2), "=f"(a3) : "l"(r23));
    } else {
      a0 = __fmul_rn(x0, kk.x); a1 = __fmul_rn(x1, kk.y);
      a2 = __fmul_rn(x2, kk.z); a3 = __fmul_rn(x3, kk.w);
    }
    asm("max.f32 %0, %0, %1, %2;" : "+f"(ma) : "f"(a0), "f"(a1));
    asm("max.f32 %0, %0, %1, %2;" : "+f"(mb) : "f"(a2), "f"(a3));
  }
  return fmaxf(ma, mb);
}

// A tiles: row r of tile qt = query q0 + qt*QPT + r / G, head r % G (the heads of a query are neighbouring
// rows, hence neighbouring TMEM lanes of one epilogue warp); K order inside each group of 8 channels is
// (even channels, odd channels), the order in which the widened key words deliver them.
template <int C, int G, int KIND, class Cfg>
__device__ __forceinline__ void tc_fill_a_tiles(const PrefillTcParams& p, uint8_t* s_a, int b, int kvh, int q0, int tid,
                                                int nthreads) {
  constexpr int QPT = 128 / G;
  constexpr int W = C / 8;
  for (int item = tid; item < TC_QT * 128 * W; item += nthreads) {
    const int w = item % W;
    const int r = (item / W) % 128;
    const int qt = item / (W * 128);
    const int qi = r / G, hd = r - qi * G;
    const int q = q0 + qt * QPT + qi;
    uint32_t ev = 0, od = 0;
    if (q < p.Tq) {
      const int64_t rowoff = ((int64_t)b * p.Hq + kvh * G + hd) * p.Tq + q;
      const uint2 x = *reinterpret_cast<const uint2*>(p.qcode + rowoff * C + 8 * w);
      ev = __byte_perm(x.x, x.y, 0x6420);          // channels 8w + 0,2,4,6
      od = __byte_perm(x.x, x.y, 0x7531);          // channels 8w + 1,3,5,7
    }
    uint8_t* tile = s_a + qt * Cfg::A_TILE + (r >> 3) * Cfg::SBO + (r & 7) * 16;
    if constexpr (KIND == 0) {
      *reinterpret_cast<uint2*>(tile + (w >> 1) * TC_LBO + (w & 1) * 8) = make_uint2(ev, od);
    } else {
      uint32_t h[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t src = i == 0 ? ev : od;
        const __half2 lo = __floats2half2_rn((float)(int8_t)(src & 0xFF), (float)(int8_t)((src >> 8) & 0xFF));
        const __half2 hi = __floats2half2_rn((float)(int8_t)((src >> 16) & 0xFF), (float)(int8_t)(src >> 24));
        h[2 * i] = *reinterpret_cast<const uint32_t*>(&lo);
        h[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
      *reinterpret_cast<uint4*>(tile + w * TC_LBO) = make_uint4(h[0], h[1], h[2], h[3]);
    }
  }
}

// The MMA issuer (one thread). Its instruction stream is the serial part of the whole CTA, so it is kept
// short: descriptors differ from a base only in their address field (low word, no carry into the other
// fields below 256 KiB), the tile loop is unrolled over the operand ring and the two accumulator stages so
// that every index is a constant, and barrier addresses are plain integers.
template <int KIND, class Cfg>
__device__ __forceinline__ void tc_issue_tiles(uint8_t* s_a, uint8_t* s_b, uint64_t* b_full, uint64_t* b_empty,
                                               uint64_t* acc_full, uint64_t* acc_empty, uint64_t* all_done,
                                               volatile uint32_t* s_dead, uint32_t tmem_base, int ntiles) {
  constexpr int BSTAGES = Cfg::BSTAGES;
  {
    const uint32_t idesc = tc_instr_desc<KIND>(128, TC_NTILE);
    const uint64_t a_desc0 = tc_smem_desc(smem_u32(s_a), TC_LBO, Cfg::SBO);
    const uint64_t b_desc0 = tc_smem_desc(smem_u32(s_b), TC_LBO, Cfg::SBO);
    const uint32_t a_lo = (uint32_t)a_desc0, a_hi = (uint32_t)(a_desc0 >> 32);
    const uint32_t b_lo = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
    auto desc = [](uint32_t lo, uint32_t hi) -> uint64_t { return ((uint64_t)hi << 32) | lo; };
    constexpr int U = (BSTAGES % 2 == 0) ? BSTAGES : 2 * BSTAGES;      // tiles per unrolled round
    bool dead = false;
    uint32_t round = 0;                                               // i0 / U
    for (int i0 = 0; i0 < ntiles && !dead; i0 += U, ++round) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + u;
        if (i >= ntiles) break;
        const int s = u % BSTAGES, a = u & 1;                          // constants after unrolling (U is even and a multiple of BSTAGES)
        const uint32_t use_b = round * (U / BSTAGES) + (uint32_t)(u / BSTAGES);   // n-th use of operand stage s
        const uint32_t use_a = round * (U / 2) + (uint32_t)(u / 2);               // n-th use of accumulator stage a
        bool ok = mbar_wait_bounded(&b_full[s], use_b & 1u);
        ok = ok && mbar_wait_bounded(&acc_empty[a], (use_a & 1u) ^ 1u);
        if (!ok) { *s_dead = 1; dead = true; break; }
        tc_fence_after();
#pragma unroll
        for (int qt = 0; qt < TC_QT; ++qt) {
          const uint32_t d = tmem_base + (uint32_t)(a * TC_QT * TC_NTILE + qt * TC_NTILE);
#pragma unroll
          for (int k = 0; k < Cfg::KSTEPS; ++k) {
            const uint64_t ad = desc(a_lo + (uint32_t)((qt * Cfg::A_TILE + k * 2 * TC_LBO) >> 4), a_hi);
            const uint64_t bd = desc(b_lo + (uint32_t)((s * Cfg::B_STAGE + k * 2 * TC_LBO) >> 4), b_hi);
            tc_mma<KIND>(d, ad, bd, idesc, k > 0 ? 1u : 0u);
          }
        }
        tc_commit(&b_empty[s]);                     // the stage may be overwritten once these MMAs have read it
        tc_commit(&acc_full[a]);
      }
    }
    tc_commit(all_done);
    mbar_wait_bounded(all_done, 0);                 // nothing of this CTA is still in flight in the tensor core
  }
}

template <int C, int G, int KIND>
__global__ void __launch_bounds__(TC_THREADS, 1) score_prefill_tc_kernel(PrefillTcParams p) {
  using Cfg = TcCfg<C, KIND>;
  constexpr int QPT = 128 / G;                      // queries per accumulator tile
  constexpr int QCTA = TC_QT * QPT;                 // queries per CTA
  constexpr int W = C / 8;                          // packed words per token
  constexpr int BSTAGES = Cfg::BSTAGES;
  extern __shared__ __align__(1024) uint8_t tc_smem[];
  uint8_t* s_a = tc_smem + Cfg::OFF_A;
  uint8_t* s_b = tc_smem + Cfg::OFF_B;
  float* s_ks = reinterpret_cast<float*>(tc_smem + Cfg::OFF_KS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tc_smem + Cfg::OFF_BAR);
  uint64_t* b_full = bars;                          // [BSTAGES] producers -> MMA (128 arrivals)
  uint64_t* b_empty = bars + BSTAGES;               // [BSTAGES] MMA -> producers (commit)
  uint64_t* acc_full = bars + 2 * BSTAGES;          // [ASTAGES] MMA -> epilogue (commit)
  uint64_t* acc_empty = acc_full + TC_ASTAGES;      // [ASTAGES] the stage's epilogue warps -> MMA (256 arrivals)
  uint64_t* all_done = acc_empty + TC_ASTAGES;      // every MMA of the CTA has completed
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tc_smem + Cfg::OFF_MISC);
  volatile uint32_t* s_dead = s_tmem + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.Hkv, kvh = bh - b * p.Hkv;
  const int q0 = blockIdx.x * QCTA;
  const int ntiles = (p.Tk + TC_NTILE - 1) / TC_NTILE;

  if (tid == 0) {
    for (int s = 0; s < BSTAGES; ++s) { mbar_init(&b_full[s], TC_PROD_WARPS * 32); mbar_init(&b_empty[s], 1); }
    for (int a = 0; a < TC_ASTAGES; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], TC_EPI_WARPS / TC_ASTAGES * 32); }
    mbar_init(all_done, 1);
    *s_dead = 0;
    fence_mbar_init();
  }
  if (warp == TC_WARPS - 1) {                       // the MMA warp owns the tensor-memory allocation
    tc_alloc(s_tmem, TC_TMEM_COLS);
    tc_relinquish();
  }

  tc_fill_a_tiles<C, G, KIND, Cfg>(p, s_a, b, kvh, q0, tid, TC_THREADS);
  fence_proxy_async_smem();                         // the tensor core reads shared memory through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;

  const uint8_t* packed_row = p.packed + (int64_t)b * p.packed_sb + (int64_t)kvh * p.packed_sh;
  const float* scale_row = p.scale + (int64_t)b * p.scale_sb + (int64_t)kvh * p.scale_sh;

  if (warp < TC_EPI_WARPS) {
    // =============================== epilogue ===============================
    // warp -> TMEM lane quadrant (warp % 4, fixed by the hardware), accumulator tile qt and stage `par`:
    // the warp handles tiles par, par + 2, ... and reads all 128 columns (two blocks) of its tile qt.
    const int quad = warp & 3, qt = (warp >> 2) & 1, par = warp >> 3;
    const int row = quad * 32 + lane;               // accumulator row = TMEM lane
    const int qi = row / G, hd = row - qi * G;
    const int q = q0 + qt * QPT + qi;
    const float qs = q < p.Tq ? p.qscale[((int64_t)b * p.Hq + kvh * G + hd) * p.Tq + q] : 0.0f;
    float* out_row = p.out + (((int64_t)b * p.Hkv + kvh) * p.Tq + (q < p.Tq ? q : 0)) * p.nblk;
    const bool writer = hd == 0 && q < p.Tq;
    float* my_ks = s_ks + warp * 2 * TC_NTILE;      // [2][128], private to the warp
    // Key scales of a tile: lane l fetches tokens 4l .. 4l+3; dead tokens get NaN, which never wins a max.
    // They are fetched two of this warp's tiles ahead, so the memory latency is never waited for.
    auto load_ks = [&](int tile) -> float4 {
      const float nan = __int_as_float(0x7fc00000);
      float4 v = make_float4(nan, nan, nan, nan);
      const int64_t t = (int64_t)tile * TC_NTILE + 4 * lane;
      if (tile < ntiles) {
        if (t + 3 < p.Tk) {
          v = *reinterpret_cast<const float4*>(scale_row + t);
        } else {
          if (t < p.Tk) v.x = scale_row[t];
          if (t + 1 < p.Tk) v.y = scale_row[t + 1];
          if (t + 2 < p.Tk) v.z = scale_row[t + 2];
        }
        if constexpr (KIND == 0) { v.x *= 0.0625f; v.y *= 0.0625f; v.z *= 0.0625f; v.w *= 0.0625f; }
      }
      return v;
    };
    auto chunk_max = [&](const uint32_t* v, const float* ks, float m) -> float {
      return tc_chunk_max<KIND, TC_CHW>(v, ks, m);
    };
    constexpr int NCH = TC_NTILE / TC_CHW;          // chunks per tile
    constexpr int CPB = 64 / TC_CHW;                // chunks per 64-token block
    const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(par * TC_QT * TC_NTILE + qt * TC_NTILE);
    float4 k_cur = load_ks(par), k_next = load_ks(par + 2);
    int buf = 0;
    for (int i = par; i < ntiles; i += TC_ASTAGES, buf ^= 1) {
      float* ksb = my_ks + buf * TC_NTILE;
      *reinterpret_cast<float4*>(ksb + 4 * lane) = k_cur;
      k_cur = k_next;
      k_next = load_ks(i + 2 * TC_ASTAGES);
      __syncwarp();
      if (*s_dead) break;
      if (!mbar_wait_bounded(&acc_full[par], (uint32_t)(i >> 1) & 1u)) { *s_dead = 1; break; }
      tc_fence_after();
      float m = -INFINITY, m0 = 0.0f;
      if constexpr (TC_DOUBLE_BUFFER) {
        uint32_t va[TC_CHW], vb[TC_CHW];
        TcLd<TC_CHW>::ld(tbase, va);
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          uint32_t* cur = (ch & 1) ? vb : va;
          uint32_t* nxt = (ch & 1) ? va : vb;
          TcLd<TC_CHW>::wait(cur);
          if (ch + 1 < NCH) {
            TcLd<TC_CHW>::ld(tbase + (uint32_t)((ch + 1) * TC_CHW), nxt);
          } else {                                  // the whole tile is in registers: the stage may be refilled
            tc_fence_before();
            mbar_arrive(&acc_empty[par]);
          }
          m = chunk_max(cur, ksb + ch * TC_CHW, m);
          if (ch == CPB - 1) { m0 = m; m = -INFINITY; }
        }
      } else {
        // one wide load at a time: the other epilogue warps of the scheduler cover its latency
        uint32_t v[TC_CHW];
#pragma unroll
        for (int ch = 0; ch < NCH; ++ch) {
          TcLd<TC_CHW>::ld(tbase + (uint32_t)(ch * TC_CHW), v);
          TcLd<TC_CHW>::wait(v);
          if (ch + 1 == NCH) {
            tc_fence_before();
            mbar_arrive(&acc_empty[par]);
          }
          m = chunk_max(v, ksb + ch * TC_CHW, m);
          if (ch == CPB - 1) { m0 = m; m = -INFINITY; }
        }
      }
      // x -> fl(x * qscale) is monotone for qscale > 0: scale the block maxima only; then the group maximum
      // over the G heads of the query, which are G neighbouring lanes
      float r0 = __fmul_rn(m0, qs), r1 = __fmul_rn(m, qs);
#pragma unroll
      for (int off = 1; off < G; off <<= 1) {
        r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, off));
        r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, off));
      }
      if (writer) {
        if (r0 == 0.0f) r0 = 0.0f;                  // -0 -> +0
        if (r1 == 0.0f) r1 = 0.0f;
        const int blk = 2 * i;
        if (blk + 1 < p.nblk && (p.nblk & 1) == 0) {
          *reinterpret_cast<float2*>(out_row + blk) = make_float2(r0, r1);
        } else {
          out_row[blk] = r0;
          if (blk + 1 < p.nblk) out_row[blk + 1] = r1;
        }
      }
    }
  } else if (warp < TC_EPI_WARPS + TC_PROD_WARPS) {
    // =============================== producers ===============================
    // thread pt widens tokens pt, pt + 32 * TC_PROD_WARPS, ... of every tile
    constexpr int PTHREADS = TC_PROD_WARPS * 32;
    constexpr int TPT = TC_NTILE / PTHREADS;        // tokens per producer thread
    constexpr int PW = W * TPT;
    const int pt = tid - TC_EPI_WARPS * 32;
    uint32_t bufA[PW], bufB[PW], bufC[PW], bufD[PW];
    auto load_tile = [&](int tile, uint32_t (&buf)[PW]) {
#pragma unroll
      for (int h = 0; h < TPT; ++h) {
        const int64_t t = (int64_t)tile * TC_NTILE + pt + h * PTHREADS;
        if (tile < ntiles && t < p.Tk) {
          const uint4* src = reinterpret_cast<const uint4*>(packed_row + t * (C / 2));
#pragma unroll
          for (int x = 0; x < W / 4; ++x) {
            const uint4 u = __ldg(src + x);
            buf[h * W + 4 * x] = u.x; buf[h * W + 4 * x + 1] = u.y;
            buf[h * W + 4 * x + 2] = u.z; buf[h * W + 4 * x + 3] = u.w;
          }
        } else {
#pragma unroll
          for (int x = 0; x < W; ++x) buf[h * W + x] = 0;
        }
      }
    };
    bool dead = false;
    auto store_tile = [&](int i, const uint32_t (&buf)[PW]) {
      const int s = i % BSTAGES;
      if (!dead) {
        const bool ok = mbar_wait_bounded(&b_empty[s], ((uint32_t)(i / BSTAGES) & 1u) ^ 1u);
        if (!ok) { *s_dead = 1; dead = true; }
      }
      if (*s_dead) dead = true;
      if (dead) return;
#pragma unroll
      for (int h = 0; h < TPT; ++h) {
        const int tok = pt + h * PTHREADS;
        uint8_t* dst = s_b + s * Cfg::B_STAGE + (tok >> 3) * Cfg::SBO + (tok & 7) * 16;
        tc_widen_token<C, KIND>(buf + h * W, dst);
      }
      fence_proxy_async_smem();
      mbar_arrive(&b_full[s]);
    };
    // four tiles of packed codes are in flight in registers
    load_tile(0, bufA);
    load_tile(1, bufB);
    load_tile(2, bufC);
    load_tile(3, bufD);
    for (int i = 0; i < ntiles; i += 4) {
      store_tile(i, bufA);
      load_tile(i + 4, bufA);
      if (i + 1 < ntiles) { store_tile(i + 1, bufB); load_tile(i + 5, bufB); }
      if (i + 2 < ntiles) { store_tile(i + 2, bufC); load_tile(i + 6, bufC); }
      if (i + 3 < ntiles) { store_tile(i + 3, bufD); load_tile(i + 7, bufD); }
    }
  } else if (lane == 0) {
    // =============================== MMA issuer ===============================
    tc_issue_tiles<KIND, Cfg>(s_a, s_b, b_full, b_empty, acc_full, acc_empty, all_done, s_dead, tmem_base, ntiles);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == TC_WARPS - 1) {
    tc_fence_after();
    tc_dealloc(tmem_base, TC_TMEM_COLS);
  }
}

// ====================================================================================================
// Second form: the key operands are widened ONCE into global memory (prefill_widen_kernel), already in the
// core-matrix layout, one contiguous B_STAGE block per tile of 128 tokens, and every CTA fetches a tile with
// one bulk copy issued by one thread. The four conversion warps and their issue slots are gone (18 warps
// instead of 21), the registers they held go to the epilogue (32-column loads, two in flight), and the
// operand ring is as deep as shared memory allows. The 64 CTAs of one (batch, KV head) read the same
// operand stream at the same pace, so it comes from L2.
constexpr int TW_EPI_WARPS = 16;
constexpr int TW_WARPS = TW_EPI_WARPS + 2;        // + the bulk-copy thread's warp + the MMA warp
constexpr int TW_THREADS = TW_WARPS * 32;
constexpr int TW_CHW = 32;                        // accumulator columns per tensor-memory load (two loads alternate)

template <int C, int KIND>
struct TwCfg {
  using Base = TcCfg<C, KIND>;
  static constexpr int SBO = Base::SBO;
  static constexpr int KSTEPS = Base::KSTEPS;
  static constexpr int A_TILE = Base::A_TILE;
  static constexpr int B_STAGE = Base::B_STAGE;
  static constexpr int FIT = (200 * 1024 - TC_QT * A_TILE) / B_STAGE;
  static constexpr int BSTAGES = FIT >= 8 ? 8 : (FIT & ~1);                 // even, at most 8
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + TC_QT * A_TILE;
  static constexpr int OFF_KS = OFF_B + BSTAGES * B_STAGE;                  // [epilogue warps][2][128] key scales
  static constexpr int OFF_BAR = OFF_KS + TW_EPI_WARPS * 2 * TC_NTILE * 4;
  static constexpr int NBAR = 2 * BSTAGES + 2 * TC_ASTAGES + 1;
  static constexpr int OFF_MISC = OFF_BAR + NBAR * 8;
  static constexpr int BYTES = OFF_MISC + 16;
};

// operands: [B*Hkv][cap_tiles][B_STAGE]; tokens at or beyond Tk are zero rows. The tiles first_tile ..
// ceil(Tk/128)-1 are written (a grown cache re-widens only its last, partly filled tile and the new ones).
template <int C, int KIND>
__global__ void __launch_bounds__(TC_NTILE) prefill_widen_kernel(const uint8_t* __restrict__ packed, int64_t packed_sb,
                                                                 int64_t packed_sh, int Hkv, int Tk, int cap_tiles,
                                                                 int first_tile, uint8_t* __restrict__ operands) {
  using Cfg = TcCfg<C, KIND>;
  constexpr int W = C / 8;
  const int tile = first_tile + blockIdx.x, bh = blockIdx.y, pt = threadIdx.x;
  const int b = bh / Hkv, kvh = bh - b * Hkv;
  const int64_t t = (int64_t)tile * TC_NTILE + pt;
  uint32_t words[W];
  if (t < Tk) {
    const uint4* src = reinterpret_cast<const uint4*>(packed + (int64_t)b * packed_sb + (int64_t)kvh * packed_sh + t * (C / 2));
#pragma unroll
    for (int x = 0; x < W / 4; ++x) {
      const uint4 u = __ldg(src + x);
      words[4 * x] = u.x; words[4 * x + 1] = u.y; words[4 * x + 2] = u.z; words[4 * x + 3] = u.w;
    }
  } else {
#pragma unroll
    for (int x = 0; x < W; ++x) words[x] = 0;
  }
  uint8_t* dst = operands + ((int64_t)bh * cap_tiles + tile) * Cfg::B_STAGE + (pt >> 3) * Cfg::SBO + (pt & 7) * 16;
  tc_widen_token<C, KIND>(words, dst);
}

struct PrefillTwParams {
  PrefillTcParams base;       // packed is unused
  const uint8_t* operands;    // see prefill_widen_kernel
  int cap_tiles;
};

template <int C, int G, int KIND>
__global__ void __launch_bounds__(TW_THREADS, 1) score_prefill_tw_kernel(PrefillTwParams pw) {
  using Cfg = TwCfg<C, KIND>;
  const PrefillTcParams& p = pw.base;
  constexpr int QPT = 128 / G;
  constexpr int QCTA = TC_QT * QPT;
  constexpr int BSTAGES = Cfg::BSTAGES;
  extern __shared__ __align__(1024) uint8_t tc_smem[];
  uint8_t* s_a = tc_smem + Cfg::OFF_A;
  uint8_t* s_b = tc_smem + Cfg::OFF_B;
  float* s_ks = reinterpret_cast<float*>(tc_smem + Cfg::OFF_KS);
  uint64_t* bars = reinterpret_cast<uint64_t*>(tc_smem + Cfg::OFF_BAR);
  uint64_t* b_full = bars;                          // [BSTAGES] bulk copy landed (transaction bytes)
  uint64_t* b_empty = bars + BSTAGES;               // [BSTAGES] MMA -> copy thread (commit)
  uint64_t* acc_full = bars + 2 * BSTAGES;          // [ASTAGES] MMA -> epilogue (commit)
  uint64_t* acc_empty = acc_full + TC_ASTAGES;      // [ASTAGES] one arrival per epilogue warp of the stage
  uint64_t* all_done = acc_empty + TC_ASTAGES;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(tc_smem + Cfg::OFF_MISC);
  volatile uint32_t* s_dead = s_tmem + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.y;
  const int b = bh / p.Hkv, kvh = bh - b * p.Hkv;
  const int q0 = blockIdx.x * QCTA;
  const int ntiles = (p.Tk + TC_NTILE - 1) / TC_NTILE;

  if (tid == 0) {
    for (int s = 0; s < BSTAGES; ++s) { mbar_init(&b_full[s], 1); mbar_init(&b_empty[s], 1); }
    for (int a = 0; a < TC_ASTAGES; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], TW_EPI_WARPS / TC_ASTAGES); }
    mbar_init(all_done, 1);
    *s_dead = 0;
    fence_mbar_init();
  }
  if (warp == TW_WARPS - 1) {
    tc_alloc(s_tmem, TC_TMEM_COLS);
    tc_relinquish();
  }
  tc_fill_a_tiles<C, G, KIND, Cfg>(p, s_a, b, kvh, q0, tid, TW_THREADS);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *s_tmem;
  const float* scale_row = p.scale + (int64_t)b * p.scale_sb + (int64_t)kvh * p.scale_sh;

  if (warp < TW_EPI_WARPS) {
    // =============================== epilogue ===============================
    // warp -> TMEM lane quadrant (warp % 4, fixed by the hardware), row tile qt and accumulator stage `par`:
    // the warp handles tiles par, par + 2, ... and reads all 128 columns (two blocks) of its row tile, so
    // the per-visit costs (barrier, scale staging, group maximum, store) are paid once per 128 columns.
    const int quad = warp & 3, qt = (warp >> 2) & 1, par = warp >> 3;
    const int row = quad * 32 + lane;
    const int qi = row / G, hd = row - qi * G;
    const int q = q0 + qt * QPT + qi;
    // (int8 operands carry 16 * code: the exact factor 1/16 goes into the query scale, a power of two)
    const float qs = (q < p.Tq ? p.qscale[((int64_t)b * p.Hq + kvh * G + hd) * p.Tq + q] : 0.0f) * (KIND == 0 ? 0.0625f : 1.0f);
    float* out_row = p.out + (((int64_t)b * p.Hkv + kvh) * p.Tq + (q < p.Tq ? q : 0)) * p.nblk;
    const bool writer = hd == 0 && q < p.Tq;
    float* my_ks = s_ks + warp * 2 * TC_NTILE;
    // Key scales of a tile: lane l fetches tokens 4l .. 4l+3; dead tokens get NaN, which never wins a max.
    // Fetched two of this warp's tiles ahead.
    auto load_ks = [&](int tile) -> float4 {
      const int64_t t = (int64_t)tile * TC_NTILE + 4 * lane;
      if ((int64_t)(tile + 1) * TC_NTILE <= (int64_t)p.Tk)                 // interior tile (all but the last one or two)
        return *reinterpret_cast<const float4*>(scale_row + t);
      const float nan = __int_as_float(0x7fc00000);
      float4 v = make_float4(nan, nan, nan, nan);
      if (tile < ntiles) {
        if (t < p.Tk) v.x = scale_row[t];
        if (t + 1 < p.Tk) v.y = scale_row[t + 1];
        if (t + 2 < p.Tk) v.z = scale_row[t + 2];
        if (t + 3 < p.Tk) v.w = scale_row[t + 3];
      }
      return v;
    };
    constexpr int NCH = TC_NTILE / TW_CHW;          // chunks per tile
    constexpr int CPB = 64 / TW_CHW;                // chunks per 64-token block
    const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(par * TC_QT * TC_NTILE + qt * TC_NTILE);
    float4 k_cur = load_ks(par), k_next = load_ks(par + 2);
    int buf = 0;
    for (int i = par; i < ntiles; i += TC_ASTAGES, buf ^= 1) {
      float* ksb = my_ks + buf * TC_NTILE;
      *reinterpret_cast<float4*>(ksb + 4 * lane) = k_cur;
      k_cur = k_next;
      k_next = load_ks(i + 2 * TC_ASTAGES);
      __syncwarp();
      // (a role that gave up stops feeding the barriers, so this bounded wait ends every warp's loop)
      if (!mbar_wait_bounded(&acc_full[par], (uint32_t)(i >> 1) & 1u)) { *s_dead = 1; break; }
      tc_fence_after();
      float m = -INFINITY, m0 = 0.0f;
      uint32_t va[TW_CHW], vb[TW_CHW];
      TcLd<TW_CHW>::ld(tbase, va);
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        uint32_t* cur = (ch & 1) ? vb : va;
        uint32_t* nxt = (ch & 1) ? va : vb;
        TcLd<TW_CHW>::wait(cur);
        if (ch + 1 < NCH) {
          TcLd<TW_CHW>::ld(tbase + (uint32_t)((ch + 1) * TW_CHW), nxt);
        } else {                                    // the whole tile is in registers: the stage may be refilled
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[par]);
        }
        m = tc_chunk_max<KIND, TW_CHW>(cur, ksb + ch * TW_CHW, m);
        if (ch == CPB - 1) { m0 = m; m = -INFINITY; }
      }
      // x -> fl(x * qscale) is monotone for qscale > 0: scale the block maxima only; then the group maximum
      // over the G heads of the query, which are G neighbouring lanes
      float r0 = __fmul_rn(m0, qs), r1 = __fmul_rn(m, qs);
#pragma unroll
      for (int off = 1; off < G; off <<= 1) {
        r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, off));
        r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, off));
      }
      if (writer) {
        if (r0 == 0.0f) r0 = 0.0f;                  // -0 -> +0
        if (r1 == 0.0f) r1 = 0.0f;
        const int blk = 2 * i;
        if (blk + 1 < p.nblk && (p.nblk & 1) == 0) {
          *reinterpret_cast<float2*>(out_row + blk) = make_float2(r0, r1);
        } else {
          out_row[blk] = r0;
          if (blk + 1 < p.nblk) out_row[blk + 1] = r1;
        }
      }
    }
  } else if (warp == TW_EPI_WARPS) {
    // =============================== operand copies ===============================
    if (lane == 0) {
      const uint8_t* src = pw.operands + (int64_t)bh * pw.cap_tiles * Cfg::B_STAGE;
      int issued = 0;
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % BSTAGES;
        if (*s_dead) break;
        if (!mbar_wait_bounded(&b_empty[s], ((uint32_t)(i / BSTAGES) & 1u) ^ 1u)) { *s_dead = 1; break; }
        mbar_arrive_expect_tx(&b_full[s], (uint32_t)Cfg::B_STAGE);
        bulk_g2s(s_b + s * Cfg::B_STAGE, src + (int64_t)i * Cfg::B_STAGE, (uint32_t)Cfg::B_STAGE, &b_full[s]);
        ++issued;
      }
      // no copy of this CTA may still be writing shared memory when the CTA leaves: wait (bounded) for the
      // copies that can be outstanding, the last BSTAGES ones
      for (int j = issued > BSTAGES ? issued - BSTAGES : 0; j < issued; ++j)
        mbar_wait_bounded(&b_full[j % BSTAGES], (uint32_t)(j / BSTAGES) & 1u, 1u << 16);
    }
  } else if (lane == 0) {
    // =============================== MMA issuer ===============================
    tc_issue_tiles<KIND, Cfg>(s_a, s_b, b_full, b_empty, acc_full, acc_empty, all_done, s_dead, tmem_base, ntiles);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == TW_WARPS - 1) {
    tc_fence_after();
    tc_dealloc(tmem_base, TC_TMEM_COLS);
  }
}

template <int C, int G, int KIND>
static int prefill_tc_launch(const PrefillTcParams& p, int device, cudaStream_t st) {
  using Cfg = TcCfg<C, KIND>;
  static_assert(Cfg::BYTES <= 227 * 1024, "shared memory budget");
  auto kern = score_prefill_tc_kernel<C, G, KIND>;
  static std::atomic<bool> attr_done[KVB_MAX_DEVICES];
  { const int arc = ensure_dynamic_smem(kern, attr_done, device, (size_t)Cfg::BYTES); if (arc != KVB_OK) return arc; }
  constexpr int QCTA = TC_QT * (128 / G);
  dim3 grid(ceil_div(p.Tq, QCTA), p.B * p.Hkv);
  kern<<<grid, TC_THREADS, Cfg::BYTES, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

template <int C, int KIND>
static int prefill_tc_dispatch_g(const PrefillTcParams& p, int G, int device, cudaStream_t st) {
  switch (G) {
    case 1: return prefill_tc_launch<C, 1, KIND>(p, device, st);
    case 2: return prefill_tc_launch<C, 2, KIND>(p, device, st);
    case 4: return prefill_tc_launch<C, 4, KIND>(p, device, st);
    case 8: return prefill_tc_launch<C, 8, KIND>(p, device, st);
    default: return KVB_BAD_SHAPE;
  }
}

// kind: 0 = int8 operands / int32 accumulators, 1 = fp16 operands / fp32 accumulators
static int prefill_tc_run(const PrefillTcParams& p, int C, int G, int kind, int device, cudaStream_t st) {
  if (kind == 0) {
    if (C == 32) return prefill_tc_dispatch_g<32, 0>(p, G, device, st);
    if (C == 64) return prefill_tc_dispatch_g<64, 0>(p, G, device, st);
    if (C == 128) return prefill_tc_dispatch_g<128, 0>(p, G, device, st);
  } else {
    if (C == 32) return prefill_tc_dispatch_g<32, 1>(p, G, device, st);
    if (C == 64) return prefill_tc_dispatch_g<64, 1>(p, G, device, st);
    if (C == 128) return prefill_tc_dispatch_g<128, 1>(p, G, device, st);
  }
  return KVB_BAD_SHAPE;
}


template <int C, int G, int KIND>
static int prefill_tw_launch(const PrefillTwParams& pw, int device, cudaStream_t st) {
  using Cfg = TwCfg<C, KIND>;
  static_assert(Cfg::BYTES <= 227 * 1024, "shared memory budget");
  static_assert(Cfg::BSTAGES >= 2, "operand ring");
  auto kern = score_prefill_tw_kernel<C, G, KIND>;
  static std::atomic<bool> attr_done[KVB_MAX_DEVICES];
  { const int arc = ensure_dynamic_smem(kern, attr_done, device, (size_t)Cfg::BYTES); if (arc != KVB_OK) return arc; }
  constexpr int QCTA = TC_QT * (128 / G);
  dim3 grid(ceil_div(pw.base.Tq, QCTA), pw.base.B * pw.base.Hkv);
  kern<<<grid, TW_THREADS, Cfg::BYTES, st>>>(pw);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

template <int C, int KIND>
static int prefill_tw_dispatch_g(const PrefillTwParams& pw, int G, int device, cudaStream_t st) {
  switch (G) {
    case 1: return prefill_tw_launch<C, 1, KIND>(pw, device, st);
    case 2: return prefill_tw_launch<C, 2, KIND>(pw, device, st);
    case 4: return prefill_tw_launch<C, 4, KIND>(pw, device, st);
    case 8: return prefill_tw_launch<C, 8, KIND>(pw, device, st);
    default: return KVB_BAD_SHAPE;
  }
}

static int prefill_tw_run(const PrefillTwParams& pw, int C, int G, int kind, int device, cudaStream_t st) {
  if (kind == 0) {
    if (C == 32) return prefill_tw_dispatch_g<32, 0>(pw, G, device, st);
    if (C == 64) return prefill_tw_dispatch_g<64, 0>(pw, G, device, st);
    if (C == 128) return prefill_tw_dispatch_g<128, 0>(pw, G, device, st);
  } else {
    if (C == 32) return prefill_tw_dispatch_g<32, 1>(pw, G, device, st);
    if (C == 64) return prefill_tw_dispatch_g<64, 1>(pw, G, device, st);
    if (C == 128) return prefill_tw_dispatch_g<128, 1>(pw, G, device, st);
  }
  return KVB_BAD_SHAPE;
}

// bytes of one widened operand tile (128 tokens)
static size_t prefill_operand_tile_bytes(int C, int kind) { return (size_t)TC_NTILE * C * (kind == 0 ? 1 : 2); }

template <int C, int KIND>
static int prefill_widen_launch(const uint8_t* packed, int64_t sb, int64_t sh, int B, int Hkv, int Tk, int cap_tiles,
                                int first_tile, uint8_t* operands, cudaStream_t st) {
  const int ntiles = ceil_div(Tk, TC_NTILE);
  if (first_tile >= ntiles) return KVB_OK;
  dim3 grid(ntiles - first_tile, B * Hkv);
  prefill_widen_kernel<C, KIND><<<grid, TC_NTILE, 0, st>>>(packed, sb, sh, Hkv, Tk, cap_tiles, first_tile, operands);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

static int prefill_widen_run(const uint8_t* packed, int64_t sb, int64_t sh, int B, int Hkv, int Tk, int C, int kind,
                             int cap_tiles, int first_tile, uint8_t* operands, cudaStream_t st) {
  if (kind == 0) {
    if (C == 32) return prefill_widen_launch<32, 0>(packed, sb, sh, B, Hkv, Tk, cap_tiles, first_tile, operands, st);
    if (C == 64) return prefill_widen_launch<64, 0>(packed, sb, sh, B, Hkv, Tk, cap_tiles, first_tile, operands, st);
    if (C == 128) return prefill_widen_launch<128, 0>(packed, sb, sh, B, Hkv, Tk, cap_tiles, first_tile, operands, st);
  } else {
    if (C == 32) return prefill_widen_launch<32, 1>(packed, sb, sh, B, Hkv, Tk, cap_tiles, first_tile, operands, st);
    if (C == 64) return prefill_widen_launch<64, 1>(packed, sb, sh, B, Hkv, Tk, cap_tiles, first_tile, operands, st);
    if (C == 128) return prefill_widen_launch<128, 1>(packed, sb, sh, B, Hkv, Tk, cap_tiles, first_tile, operands, st);
  }
  return KVB_BAD_SHAPE;
}

}  // namespace kvb

