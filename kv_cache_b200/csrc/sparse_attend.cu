// Stage 4: exact attention of one decode query per sequence over a list of gathered K/V rows.
//
// One CTA handles a chunk of the index list of one (batch, index-head) pair and ALL query heads
// that share that list (the G heads of a KV head), so each 256-byte K row and V row is fetched
// once per KV head. Rows are gathered with 16-byte cp.async copies into a 3-stage ring of
// 32-row tiles (row pitch 272 bytes, bank-conflict free for the fragment loads below). QK^T and
// PV run on mma.sync m16n8k16 bf16 with fp32 accumulators (heads padded to the 16-row A tile),
// softmax is online in fp32, and the chunks of a list are combined by the last CTA to finish
// (log-sum-exp merge), so no second launch and no spinning is needed.
#include "common.cuh"

namespace kvb {

constexpr int AT_THREADS = 128;
constexpr int AT_TILE = 32;                 // rows per tile
constexpr int AT_D = 128;
constexpr int AT_PITCH = 272;               // bytes per staged row (256 + 16)
constexpr int AT_STAGES = 3;
constexpr int AT_TILE_BYTES = AT_TILE * AT_PITCH;        // 8704
constexpr int AT_STAGE_BYTES = 2 * AT_TILE_BYTES;        // K then V
constexpr int AT_MAX_TILES_PER_CTA = 32;
constexpr int AT_MAX_ROWS_PER_CTA = AT_MAX_TILES_PER_CTA * AT_TILE;
constexpr int AT_S_PITCH = 40;              // floats per score row
constexpr int AT_TARGET_CTAS = 444;         // one wave: 148 SMs x 3 resident CTAs (shared memory bound)

struct AttendParams {
  const __nv_bfloat16* query; int64_t q_sb, q_sh;
  const __nv_bfloat16* key;   int64_t k_sb, k_sh, k_st;
  const __nv_bfloat16* value; int64_t v_sb, v_sh, v_st;
  const void* indices; int idx_is_i64;
  const uint8_t* valid;
  const float* mask; int64_t mask_sb;
  int B, Hq, Hkv, Hi, Tk, S;
  int G;                      // Hq / Hkv
  float scaling;
  __nv_bfloat16* out;
  float* out_partial;
  float* ws_partial;          // [B*Hi, nsplit, GG, D+2]
  uint32_t* ws_counter;       // [B*Hi]
  int nsplit, tiles_per_cta;
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3,
                                                  uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(smem_addr)
               : "memory");
}

// GG = query heads that share one index list (1, 2, 4 or 8).
template <int GG>
__global__ void __launch_bounds__(AT_THREADS) sparse_attend_kernel(AttendParams p) {
  extern __shared__ __align__(128) uint8_t at_smem[];
  uint8_t* s_stage = at_smem;                                                  // [stages][K|V][32][272]
  float* s_S = reinterpret_cast<float*>(s_stage + AT_STAGES * AT_STAGE_BYTES);  // [8][40]
  int* s_idx = reinterpret_cast<int*>(s_S + 8 * AT_S_PITCH);                    // [rows of this CTA]
  float* s_maskv = reinterpret_cast<float*>(s_idx + AT_MAX_ROWS_PER_CTA);       // [rows of this CTA]
  __shared__ int s_is_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int split = blockIdx.x;
  const int row = blockIdx.y;                         // (b, index head)
  const int b = row / p.Hi, hi = row - b * p.Hi;
  const int head0 = hi * GG;                          // first query head served
  const int kvh = head0 / p.G;

  const int s_begin = split * p.tiles_per_cta * AT_TILE;
  int s_end = s_begin + p.tiles_per_cta * AT_TILE;
  if (s_end > p.S) s_end = p.S;
  const int nrows = s_end - s_begin;                  // >= 1 by construction of nsplit
  const int ntile = (nrows + AT_TILE - 1) / AT_TILE;

  // Index list of this chunk: -1 marks an entry that contributes nothing.
  {
    const int64_t base = (int64_t)row * p.S + s_begin;
    for (int i = tid; i < ntile * AT_TILE; i += AT_THREADS) {
      int tok = -1;
      float mv = 0.0f;
      if (i < nrows) {
        const int64_t raw = p.idx_is_i64 ? reinterpret_cast<const int64_t*>(p.indices)[base + i]
                                         : (int64_t) reinterpret_cast<const int32_t*>(p.indices)[base + i];
        const bool ok = (p.valid == nullptr || p.valid[base + i] != 0) && raw >= 0 && raw < (int64_t)p.Tk;
        if (ok) {
          tok = (int)raw;
          if (p.mask) mv = p.mask[(int64_t)b * p.mask_sb + raw];
        }
      }
      s_idx[i] = tok;
      s_maskv[i] = mv;
    }
  }
  __syncthreads();

  const __nv_bfloat16* kbase = p.key + (int64_t)b * p.k_sb + (int64_t)kvh * p.k_sh;
  const __nv_bfloat16* vbase = p.value + (int64_t)b * p.v_sb + (int64_t)kvh * p.v_sh;

  auto load_tile = [&](int tile) {
    uint8_t* sk = s_stage + (tile % AT_STAGES) * AT_STAGE_BYTES;
    uint8_t* sv = sk + AT_TILE_BYTES;
    const int c16 = tid & 15;
    const int r0 = tid >> 4;
#pragma unroll
    for (int j = 0; j < AT_TILE / 8; ++j) {
      const int r = r0 + 8 * j;
      int tok = s_idx[tile * AT_TILE + r];
      if (tok < 0) tok = 0;                            // weight is forced to zero later; any live row will do
      cp_async_16(sk + r * AT_PITCH + c16 * 16, kbase + (int64_t)tok * p.k_st + c16 * 8);
      cp_async_16(sv + r * AT_PITCH + c16 * 16, vbase + (int64_t)tok * p.v_st + c16 * 8);
    }
  };

  // Query fragments (A operand, rows = heads; rows >= GG are zero).
  uint32_t qa[8][2];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qa[ks][0] = 0u;
    qa[ks][1] = 0u;
    if (g < GG) {
      const __nv_bfloat16* qrow = p.query + (int64_t)b * p.q_sb + (int64_t)(head0 + g) * p.q_sh;
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t4);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t4 + 8);
    }
  }

  float o[4][4];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nt][i] = 0.0f;
  float m_run = -INFINITY, l_run = 0.0f;

#pragma unroll
  for (int s = 0; s < AT_STAGES - 1; ++s) {
    if (s < ntile) load_tile(s);
    cp_async_commit();
  }

  for (int i = 0; i < ntile; ++i) {
    if (i + AT_STAGES - 1 < ntile) load_tile(i + AT_STAGES - 1);
    cp_async_commit();
    cp_async_wait<AT_STAGES - 1>();
    __syncthreads();

    const uint8_t* sk = s_stage + (i % AT_STAGES) * AT_STAGE_BYTES;
    const uint8_t* sv = sk + AT_TILE_BYTES;

    // ---- S = Q K^T for this warp's 8 rows of the tile ----
    {
      float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const uint8_t* krow = sk + (8 * warp + g) * AT_PITCH;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + (16 * ks + 2 * t4) * 2);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + (16 * ks + 2 * t4 + 8) * 2);
        mma_bf16_16816(c, qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
      }
      const int r = 8 * warp + 2 * t4;                 // tile-local rows of c[0], c[1]
      const int gi = i * AT_TILE + r;
      float s0 = c[0] * p.scaling + s_maskv[gi];
      float s1 = c[1] * p.scaling + s_maskv[gi + 1];
      if (s_idx[gi] < 0) s0 = -INFINITY;
      if (s_idx[gi + 1] < 0) s1 = -INFINITY;
      *reinterpret_cast<float2*>(&s_S[g * AT_S_PITCH + r]) = make_float2(s0, s1);
    }
    __syncthreads();

    // ---- online softmax (every warp keeps the same running statistics for head g) ----
    float sc[8];
    {
      const float* srow = s_S + g * AT_S_PITCH;
      const float2 v0 = *reinterpret_cast<const float2*>(srow + 2 * t4);
      const float2 v1 = *reinterpret_cast<const float2*>(srow + 2 * t4 + 8);
      const float2 v2 = *reinterpret_cast<const float2*>(srow + 2 * t4 + 16);
      const float2 v3 = *reinterpret_cast<const float2*>(srow + 2 * t4 + 24);
      sc[0] = v0.x; sc[1] = v0.y; sc[2] = v1.x; sc[3] = v1.y;
      sc[4] = v2.x; sc[5] = v2.y; sc[6] = v3.x; sc[7] = v3.y;
    }
    float mx = sc[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) mx = fmaxf(mx, sc[j]);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
    const float alpha = __expf(m_run - m_use);          // 0 when m_run == -inf
    float psum = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      sc[j] = __expf(sc[j] - m_use);                    // 0 for -inf
      psum += sc[j];
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l_run = l_run * alpha + psum;
    m_run = m_new;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      o[nt][0] *= alpha;
      o[nt][1] *= alpha;
    }
    // P fragments (A operand): k-step 0 = rows 0..15 of the tile, k-step 1 = rows 16..31
    const uint32_t pa[2][2] = {{pack_bf16x2(sc[0], sc[1]), pack_bf16x2(sc[2], sc[3])},
                               {pack_bf16x2(sc[4], sc[5]), pack_bf16x2(sc[6], sc[7])}};

    // ---- O += P V for this warp's 32 output dims ----
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int jp = 0; jp < 2; ++jp) {
        const int vrow = 16 * ks + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int vdim = 32 * warp + 16 * jp + (lane >> 4) * 8;
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans(r0, r1, r2, r3, smem_u32(sv + vrow * AT_PITCH + vdim * 2));
        mma_bf16_16816(o[2 * jp], pa[ks][0], 0u, pa[ks][1], 0u, r0, r1);
        mma_bf16_16816(o[2 * jp + 1], pa[ks][0], 0u, pa[ks][1], 0u, r2, r3);
      }
    }
    __syncthreads();   // s_S and this stage are rewritten by the next iterations
  }
  cp_async_wait<0>();

  // ---- partial result of this chunk ----
  constexpr int PW = AT_D + 2;
  float* part = p.ws_partial + ((int64_t)row * p.nsplit + split) * GG * PW;
  if (g < GG) {
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int d = 32 * warp + 8 * nt + 2 * t4;
      *reinterpret_cast<float2*>(&part[g * PW + d]) = make_float2(o[nt][0], o[nt][1]);
    }
    if (warp == 0 && t4 == 0) {
      part[g * PW + AT_D] = m_run;
      part[g * PW + AT_D + 1] = l_run;
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t prev = atomicAdd(&p.ws_counter[row], 1u);
    s_is_last = (prev == (uint32_t)(p.nsplit - 1));
    if (s_is_last) p.ws_counter[row] = 0;              // leave the counter ready for the next call
  }
  __syncthreads();
  if (!s_is_last) return;
  __threadfence();

  // ---- log-sum-exp merge of the chunks by the last CTA: thread d handles output dim d ----
  const float* parts = p.ws_partial + (int64_t)row * p.nsplit * GG * PW;
  for (int hd = 0; hd < GG; ++hd) {
    float M = -INFINITY;
    for (int sp = 0; sp < p.nsplit; ++sp) M = fmaxf(M, __ldcg(&parts[(sp * GG + hd) * PW + AT_D]));
    const float Mu = (M == -INFINITY) ? 0.0f : M;
    float L = 0.0f, O = 0.0f;
    for (int sp = 0; sp < p.nsplit; ++sp) {
      const float* ps = parts + (sp * GG + hd) * PW;
      const float w = __expf(__ldcg(&ps[AT_D]) - Mu);
      L += __ldcg(&ps[AT_D + 1]) * w;
      O += __ldcg(&ps[tid]) * w;
    }
    const int head = head0 + hd;
    if (p.out) p.out[((int64_t)b * p.Hq + head) * AT_D + tid] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
    if (p.out_partial) {
      float* op = p.out_partial + ((int64_t)b * p.Hq + head) * PW;
      op[tid] = O;
      if (tid == 0) {
        op[AT_D] = M;
        op[AT_D + 1] = L;
      }
    }
  }
}

// Combine N shard partials into the final bf16 output: grid B*Hq, 128 threads (one per dim).
__global__ void __launch_bounds__(AT_THREADS) lse_merge_kernel(const float* partials, int N, int BH, __nv_bfloat16* out) {
  constexpr int PW = AT_D + 2;
  const int bh = blockIdx.x, d = threadIdx.x;
  float M = -INFINITY;
  for (int r = 0; r < N; ++r) {
    const float* ps = partials + ((int64_t)r * BH + bh) * PW;
    if (ps[AT_D + 1] > 0.0f) M = fmaxf(M, ps[AT_D]);
  }
  float L = 0.0f, O = 0.0f;
  if (M != -INFINITY) {
    for (int r = 0; r < N; ++r) {
      const float* ps = partials + ((int64_t)r * BH + bh) * PW;
      const float l = ps[AT_D + 1];
      if (l > 0.0f) {
        const float w = __expf(ps[AT_D] - M);
        L += l * w;
        O += ps[d] * w;
      }
    }
  }
  out[(int64_t)bh * AT_D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
}

// selected || sink || recent || self, with the protected ranges removed from the selected part.
__global__ void build_final_indices_kernel(const int32_t* sel_idx, const uint8_t* sel_valid, int R, int kk, int S,
                                           int history, int key_count, int sink_end, int recent_on, int recent_start,
                                           int recent_from, int n_recent, int keep_self, int append_protected,
                                           int32_t* out_idx, uint8_t* out_valid) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)R * S) return;
  const int r = (int)(i / S), s = (int)(i - (int64_t)r * S);
  int idx;
  bool ok = true;
  if (s < kk) {
    idx = sel_idx[(int64_t)r * kk + s];
    ok = sel_valid ? (sel_valid[(int64_t)r * kk + s] != 0) : true;
    if (!append_protected) {
      if (recent_on && idx >= recent_start && idx < history) ok = false;
      if (sink_end > 0 && idx < sink_end) ok = false;
    }
  } else if (s < kk + sink_end) {
    idx = s - kk;
  } else if (s < kk + sink_end + n_recent) {
    idx = recent_from + (s - kk - sink_end);
  } else {
    idx = key_count - 1;
  }
  out_idx[i] = idx;
  out_valid[i] = ok ? 1 : 0;
}

struct FinalLayout {
  int sink_end, recent_on, recent_start, recent_from, n_recent, S;
};

static FinalLayout final_layout(int kk, int history, int sink, int recent, int keep_self) {
  FinalLayout f;
  f.sink_end = sink > 0 ? (sink < history ? sink : history) : 0;
  f.recent_on = recent > 0 ? 1 : 0;
  f.recent_start = history;
  f.recent_from = history;
  f.n_recent = 0;
  if (recent > 0) {
    f.recent_start = history - recent > 0 ? history - recent : 0;
    if (f.recent_start < history) {
      f.recent_from = f.recent_start > f.sink_end ? f.recent_start : f.sink_end;
      if (f.recent_from < history) f.n_recent = history - f.recent_from;
    }
  }
  f.S = kk + f.sink_end + f.n_recent + (keep_self ? 1 : 0);
  return f;
}

struct AttendPlan {
  int tiles_per_cta, nsplit;
  size_t counter_bytes, partial_bytes, bytes;
};

static AttendPlan attend_plan(int B, int Hq, int Hi, int S) {
  AttendPlan a;
  const int R = B * Hi;
  const int GG = Hq / Hi;
  const int ntiles = ceil_div(S, AT_TILE);
  // As many chunks per list as fit in ONE wave of resident CTAs: long chunks keep the 3-stage
  // gather pipeline full and make the final merge short.
  int want_splits = AT_TARGET_CTAS / R;
  if (want_splits < 1) want_splits = 1;
  int tpc = ceil_div(ntiles, want_splits);
  if (tpc < 1) tpc = 1;
  if (tpc > AT_MAX_TILES_PER_CTA) tpc = AT_MAX_TILES_PER_CTA;
  a.tiles_per_cta = tpc;
  a.nsplit = ceil_div(ntiles, tpc);
  a.counter_bytes = round_up(sizeof(uint32_t) * (size_t)R, 256);
  a.partial_bytes = round_up(sizeof(float) * (size_t)R * a.nsplit * GG * (AT_D + 2), 256);
  a.bytes = a.counter_bytes + a.partial_bytes;
  return a;
}

template <int GG>
static int attend_launch(const AttendParams& p, int device, cudaStream_t st) {
  const size_t smem = (size_t)AT_STAGES * AT_STAGE_BYTES + sizeof(float) * 8 * AT_S_PITCH +
                      (sizeof(int) + sizeof(float)) * AT_MAX_ROWS_PER_CTA;
  auto kern = sparse_attend_kernel<GG>;
  static bool attr_done[64] = {false};
  if (device < 64 && !attr_done[device]) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr_done[device] = true;
  }
  kern<<<dim3(p.nsplit, p.B * p.Hi), AT_THREADS, smem, st>>>(p);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_sparse_attend_workspace_bytes(int B, int Hq, int Hi, int S) {
  if (B <= 0 || Hq <= 0 || Hi <= 0 || S <= 0 || (Hq % Hi)) return 0;
  return kvb::attend_plan(B, Hq, Hi, S).bytes;
}

namespace kvb {

// Shared by kvb_sparse_attend and the fused step. `counters_zeroed` tells that the caller already
// cleared ws_counter on this stream.
static int attend_run(const void* query, int64_t q_sb, int64_t q_sh, const void* key, int64_t k_sb, int64_t k_sh,
                      int64_t k_st, const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st,
                      const void* indices, int idx_is_i64, const uint8_t* valid, const float* mask, int64_t mask_sb,
                      int B, int Hq, int Hkv, int Hi, int Tk, int D, int S, float scaling, void* out,
                      float* out_partial, uint32_t* ws_counter, float* ws_partial, bool counters_zeroed, int device,
                      cudaStream_t st) {
  if (!query || !key || !value || !indices || !ws_counter || !ws_partial) return KVB_BAD_ARG;
  if (!out && !out_partial) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hi <= 0 || Tk <= 0 || S <= 0) return KVB_BAD_SHAPE;
  if (D != AT_D || (Hq % Hkv) || (Hi != Hkv && Hi != Hq)) return KVB_BAD_SHAPE;
  const int GG = Hq / Hi;
  if (GG != 1 && GG != 2 && GG != 4 && GG != 8) return KVB_BAD_SHAPE;
  if ((int64_t)B * Hi > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(query, 16) || !aligned_to(key, 16) || !aligned_to(value, 16)) return KVB_BAD_ALIGN;
  if ((q_sb % 8) || (q_sh % 8) || (k_sb % 8) || (k_sh % 8) || (k_st % 8) || (v_sb % 8) || (v_sh % 8) || (v_st % 8))
    return KVB_BAD_ALIGN;
  if (!aligned_to(indices, idx_is_i64 ? 8 : 4) || !aligned_to(ws_partial, 16)) return KVB_BAD_ALIGN;
  if (out && !aligned_to(out, 2)) return KVB_BAD_ALIGN;
  const AttendPlan plan = attend_plan(B, Hq, Hi, S);
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;

  AttendParams p;
  p.query = reinterpret_cast<const __nv_bfloat16*>(query); p.q_sb = q_sb; p.q_sh = q_sh;
  p.key = reinterpret_cast<const __nv_bfloat16*>(key); p.k_sb = k_sb; p.k_sh = k_sh; p.k_st = k_st;
  p.value = reinterpret_cast<const __nv_bfloat16*>(value); p.v_sb = v_sb; p.v_sh = v_sh; p.v_st = v_st;
  p.indices = indices; p.idx_is_i64 = idx_is_i64; p.valid = valid;
  p.mask = mask; p.mask_sb = mask_sb;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Hi = Hi; p.Tk = Tk; p.S = S; p.G = Hq / Hkv;
  p.scaling = scaling;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_partial = out_partial;
  p.ws_counter = ws_counter;
  p.ws_partial = ws_partial;
  p.nsplit = plan.nsplit; p.tiles_per_cta = plan.tiles_per_cta;

  if (!counters_zeroed) KVB_CHECK_CUDA(cudaMemsetAsync(p.ws_counter, 0, sizeof(uint32_t) * (size_t)B * Hi, st));
  switch (GG) {
    case 1: return attend_launch<1>(p, device, st);
    case 2: return attend_launch<2>(p, device, st);
    case 4: return attend_launch<4>(p, device, st);
    default: return attend_launch<8>(p, device, st);
  }
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_sparse_attend(
    const void* query, int64_t q_sb, int64_t q_sh, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
    const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st, const void* indices, int idx_is_i64,
    const uint8_t* valid, const float* mask, int64_t mask_sb, int B, int Hq, int Hkv, int Hi, int Tk, int D, int S,
    float scaling, void* out, float* out_partial, void* workspace, size_t workspace_bytes, int device, void* stream) {
  using namespace kvb;
  if (!workspace) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hi <= 0 || S <= 0 || (Hq % Hi)) return KVB_BAD_SHAPE;
  if (!aligned_to(workspace, 256)) return KVB_BAD_ALIGN;
  const AttendPlan plan = attend_plan(B, Hq, Hi, S);
  if (workspace_bytes < plan.bytes) return KVB_WORKSPACE_TOO_SMALL;
  return attend_run(query, q_sb, q_sh, key, k_sb, k_sh, k_st, value, v_sb, v_sh, v_st, indices, idx_is_i64, valid,
                    mask, mask_sb, B, Hq, Hkv, Hi, Tk, D, S, scaling, out, out_partial,
                    reinterpret_cast<uint32_t*>(workspace),
                    reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + plan.counter_bytes),
                    /*counters_zeroed=*/false, device, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int kvb_lse_merge(const float* partials, int N, int B, int Hq, int D, void* out, int device,
                             void* stream) {
  using namespace kvb;
  if (!partials || !out) return KVB_BAD_ARG;
  if (N <= 0 || B <= 0 || Hq <= 0 || D != AT_D) return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  lse_merge_kernel<<<B * Hq, AT_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      partials, N, B * Hq, reinterpret_cast<__nv_bfloat16*>(out));
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}

extern "C" __attribute__((visibility("default"))) int kvb_final_index_count(int kk, int history_count, int protect_sink, int protect_recent,
                                     int keep_self) {
  if (kk < 0 || history_count < 0) return -1;
  return kvb::final_layout(kk, history_count, protect_sink, protect_recent, keep_self).S;
}

extern "C" __attribute__((visibility("default"))) int kvb_build_final_indices(const int32_t* sel_idx, const uint8_t* sel_valid, int R, int kk,
                                       int history_count, int key_count, int protect_sink, int protect_recent,
                                       int keep_self, int append_protected, int32_t* out_idx, uint8_t* out_valid,
                                       int device, void* stream) {
  using namespace kvb;
  if ((!sel_idx && kk > 0) || !out_idx || !out_valid) return KVB_BAD_ARG;
  if (R <= 0 || kk < 0 || history_count < 0 || key_count <= 0) return KVB_BAD_SHAPE;
  const FinalLayout f = final_layout(kk, history_count, protect_sink, protect_recent, keep_self);
  if (f.S == 0) return KVB_OK;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  const int64_t n = (int64_t)R * f.S;
  const int threads = 256;
  const unsigned blocks = (unsigned)((n + threads - 1) / threads);
  build_final_indices_kernel<<<blocks, threads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      sel_idx, sel_valid, R, kk, f.S, history_count, key_count, f.sink_end, f.recent_on, f.recent_start,
      f.recent_from, f.n_recent, keep_self, append_protected, out_idx, out_valid);
  KVB_CHECK_CUDA(cudaGetLastError());
  return KVB_OK;
}
