// Stage 4: exact attention of one decode query per sequence over a list of gathered K/V rows.
//
// Work item = one chunk of the index list of one (batch, index-head) pair, handled by ONE WARP for
// all query heads that share the list (the G heads of a KV head), so each 256-byte K row and V
// row is fetched once per KV head. The warp gathers rows with 16-byte cp.async copies into its own
// 3-stage ring of 16-row tiles (row pitch 272 bytes: conflict-free fragment loads), computes
// Q K^T and P V with mma.sync m16n8k16 bf16 / fp32 accumulate (heads padded to the 16-row A tile;
// the score fragment is re-used in registers as the P fragment), keeps an online softmax in fp32,
// and never waits for another warp. The chunks of a list are combined by a small second launch
// (log-sum-exp merge, one CTA per (list, head)): folding it into the last warp to finish put a
// long chain of dependent L2 round trips on the tail of the kernel.
#include "common.cuh"

namespace kvb {

constexpr int AT_WARPS = 4;
constexpr int AT_THREADS = AT_WARPS * 32;
constexpr int AT_TILE = 16;                 // rows per tile
constexpr int AT_D = 128;
constexpr int AT_PITCH = 272;               // bytes per staged row (256 + 16)
constexpr int AT_STAGES = 3;
constexpr int AT_TILE_BYTES = AT_TILE * AT_PITCH;        // 4352
constexpr int AT_STAGE_BYTES = 2 * AT_TILE_BYTES;        // K then V
constexpr int AT_WARP_SMEM = AT_STAGES * (AT_STAGE_BYTES + AT_TILE * 8);   // stages + per-row (token, mask)
constexpr int AT_TARGET_WARPS = 1184;       // one wave: 148 SMs x 2 CTAs x 4 warps

struct FinalLayout {
  int sink_end, recent_on, recent_start, recent_from, n_recent, S;
};

__host__ __device__ inline FinalLayout final_layout(int kk, int history, int sink, int recent, int keep_self) {
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

// How the logical list of S entries is produced.
//   explicit: indices[row, s] (+ valid[row, s])
//   implicit: selected[row, 0..kk) || [0, sink_end) || [recent_from, recent_from + n_recent) || self
//             with the protected ranges removed from the selected part (the rule of
//             _qabs_final_indices_from_selected, or of ..._append_protected when append_protected)
struct AttendList {
  const void* indices; int idx_is_i64; const uint8_t* valid;      // explicit
  int implicit;
  const int32_t* selected; int kk; int sel_pitch;   // kk entries used of rows sel_pitch apart
  int64_t sel_base; int sel_limit;       // selected ids are global: local row = id - sel_base, kept iff in [0, sel_limit)
  const int32_t* sel_count;              // optional: row r uses only its first sel_count[r] (<= kk) selected entries
  int sink_end, n_recent, recent_from, recent_start, recent_on, history, append_protected;
};

// Optional extra duty of the warp that owns chunk 0 of a list: quantize the newest K row into the
// int4 side cache (the append of the fused decode step).
struct AttendAppend {
  int enabled;
  const int32_t* channel_idx; int C;
  uint8_t* packed; int64_t packed_sb, packed_sh;
  float* scale; int64_t scale_sb, scale_sh;
  int64_t t_src, t_dst;
};

struct AttendParams {
  const __nv_bfloat16* query; int64_t q_sb, q_sh;
  const __nv_bfloat16* key;   int64_t k_sb, k_sh, k_st;
  const __nv_bfloat16* value; int64_t v_sb, v_sh, v_st;
  AttendList list;
  const float* mask; int64_t mask_sb;
  int B, Hq, Hkv, Hi, Tk, S;
  int G;                      // Hq / Hkv
  float scaling;
  __nv_bfloat16* out;
  float* out_partial;
  float* ws_partial;          // [B*Hi, nsplit, GG, D+2]
  uint32_t* ws_counter;       // [B*Hi]
  int nsplit, tiles_per_split;
  AttendAppend append;
  // optional (fused step): the history length lives on the device; the list layout is then derived
  // in the kernel from the raw policy below, and the host-side figures are upper bounds
  const int32_t* T_dev;
  int top_k, protect_sink, protect_recent, keep_self;
  int advance_history;        // the merge kernel adds one to *T_dev when everything else is done
  PartialPush ppush;          // sequence-sharded step: the merged (o, m, l) of every head goes to all ranks' inboxes
  // optional mean-value blend (SparQ): out = mean + alpha * (attention - mean)
  const float* blend_alpha;   // fp32 [B*Hq] or NULL
  const float* blend_mean;    // fp32 [B,Hkv,D] dense
  KvPages pages;              // optional: key / value are page pools (rows of D contiguous elements)
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

// Entry s of the logical list of `row`: token id, or -1 when it contributes nothing.
__device__ __forceinline__ int attend_fetch(const AttendParams& p, int row, int s) {
  const AttendList& L = p.list;
  int64_t raw;
  bool ok = true;
  if (!L.implicit) {
    const int64_t o = (int64_t)row * p.S + s;
    raw = L.idx_is_i64 ? reinterpret_cast<const int64_t*>(L.indices)[o]
                       : (int64_t) reinterpret_cast<const int32_t*>(L.indices)[o];
    ok = (L.valid == nullptr) || (L.valid[o] != 0);
  } else if (s < L.kk) {
    raw = (int64_t)L.selected[(int64_t)row * L.sel_pitch + s] - L.sel_base;
    if (raw >= L.sel_limit) ok = false;
    if (!L.append_protected) {
      if (L.recent_on && raw >= L.recent_start && raw < L.history) ok = false;
      if (L.sink_end > 0 && raw < L.sink_end) ok = false;
    }
  } else if (s < L.kk + L.sink_end) {
    raw = s - L.kk;
  } else if (s < L.kk + L.sink_end + L.n_recent) {
    raw = L.recent_from + (s - L.kk - L.sink_end);
  } else {
    raw = (int64_t)p.Tk - 1;                                   // the token being decoded
  }
  return (ok && raw >= 0 && raw < (int64_t)p.Tk) ? (int)raw : -1;
}

// One warp quantizes one bf16 K row to int4 (same arithmetic as quantize_pack_kernel).
__device__ __forceinline__ void quantize_row_warp(const __nv_bfloat16* krow, const int32_t* ch, int C, uint8_t* dst,
                                                  float* scale_dst, int lane) {
  const int nb = C >> 1;                       // <= 64 bytes: at most two per lane
  float x[4];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int byte = lane + 32 * j;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      x[2 * j + i] = (byte < nb) ? __bfloat162float(krow[ch[2 * byte + i]]) : 0.0f;
      amax = fmaxf(amax, fabsf(x[2 * j + i]));
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  const float sc = __fdiv_rn(fmaxf(amax, 5.9604644775390625e-08f /* 2^-24 */), 7.0f);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int byte = lane + 32 * j;
    if (byte < nb) {
      float lo = rintf(__fdiv_rn(x[2 * j], sc)), hi = rintf(__fdiv_rn(x[2 * j + 1], sc));
      lo = fminf(fmaxf(lo, -7.0f), 7.0f);
      hi = fminf(fmaxf(hi, -7.0f), 7.0f);
      dst[byte] = (uint8_t)((((int)lo) & 0xF) | ((((int)hi) & 0xF) << 4));
    }
  }
  if (lane == 0) *scale_dst = sc;
}

// GG = query heads that share one index list (1, 2, 4 or 8).
template <int GG>
__global__ void __launch_bounds__(AT_THREADS, 2) sparse_attend_kernel(AttendParams pin) {
  extern __shared__ __align__(128) uint8_t at_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int task = blockIdx.x * AT_WARPS + warp;
  pdl_launch_dependents();
  pdl_wait();
  if (task >= pin.B * pin.Hi * pin.nsplit) return;       // warps are independent: no block barrier below
  AttendParams p = pin;
  if (p.T_dev) {
    // history length from the device: rebuild the implicit list's layout for it
    int T = *p.T_dev;
    if (T > pin.list.history) T = pin.list.history;      // never beyond what the host sized for
    const int kk = p.top_k < T ? p.top_k : T;
    const FinalLayout f = final_layout(kk, T, p.protect_sink, p.protect_recent, p.keep_self);
    p.list.kk = kk; p.list.sel_limit = T; p.list.history = T;
    p.list.sink_end = f.sink_end; p.list.n_recent = f.n_recent; p.list.recent_from = f.recent_from;
    p.list.recent_start = f.recent_start; p.list.recent_on = f.recent_on;
    p.S = f.S;
    p.Tk = T + (p.keep_self ? 1 : 0);
    p.append.t_src = T; p.append.t_dst = T;
  }
  const int row = task / p.nsplit;                       // (b, index head)
  const int split = task - row * p.nsplit;
  const int b = row / p.Hi, hi = row - b * p.Hi;
  if (p.list.implicit && p.list.sel_count) {
    // a shorter selected part for this row: the list and the chunking shrink with it
    int c = p.list.sel_count[row];
    if (c < 0) c = 0;
    if (c < p.list.kk) {
      p.S -= p.list.kk - c;
      p.list.kk = c;
      const int tiles = (p.S + AT_TILE - 1) / AT_TILE;
      p.tiles_per_split = (tiles + p.nsplit - 1) / p.nsplit;
      if (p.tiles_per_split < 1) p.tiles_per_split = 1;
    }
  }
  const int head0 = hi * GG;                             // first query head served
  const int kvh = head0 / p.G;

  uint8_t* my = at_smem + warp * AT_WARP_SMEM;           // [stages][K|V][16][272] | tok[stages][16] | mask[stages][16]
  int* s_tok = reinterpret_cast<int*>(my + AT_STAGES * AT_STAGE_BYTES);
  float* s_msk = reinterpret_cast<float*>(s_tok + AT_STAGES * AT_TILE);

  const int s_begin = split * p.tiles_per_split * AT_TILE;
  int s_end = s_begin + p.tiles_per_split * AT_TILE;
  if (s_end > p.S) s_end = p.S;
  const int nrows = s_end - s_begin;                     // >= 1 by construction of nsplit unless the device-side length shrank the list
  const int ntile = nrows > 0 ? (nrows + AT_TILE - 1) / AT_TILE : 0;

  // paged pools: rows are addressed by their row number inside the pool (see kv_paged_row), D elements apart
  const bool paged = p.pages.table != nullptr;
  const __nv_bfloat16* kbase = paged ? p.key : p.key + (int64_t)b * p.k_sb + (int64_t)kvh * p.k_sh;
  const __nv_bfloat16* vbase = paged ? p.value : p.value + (int64_t)b * p.v_sb + (int64_t)kvh * p.v_sh;
  const int64_t k_st = paged ? AT_D : p.k_st, v_st = paged ? AT_D : p.v_st;

  if (p.append.enabled && split == 0) {
    const AttendAppend& A = p.append;
    const int64_t src_row = paged ? kv_paged_row(p.pages, p.Hkv, b, kvh, A.t_src) : (int64_t)A.t_src;
    quantize_row_warp(kbase + src_row * k_st, A.channel_idx + (int64_t)kvh * A.C, A.C,
                      A.packed + (int64_t)b * A.packed_sb + (int64_t)kvh * A.packed_sh + A.t_dst * (A.C >> 1),
                      A.scale + (int64_t)b * A.scale_sb + (int64_t)kvh * A.scale_sh + A.t_dst, lane);
  }

  // List entries are fetched one tile AHEAD of the gather that uses them, so the global-memory
  // latency of the index (and mask) read overlaps the math of the tile in between.
  auto fetch_tile = [&](int tile, int& tok, float& mv) {
    const int s = s_begin + tile * AT_TILE + (lane & 15);      // lanes 16..31 mirror lanes 0..15
    tok = (tile < ntile && s < s_end) ? attend_fetch(p, row, s) : -1;
    mv = (tok >= 0 && p.mask) ? p.mask[(int64_t)b * p.mask_sb + tok] : 0.0f;
  };
  auto load_tile = [&](int tile, int tok, float mv) {
    const int stage = tile % AT_STAGES;
    uint8_t* sk = my + stage * AT_STAGE_BYTES;
    uint8_t* sv = sk + AT_TILE_BYTES;
    if (lane < AT_TILE) {
      s_tok[stage * AT_TILE + lane] = tok;
      s_msk[stage * AT_TILE + lane] = mv;
    }
    if (tok < 0) tok = 0;                                 // weight is forced to zero later; any live row will do
    int prow = tok;                                       // row number: the token itself, or its place in the pool (< 2^31)
    if (paged) prow = (int)kv_paged_row(p.pages, p.Hkv, b, kvh, tok);
    const int c16 = lane & 15;
    const int r0 = lane >> 4;
#pragma unroll
    for (int j = 0; j < AT_TILE / 2; ++j) {
      const int r = r0 + 2 * j;
      const int tr = __shfl_sync(0xffffffffu, prow, r);
      cp_async_16(sk + r * AT_PITCH + c16 * 16, kbase + (int64_t)tr * k_st + c16 * 8);
      cp_async_16(sv + r * AT_PITCH + c16 * 16, vbase + (int64_t)tr * v_st + c16 * 8);
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

  float o[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nt][i] = 0.0f;
  float m_run = -INFINITY, l_run = 0.0f;

  int tok_cur, tok_nxt;
  float mv_cur, mv_nxt;
  {
    int tk[AT_STAGES];
    float mk[AT_STAGES];
#pragma unroll
    for (int s = 0; s < AT_STAGES; ++s) fetch_tile(s, tk[s], mk[s]);      // all in flight together
#pragma unroll
    for (int s = 0; s < AT_STAGES - 1; ++s) {
      if (s < ntile) load_tile(s, tk[s], mk[s]);
      cp_async_commit();
    }
    tok_cur = tk[AT_STAGES - 1];
    mv_cur = mk[AT_STAGES - 1];
  }

  for (int i = 0; i < ntile; ++i) {
    fetch_tile(i + AT_STAGES, tok_nxt, mv_nxt);           // used by the NEXT iteration's gather
    if (i + AT_STAGES - 1 < ntile) load_tile(i + AT_STAGES - 1, tok_cur, mv_cur);
    cp_async_commit();
    tok_cur = tok_nxt;
    mv_cur = mv_nxt;
    cp_async_wait<AT_STAGES - 1>();
    __syncwarp();

    const int stage = i % AT_STAGES;
    const uint8_t* sk = my + stage * AT_STAGE_BYTES;
    const uint8_t* sv = sk + AT_TILE_BYTES;

    // ---- S = Q K^T: two 8-row halves of the tile, independent accumulators ----
    float c[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.0f;
      const uint8_t* krow = sk + (8 * nt + g) * AT_PITCH;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + (16 * ks + 2 * t4) * 2);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + (16 * ks + 2 * t4 + 8) * 2);
        mma_bf16_16816(c[nt], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
      }
    }
    // c[nt][0], c[nt][1]: head g, tile rows 8*nt + 2*t4, + 1
    float sc[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int r = 8 * nt + 2 * t4 + e;
        const float v = c[nt][e] * p.scaling + s_msk[stage * AT_TILE + r];
        sc[2 * nt + e] = (s_tok[stage * AT_TILE + r] < 0) ? -INFINITY : v;
      }

    // ---- online softmax for head g (the four lanes of a quad hold the 16 rows) ----
    float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
    const float alpha = __expf(m_run - m_use);          // 0 when m_run == -inf
    float psum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      sc[j] = __expf(sc[j] - m_use);                    // 0 for -inf
      psum += sc[j];
    }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l_run = l_run * alpha + psum;
    m_run = m_new;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      o[nt][0] *= alpha;
      o[nt][1] *= alpha;
    }
    // The score fragment is already laid out as the A fragment of P V: rows 2*t4, 2*t4+1 and +8.
    const uint32_t pa0 = pack_bf16x2(sc[0], sc[1]);
    const uint32_t pa2 = pack_bf16x2(sc[2], sc[3]);

    // ---- O += P V over all 128 output dims ----
#pragma unroll
    for (int jp = 0; jp < 8; ++jp) {
      const int vrow = ((lane >> 3) & 1) * 8 + (lane & 7);
      const int vdim = 16 * jp + (lane >> 4) * 8;
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4_trans(r0, r1, r2, r3, smem_u32(sv + vrow * AT_PITCH + vdim * 2));
      mma_bf16_16816(o[2 * jp], pa0, 0u, pa2, 0u, r0, r1);
      mma_bf16_16816(o[2 * jp + 1], pa0, 0u, pa2, 0u, r2, r3);
    }
    __syncwarp();   // the stage is refilled by the load issued at the top of the next iteration
  }
  cp_async_wait<0>();

  // ---- partial result of this chunk ----
  constexpr int PW = AT_D + 2;
  float* part = p.ws_partial + ((int64_t)row * p.nsplit + split) * GG * PW;
  if (g < GG) {
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      const int d = 8 * nt + 2 * t4;
      *reinterpret_cast<float2*>(&part[g * PW + d]) = make_float2(o[nt][0], o[nt][1]);
    }
    if (t4 == 0) {
      part[g * PW + AT_D] = m_run;
      part[g * PW + AT_D + 1] = l_run;
    }
  }
}

// Log-sum-exp merge of the nsplit chunk partials of every (list, head): one CTA per (row, head),
// thread d owns output dim d. Chunk maxima / sums are staged in shared memory (one round trip),
// then every thread streams its column with independent loads.
template <int GG>
__global__ void __launch_bounds__(AT_D) attend_merge_kernel(AttendParams p) {
  constexpr int PW = AT_D + 2;
  __shared__ float s_w[64];
  __shared__ float s_ml[2];
  const int row = blockIdx.x / GG, hd = blockIdx.x - row * GG;
  const int b = row / p.Hi, hi = row - b * p.Hi;
  const int head = hi * GG + hd;
  const int d = threadIdx.x;
  pdl_wait();
  const float* parts = p.ws_partial + (int64_t)row * p.nsplit * GG * PW;
  // the first eight partial outputs are requested before the weights are known: one round trip to L2, not two
  const float* col = parts + hd * PW + d;
  float x0[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) x0[u] = (u < p.nsplit) ? __ldcg(col + (int64_t)u * GG * PW) : 0.0f;
  if (d < 32) {
    float m_a = -INFINITY, l_a = 0.0f, m_b = -INFINITY, l_b = 0.0f;
    if (d < p.nsplit) {
      m_a = __ldcg(&parts[(d * GG + hd) * PW + AT_D]);
      l_a = __ldcg(&parts[(d * GG + hd) * PW + AT_D + 1]);
    }
    if (d + 32 < p.nsplit) {
      m_b = __ldcg(&parts[((d + 32) * GG + hd) * PW + AT_D]);
      l_b = __ldcg(&parts[((d + 32) * GG + hd) * PW + AT_D + 1]);
    }
    float M = fmaxf(m_a, m_b);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float Mu = (M == -INFINITY) ? 0.0f : M;
    const float w_a = __expf(m_a - Mu), w_b = __expf(m_b - Mu);    // 0 for absent chunks (m = -inf)
    float L = l_a * w_a + l_b * w_b;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    s_w[d] = w_a;
    s_w[d + 32] = w_b;
    if (d == 0) { s_ml[0] = M; s_ml[1] = L; }
  }
  __syncthreads();
  float O = 0.0f;
#pragma unroll
  for (int u = 0; u < 8; ++u) O += (u < p.nsplit) ? x0[u] * s_w[u] : 0.0f;
  for (int sp = 8; sp < p.nsplit; sp += 8) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = (sp + u < p.nsplit) ? __ldcg(col + (int64_t)(sp + u) * GG * PW) : 0.0f;
#pragma unroll
    for (int u = 0; u < 8; ++u) O += (sp + u < p.nsplit) ? x[u] * s_w[sp + u] : 0.0f;
  }
  const float M = s_ml[0], L = s_ml[1];
  if (p.out) {
    float res = L > 0.0f ? O / L : 0.0f;
    if (p.blend_alpha) {
      const float a = p.blend_alpha[(int64_t)b * p.Hq + head];
      const float vm = p.blend_mean[((int64_t)b * p.Hkv + head / p.G) * AT_D + d];
      res = fmaf(a, res - vm, vm);
    }
    p.out[((int64_t)b * p.Hq + head) * AT_D + d] = __float2bfloat16_rn(res);
  }
  if (p.advance_history && p.T_dev && blockIdx.x == 0 && d == 0) *const_cast<int32_t*>(p.T_dev) += 1;
  if (p.out_partial) {
    float* op = p.out_partial + ((int64_t)b * p.Hq + head) * PW;
    op[d] = O;
    if (d == 0) {
      op[AT_D] = M;
      op[AT_D + 1] = L;
    }
  }
  if (p.ppush.n > 0) {
    // every value goes to every rank as a {bits, step number} pair: no barrier, fence or flag behind it
    const uint32_t epoch = *p.ppush.epoch;
    const int64_t bh = (int64_t)b * p.Hq + head;
    const int64_t o = ((int64_t)p.ppush.rank * p.B * p.Hq + bh) * PW;
    for (int q = 0; q < p.ppush.n; ++q) {
      uint2* op = p.ppush.inbox[q] + o;
      st_pair(op + d, __float_as_uint(O), epoch);
      if (d == 0) {
        st_pair(op + AT_D, __float_as_uint(M), epoch);
        st_pair(op + AT_D + 1, __float_as_uint(L), epoch);
      }
    }
  }
}

// Combine N shard partials into the final bf16 output: grid B*Hq, 128 threads (one per dim).
// With `wait` the partials are an inbox that the ranks fill over NVLink: the CTA first waits (bounded) for
// every rank's flag of its (batch, head).
__global__ void __launch_bounds__(AT_THREADS) lse_merge_kernel(const float* partials, int N, int BH, __nv_bfloat16* out,
                                                               PartialWait wait) {
  constexpr int PW = AT_D + 2;
  const int bh = blockIdx.x, d = threadIdx.x;
  pdl_wait();
  (void)wait;
  float M = -INFINITY;
  for (int r = 0; r < N; ++r) {
    const float* ps = partials + ((int64_t)r * BH + bh) * PW;
    if (__ldcg(ps + AT_D + 1) > 0.0f) M = fmaxf(M, __ldcg(ps + AT_D));
  }
  float L = 0.0f, O = 0.0f;
  if (M != -INFINITY) {
    for (int r = 0; r < N; ++r) {
      const float* ps = partials + ((int64_t)r * BH + bh) * PW;
      const float l = __ldcg(ps + AT_D + 1);
      if (l > 0.0f) {
        const float w = __expf(__ldcg(ps + AT_D) - M);
        L += l * w;
        O += __ldcg(ps + d) * w;
      }
    }
  }
  out[(int64_t)bh * AT_D + d] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
}

// The same combine over pairs {fp32 bits, step number} that the ranks' chunk merges store into this rank's
// inbox: every thread polls (bounded) the pairs it needs until they carry this step's number.
__global__ void __launch_bounds__(AT_THREADS) lse_merge_pairs_kernel(const uint2* partials, int N, int BH,
                                                                     __nv_bfloat16* out, PartialWait wait) {
  constexpr int PW = AT_D + 2;
  const int bh = blockIdx.x, d = threadIdx.x;
  // (no wait for the kernel before it: everything this kernel reads arrives as tagged pairs)
  const uint32_t epoch = *wait.epoch;
  float M = -INFINITY;
  float m_r[KVB_MAX_RANKS], l_r[KVB_MAX_RANKS], o_r[KVB_MAX_RANKS];
#pragma unroll
  for (int r = 0; r < KVB_MAX_RANKS; ++r) {
    m_r[r] = -INFINITY; l_r[r] = 0.0f; o_r[r] = 0.0f;
    if (r < N) {
      const uint2* ps = partials + ((int64_t)r * BH + bh) * PW;
      uint32_t bm, bl, bo;
      if (!wait_pair(ps + AT_D, epoch, wait.limit, bm) || !wait_pair(ps + AT_D + 1, epoch, wait.limit, bl) ||
          !wait_pair(ps + d, epoch, wait.limit, bo))
        return;                                         // gave up (status word set): the output keeps its old contents
      m_r[r] = __uint_as_float(bm); l_r[r] = __uint_as_float(bl); o_r[r] = __uint_as_float(bo);
      if (l_r[r] > 0.0f) M = fmaxf(M, m_r[r]);
    }
  }
  float L = 0.0f, O = 0.0f;
  if (M != -INFINITY) {
#pragma unroll
    for (int r = 0; r < KVB_MAX_RANKS; ++r) {
      if (r < N && l_r[r] > 0.0f) {
        const float w = __expf(m_r[r] - M);
        L += l_r[r] * w;
        O += o_r[r] * w;
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

struct AttendPlan {
  int tiles_per_split, nsplit;
  size_t counter_bytes, partial_bytes, bytes;
};

static AttendPlan attend_plan(int B, int Hq, int Hi, int S) {
  AttendPlan a;
  const int R = B * Hi;
  const int GG = Hq / Hi;
  const int ntiles = ceil_div(S, AT_TILE);
  // As many chunks per list as fit in ONE wave of resident warps: long chunks keep the 3-stage
  // gather pipeline full and make the final merge short.
  int want_splits = AT_TARGET_WARPS / R;
  if (want_splits < 1) want_splits = 1;
  if (want_splits > 64) want_splits = 64;
  int tps = ceil_div(ntiles, want_splits);
  if (tps < 1) tps = 1;
  a.tiles_per_split = tps;
  a.nsplit = ceil_div(ntiles, tps);
  a.counter_bytes = round_up(sizeof(uint32_t) * (size_t)R, 256);
  a.partial_bytes = round_up(sizeof(float) * (size_t)R * a.nsplit * GG * (AT_D + 2), 256);
  a.bytes = a.counter_bytes + a.partial_bytes;
  return a;
}

template <int GG>
static int attend_launch(const AttendParams& p, int device, cudaStream_t st) {
  const size_t smem = (size_t)AT_WARPS * AT_WARP_SMEM;
  auto kern = sparse_attend_kernel<GG>;
  static std::atomic<bool> attr_done[KVB_MAX_DEVICES];
  { const int arc = ensure_dynamic_smem(kern, attr_done, device, smem); if (arc != KVB_OK) return arc; }
  const int tasks = p.B * p.Hi * p.nsplit;
  KVB_CHECK_CUDA(launch_kernel(kern, dim3(ceil_div(tasks, AT_WARPS)), dim3(AT_THREADS), smem, st, p));
  KVB_CHECK_CUDA(cudaGetLastError());
  KVB_CHECK_CUDA(launch_kernel(attend_merge_kernel<GG>, dim3(p.B * p.Hi * GG), dim3(AT_D), 0, st, p));
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
// Device-side history length of the fused step (see AttendParams).
struct AttendDeviceLength {
  const int32_t* T_dev;
  int top_k, protect_sink, protect_recent, keep_self, advance_history;
};

static int attend_run(const void* query, int64_t q_sb, int64_t q_sh, const void* key, int64_t k_sb, int64_t k_sh,
                      int64_t k_st, const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st,
                      const AttendList& list, const AttendAppend* append, const AttendDeviceLength* dev,
                      const float* mask, int64_t mask_sb,
                      int B, int Hq, int Hkv, int Hi, int Tk, int D, int S, float scaling, void* out,
                      float* out_partial, uint32_t* ws_counter, float* ws_partial, bool counters_zeroed, int device,
                      cudaStream_t st, const PartialPush* ppush = nullptr, const float* blend_alpha = nullptr,
                      const float* blend_mean = nullptr, const KvPages* pages = nullptr) {
  if (!query || !key || !value || !ws_counter || !ws_partial) return KVB_BAD_ARG;
  if (list.implicit ? (!list.selected && list.kk > 0) : !list.indices) return KVB_BAD_ARG;
  if (!out && !out_partial && !ppush) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hi <= 0 || Tk <= 0 || S <= 0) return KVB_BAD_SHAPE;
  if (D != AT_D || (Hq % Hkv) || (Hi != Hkv && Hi != Hq)) return KVB_BAD_SHAPE;
  const int GG = Hq / Hi;
  if (GG != 1 && GG != 2 && GG != 4 && GG != 8) return KVB_BAD_SHAPE;
  if ((int64_t)B * Hi > 65535) return KVB_BAD_SHAPE;
  if (!aligned_to(query, 16) || !aligned_to(key, 16) || !aligned_to(value, 16)) return KVB_BAD_ALIGN;
  const bool paged = pages && pages->table;
  if ((q_sb % 8) || (q_sh % 8)) return KVB_BAD_ALIGN;
  if (!paged && ((k_sb % 8) || (k_sh % 8) || (k_st % 8) || (v_sb % 8) || (v_sh % 8) || (v_st % 8))) return KVB_BAD_ALIGN;
  if (!list.implicit && !aligned_to(list.indices, list.idx_is_i64 ? 8 : 4)) return KVB_BAD_ALIGN;
  if (!aligned_to(ws_partial, 16)) return KVB_BAD_ALIGN;
  if (append && append->enabled && (append->C > 128 || (append->C & 1))) return KVB_BAD_SHAPE;
  if (out && !aligned_to(out, 8)) return KVB_BAD_ALIGN;
  const AttendPlan plan = attend_plan(B, Hq, Hi, S);
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;

  AttendParams p;
  p.query = reinterpret_cast<const __nv_bfloat16*>(query); p.q_sb = q_sb; p.q_sh = q_sh;
  p.key = reinterpret_cast<const __nv_bfloat16*>(key); p.k_sb = k_sb; p.k_sh = k_sh; p.k_st = k_st;
  p.value = reinterpret_cast<const __nv_bfloat16*>(value); p.v_sb = v_sb; p.v_sh = v_sh; p.v_st = v_st;
  p.list = list;
  p.mask = mask; p.mask_sb = mask_sb;
  if (append) p.append = *append; else p.append.enabled = 0;
  p.T_dev = dev ? dev->T_dev : nullptr;
  p.top_k = dev ? dev->top_k : 0; p.protect_sink = dev ? dev->protect_sink : 0;
  p.protect_recent = dev ? dev->protect_recent : 0; p.keep_self = dev ? dev->keep_self : 0;
  p.advance_history = dev ? dev->advance_history : 0;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Hi = Hi; p.Tk = Tk; p.S = S; p.G = Hq / Hkv;
  p.scaling = scaling;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.out_partial = out_partial;
  p.ws_counter = ws_counter;
  p.ws_partial = ws_partial;
  p.nsplit = plan.nsplit; p.tiles_per_split = plan.tiles_per_split;
  if (ppush) p.ppush = *ppush;
  p.blend_alpha = blend_alpha; p.blend_mean = blend_mean;
  if (paged) p.pages = *pages;

  (void)counters_zeroed;   // the chunk merge is its own launch: no arrival counters to clear
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
  AttendList list{};
  list.indices = indices; list.idx_is_i64 = idx_is_i64; list.valid = valid; list.implicit = 0;
  return attend_run(query, q_sb, q_sh, key, k_sb, k_sh, k_st, value, v_sb, v_sh, v_st, list, nullptr, nullptr,
                    mask, mask_sb, B, Hq, Hkv, Hi, Tk, D, S, scaling, out, out_partial,
                    reinterpret_cast<uint32_t*>(workspace),
                    reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + plan.counter_bytes),
                    /*counters_zeroed=*/false, device, reinterpret_cast<cudaStream_t>(stream));
}

namespace kvb {
static int attend_selected_impl(
    const void* query, int64_t q_sb, int64_t q_sh, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
    const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st, const int32_t* selected, int kk,
    const int32_t* sel_count, int64_t id_base,
    int history_count, int protect_sink, int protect_recent, int keep_self, int append_protected, const float* mask,
    int64_t mask_sb, int B, int Hq, int Hkv, int Tk, int D, float scaling, void* out, float* out_partial,
    void* workspace, size_t workspace_bytes, const float* blend_alpha, const float* blend_mean, int device,
    void* stream) {
  if (!workspace || (!selected && kk > 0)) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || kk < 0 || history_count < 0 || (Hq % Hkv)) return KVB_BAD_SHAPE;
  if (Tk < history_count + (keep_self ? 1 : 0)) return KVB_BAD_SHAPE;
  if ((blend_alpha == nullptr) != (blend_mean == nullptr)) return KVB_BAD_ARG;
  if (blend_alpha && !out) return KVB_BAD_ARG;
  if (!aligned_to(workspace, 256)) return KVB_BAD_ALIGN;
  const FinalLayout f = final_layout(kk, history_count, protect_sink, protect_recent, keep_self);
  if (f.S <= 0) return KVB_BAD_SHAPE;
  const AttendPlan plan = attend_plan(B, Hq, Hkv, f.S);
  if (workspace_bytes < plan.bytes) return KVB_WORKSPACE_TOO_SMALL;
  AttendList list{};
  list.implicit = 1;
  list.selected = selected; list.kk = kk; list.sel_pitch = kk;
  list.sel_count = sel_count;
  list.sel_base = id_base; list.sel_limit = history_count;
  list.sink_end = f.sink_end; list.n_recent = f.n_recent; list.recent_from = f.recent_from;
  list.recent_start = f.recent_start; list.recent_on = f.recent_on; list.history = history_count;
  list.append_protected = append_protected;
  // the "self" entry of the implicit list is row Tk - 1, so the view must end at the decoded token
  return attend_run(query, q_sb, q_sh, key, k_sb, k_sh, k_st, value, v_sb, v_sh, v_st, list, nullptr, nullptr, mask, mask_sb,
                    B, Hq, Hkv, Hkv, keep_self ? history_count + 1 : history_count, D, f.S, scaling, out, out_partial,
                    reinterpret_cast<uint32_t*>(workspace),
                    reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + plan.counter_bytes),
                    /*counters_zeroed=*/false, device, reinterpret_cast<cudaStream_t>(stream), nullptr, blend_alpha,
                    blend_mean);
}
}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_attend_selected(
    const void* query, int64_t q_sb, int64_t q_sh, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
    const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st, const int32_t* selected, int kk,
    const int32_t* sel_count, int64_t id_base,
    int history_count, int protect_sink, int protect_recent, int keep_self, int append_protected, const float* mask,
    int64_t mask_sb, int B, int Hq, int Hkv, int Tk, int D, float scaling, void* out, float* out_partial,
    void* workspace, size_t workspace_bytes, int device, void* stream) {
  return kvb::attend_selected_impl(query, q_sb, q_sh, key, k_sb, k_sh, k_st, value, v_sb, v_sh, v_st, selected, kk,
                                   sel_count, id_base, history_count, protect_sink, protect_recent, keep_self,
                                   append_protected, mask, mask_sb, B, Hq, Hkv, Tk, D, scaling, out, out_partial,
                                   workspace, workspace_bytes, nullptr, nullptr, device, stream);
}

extern "C" __attribute__((visibility("default"))) int kvb_attend_selected_blend(
    const void* query, int64_t q_sb, int64_t q_sh, const void* key, int64_t k_sb, int64_t k_sh, int64_t k_st,
    const void* value, int64_t v_sb, int64_t v_sh, int64_t v_st, const int32_t* selected, int kk,
    const int32_t* sel_count, int history_count, int keep_self, const float* mask, int64_t mask_sb,
    const float* alpha, const float* value_mean, int B, int Hq, int Hkv, int Tk, int D, float scaling, void* out,
    void* workspace, size_t workspace_bytes, int device, void* stream) {
  if (!alpha || !value_mean || !out) return KVB_BAD_ARG;
  return kvb::attend_selected_impl(query, q_sb, q_sh, key, k_sb, k_sh, k_st, value, v_sb, v_sh, v_st, selected, kk,
                                   sel_count, 0, history_count, 0, 0, keep_self, 0, mask, mask_sb, B, Hq, Hkv, Tk, D,
                                   scaling, out, nullptr, workspace, workspace_bytes, alpha, value_mean, device, stream);
}

extern "C" __attribute__((visibility("default"))) int kvb_lse_merge(const float* partials, int N, int B, int Hq, int D, void* out, int device,
                             void* stream) {
  using namespace kvb;
  if (!partials || !out) return KVB_BAD_ARG;
  if (N <= 0 || B <= 0 || Hq <= 0 || D != AT_D) return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  lse_merge_kernel<<<B * Hq, AT_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      partials, N, B * Hq, reinterpret_cast<__nv_bfloat16*>(out), PartialWait{});
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
