// Sequence-sharded decode step as ONE chain of launches with no collective call in it.
//
// Every rank owns a contiguous token range of the K/V cache and of the int4 side cache. A step is
//   1. sample -> candidate scorer -> exact local top-k, whose kernel also PUSHES its best entries into
//      every rank's inbox (plain 8-byte stores into peer memory over NVLink) and raises a flag there,
//   2. global merge: waits (bounded) for the N flags of its row, selects the global top-k from the local
//      inbox and compacts the winners this rank owns -> attention over those rows -> chunk merge, which
//      pushes the (o, m, l) partial of every (batch, head) to every rank and raises a second flag,
//   3. combine: waits for the N partial flags and merges them by log-sum-exp.
// The flags hold the step number, so nothing is cleared between steps; a rank cannot overwrite data its
// peers still read because it cannot finish step e before it has seen every peer's partial of step e,
// which a peer emits only after its merge of step e has finished. All waits are bounded: a rank that
// never arrives costs a KVB_TIMEOUT in the status word, not a hang.
// Only plain loads and stores touch peer memory: no bulk or tensor copies of any kind.
#include "common.cuh"
#include "score_common.cuh"

namespace kvb {

struct ExchangeLayout {
  int R, BH, kk, prefix;
  size_t off_epoch, off_full, off_inbox, off_flags, off_part, bytes;
};

// Identical on every rank (it depends on the problem shape and the world size only).
static ExchangeLayout exchange_layout(int B, int Hq, int Hkv, int top_k, int world) {
  ExchangeLayout L;
  L.R = B * Hkv;
  L.BH = B * Hq;
  L.kk = top_k;
  L.prefix = 8192 / world < top_k ? 8192 / world : top_k;
  size_t off = 0;
  L.off_epoch = off;  off += 256;
  L.off_full = off;   off += round_up(sizeof(uint64_t) * (size_t)L.R * L.kk, 256);
  L.off_inbox = off;  off += round_up(sizeof(uint4) * (size_t)world * L.R * L.prefix, 256);      // tagged pairs (st_pair2)
  L.off_flags = off;  off += round_up(sizeof(uint32_t) * (size_t)world * L.R, 256);
  L.off_part = off;   off += round_up(sizeof(uint2) * (size_t)world * L.BH * (AT_D + 2), 256);    // {bits, step} pairs
  L.bytes = off;
  return L;
}

struct ShardedStepLayout {
  ShardLayout shard;
  AttendPlan attend;
  size_t off_shard, off_sel, off_owned, off_owned_count, off_attcnt, off_attpart, bytes;
};

static ShardedStepLayout sharded_step_layout(int B, int Hq, int Hkv, int t_local, int top_k, int keep_self) {
  ShardedStepLayout L;
  L.shard = shard_layout(B, Hkv, t_local, top_k);
  // the chunking of the attention differs between a list with and without the decoded token's entry, and
  // the shorter list can have MORE chunks: size for the larger of the two plans
  (void)keep_self;
  const AttendPlan with_self = attend_plan(B, Hq, Hkv, final_layout(top_k, t_local, 0, 0, 1).S);
  const AttendPlan without = attend_plan(B, Hq, Hkv, top_k > 0 ? top_k : 1);
  L.attend = with_self.partial_bytes >= without.partial_bytes ? with_self : without;
  const size_t R = (size_t)B * Hkv;
  size_t off = 0;
  L.off_shard = off;       off += round_up(L.shard.bytes, 256);
  L.off_sel = off;         off += round_up(sizeof(int32_t) * R * top_k, 256);
  L.off_owned = off;       off += round_up(sizeof(int32_t) * R * top_k, 256);
  L.off_owned_count = off; off += round_up(sizeof(int32_t) * R, 256);
  L.off_attcnt = off;      off += L.attend.counter_bytes;
  L.off_attpart = off;     off += L.attend.partial_bytes;
  L.bytes = off;
  return L;
}

// The local top-k of a shard as composites with global ids (sample -> scorer -> exact finish); with `push`
// the finish kernel also delivers the best entries to the ranks' inboxes.
static int shard_candidates_run(const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb,
                                int64_t packed_sh, const float* scale, int64_t scale_sb, int64_t scale_sh,
                                const int32_t* channel_idx, int B, int Hq, int Hkv, int T, int D, int C, int top_k,
                                int split_k, int64_t id_offset, uint64_t* out_comp, void* workspace,
                                size_t workspace_bytes, const PeerPush* push, uint32_t* step_counter,
                                ChainLaunchScope* chain, int device, cudaStream_t st, int32_t* out_idx = nullptr,
                                bool ascending = false) {
  if (!query || !packed || !scale || !channel_idx || (!out_comp && !out_idx) || !workspace) return KVB_BAD_ARG;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || T <= 0 || top_k <= 0 || split_k < 0 || (Hq % Hkv)) return KVB_BAD_SHAPE;
  if (id_offset < 0 || id_offset + T > 0x7fffffffLL) return KVB_BAD_SHAPE;
  if (!aligned_to(workspace, 256)) return KVB_BAD_ALIGN;
  const ShardLayout L = shard_layout(B, Hkv, T, top_k);
  if (workspace_bytes < L.bytes) return KVB_WORKSPACE_TOO_SMALL;
  if (!fast_front_ok(C, Hq / Hkv, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, T, L.kk, L.cap))
    return KVB_BAD_SHAPE;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  uint32_t* count = reinterpret_cast<uint32_t*>(ws + L.off_count);
  float* tau = reinterpret_cast<float*>(ws + L.off_tau);
  uint64_t* cand = reinterpret_cast<uint64_t*>(ws + L.off_cand);
  float* gmax = reinterpret_cast<float*>(ws + L.off_gmax);

  ScoreParams base;
  fill_score_params(base, query, q_sb, q_sh, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, channel_idx, B,
                    Hq, Hkv, T, D, C, nullptr);
  int rc = sample_run(base, tau, top_k, L.cap, st, count, reinterpret_cast<uint32_t*>(ws + L.off_failed), nullptr,
                      step_counter, gmax, device);
  if (rc != KVB_OK) return rc;
  if (chain) chain->on();                       // the kernels after the first start early and wait inside
  ScoreEmit emit{tau, cand, count, L.cap};
  rc = score_run(query, q_sb, q_sh, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, channel_idx, B, Hq, Hkv, T,
                 D, C, nullptr, nullptr, nullptr, nullptr, &emit, nullptr, device, st);
  if (rc != KVB_OK) return rc;
  SelectParams sp;
  sp.scores = gmax; sp.row_stride = T; sp.payload = nullptr;
  sp.R = L.R; sp.T = T; sp.k = top_k; sp.kk = L.kk; sp.idx_offset = id_offset;
  sp.out_idx32 = out_idx; sp.out_idx64 = nullptr; sp.out_scores = nullptr; sp.out_comp = out_comp;
  sp.hist = nullptr; sp.cand = cand; sp.cand_count = count; sp.cap = L.cap;
  sp.tokens_per_cta = 0; sp.thresholds = nullptr;
  sp.order_by_index = 2; sp.use_bitmap = 0;
  sp.from_candidates = 1; sp.row_failed = nullptr; sp.T_dev = nullptr;
  sp.gather = nullptr; sp.gather_n = 0; sp.gather_len = 0; sp.gather_stride = 0;
  sp.rescue = 1; sp.rescue_sp = base;
  sp.split_k = split_k;
  if (push) sp.push = *push;
  size_t smem = (size_t)L.cap * 8 + SEL_FINAL_FIXED_SMEM;
  const size_t bitmap_bytes = sizeof(uint32_t) * (size_t)((T + 31) / 32);
  if (ascending && !out_comp && smem + bitmap_bytes <= SEL_SMEM_LIMIT) {      // ids in ascending order (on-chip bitmap)
    sp.order_by_index = 1; sp.use_bitmap = 1; smem += bitmap_bytes;
  } else if (sp.order_by_index == 2 && smem + select_stage_bytes(L.kk) <= SEL_SMEM_LIMIT) {
    sp.stage = 1; smem += select_stage_bytes(L.kk);                             // coalesced output and pushes
  }
  { const int prc = select_final_prepare(device); if (prc != KVB_OK) return prc; }
  KVB_CHECK_CUDA(launch_kernel(select_final_kernel, dim3(L.R), dim3(SEL_FINAL_THREADS), smem, st, sp));
  return KVB_OK;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) int kvb_shard_candidates(
    const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, const int32_t* channel_idx, int B, int Hq, int Hkv, int T,
    int D, int C, int top_k, int split_k, int64_t id_offset, uint64_t* out_comp, void* workspace,
    size_t workspace_bytes, int device, void* stream) {
  return kvb::shard_candidates_run(query, q_sb, q_sh, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, channel_idx,
                                   B, Hq, Hkv, T, D, C, top_k, split_k, id_offset, out_comp, workspace, workspace_bytes,
                                   nullptr, nullptr, nullptr, device, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" __attribute__((visibility("default"))) int kvb_score_select(
    const void* query, int64_t q_sb, int64_t q_sh, const uint8_t* packed, int64_t packed_sb, int64_t packed_sh,
    const float* scale, int64_t scale_sb, int64_t scale_sh, const int32_t* channel_idx, int B, int Hq, int Hkv, int T,
    int D, int C, int top_k, int ascending, int32_t* out_idx, void* workspace, size_t workspace_bytes, int device,
    void* stream) {
  if (!out_idx) return KVB_BAD_ARG;
  return kvb::shard_candidates_run(query, q_sb, q_sh, packed, packed_sb, packed_sh, scale, scale_sb, scale_sh, channel_idx,
                                   B, Hq, Hkv, T, D, C, top_k, 0, 0, nullptr, workspace, workspace_bytes, nullptr, nullptr,
                                   nullptr, device, reinterpret_cast<cudaStream_t>(stream), out_idx, ascending != 0);
}

// ---- exchange buffers: the only entry points of the library that allocate -------------------------------

extern "C" __attribute__((visibility("default"))) size_t kvb_sharded_exchange_bytes(int B, int Hq, int Hkv, int top_k,
                                                                                    int world) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || top_k <= 0 || world <= 0 || world > kvb::KVB_MAX_RANKS || (Hq % Hkv)) return 0;
  return kvb::exchange_layout(B, Hq, Hkv, top_k, world).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_exchange_alloc(size_t bytes, int device, void** out_ptr,
                                                                         void* out_handle) {
  using namespace kvb;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is published as 64 opaque bytes");
  if (!out_ptr || !out_handle || bytes == 0) return KVB_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  void* ptr = nullptr;
  KVB_CHECK_CUDA(cudaMalloc(&ptr, bytes));
  if (cudaMemset(ptr, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    cudaFree(ptr);
    return KVB_CUDA_ERROR;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
    cudaFree(ptr);
    return KVB_CUDA_ERROR;
  }
  memcpy(out_handle, &h, sizeof(h));
  *out_ptr = ptr;
  return KVB_OK;
}

extern "C" __attribute__((visibility("default"))) int kvb_exchange_open(const void* handle, int device, void** out_ptr) {
  using namespace kvb;
  if (!handle || !out_ptr) return KVB_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* ptr = nullptr;
  KVB_CHECK_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  *out_ptr = ptr;
  return KVB_OK;
}

extern "C" __attribute__((visibility("default"))) int kvb_exchange_close(void* ptr, int device) {
  using namespace kvb;
  if (!ptr) return KVB_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  KVB_CHECK_CUDA(cudaIpcCloseMemHandle(ptr));
  return KVB_OK;
}

extern "C" __attribute__((visibility("default"))) int kvb_exchange_free(void* ptr, int device) {
  using namespace kvb;
  if (!ptr) return KVB_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  KVB_CHECK_CUDA(cudaFree(ptr));
  return KVB_OK;
}

// ---- the step ---------------------------------------------------------------------------------------------

extern "C" __attribute__((visibility("default"))) size_t kvb_sharded_step_workspace_bytes(int B, int Hq, int Hkv,
                                                                                          int t_local, int top_k) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || t_local <= 0 || top_k <= 0 || (Hq % Hkv)) return 0;
  return kvb::sharded_step_layout(B, Hq, Hkv, t_local, top_k, 1).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_sharded_decode_step(const kvb_sharded_step_params* p,
                                                                              int device, void* stream) {
  using namespace kvb;
  if (!p || !p->query || !p->key || !p->value || !p->packed || !p->scale || !p->channel_idx || !p->workspace)
    return KVB_BAD_ARG;
  const int N = p->world, me = p->rank;
  if (N <= 0 || N > KVB_MAX_RANKS || me < 0 || me >= N) return KVB_BAD_ARG;
  if ((p->phases & 7) == 0 || (p->phases & ~7)) return KVB_BAD_ARG;
  if ((p->phases & 4) && !p->out) return KVB_BAD_ARG;
  for (int r = 0; r < N; ++r)
    if (!p->exchange[r] || !aligned_to(p->exchange[r], 256)) return KVB_BAD_ARG;
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || (p->Hq % p->Hkv) || p->t_local <= 0 || p->top_k <= 0 || p->D != AT_D)
    return KVB_BAD_SHAPE;
  if (p->top_k > p->t_local) return KVB_BAD_SHAPE;          // every shard brings top_k entries
  if (p->id_offset < 0 || p->total_tokens <= 0 || p->id_offset + p->t_local > p->total_tokens ||
      p->total_tokens > 0x7fffffffLL)
    return KVB_BAD_SHAPE;
  if (!aligned_to(p->workspace, 256)) return KVB_BAD_ALIGN;
  const int B = p->B, Hq = p->Hq, Hkv = p->Hkv, T = p->t_local, k = p->top_k;
  const int keep_self = me == N - 1 ? 1 : 0;                // the decoded token's row belongs to the last shard
  const ExchangeLayout X = exchange_layout(B, Hq, Hkv, k, N);
  if (p->exchange_bytes < X.bytes) return KVB_WORKSPACE_TOO_SMALL;
  if ((int64_t)N * X.prefix < (int64_t)k) return KVB_BAD_SHAPE;
  const ShardedStepLayout L = sharded_step_layout(B, Hq, Hkv, T, k, 1);
  if (p->workspace_bytes < L.bytes) return KVB_WORKSPACE_TOO_SMALL;
  uint8_t* ws = reinterpret_cast<uint8_t*>(p->workspace);
  uint8_t* mine = reinterpret_cast<uint8_t*>(p->exchange[me]);
  uint32_t* epoch = reinterpret_cast<uint32_t*>(mine + X.off_epoch);
  const uint32_t polls = p->wait_polls ? p->wait_polls : KVB_DEFAULT_WAIT_POLLS;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int32_t* sel = p->sel_idx_out ? p->sel_idx_out : reinterpret_cast<int32_t*>(ws + L.off_sel);
  int32_t* owned = reinterpret_cast<int32_t*>(ws + L.off_owned);
  int32_t* owned_count = reinterpret_cast<int32_t*>(ws + L.off_owned_count);
  ChainLaunchScope chain;
  int rc;

  if (p->phases & 1) {
    PeerPush push;
    push.n = N; push.rank = me; push.prefix = X.prefix; push.epoch = epoch;
    for (int r = 0; r < N; ++r) {
      uint8_t* xr = reinterpret_cast<uint8_t*>(p->exchange[r]);
      push.inbox[r] = reinterpret_cast<uint4*>(xr + X.off_inbox);
      push.flags[r] = reinterpret_cast<uint32_t*>(xr + X.off_flags);
    }
    rc = shard_candidates_run(p->query, p->q_sb, p->q_sh, p->packed, p->packed_sb, p->packed_sh, p->scale, p->scale_sb,
                              p->scale_sh, p->channel_idx, B, Hq, Hkv, T, p->D, p->C, k,
                              X.prefix < k ? X.prefix : 0, p->id_offset, reinterpret_cast<uint64_t*>(mine + X.off_full),
                              ws + L.off_shard, L.shard.bytes, &push, epoch, &chain, device, st);
    if (rc != KVB_OK) return rc;
  }
  if (p->phases & 2) {
    DeviceGuard guard(device);
    if (!guard.ok) return KVB_BAD_DEVICE;
    SelectParams sp;
    sp.scores = nullptr; sp.row_stride = 0; sp.payload = nullptr;
    sp.R = X.R; sp.T = (int)p->total_tokens; sp.k = k; sp.kk = k; sp.idx_offset = 0;
    sp.out_idx32 = sel; sp.out_idx64 = nullptr; sp.out_scores = nullptr; sp.out_comp = nullptr;
    sp.hist = nullptr; sp.cand = nullptr; sp.cand_count = nullptr; sp.cap = select_cap(k);
    sp.tokens_per_cta = 0; sp.thresholds = nullptr;
    sp.from_candidates = 0; sp.row_failed = nullptr; sp.T_dev = nullptr;
    sp.gather = nullptr;                                    // (the prefixes are read from wait.inbox)
    sp.wait.inbox = reinterpret_cast<const uint4*>(mine + X.off_inbox);
    sp.gather_n = N; sp.gather_len = X.kk; sp.gather_stride = (int64_t)X.R * X.prefix; sp.gather_pitch = X.prefix;
    sp.gather_prefix = X.prefix;
    sp.rescue = 0;
    sp.out_owned = owned; sp.out_owned_count = owned_count;
    sp.own_base = p->id_offset; sp.own_limit = p->id_offset + T;
    sp.order_by_index = 2; sp.use_bitmap = 0;
    sp.wait.n = N; sp.wait.flags = reinterpret_cast<const uint32_t*>(mine + X.off_flags); sp.wait.epoch = epoch;
    sp.wait.limit = polls; sp.wait.full_len = X.kk;
    for (int r = 0; r < N; ++r)
      sp.wait.full[r] = reinterpret_cast<const uint64_t*>(reinterpret_cast<uint8_t*>(p->exchange[r]) + X.off_full);
    if ((int64_t)N * X.prefix > (int64_t)sp.cap) return KVB_BAD_SHAPE;
    size_t smem = (size_t)sp.cap * 8 + SEL_FINAL_FIXED_SMEM;
    if (smem + select_stage_bytes(sp.kk) <= SEL_SMEM_LIMIT) { sp.stage = 1; smem += select_stage_bytes(sp.kk); }
    { const int prc = select_final_prepare(device); if (prc != KVB_OK) return prc; }
    KVB_CHECK_CUDA(launch_kernel(select_final_kernel, dim3(X.R), dim3(SEL_FINAL_THREADS), smem, st, sp));
    chain.on();

    const FinalLayout f = final_layout(k, T, 0, 0, keep_self);
    AttendList list{};
    list.implicit = 1;
    list.selected = owned; list.kk = k; list.sel_pitch = k;
    list.sel_count = owned_count;
    list.sel_base = p->id_offset; list.sel_limit = T;
    list.sink_end = f.sink_end; list.n_recent = f.n_recent; list.recent_from = f.recent_from;
    list.recent_start = f.recent_start; list.recent_on = f.recent_on; list.history = T;
    list.append_protected = 0;
    PartialPush pp;
    pp.n = N; pp.rank = me; pp.epoch = epoch;
    for (int r = 0; r < N; ++r) {
      uint8_t* xr = reinterpret_cast<uint8_t*>(p->exchange[r]);
      pp.inbox[r] = reinterpret_cast<uint2*>(xr + X.off_part);
    }
    rc = attend_run(p->query, p->q_sb, p->q_sh, p->key, p->k_sb, p->k_sh, p->k_st, p->value, p->v_sb, p->v_sh, p->v_st,
                    list, nullptr, nullptr, nullptr, 0, B, Hq, Hkv, Hkv, keep_self ? T + 1 : T, p->D, f.S, p->scaling,
                    nullptr, nullptr, reinterpret_cast<uint32_t*>(ws + L.off_attcnt),
                    reinterpret_cast<float*>(ws + L.off_attpart), /*counters_zeroed=*/false, device, st, &pp);
    if (rc != KVB_OK) return rc;
  }
  if (p->phases & 4) {
    DeviceGuard guard(device);
    if (!guard.ok) return KVB_BAD_DEVICE;
    PartialWait pw;
    pw.n = N; pw.epoch = epoch; pw.limit = polls;
    KVB_CHECK_CUDA(launch_kernel(lse_merge_pairs_kernel, dim3(X.BH), dim3(AT_THREADS), 0, st,
                                 reinterpret_cast<const uint2*>(mine + X.off_part), N, X.BH,
                                 reinterpret_cast<__nv_bfloat16*>(p->out), pw));
  }
  return KVB_OK;
}
