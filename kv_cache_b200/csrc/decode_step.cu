// Fused per-layer decode step: quantize-append, score (+histogram), select, final index list,
// attend — six stream-ordered launches sharing one caller-provided workspace. Intermediate
// tensors (group-max scores, histogram, selected ids, final list) never leave the workspace.
#include "common.cuh"

namespace kvb {

// Workspace of the fused step. The regions that must start at zero (attention split counters,
// select candidate counters, histogram) are adjacent so ONE memset per step clears them.
struct StepLayout {
  int R, kk, S;
  size_t off_attcnt, off_selws, off_attpart, off_gmax, off_sel;
  size_t zero_bytes, selws_bytes, bytes;
};

static StepLayout step_layout(int B, int Hq, int Hkv, int T, int k, int sink, int recent, int keep_self) {
  StepLayout L;
  L.R = B * Hkv;
  L.kk = k < T ? k : T;
  L.S = kvb_final_index_count(L.kk, T, sink, recent, keep_self);
  const SelectWorkspace sw = select_carve(nullptr, L.R, L.kk > 0 ? L.kk : 1);
  const AttendPlan ap = attend_plan(B, Hq, Hkv, L.S > 0 ? L.S : 1);
  size_t off = 0;
  L.off_attcnt = off;  off += ap.counter_bytes;
  L.off_selws = off;   off += round_up(sw.bytes, 256);
  L.selws_bytes = sw.bytes;
  L.zero_bytes = ap.counter_bytes + sw.zero_bytes;       // attention counters + select counters + histogram
  L.off_attpart = off; off += ap.partial_bytes;
  L.off_gmax = off;    off += round_up(sizeof(float) * (size_t)L.R * (size_t)T, 256);
  L.off_sel = off;     off += round_up(sizeof(int32_t) * (size_t)L.R * (size_t)(L.kk > 0 ? L.kk : 1), 256);
  L.bytes = off;
  return L;
}

}  // namespace kvb

extern "C" __attribute__((visibility("default"))) size_t kvb_decode_step_workspace_bytes(
    int B, int Hq, int Hkv, int history_count, int top_k, int protect_sink, int protect_recent, int keep_self) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || history_count < 0 || top_k <= 0 || (Hq % Hkv)) return 0;
  return kvb::step_layout(B, Hq, Hkv, history_count, top_k, protect_sink, protect_recent, keep_self).bytes;
}

extern "C" __attribute__((visibility("default"))) int kvb_decode_step(const kvb_decode_step_params* p, int device,
                                                                      void* stream) {
  using namespace kvb;
  if (!p || !p->query || !p->key || !p->value || !p->packed || !p->scale || !p->channel_idx || !p->out ||
      !p->workspace)
    return KVB_BAD_ARG;
  if (p->B <= 0 || p->Hq <= 0 || p->Hkv <= 0 || (p->Hq % p->Hkv) || p->history_count <= 0 || p->top_k <= 0)
    return KVB_BAD_SHAPE;
  if (p->top_k > SEL_MAX_K && p->history_count > SEL_MAX_K) return KVB_BAD_SHAPE;
  if (!aligned_to(p->workspace, 256)) return KVB_BAD_ALIGN;
  const int T = p->history_count;
  const StepLayout L = step_layout(p->B, p->Hq, p->Hkv, T, p->top_k, p->protect_sink, p->protect_recent,
                                   p->keep_self);
  if (p->workspace_bytes < L.bytes) return KVB_WORKSPACE_TOO_SMALL;
  if (L.S <= 0) return KVB_BAD_SHAPE;
  uint8_t* ws = reinterpret_cast<uint8_t*>(p->workspace);
  uint32_t* attcnt = reinterpret_cast<uint32_t*>(ws + L.off_attcnt);
  void* selws = ws + L.off_selws;
  const SelectWorkspace sw = select_carve(selws, L.R, L.kk);
  float* attpart = reinterpret_cast<float*>(ws + L.off_attpart);
  float* gmax = reinterpret_cast<float*>(ws + L.off_gmax);
  int32_t* sel = p->sel_idx_out ? p->sel_idx_out : reinterpret_cast<int32_t*>(ws + L.off_sel);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc;

  {
    DeviceGuard guard(device);
    if (!guard.ok) return KVB_BAD_DEVICE;
    KVB_CHECK_CUDA(cudaMemsetAsync(ws + L.off_attcnt, 0, L.zero_bytes, st));
  }
  rc = kvb_score_decode(p->query, p->q_sb, p->q_sh, p->packed, p->packed_sb, p->packed_sh, p->scale, p->scale_sb,
                        p->scale_sh, p->channel_idx, p->B, p->Hq, p->Hkv, T, p->D, p->C, gmax, nullptr, nullptr,
                        sw.hist, device, stream);
  if (rc != KVB_OK) return rc;
  // ascending-index order: the set is what matters to the attention, and it is the cheapest to emit
  rc = select_run(gmax, T, nullptr, L.R, T, p->top_k, 0, /*order=*/1, sel, nullptr, nullptr, nullptr,
                  /*hist_in_workspace=*/true, /*zeroed=*/true, selws, L.selws_bytes, device, st);
  if (rc != KVB_OK) return rc;
  // The attention kernel reads the list  selected || sink || recent || self  implicitly (no list is
  // materialised) and its chunk-0 warps append the decoded token's K row to the int4 cache.
  const FinalLayout f = final_layout(L.kk, T, p->protect_sink, p->protect_recent, p->keep_self);
  AttendList list{};
  list.implicit = 1;
  list.selected = sel; list.kk = L.kk;
  list.sel_base = 0; list.sel_limit = T;
  list.sink_end = f.sink_end; list.n_recent = f.n_recent; list.recent_from = f.recent_from;
  list.recent_start = f.recent_start; list.recent_on = f.recent_on; list.history = T;
  list.append_protected = p->append_protected;
  AttendAppend ap{};
  ap.enabled = p->append_self ? 1 : 0;
  ap.channel_idx = p->channel_idx; ap.C = p->C;
  ap.packed = p->packed; ap.packed_sb = p->packed_sb; ap.packed_sh = p->packed_sh;
  ap.scale = p->scale; ap.scale_sb = p->scale_sb; ap.scale_sh = p->scale_sh;
  ap.t_src = T; ap.t_dst = T;
  rc = attend_run(p->query, p->q_sb, p->q_sh, p->key, p->k_sb, p->k_sh, p->k_st, p->value, p->v_sb, p->v_sh, p->v_st,
                  list, &ap, p->mask, p->mask_sb, p->B, p->Hq, p->Hkv, p->Hkv, T + 1, p->D, L.S, p->scaling,
                  p->out, nullptr, attcnt, attpart, /*counters_zeroed=*/true, device, st);
  if (rc != KVB_OK) return rc;
  return KVB_OK;
}
