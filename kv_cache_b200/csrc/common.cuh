// Shared device/host helpers for the sm_100a kernels of this library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "../../include/kvcache_b200.h"

namespace kvb {

constexpr int KVB_MAX_DEVICES = 64;              // device ordinals the per-device set-up tables cover

// ---- host side -------------------------------------------------------------------------

#define KVB_CHECK_CUDA(expr)                         \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) return KVB_CUDA_ERROR;    \
  } while (0)

// Makes `device` current for the lifetime of the object and restores the previous one.
struct DeviceGuard {
  int prev = -1;
  bool ok = false;
  explicit DeviceGuard(int device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) return;
    if (device < 0 || device >= count) return;
    if (cudaGetDevice(&prev) != cudaSuccess) return;
    if (prev != device && cudaSetDevice(device) != cudaSuccess) return;
    target = device;
    ok = true;
  }
  ~DeviceGuard() {
    if (ok && prev >= 0 && prev != target) cudaSetDevice(prev);
  }
  int target = -1;
};

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Number of SMs of a device (cached per device ordinal).
inline int sm_count(int device) {
  static std::atomic<int> cached[KVB_MAX_DEVICES];
  if (device < 0 || device >= KVB_MAX_DEVICES) return 148;
  int n = cached[device].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cached[device].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Opts `kern` into `bytes` of dynamic shared memory once per device (which must be current). `done` is the
// call site's own table of KVB_MAX_DEVICES flags; concurrent first calls only repeat an idempotent attribute call.
template <typename K>
static inline int ensure_dynamic_smem(K kern, std::atomic<bool>* done, int device, size_t bytes) {
  if (device < 0 || device >= KVB_MAX_DEVICES) return KVB_BAD_DEVICE;
  if (!done[device].load(std::memory_order_acquire)) {
    KVB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    done[device].store(true, std::memory_order_release);
  }
  return KVB_OK;
}

// Sticky device status word. The library is built as ONE translation unit (kvcache_b200.cu
// includes every kernel file), so there is one copy per loaded library per device.
static __device__ int g_device_status = 0;

// ---- device side -----------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Order-preserving map fp32 -> uint32 (larger float <=> larger key); -0 is folded into +0
// first so both zeros share one key.
__device__ __forceinline__ uint32_t float_to_key(float v) {
  uint32_t u = __float_as_uint(v);
  if (u == 0x80000000u) u = 0u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_to_float(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// Unique 64-bit sort key of (score, index): larger composite <=> better score, then LOWER index.
__device__ __forceinline__ uint64_t make_composite(float score, uint32_t idx) {
  return ((uint64_t)float_to_key(score) << 32) | (uint64_t)(0xFFFFFFFFu - idx);
}

// ---- mbarrier + bulk async copy (TMA engine, 1-D, no tensor map, one destination CTA) ----------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll itself blocks for a hardware time
// slice), records KVB_TIMEOUT in the sticky status word and reports failure to the caller,
// which must then leave its loop without touching the stage.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  atomicExch(&g_device_status, (int)KVB_TIMEOUT);
  return false;
}
// global -> shared bulk copy; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// Same with an L2 evict-first policy: the packed K stream is read exactly once per step.
__device__ __forceinline__ void bulk_g2s_evict_first(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                                     uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
          "r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

__device__ __forceinline__ void st_global_hint_f32(float* p, float v, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(p), "f"(v), "l"(policy) : "memory");
}

// ---- cp.async (LDGSTS) 16-byte copies ---------------------------------------------------

__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src_gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- misc ------------------------------------------------------------------------------

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}


// ---- exchange between the ranks of a sequence-sharded step (plain loads/stores over NVLink) ------
// A rank publishes data into a buffer that lives in ANOTHER rank's memory (mapped into this process),
// then raises a flag there; the consumer polls its own local flag and reads its own local memory.
// Flags carry the step number, so nothing is ever cleared.
constexpr int KVB_MAX_RANKS = 8;

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait for *flag == want: gives up after `limit` polls, records KVB_TIMEOUT in the sticky status
// word and returns false; the caller must then finish without using the data the flag guards.
__device__ __forceinline__ bool wait_flag_bounded(const uint32_t* flag, uint32_t want, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (ld_acquire_sys_u32(flag) == want) return true;
    __nanosleep(128);
  }
  atomicExch(&g_device_status, (int)KVB_TIMEOUT);
  return false;
}
constexpr uint32_t KVB_DEFAULT_WAIT_POLLS = 1u << 22;       // a few seconds at ~1 us per poll

// Producer side of the candidate exchange (local top-k kernel): the `prefix` best composites of every row
// go to slot [rank, row, 0..prefix) of every rank's inbox, then flag [rank, row] of that rank is set.
struct PeerPush {
  int n = 0;                              // ranks; 0 = no exchange
  int rank = 0;
  int prefix = 0;                         // entries per (rank, row) slot
  uint4* inbox[KVB_MAX_RANKS] = {};       // rank q's inbox  [n, R, prefix] composites as tagged pairs (st_pair2)
  uint32_t* flags[KVB_MAX_RANKS] = {};    // rank q's flags  uint32 [n, R]: raised when the rank's WHOLE list may be read
  const uint32_t* epoch = nullptr;        // this rank's step counter
};
// Consumer side (global merge kernel): polls the tagged pairs of the local inbox; `full[s]` is rank s's whole
// local list uint64 [R, full_len] (peer memory, read only when the prefixes cannot decide a row, and then only
// after flags [s, row] == epoch for every rank s).
struct PeerWait {
  int n = 0;
  const uint4* inbox = nullptr;           // local, [n, R, prefix]
  const uint32_t* flags = nullptr;        // local, uint32 [n, R]
  const uint32_t* epoch = nullptr;
  uint32_t limit = KVB_DEFAULT_WAIT_POLLS;
  const uint64_t* full[KVB_MAX_RANKS] = {};
  int full_len = 0;
};
// Flag-in-data pairs: a value travels as one naturally aligned 8-byte store {value bits, step number}; a reader
// that sees the step number it expects has the value of that step, with no fence on either side and no
// separate flag (an 8-byte store is delivered whole). A system-scope release after a CTA's stores costs about
// 3.5 us here; this costs the flight time of the store.
__device__ __forceinline__ void st_pair(uint2* p, uint32_t bits, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(bits), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
// Polls (bounded) until the pair carries `tag`; false (status word set) when it gives up.
__device__ __forceinline__ bool wait_pair(const uint2* p, uint32_t tag, uint32_t limit, uint32_t& bits) {
  for (uint32_t i = 0; i < limit; ++i) {
    const uint2 v = ld_pair(p);
    if (v.y == tag) { bits = v.x; return true; }
    __nanosleep(64);
  }
  atomicExch(&g_device_status, (int)KVB_TIMEOUT);
  return false;
}

// A 64-bit value as two pairs in one 16-byte store {high word, step number, low word, step number}: each 8-byte
// half carries its own tag, so the halves may arrive apart.
__device__ __forceinline__ void st_pair2(uint4* p, uint64_t v, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"((uint32_t)(v >> 32)), "r"(tag),
               "r"((uint32_t)v), "r"(tag)
               : "memory");
}
__device__ __forceinline__ uint4 ld_pair2(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// `first` is an earlier load of the same place; polls (bounded) until both halves carry `tag`.
__device__ __forceinline__ bool wait_pair2(const uint4* p, uint4 first, uint32_t tag, uint32_t limit, uint64_t& v) {
  uint4 w = first;
  for (uint32_t i = 0; i < limit; ++i) {
    if (w.y == tag && w.w == tag) { v = ((uint64_t)w.x << 32) | w.z; return true; }
    __nanosleep(64);
    w = ld_pair2(p);
  }
  atomicExch(&g_device_status, (int)KVB_TIMEOUT);
  return false;
}

// The attention partials of every (rank, batch, query head): D+2 pairs {fp32 bits, step number} [n, B*Hq, D+2].
struct PartialPush {
  int n = 0, rank = 0;
  uint2* inbox[KVB_MAX_RANKS] = {};
  const uint32_t* epoch = nullptr;
};
struct PartialWait {
  int n = 0;
  const uint32_t* epoch = nullptr;
  uint32_t limit = KVB_DEFAULT_WAIT_POLLS;
};

// ---- programmatic dependent launch ------------------------------------------------------------
// Inside a chain of kernels on one stream the next kernel may be made resident while the current
// one still runs: its blocks start, do whatever does not depend on the predecessor and then block
// in pdl_wait() until the predecessor has completed and its writes are visible. Both instructions
// are no-ops in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- paged K/V: pools bf16 [num_pages, Hkv, page_tokens, D] addressed through a per-sequence page table ----
struct KvPages {
  const int32_t* table = nullptr;   // int32 [B, table_stride]: page id of logical page t >> shift of batch row b
  int64_t table_stride = 0;
  int shift = 0;                    // log2(page_tokens)
};
// Row of token t of (batch row b, KV head h) inside a pool, in units of one D-element row.
__device__ __forceinline__ int64_t kv_paged_row(const KvPages& pg, int Hkv, int b, int h, int t) {
  const int page = pg.table[(int64_t)b * pg.table_stride + (t >> pg.shift)];
  return (((int64_t)page * Hkv + h) << pg.shift) + (int64_t)(t & ((1 << pg.shift) - 1));
}

// Whether launches made by this host thread ask for the early start (set only while a fused chain
// whose kernels all begin with pdl_wait() is being enqueued).
static thread_local bool t_chain_launch = false;
struct ChainLaunchScope {
  bool prev;
  ChainLaunchScope() : prev(t_chain_launch) {}
  void on() { t_chain_launch = true; }
  ~ChainLaunchScope() { t_chain_launch = prev; }
};

template <typename... KArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                        Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = t_chain_launch ? attr : nullptr;
  cfg.numAttrs = t_chain_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

}  // namespace kvb
