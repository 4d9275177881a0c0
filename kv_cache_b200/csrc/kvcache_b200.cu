// The whole library as ONE translation unit: every kernel file is included here so that the
// sticky device status word and the helpers of common.cuh exist once per loaded library.
#include "common.cuh"

#include "quantize.cu"
#include "score_decode.cu"
#include "select_topk.cu"
#include "sparse_attend.cu"
#include "decode_step.cu"
#include "sharded_step.cu"
#include "rerank.cu"
#include "sparq.cu"
#include "score_prefill_tc.cu"
#include "score_prefill.cu"
#include "qabs_fp32.cu"

extern "C" __attribute__((visibility("default"))) int kvb_version(void) { return 100; /* 0.1.0 */ }

extern "C" __attribute__((visibility("default"))) const char* kvb_status_string(int status) {
  switch (status) {
    case KVB_OK: return "ok";
    case KVB_BAD_SHAPE: return "bad shape";
    case KVB_BAD_ALIGN: return "bad alignment";
    case KVB_BAD_DEVICE: return "bad device";
    case KVB_WORKSPACE_TOO_SMALL: return "workspace too small";
    case KVB_TIMEOUT: return "device-side wait timed out";
    case KVB_CUDA_ERROR: return "CUDA error";
    case KVB_BAD_ARG: return "bad argument";
    case KVB_SCRATCH_LIMIT: return "problem exceeds the built-in scratch";
    default: return "unknown status";
  }
}

extern "C" __attribute__((visibility("default"))) int kvb_device_status(int device, int* out_status) {
  using namespace kvb;
  if (!out_status) return KVB_BAD_ARG;
  DeviceGuard guard(device);
  if (!guard.ok) return KVB_BAD_DEVICE;
  int v = 0;
  KVB_CHECK_CUDA(cudaDeviceSynchronize());
  KVB_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
  const int zero = 0;
  KVB_CHECK_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
  *out_status = v;
  return KVB_OK;
}
