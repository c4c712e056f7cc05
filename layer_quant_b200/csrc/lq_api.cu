// Library-level entry points: ABI version, last-error text, device properties.
#include "lq_common.cuh"

namespace lq {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int int4_read_device_status(int32_t* status);  // lq_int4_kv.cu

}  // namespace lq

LQ_EXPORT int lq_abi_version(void) { return LQ_ABI_VERSION; }

// sizeof of the ABI structs, so that a binding can check its own mirror of them
LQ_EXPORT int lq_abi_sizeof(int which) {
  switch (which) {
    case 0: return (int)sizeof(lq_mx_state);
    case 1: return (int)sizeof(lq_rounding);
    case 2: return (int)sizeof(lq_mx_update_args);
    case 3: return (int)sizeof(lq_int4_cache);
    case 4: return (int)sizeof(lq_int4_decode_args);
    case 5: return (int)sizeof(lq_dense_update_args);
    case 6: return (int)sizeof(lq_conv1d_update_args);
    case 7: return (int)sizeof(lq_int4_prefill_args);
    default: return -1;
  }
}

LQ_EXPORT const char* lq_last_error_string(void) { return lq::last_error_buffer(); }

LQ_EXPORT int lq_device_status(int32_t* status) {
  LQ_CHECK_ARG(status != nullptr, "lq_device_status: null pointer");
  return lq::int4_read_device_status(status);
}
