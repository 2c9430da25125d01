// Library-level entry points: version, status text, device check.
#include "plq_common.cuh"

namespace plq {

thread_local int g_last_cuda_error = 0;

namespace {
struct DevInfo { int checked; int ok; int sms; };
DevInfo g_dev[64];
}  // namespace

static DevInfo* dev_info() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  DevInfo* d = &g_dev[dev];
  if (!d->checked) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) return nullptr;
    d->ok = (p.major == 10);
    d->sms = p.multiProcessorCount;
    d->checked = 1;
  }
  return d;
}

int device_check() {
  DevInfo* d = dev_info();
  return (d && d->ok) ? PLQ_OK : PLQ_ERR_ARCH;
}

int sm_count() {
  DevInfo* d = dev_info();
  return d ? d->sms : 0;
}

}  // namespace plq

extern "C" int plq_version(void) { return 100; }

extern "C" const char* plq_status_string(int status) {
  switch (status) {
    case PLQ_OK: return "ok";
    case PLQ_ERR_NULL: return "a required pointer is NULL";
    case PLQ_ERR_SHAPE: return "unsupported shape (need K_lo % 64 == 0, K_hi % 32 == 0, K % 128 == 0 with rotation/norm, N % 8 == 0, 1 <= m)";
    case PLQ_ERR_ALIGN: return "a pointer or leading dimension is not 16-byte aligned";
    case PLQ_ERR_ARCH: return "the current CUDA device is not compute capability 10.x (B200); there is no fallback path";
    case PLQ_ERR_CUDA: return "a CUDA runtime call failed (see plq_last_cuda_error)";
    case PLQ_ERR_TENSORMAP: return "cuTensorMapEncodeTiled rejected a tensor map";
    case PLQ_ERR_LIMIT: return "a size exceeds a documented maximum";
    case PLQ_DEV_TIMEOUT: return "a bounded wait inside a kernel ran out; the output is undefined";
    case PLQ_DEV_PROTOCOL: return "a fused reduction was called on the wrong one of its two buffer sets (calls must alternate; a replayed CUDA graph must hold an even number of them); the output is undefined";
    case PLQ_DEV_RANGE: return "a cache position read from device memory was outside the cache; nothing was stored for it";
    default: return "unknown status";
  }
}

extern "C" int plq_last_cuda_error(void) { return plq::g_last_cuda_error; }

extern "C" int plq_device_check(void) { return plq::device_check(); }

extern "C" int64_t plq_sf_tiled_bytes(int64_t rows, int64_t n_sf) {
  if (rows < 0 || n_sf < 0) return 0;
  return ((rows + 127) / 128) * ((n_sf + 3) / 4) * 512;
}
