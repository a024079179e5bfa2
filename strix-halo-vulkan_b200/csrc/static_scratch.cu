// One projection entry point for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off the table: inside a stream capture,
// inside a real-time audio/serving thread that may not take the allocator's lock, or in a
// process whose memory budget was handed out up front and is policed. b200_qgemv() stages the
// activations as fp16 in a temporary it allocates per call; this variant keeps that staging
// area in a file-scope device array instead, so the call allocates nothing.
#include "kernels.cuh"
#include "model.h"

namespace b200 {

constexpr int STATIC_MAX_ROWS = 8;        // activation rows per call
constexpr int STATIC_MAX_K = 16384;       // row length
// fp16 staging of the activations: 8 x 16384 halves = 256 KiB, held by every device that loads
// the library until the process exits. Shared by all calls and never cleared: each call
// overwrites the part it reads, so calls that overlap on the device race on it.
static __device__ __align__(256) __half g_static_x16[STATIC_MAX_ROWS * STATIC_MAX_K];

constexpr int MAX_DEVICES = 64;
static __half* g_scratch_ptr[MAX_DEVICES];
static bool g_scratch_ready[MAX_DEVICES];

// The array's name is only a host-side stand-in; the kernel needs the device address, looked
// up once per device with that device current.
static int scratch_for_current_device(__half** out) {
  int dev = 0;
  B200_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) { set_error("qgemv_static: device index out of range"); return EINVAL_; }
  if (!g_scratch_ready[dev]) {
    __half* p = nullptr;
    B200_CUDA(cudaGetSymbolAddress((void**)&p, g_static_x16));
    g_scratch_ptr[dev] = p;
    g_scratch_ready[dev] = true;
  }
  *out = g_scratch_ptr[dev];
  return OK;
}

int qgemv_static(uint32_t type, const void* dev_w, int64_t rows, int64_t k, const float* dev_x, int32_t m, float* dev_y) {
  if (!dev_w || !dev_x || !dev_y) { set_error("qgemv_static: null pointer"); return EINVAL_; }
  if (type != T_Q4_K && type != T_Q5_K) { set_error("qgemv_static: Q4_K and Q5_K only (their checkpoint layout is the device layout)"); return EINVAL_; }
  if (m < 1 || m > STATIC_MAX_ROWS) { set_error("qgemv_static: at most 8 activation rows per call"); return ECAPACITY; }
  if (k < 256 || k > STATIC_MAX_K || k % 256) { set_error("qgemv_static: row length must be a multiple of 256, at most 16384"); return ECAPACITY; }
  if (rows < 1 || rows > (1 << 24)) { set_error("qgemv_static: row count out of range"); return ECAPACITY; }
  if (((uintptr_t)dev_w & 15) || ((uintptr_t)dev_x & 15)) { set_error("qgemv_static: weights and activations must be 16-byte aligned"); return EINVAL_; }
  __half* x16 = nullptr;
  B200_TRY(scratch_for_current_device(&x16));
  B200_TRY(quantize_rows_device(T_F16, dev_x, m, k, (uint8_t*)x16, 0));
  QGemvParams p{};
  p.w[0] = (const uint8_t*)dev_w; p.seg_end[0] = (int)rows; p.nseg = 1; p.stride = device_row_stride(type, k);
  p.K = (int)k; p.N = (int)rows; p.M = m; p.xcols = m; p.x = x16; p.ldx = k; p.y = dev_y; p.ldy = rows; p.x_div = 1;
  B200_TRY(launch_qgemv(type, PRO_F16, EPI_STORE, false, false, p, 0, false, 0));
  B200_CUDA(cudaStreamSynchronize(0));
  return OK;
}

}  // namespace b200
