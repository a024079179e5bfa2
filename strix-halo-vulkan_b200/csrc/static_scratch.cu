// One projection entry point for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off the table at the moment a projection
// is needed: a latency-critical serving or audio thread that may not block on the allocator's
// lock (cudaMalloc and cudaFree serialise on it and may synchronise the device), or a process
// whose device memory was handed out up front and is policed. b200_qgemv() stages the
// activations as fp16 in a temporary that it allocates per call; this variant keeps that
// staging area, and the word a timed-out wait is reported through, in file-scope device
// arrays instead, so the call allocates nothing.
#include "kernels.cuh"
#include "model.h"

namespace b200 {

constexpr int STATIC_MAX_ROWS = 8;        // activation rows per call
constexpr int STATIC_MAX_K = 16384;       // row length
// fp16 staging of the activations: 8 x 16384 halves = 256 KiB, held by every device that loads
// the library until the process exits. Shared by all calls and never cleared: each call
// overwrites the part it reads, so calls that overlap on the device race on it.
static __device__ __align__(256) __half g_static_x16[STATIC_MAX_ROWS * STATIC_MAX_K];
// set by the kernel when one of its bounded waits gives up; cleared at the start of every call
static __device__ __align__(256) int g_static_err[64];

struct StaticScratch { __half* x16; int* err; };
static StaticScratch g_scratch[MAX_DEVICES];
static std::atomic<int> g_scratch_ready[MAX_DEVICES];

// In host code the arrays' names are host-side stand-ins, not device addresses; the kernels need the
// device addresses, looked up once per device with that device current.
static int scratch_for_current_device(StaticScratch* out) {
  const int slot = current_device_slot();
  if (g_scratch_ready[slot].load(std::memory_order_acquire) == 0) {
    StaticScratch s{};
    B200_CUDA(cudaGetSymbolAddress((void**)&s.x16, g_static_x16));
    B200_CUDA(cudaGetSymbolAddress((void**)&s.err, g_static_err));
    g_scratch[slot] = s;
    g_scratch_ready[slot].store(1, std::memory_order_release);
  }
  *out = g_scratch[slot];
  return OK;
}

// Shared memory the projection kernel needs for m staged rows of length k plus one stage of weight
// tiles; the launch is refused when it exceeds what an SM offers (the same sum launch_qgemv checks).
static size_t static_smem_need(uint32_t type, int64_t k, int m) {
  return qg_fixed_smem((int)k, m, false) + qg_stage_bytes((int)k, device_row_stride(type, k), false);
}
constexpr size_t STATIC_SMEM_BUDGET = 220 * 1024;

int qgemv_static(uint32_t type, const void* dev_w, int64_t rows, int64_t k, const float* dev_x, int32_t m, float* dev_y) {
  if (!dev_w || !dev_x || !dev_y) { set_error("qgemv_static: null pointer"); return EINVAL_; }
  if (type != T_Q4_K && type != T_Q5_K) { set_error("qgemv_static: Q4_K and Q5_K only (their checkpoint layout is the device layout)"); return EINVAL_; }
  if (m < 1 || m > STATIC_MAX_ROWS) { set_error("qgemv_static: at most 8 activation rows per call"); return ECAPACITY; }
  if (k < 256 || k > STATIC_MAX_K || k % 256) { set_error("qgemv_static: row length must be a multiple of 256, at most 16384"); return ECAPACITY; }
  if (rows < 1 || rows > (1 << 24)) { set_error("qgemv_static: row count out of range"); return ECAPACITY; }
  if (((uintptr_t)dev_w & 15) || ((uintptr_t)dev_x & 15)) { set_error("qgemv_static: weights and activations must be 16-byte aligned"); return EINVAL_; }
  if (static_smem_need(type, k, m) > STATIC_SMEM_BUDGET) {
    int fit = 0;
    for (int mm = 1; mm < m; mm++) if (static_smem_need(type, k, mm) <= STATIC_SMEM_BUDGET) fit = mm;
    set_error("qgemv_static: " + std::to_string(m) + " rows of " + std::to_string(k) + " elements need " + std::to_string(static_smem_need(type, k, m)) +
              " bytes of shared-memory staging and the kernel has " + std::to_string(STATIC_SMEM_BUDGET) + ": at this row length " +
              (fit > 0 ? "at most " + std::to_string(fit) + " rows fit" : std::string("no row fits")));
    return ECAPACITY;
  }
  StaticScratch sc{};
  B200_TRY(scratch_for_current_device(&sc));
  B200_CUDA(cudaMemsetAsync(sc.err, 0, sizeof(int), 0));
  B200_TRY(quantize_rows_device(T_F16, dev_x, m, k, (uint8_t*)sc.x16, 0));
  QGemvParams p{};
  p.w[0] = (const uint8_t*)dev_w; p.seg_end[0] = (int)rows; p.nseg = 1; p.stride = device_row_stride(type, k);
  p.K = (int)k; p.N = (int)rows; p.M = m; p.xcols = m; p.x = sc.x16; p.ldx = k; p.y = dev_y; p.ldy = rows; p.x_div = 1; p.err = sc.err;
  B200_TRY(launch_qgemv(type, PRO_F16, EPI_STORE, false, false, p, 0, false, 0));
  int herr = 0;
  B200_CUDA(cudaMemcpy(&herr, sc.err, sizeof(int), cudaMemcpyDeviceToHost));  // also waits for the work
  if (herr != 0) { set_error("qgemv_static: a bounded wait for the weight copies gave up; dev_y is not valid"); return ETIMEOUT; }
  return OK;
}

}  // namespace b200
