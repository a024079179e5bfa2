// Shared declarations of the B200 token-loop library: status codes, ggml type ids,
// device-side tensor descriptors and small device helpers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <string>

namespace b200 {

enum Status : int32_t { OK = 0, EINVAL_ = 1, ECAPACITY = 2, ECUDA = 3, ENCCL = 4, ETIMEOUT = 5, ESTATE = 6, ENOMEM_ = 7, EIO_ = 8 };

// ggml tensor types (reference: gguf/gguf.go:53-88)
enum : uint32_t { T_F32 = 0, T_F16 = 1, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ4_NL = 20, T_BF16 = 30 };

bool block_geometry(uint32_t type, int* elems, int* nbytes);  // reference: gguf/gguf.go:101-134
int64_t gguf_row_bytes(uint32_t type, int64_t n);

// A weight matrix on the device. Q4_K / Q5_K keep the checkpoint's own 144 / 176-byte
// super-blocks (16-byte aligned). Q6_K and Q8_0 blocks are 210 / 34 bytes, which no
// 128-bit load can address, so each ROW is re-laid as planes (same bytes, permuted):
//   Q6_K row of nb blocks: ql[nb][128] | qh[nb][64] | scales[nb][16] | d[nb] (fp16)
//   Q8_0 row of nb blocks: qs[nb][32] | d[nb] (fp16)
// with the row stride rounded up to 16 bytes.
struct DTensor {
  uint32_t type = 0;
  int64_t k = 0;        // row length (ggml dims[0])
  int64_t rows = 0;     // product of the remaining dims
  int64_t stride = 0;   // bytes per row on the device
  uint8_t* data = nullptr;
  bool ok() const { return data != nullptr; }
};

void set_error(const std::string& s);
const char* last_error();

#define B200_CUDA(expr)                                                                          \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess) {                                                                     \
      b200::set_error(std::string(#expr) + ": " + cudaGetErrorString(_e));                       \
      return b200::ECUDA;                                                                        \
    }                                                                                            \
  } while (0)

// Settings made with cudaFuncSetAttribute, and the SM count, belong to the device that is current when
// they are made or read, and one process may hold graphs on several devices (the ABI takes a device
// index per model): "done once" is therefore kept per device. Handles may be driven from different
// threads, so the marks are atomic; two threads that both find a mark unset both make the (idempotent) setting.
constexpr int MAX_DEVICES = 64;
struct OncePerDevice {
  std::atomic<int> done[MAX_DEVICES];
};
inline int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
  return dev % MAX_DEVICES;
}
// SM count of the current device (cached per device); 0 on failure with the error set
int sm_count_current();

#define B200_ONCE_PER_DEVICE(expr)                                   \
  do {                                                               \
    static b200::OncePerDevice _once;                                \
    const int _slot = b200::current_device_slot();                   \
    if (_once.done[_slot].load(std::memory_order_acquire) == 0) {    \
      B200_CUDA(expr);                                               \
      _once.done[_slot].store(1, std::memory_order_release);         \
    }                                                                \
  } while (0)

#define B200_TRY(expr)                   \
  do {                                   \
    int _s = (expr);                     \
    if (_s != b200::OK) return _s;       \
  } while (0)

// Optional per-launch phase timestamps (the reference keeps GPU timestamps per dispatch:
// vk/shim.h:222-229, llm/graph.go:527-589). buf == nullptr switches them off.
struct Timeline {
  long long* buf;  // [launch][8] globaltimer nanoseconds
  int slot;
};

#ifdef __CUDACC__
__device__ __forceinline__ void tl_mark(const Timeline& t, int phase, bool any_block = false) {
  if (t.buf != nullptr && threadIdx.x == 0 && (any_block || (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0))) {
    long long v;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
    t.buf[t.slot * 8 + phase] = v;
  }
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_acc(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Programmatic dependent launch: wait for the producer grid's memory, and let the
// consumer grid start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}

// ---- bulk asynchronous copies (TMA, untiled) completing on an mbarrier -------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(bar)), "r"(bytes) : "memory");
}
// global -> shared, both 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)),
               "l"(src), "r"(bytes), "r"((uint32_t)__cvta_generic_to_shared(bar))
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Bounded wait: returns false if the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(bar);
  for (uint32_t i = 0; i < limit; i++) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

// D = A(16x16, row) * B(16x8, col) + C, fp16 inputs, f32 accumulate.
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t hadd2_u(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t lop3_or_and(uint32_t a, uint32_t mask, uint32_t orv) {  // (a & mask) | orv
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(orv));
  return d;
}
__device__ __forceinline__ uint32_t lop3_or_andb(uint32_t a, uint32_t b, uint32_t mask) {  // a | (b & mask)
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xF8;" : "=r"(d) : "r"(a), "r"(b), "r"(mask));
  return d;
}
__device__ __forceinline__ float h2f_lo(uint32_t h2) { return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffff))); }
__device__ __forceinline__ float h2f_hi(uint32_t h2) { return __half2float(__ushort_as_half((unsigned short)(h2 >> 16))); }
#endif

}  // namespace b200
