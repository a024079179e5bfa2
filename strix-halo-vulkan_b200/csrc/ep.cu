// Expert-parallel exchanges (see ep.cuh) and the graph's side of setting them up.
#include "ep.cuh"

#include "graph.h"

#include <cstring>

namespace b200 {

__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ long long global_ns() {
  long long v;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
  return v;
}

// Polls a flag that a peer raises until it reaches `want`, for at most limit_ns. A wait that runs out sets
// the error word and returns; once the word is set, later waits do not wait at all (a peer that is gone
// costs one limit, not one per exchange).
__device__ bool wait_flag(const int* flag, int want, long long limit_ns, int* err) {
  if (ld_acquire_sys(flag) >= want) return true;
  if (*reinterpret_cast<volatile int*>(err) != 0) return false;
  const long long t0 = global_ns();
  for (;;) {
    if (ld_acquire_sys(flag) >= want) return true;
    if (global_ns() - t0 > limit_ns) { atomicExch(err, 2); return false; }
    __nanosleep(40);
  }
}

// Dispatch: CTA q stores this rank's rows and routing into rank q's gathered buffers, raises this rank's
// flag there, then waits for rank q's flag here. grid `world`, block 512.
__global__ void __launch_bounds__(512) ep_dispatch_kernel(EpParams p) {
  __shared__ int epoch_next;
  pdl_wait();   // the rows and the routing come from the router kernel
  pdl_launch();
  const int q = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) epoch_next = *reinterpret_cast<volatile int*>(p.epoch) + 1;
  __syncthreads();
  const int e = epoch_next;
  uint8_t* dst = p.base[q];
  const size_t row_units = (size_t)p.rows * p.H / 8;   // 16-byte units
  const uint4* src = reinterpret_cast<const uint4*>(p.xn);
  uint4* d = reinterpret_cast<uint4*>(dst + p.off_xg) + (size_t)p.rank * row_units;
  for (size_t i = tid; i < row_units; i += 512) d[i] = __ldcg(src + i);
  int* dt = reinterpret_cast<int*>(dst + p.off_topk) + (size_t)p.rank * p.rows * p.used;
  for (int i = tid; i < p.rows * p.used; i += 512) dt[i] = __ldcg(p.topk + i);
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    st_release_sys(reinterpret_cast<int*>(dst + p.off_flags) + p.rank, e);
    wait_flag(reinterpret_cast<const int*>(p.base[p.rank] + p.off_flags) + q, e, p.limit_ns, p.err);
    __threadfence();
    // the last CTA to get here closes the exchange (every CTA read the epoch before taking its ticket)
    if (atomicAdd(p.done, 1) == p.world - 1) { *p.done = 0; *p.epoch = e; __threadfence(); }
  }
}

// Combine: CTA i copies the output row of the i-th pair this rank computed into the `down` buffer of the rank
// that owns the pair's row (16-byte stores: a row crosses NVLink as whole sectors). The last CTA to finish raises
// this rank's flag at every rank and waits for theirs: when it returns, all pairs of this rank's rows have landed.
// grid: an upper bound of the pair count, block 256.
__global__ void __launch_bounds__(256) ep_combine_kernel(EpParams p) {
  __shared__ int last;
  pdl_wait();   // the down projections
  pdl_launch();
  const int i = blockIdx.x, tid = threadIdx.x;
  const int e = *reinterpret_cast<volatile int*>(p.epoch) + 1;   // read before this CTA takes its ticket
  if (i < __ldcg(p.n_pairs)) {
    const int pair = __ldcg(p.cols + i);
    const int owner = pair / p.pairs_per_rank, local = pair - owner * p.pairs_per_rank;
    const uint4* src = reinterpret_cast<const uint4*>(p.y_local + (size_t)pair * p.H);
    uint4* dst = reinterpret_cast<uint4*>(p.base[owner] + p.off_down) + (size_t)local * (p.H / 4);
    for (int k = tid; k < p.H / 4; k += 256) dst[k] = __ldcg(src + k);
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) last = atomicAdd(p.done, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence_system();
  if (tid < p.world) {
    st_release_sys(reinterpret_cast<int*>(p.base[tid] + p.off_flags) + p.rank, e);
    wait_flag(reinterpret_cast<const int*>(p.base[p.rank] + p.off_flags) + tid, e, p.limit_ns, p.err);
  }
  __syncthreads();
  if (tid == 0) { *p.done = 0; *p.epoch = e; __threadfence(); }
}

static int launch_ep(void (*kernel)(EpParams), int grid, int block, const EpParams& p, bool pdl, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(block); cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
  B200_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
  return OK;
}
int launch_ep_dispatch(const EpParams& p, bool pdl, cudaStream_t st) { return launch_ep(ep_dispatch_kernel, p.world, 512, p, pdl, st); }
int launch_ep_combine(const EpParams& p, int max_pairs, bool pdl, cudaStream_t st) { return launch_ep(ep_combine_kernel, max_pairs, 256, p, pdl, st); }

// ---- the graph's side -----------------------------------------------------------------------
// One device allocation per rank holds everything peers write: flags, the gathered rows and routing, and
// the down-projection outputs of this rank's rows. Offsets depend on the graph's shape only, so every rank
// computes the same ones.
int Graph::ep_prepare(int rank, int world) {
  const b200_config& c = m->c;
  if (world < 1 || world > EP_MAX_RANKS || rank < 0 || rank >= world) { set_error("ep: rank / world out of range (at most 8 ranks)"); return EINVAL_; }
  if (c.n_expert % world) { set_error("ep: the expert count must divide evenly over the ranks"); return EINVAL_; }
  if (ep_arena != nullptr) { set_error("ep: already prepared"); return ESTATE; }
  B200_CUDA(cudaSetDevice(m->device));
  const size_t slots1 = (size_t)c.n_expert_used + 1;
  auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
  ep.off_flags = 0;
  ep.off_xg = up(EP_MAX_RANKS * sizeof(int));
  ep.off_topk = ep.off_xg + up((size_t)MR * c.n_embd * sizeof(__half));
  ep.off_down = ep.off_topk + up((size_t)MR * c.n_expert_used * sizeof(int32_t));
  ep_arena_bytes = ep.off_down + up((size_t)MR * slots1 * c.n_embd * sizeof(float));
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, ep_arena_bytes);
  if (e != cudaSuccess) { set_error(std::string("ep: arena allocation failed: ") + cudaGetErrorString(e)); return ENOMEM_; }
  B200_CUDA(cudaMemset(p, 0, ep_arena_bytes));
  allocs.push_back(p);
  ep_arena = (uint8_t*)p;
  B200_TRY(dalloc(&ep_epoch, 4));   // epoch, ticket, pair count
  ep.rank = rank; ep.world = world; ep.epoch = ep_epoch; ep.done = ep_epoch + 1; ep.err = err_flag;
  ep.H = c.n_embd; ep.used = c.n_expert_used; ep.limit_ns = 2000000000ll;
  for (int q = 0; q < EP_MAX_RANKS; q++) ep.base[q] = nullptr;
  ep.base[rank] = ep_arena;
  return OK;
}

int Graph::ep_export(int rank, int world, void* handle64) {
  B200_TRY(ep_prepare(rank, world));
  cudaIpcMemHandle_t h;
  B200_CUDA(cudaIpcGetMemHandle(&h, ep_arena));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, sizeof(h));
  return OK;
}

int Graph::ep_attach(const void* handles64) {
  if (ep_arena == nullptr) { set_error("ep: export first"); return ESTATE; }
  B200_CUDA(cudaSetDevice(m->device));
  for (int q = 0; q < ep.world; q++) {
    if (q == ep.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const uint8_t*)handles64 + (size_t)q * 64, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { set_error("ep: cannot map rank " + std::to_string(q) + "'s exchange buffers: " + cudaGetErrorString(e)); return ECUDA; }
    ep.base[q] = (uint8_t*)p;
    ep_mapped.push_back(p);
  }
  ep_ready = true;
  return OK;
}

// Ranks that live in one process (one graph per device) exchange plain device pointers instead of IPC handles.
int Graph::ep_attach_local(Graph* const* peers, int world) {
  if (ep_arena == nullptr || world != ep.world) { set_error("ep: prepare every rank first, with the same world size"); return ESTATE; }
  B200_CUDA(cudaSetDevice(m->device));
  for (int q = 0; q < world; q++) {
    if (q == ep.rank) continue;
    if (peers[q] == nullptr || peers[q]->ep_arena == nullptr || peers[q]->ep.rank != q) { set_error("ep: rank " + std::to_string(q) + " is not prepared"); return ESTATE; }
    // two ranks on one GPU would be kernels that wait for each other with no guarantee that both are running
    if (peers[q]->m->device == m->device) { set_error("ep: every rank needs a GPU of its own"); return EINVAL_; }
    {
      int can = 0;
      B200_CUDA(cudaDeviceCanAccessPeer(&can, m->device, peers[q]->m->device));
      if (!can) { set_error("ep: device " + std::to_string(m->device) + " cannot reach device " + std::to_string(peers[q]->m->device)); return ECUDA; }
      cudaError_t e = cudaDeviceEnablePeerAccess(peers[q]->m->device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { set_error(std::string("ep: enabling peer access failed: ") + cudaGetErrorString(e)); return ECUDA; }
      cudaGetLastError();
    }
    ep.base[q] = peers[q]->ep_arena;
  }
  ep_ready = true;
  return OK;
}

}  // namespace b200
