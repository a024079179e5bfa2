// Expert parallelism over NVLink peer memory: ranks own disjoint ranges of every layer's routed experts,
// slots are split over the ranks, and the two exchanges a MoE layer needs are peer stores into buffers
// every rank exposes, ordered by flags that are polled with a time limit.
//
// The reference keeps all experts on one device (llm/gpu_moe.go:693-705) and has nothing to compare with;
// what must hold is that the exchange changes no arithmetic: a (row, expert) pair is computed by the same
// kernels whichever rank owns the expert, and the owner of the ROW adds its pairs in slot order
// (llm/moe.go:347-357), so the result is the single-device one.
//
// Per MoE layer, rank r with its n local rows (world * n rows in all, row i of rank q is global row q*n + i):
//   1. dispatch  every rank stores its normalised fp16 rows and their routed expert ids into every peer's
//                gathered buffers (xg, topk_g) and raises its flag there; it then waits for all peers' flags;
//   2. work list built from the gathered routing, restricted to the experts [r*E/world, (r+1)*E/world) that
//                this rank owns (plus the shared expert for its own rows);
//   3. experts   gate/up + SwiGLU, then down into local memory;
//   4. combine   every pair's output row is copied, as whole 16-byte stores, into the `down` buffer of the rank
//                that owns the pair's row; flags again (all pairs of my rows have landed), then the ordinary
//                slot-order sum.
// No load ever reads another GPU's memory: remote data always lands in local HBM first.
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int EP_MAX_RANKS = 8;

struct EpParams {
  int rank, world;
  uint8_t* base[EP_MAX_RANKS];       // exchange arena of every rank as mapped in this process (base[rank] = own)
  size_t off_flags, off_xg, off_topk, off_down;
  int* epoch;                        // local: exchanges completed so far
  int* done;                         // local: ticket of the exchange kernel's CTAs
  int* err;                          // the graph's error word
  int rows, H, used;                 // local rows of this pass, row length, experts per row
  const __half* xn;                  // [rows][H] local normalised rows
  const int32_t* topk;               // [rows][used] local routing
  long long limit_ns;                // how long a wait may last
  // combine: the down projections' outputs of the pairs this rank computed, [pair id][H] f32 in local memory, the
  // pair ids in work-list order and their count (written by the work-list kernel)
  const float* y_local;
  const int* cols;
  const int* n_pairs;
  int pairs_per_rank;                // rows * (used + 1): pair id / pairs_per_rank owns the pair's row
};

int launch_ep_dispatch(const EpParams& p, bool pdl, cudaStream_t st);
int launch_ep_combine(const EpParams& p, int max_pairs, bool pdl, cudaStream_t st);

}  // namespace b200
