// Shared helpers for the libmie kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>
#include "mie.h"

#define MIE_TILE 8
#define MIE_SM_COUNT 148  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

namespace mie {

// Records the text of a failed CUDA runtime call for mie_last_cuda_error(); defined in mie_mask.cu.
void set_cuda_error(cudaError_t e);

static inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_cuda_error(e);
    return MIE_ECUDA;
  }
  return MIE_OK;
}

// Programmatic dependent launch.  The kernels of one timestep form a chain of short launches, each reading what the one
// before wrote.  A kernel launched through launch_chained() may become resident while its predecessor in the stream is
// still running: whatever it does before grid_dependency_wait() (barrier and tensor-memory set-up, nothing that
// touches global memory) overlaps the predecessor's tail; the wait returns once the predecessor has finished and its
// writes are visible.  grid_dependency_trigger() lets the next kernel of the chain start its own set-up.
// Rule: every kernel launched through launch_chained() executes grid_dependency_wait() in every thread before its
// first global-memory access.  MIE_PDL=0 in the environment launches without the attribute (plain stream order).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool chained_launch_enabled() {
  static const bool on = []() { const char *e = getenv("MIE_PDL"); return !(e && e[0] == '0'); }();
  return on;
}

template <typename... KArgs, typename... Args>
static inline void launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launch_enabled() ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  (void)e;  // picked up by check_launch() through cudaGetLastError()
}

static inline int divup(int a, int b) { return (a + b - 1) / b; }
static inline int64_t divup64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ float act_apply(int op, float x) {
  // expf/tanhf are the accurate libm-class device functions (no fast-math): parity with
  // torch.sigmoid / torch.tanh is required to 1e-4 of the output range.
  switch (op) {
    case MIE_ACT_RELU: return fmaxf(x, 0.0f);
    case MIE_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case MIE_ACT_TANH: return tanhf(x);
    default: return x;
  }
}

template <int OP>
__device__ __forceinline__ float act_t(float x) {
  if (OP == MIE_ACT_RELU) return fmaxf(x, 0.0f);
  if (OP == MIE_ACT_SIGMOID) return 1.0f / (1.0f + expf(-x));
  if (OP == MIE_ACT_TANH) return tanhf(x);
  return x;
}

// Bit mask of the valid pixels of tile (ty, tx) in an H x W image (ragged right / bottom tiles).
__device__ __forceinline__ unsigned long long tile_valid_mask(int ty, int tx, int H, int W) {
  int rows = min(MIE_TILE, H - ty * MIE_TILE);
  int cols = min(MIE_TILE, W - tx * MIE_TILE);
  unsigned long long rowm = (1ull << cols) - 1ull;  // cols <= 8
  unsigned long long m = 0;
  for (int r = 0; r < rows; ++r) m |= rowm << (r * 8);
  return m;
}

// Ordered compaction run by ONE thread block: list <- ascending i in [0,n) with pred(i) != 0.
// Returns the count to every thread.  blockDim.x must be a multiple of 32, at most 1024.
template <typename Pred>
__device__ int block_ordered_compact(Pred pred, int n, int32_t *list) {
  __shared__ int s_warp[32];
  __shared__ int s_base;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) s_base = 0;
  __syncthreads();
  for (int start = 0; start < n; start += blockDim.x) {
    int i = start + threadIdx.x;
    bool p = (i < n) && pred(i);
    unsigned ballot = __ballot_sync(0xffffffffu, p);
    int within = __popc(ballot & ((1u << lane) - 1u));
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int warp_off = 0, total = 0;
    for (int w2 = 0; w2 < nwarps; ++w2) {
      int c = s_warp[w2];
      if (w2 < warp) warp_off += c;
      total += c;
    }
    int base = s_base;
    if (p) list[base + warp_off + within] = i;
    __syncthreads();
    if (threadIdx.x == 0) s_base = base + total;
    __syncthreads();
  }
  return s_base;
}

// Two ordered compactions in one sweep (same barriers as one): listA <- i with flag(i) == 1, listB <- i with
// flag(i) == 2 (listB may be null: then only counted as 0).  Returns the two counts through na / nb.
template <typename Flag>
__device__ void block_ordered_compact2(Flag flag, int n, int32_t *listA, int32_t *listB, int *na, int *nb) {
  __shared__ int s_wa[32], s_wb[32];
  __shared__ int s_ba, s_bb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (threadIdx.x == 0) { s_ba = 0; s_bb = 0; }
  __syncthreads();
  for (int start = 0; start < n; start += blockDim.x) {
    const int i = start + threadIdx.x;
    const int f = (i < n) ? flag(i) : 0;
    const bool pa = f == 1, pb = (f == 2) && listB;
    const unsigned ba = __ballot_sync(0xffffffffu, pa), bb = __ballot_sync(0xffffffffu, pb);
    const unsigned below = (1u << lane) - 1u;
    if (lane == 0) { s_wa[warp] = __popc(ba); s_wb[warp] = __popc(bb); }
    __syncthreads();
    int offa = 0, tota = 0, offb = 0, totb = 0;
    for (int w2 = 0; w2 < nwarps; ++w2) {
      const int ca = s_wa[w2], cb = s_wb[w2];
      if (w2 < warp) { offa += ca; offb += cb; }
      tota += ca; totb += cb;
    }
    const int basea = s_ba, baseb = s_bb;
    if (pa) listA[basea + offa + __popc(ba & below)] = i;
    if (pb) listB[baseb + offb + __popc(bb & below)] = i;
    __syncthreads();
    if (threadIdx.x == 0) { s_ba = basea + tota; s_bb = baseb + totb; }
    __syncthreads();
  }
  *na = s_ba;
  *nb = s_bb;
}

}  // namespace mie
