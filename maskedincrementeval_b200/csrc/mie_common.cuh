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

// Kernels enqueued through launch_chained() since the last reset (MIE_OPT_LAUNCH_COUNT); defined in mie_mask.cu.
extern unsigned long long g_launch_count;

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
  if (e == cudaSuccess) __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
  // a failure is picked up by check_launch() through cudaGetLastError()
}

// The same for a kernel that runs as thread-block clusters of `cluster_x` CTAs (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
static inline void launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                          unsigned cluster_x, Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained_launch_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  if (e == cudaSuccess) __atomic_fetch_add(&g_launch_count, 1ull, __ATOMIC_RELAXED);
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

// ---------------------------------------------------------------------------------------------
// dilated output-tile set of a convolution: the per-tile test shared by the dilation kernels and the tail job
// ---------------------------------------------------------------------------------------------
// Bit j of the result is set when input row (base + j) feeds one of the valid output rows
// [o0, o0 + cnt) of a tile: rows o*stride - pad + t for t in [0, k).
__device__ __forceinline__ unsigned feed_set(int o0, int cnt, int k, int stride, int pad, int base, int limit) {
  if (stride <= k) {
    // consecutive outputs read adjacent or overlapping input ranges: their union is one interval [lo, hi)
    const int lo = max(o0 * stride - pad, 0), hi = min((o0 + cnt - 1) * stride - pad + k, limit);
    if (hi <= lo) return 0u;
    return ((1u << (hi - base)) - 1u) & ~((1u << (lo - base)) - 1u);   // 0 <= lo - base < hi - base <= 21
  }
  unsigned set = 0;
  for (int o = 0; o < cnt; ++o)
    for (int t = 0; t < k; ++t) {
      const int i = (o0 + o) * stride - pad + t;
      if (i >= 0 && i < limit) set |= 1u << (i - base);
    }
  return set;
}

// 0: inactive, 1: active, 2: inactive now but the output tile holds data from the previous step (stale).
// Also clears the output word (clear_active = false: only that of a stale tile; the word of an active tile is then
// stored, not ORed into, by whoever finishes the tile).
__device__ __forceinline__ uint8_t dilate_flag(int t, const uint64_t *in_bits, int Hin, int Win, int Hout,
                                               int Wout, int k, int stride, int pad,
                                               const uint64_t *union_bits, uint64_t *out_bits, bool clear_active = true) {
  const int THi = (Hin + 7) >> 3, TWi = (Win + 7) >> 3;
  const int THo = (Hout + 7) >> 3, TWo = (Wout + 7) >> 3;
  const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
  const int rows = min(8, Hout - ty * 8), cols = min(8, Wout - tx * 8);
  const int ybase = ty * 8 * stride - pad, xbase = tx * 8 * stride - pad;  // span <= 7*stride + k <= 21 < 32
  // issued before the neighbourhood test so that the three latencies overlap
  const uint64_t prev = out_bits ? __ldcg(out_bits + t) : 0ull;
  const uint64_t uni = union_bits ? __ldcg(union_bits + t) : 0ull;
  const unsigned rset = feed_set(ty * 8, rows, k, stride, pad, ybase, Hin);
  const unsigned cset = feed_set(tx * 8, cols, k, stride, pad, xbase, Win);
  bool active = false;
  if (rset && cset) {
    const int ylo = ybase + __ffs(rset) - 1, yhi = ybase + 31 - __clz(rset);
    const int xlo = xbase + __ffs(cset) - 1, xhi = xbase + 31 - __clz(cset);
    // The receptive field spans at most 7 * stride + k <= 21 rows / columns = at most 4 x 4 input tiles.  All their
    // words are loaded before any is tested: with an early exit each load waited for the test of the one before --
    // a chain of up to nine round trips to L2 or DRAM per thread, which was this kernel's whole run time.
    const int ity0 = ylo >> 3, ity1 = yhi >> 3, itx0 = xlo >> 3, itx1 = xhi >> 3;
    uint64_t w[4][4];
#pragma unroll
    for (int dy = 0; dy < 4; ++dy)
#pragma unroll
      for (int dx = 0; dx < 4; ++dx) {
        const int ity = ity0 + dy, itx = itx0 + dx;
        w[dy][dx] = (ity <= ity1 && itx <= itx1) ? __ldcg(in_bits + ((int64_t)n * THi + ity) * TWi + itx) : 0ull;
      }
    unsigned selr[4], selc[4];
#pragma unroll
    for (int d = 0; d < 4; ++d) {
      // bits of rset / cset that fall into input tile ity0 + d / itx0 + d, as an 8-bit row / column selection
      const int jr = (ity0 + d) * 8 - ybase, jc = (itx0 + d) * 8 - xbase;   // in (-8, 32)
      selr[d] = (jr >= 0 ? (jr < 32 ? rset >> jr : 0u) : rset << -jr) & 0xFFu;
      selc[d] = (jc >= 0 ? (jc < 32 ? cset >> jc : 0u) : cset << -jc) & 0xFFu;
    }
    uint64_t hit = 0ull;
#pragma unroll
    for (int dy = 0; dy < 4; ++dy) {
      // row selection spread to bytes: byte py = 0xFF when row py is selected
      uint64_t rowsel = 0ull;
#pragma unroll
      for (int py = 0; py < 8; ++py)
        if ((selr[dy] >> py) & 1u) rowsel |= 0xFFull << (py * 8);
#pragma unroll
      for (int dx = 0; dx < 4; ++dx) hit |= w[dy][dx] & rowsel & (0x0101010101010101ull * (uint64_t)selc[dx]);
    }
    active = hit != 0ull;
  }
  if (uni != 0ull) active = true;
  uint8_t f = active ? 1 : 0;
  if (out_bits) {
    if (!active && prev != 0ull) f = 2;
    if (prev != 0ull && (clear_active || !active)) out_bits[t] = 0ull;
  }
  return f;
}


// ---------------------------------------------------------------------------------------------
// Tail job: the tile dilation of the NEXT convolution, run by the last thread block of the kernel that produces
// that convolution's input mask (see mie_tail_job in mie.h).  Every thread of every block of the producing kernel
// calls run_tail_job() once, as its last action, with no thread having left the kernel before; blockDim.x must be a
// multiple of 32.  All loads of mask words are L2-coherent (__ldcg): the words were written by other blocks of the
// same launch.
// ---------------------------------------------------------------------------------------------
constexpr int TAIL_MAX_TILES = MIE_TAIL_MAX_TILES;   // larger fields keep the separate, multi-block dilation launch

// Arguments by value (registers): a reference to a kernel parameter would make the caller copy its whole parameter
// block to local memory.
static __device__ __noinline__ void run_tail_job_last(const uint64_t *in_bits, int N, int Hin, int Win, int Hout, int Wout,
                                                      int k, int stride, int pad, const uint64_t *union_bits,
                                                      uint64_t *out_bits, int32_t *list, int32_t *stale, int32_t *counts,
                                                      uint8_t *flags, bool clear_ticket) {
  // the per-tile flags stay in shared memory (at most TAIL_MAX_TILES of them: the host sends larger fields to the
  // separate launch); `flags` is the global scratch of that launch and is not touched here
  (void)flags;
  __shared__ uint8_t s_tile_flags[TAIL_MAX_TILES];
  const int ntiles = N * ((Hout + 7) >> 3) * ((Wout + 7) >> 3);
  for (int t = threadIdx.x; t < ntiles; t += blockDim.x)
    s_tile_flags[t] = dilate_flag(t, in_bits, Hin, Win, Hout, Wout, k, stride, pad, union_bits, out_bits);
  __syncthreads();
  int na, ns;
  block_ordered_compact2([&](int i) { return (int)s_tile_flags[i]; }, ntiles, list, stale, &na, &ns);
  if (threadIdx.x == 0) {
    counts[0] = na;
    counts[1] = ns;
    if (clear_ticket) counts[2] = 0;
  }
}

// ---------------------------------------------------------------------------------------------
// Head job: a convolution's OWN tile dilation, run by block 0 of the convolution kernel while the other blocks of the
// launch wait for it (mie_conv_args.head).  One launch instead of two, and no race: no block reads the lists, clears or
// sets a tile word before block 0 has published them.  counts[2] carries the hand-over: bit 30 = "lists ready", the low
// bits count the blocks that have left; the last one to leave puts the word back to 0 for the next launch.
// All blocks of one launch are resident together or are dispatched in index order, so block 0 runs while the others
// poll; the poll is bounded all the same (MIE_ERR_WAIT_EXPIRED, the layer is then treated as empty).
// run_head_job(): every thread of every block, right after grid_dependency_wait() and before the first read of the
// lists; returns false when the wait ran out.  count_head_job_passed(): one thread of every block, any time after.
// ---------------------------------------------------------------------------------------------
constexpr int HEAD_READY = 1 << 30;

__device__ __forceinline__ bool run_head_job(const mie_tail_job &j, unsigned spin_limit) {
  if (j.list == nullptr) return true;     // uniform over the grid
  if (blockIdx.x == 0) {
    run_tail_job_last(j.in_bits, j.N, j.Hin, j.Win, j.Hout, j.Wout, j.k, j.stride, j.pad, j.union_bits, j.out_bits, j.list,
                      j.stale, j.counts, j.flags, false);
    // block barrier, then one fence and the flag by one thread: the fence is cumulative over what the barrier ordered
    // before it (the hand-over a grid-wide barrier uses)
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      atomicOr(&j.counts[2], HEAD_READY);
    }
    return true;
  }
  __shared__ int s_head_ok;
  if (threadIdx.x == 0) {
    int ok = 0;
    for (unsigned it = 0; it < spin_limit && !ok; ++it) {
      int v;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(j.counts + 2) : "memory");
      ok = (v & HEAD_READY) != 0;
      if (!ok) __nanosleep(128);   // a hundred-odd blocks poll one word that shares its line with the counts block 0 writes
    }
    if (!ok) atomicOr(&j.counts[3], MIE_ERR_WAIT_EXPIRED);
    s_head_ok = ok;
  }
  __syncthreads();
  return s_head_ok != 0;
}

// Counts this block among those that have passed the wait; the last one puts the word back to 0 for the next launch
// (nobody polls it any more).  Called once per block by ONE thread that is off the block's critical path -- the
// atomic's round trip then overlaps the block's work instead of delaying its exit.
__device__ __forceinline__ void count_head_job_passed(const mie_tail_job &j) {
  if (j.list == nullptr) return;
  const int old = atomicAdd(&j.counts[2], 1);
  if ((old & (HEAD_READY - 1)) == (int)(gridDim.x * gridDim.y * gridDim.z) - 1) j.counts[2] = 0;
}

__device__ __forceinline__ void run_tail_job(const mie_tail_job &j) {
  if (j.list == nullptr) return;          // uniform over the grid
  __shared__ int s_tail_last;
  __threadfence();                        // this thread's mask words and data, before the ticket
  __syncthreads();
  if (threadIdx.x == 0)
    s_tail_last = atomicAdd(&j.counts[2], 1) == (int)(gridDim.x * gridDim.y * gridDim.z) - 1;
  __syncthreads();
  if (!s_tail_last) return;
  __threadfence();
  run_tail_job_last(j.in_bits, j.N, j.Hin, j.Win, j.Hout, j.Wout, j.k, j.stride, j.pad, j.union_bits, j.out_bits, j.list,
                    j.stale, j.counts, j.flags, true);
}

// ---- host side of the tail job -----------------------------------------------------------------------------------
// An entry point with a `tail` argument (1) validates it (tail_check: the job must read the tile words this call
// writes), (2) hands tail_for_kernel() to a kernel that ends in run_tail_job() -- an empty job when there is none or
// when it is too large for one block -- and (3) finishes with tail_after_launch(), which enqueues the separate
// dilation launch whenever the kernel did not carry the job.  Either way the dilation is in the stream on return.
static inline bool tail_fits(const mie_tail_job *t) {
  return (int64_t)t->N * divup(t->Hout, 8) * divup(t->Wout, 8) <= TAIL_MAX_TILES;
}
static inline int tail_check(const mie_tail_job *t, const void *produced_bits) {
  if (!t) return MIE_OK;
  if (!t->in_bits || !t->list || !t->counts || !t->flags || t->N <= 0 || t->Hin <= 0 || t->Win <= 0 || t->Hout <= 0 || t->Wout <= 0)
    return MIE_EINVAL;
  if (t->k < 1 || t->k > 7 || t->stride < 1 || t->stride > 2 || t->pad < 0 || t->pad > t->k) return MIE_EINVAL;
  if (t->out_bits && !t->stale) return MIE_EINVAL;
  if (static_cast<const void *>(t->in_bits) != produced_bits) return MIE_EINVAL;
  return MIE_OK;
}
// A head job must fill exactly the lists the convolution call reads.
static inline int head_check(const mie_tail_job *t, const mie_conv_args *a) {
  if (!t) return MIE_OK;
  if (tail_check(t, t->in_bits) != MIE_OK) return MIE_EINVAL;
  if (t->list != a->list || t->counts != a->counts || t->stale != a->stale || t->out_bits != a->out_bits) return MIE_EINVAL;
  if (t->N != a->n || t->Hin != a->hin || t->Win != a->win || t->Hout != a->hout || t->Wout != a->wout || t->k != a->k ||
      t->stride != a->stride || t->pad != a->pad)
    return MIE_EINVAL;
  return MIE_OK;
}
static inline mie_tail_job tail_for_kernel(const mie_tail_job *t) {
  mie_tail_job j = {};
  if (t && tail_fits(t)) j = *t;
  return j;
}
static inline int tail_after_launch(int status, const mie_tail_job *t, bool kernel_carries_tails, void *stream) {
  if (status != MIE_OK || !t || (kernel_carries_tails && tail_fits(t))) return status;
  return mie_tiles_dilate(t->in_bits, t->N, t->Hin, t->Win, t->Hout, t->Wout, t->k, t->stride, t->pad, t->union_bits,
                          t->out_bits, t->list, t->stale, t->counts, t->flags, stream);
}

}  // namespace mie
