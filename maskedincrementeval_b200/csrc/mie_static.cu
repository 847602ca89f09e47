// mie_tiles_dilate_static: the output-tile set of a convolution for callers that may not allocate.
//
// mie_tiles_dilate needs two pieces of device scratch from its caller: one flag byte per output tile and a
// ticket word.  Some hosts of this library cannot provide them.  An event-camera pipeline that embeds the
// library typically carves up device memory once at start-up (the capture driver, the inference runtime and
// the display path each get a fixed pool) and forbids cudaMalloc afterwards, because an allocation synchronises
// the whole device, can fail under fragmentation hours into a recording, and is illegal while a stream is
// being captured into a graph.  A plugin loaded into such a host has no pool of its own to draw from.
//
// For those callers the scratch lives in this translation unit, in a fixed-size array in device memory that
// every GPU loading the library carries until the process exits (MIE_STATIC_MAX_TILES flag bytes plus one
// 256-byte header: 256.25 KiB).  Nothing here calls cudaMalloc, cudaFree or any allocating routine.
//
// Consequences the caller must know about:
//  * Larger problems are refused with MIE_ETOOBIG (more than MIE_STATIC_MAX_TILES output tiles).
//  * The array is shared by every call on a device and keeps what the last call left in it.  The one word that
//    has to start at zero (the ticket) is cleared on the caller's stream before each launch; the flag bytes
//    are fully rewritten for the tiles of the call before they are read.
//  * Because of that sharing, two calls that overlap on the GPU (different streams, or two host threads)
//    race on the array.  Serialise them.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress).  Make that
//    first call before any stream capture begins; later calls only enqueue a 4-byte memset and one kernel.
#include <mutex>
#include "mie_common.cuh"

using namespace mie;

namespace {

constexpr int HEADER_BYTES = 256;
constexpr size_t SCRATCH_BYTES = HEADER_BYTES + (size_t)MIE_STATIC_MAX_TILES;

// In host code this name is only a handle for the runtime's symbol table, not a device address.
static __device__ __align__(256) unsigned char g_scratch[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
void *g_scratch_addr[MAX_DEVICES];
bool g_scratch_known[MAX_DEVICES];

// Device address of g_scratch on the current device; looked up once per device.
int scratch_address(unsigned char **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  if (dev < 0 || dev >= MAX_DEVICES) return MIE_EUNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_known[dev]) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      if (e != cudaSuccess) set_cuda_error(e);
      return MIE_ECUDA;
    }
    g_scratch_addr[dev] = p;
    g_scratch_known[dev] = true;
  }
  *out = static_cast<unsigned char *>(g_scratch_addr[dev]);
  return MIE_OK;
}

// Input rows (or columns) base .. base+31 that feed the valid outputs [o0, o0 + cnt) of a tile.
__device__ __forceinline__ unsigned feeders(int o0, int cnt, int k, int stride, int pad, int base, int limit) {
  unsigned set = 0;
  for (int o = 0; o < cnt; ++o)
    for (int t = 0; t < k; ++t) {
      const int i = (o0 + o) * stride - pad + t;
      if (i >= 0 && i < limit) set |= 1u << (i - base);
    }
  return set;
}

__device__ __forceinline__ unsigned select8(unsigned set, int tile, int base) {
  unsigned sel = 0;
  for (int q = 0; q < 8; ++q) {
    const int j = tile * 8 + q - base;
    if (j >= 0 && j < 32 && ((set >> j) & 1u)) sel |= 1u << q;
  }
  return sel;
}

__global__ void __launch_bounds__(256) tiles_dilate_static_kernel(
    const uint64_t *__restrict__ in_bits, int N, int Hin, int Win, int Hout, int Wout, int k, int stride, int pad,
    const uint64_t *__restrict__ union_bits, uint64_t *__restrict__ out_bits, int32_t *__restrict__ list,
    int32_t *__restrict__ stale, int32_t *__restrict__ counts, unsigned char *__restrict__ scratch) {
  int *ticket = reinterpret_cast<int *>(scratch);
  unsigned char *flags = scratch + HEADER_BYTES;
  const int THi = (Hin + 7) >> 3, TWi = (Win + 7) >> 3;
  const int THo = (Hout + 7) >> 3, TWo = (Wout + 7) >> 3;
  const int ntiles = N * THo * TWo;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < ntiles) {
    const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
    const int rows = min(8, Hout - ty * 8), cols = min(8, Wout - tx * 8);
    const int ybase = ty * 8 * stride - pad, xbase = tx * 8 * stride - pad;
    const unsigned rset = feeders(ty * 8, rows, k, stride, pad, ybase, Hin);
    const unsigned cset = feeders(tx * 8, cols, k, stride, pad, xbase, Win);
    bool active = false;
    if (rset && cset) {
      const int ylo = ybase + __ffs(rset) - 1, yhi = ybase + 31 - __clz(rset);
      const int xlo = xbase + __ffs(cset) - 1, xhi = xbase + 31 - __clz(cset);
      for (int ity = ylo >> 3; ity <= (yhi >> 3) && !active; ++ity) {
        const unsigned selr = select8(rset, ity, ybase);
        for (int itx = xlo >> 3; itx <= (xhi >> 3); ++itx) {
          const unsigned selc = select8(cset, itx, xbase);
          uint64_t m = 0;
          for (int py = 0; py < 8; ++py)
            if ((selr >> py) & 1u) m |= (uint64_t)selc << (py * 8);
          if (in_bits[((int64_t)n * THi + ity) * TWi + itx] & m) { active = true; break; }
        }
      }
    }
    if (!active && union_bits && union_bits[t] != 0ull) active = true;
    unsigned char f = active ? 1 : 0;
    if (out_bits) {
      if (!active && out_bits[t] != 0ull) f = 2;
      out_bits[t] = 0ull;
    }
    flags[t] = f;
  }
  __shared__ bool s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(ticket, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int na = block_ordered_compact([&](int i) { return __ldcg(flags + i) == 1; }, ntiles, list);
  __syncthreads();
  int ns = 0;
  if (stale) ns = block_ordered_compact([&](int i) { return __ldcg(flags + i) == 2; }, ntiles, stale);
  if (threadIdx.x == 0) {
    counts[0] = na;
    counts[1] = ns;
    *ticket = 0;
  }
}

}  // namespace

extern "C" int mie_tiles_dilate_static(const uint64_t *in_bits, int N, int Hin, int Win, int Hout, int Wout, int k,
                                       int stride, int pad, const uint64_t *union_bits, uint64_t *out_bits,
                                       int32_t *list, int32_t *stale, int32_t *counts, void *stream) {
  if (!in_bits || !list || !counts || N <= 0 || Hin <= 0 || Win <= 0 || Hout <= 0 || Wout <= 0) return MIE_EINVAL;
  if (k < 1 || k > 7 || stride < 1 || stride > 2 || pad < 0 || pad > k) return MIE_EUNSUPPORTED;
  if (out_bits && !stale) return MIE_EINVAL;
  const int64_t ntiles = (int64_t)N * divup(Hout, 8) * divup(Wout, 8);
  if (ntiles > MIE_STATIC_MAX_TILES) return MIE_ETOOBIG;  // the built-in scratch holds MIE_STATIC_MAX_TILES flags
  unsigned char *scratch = nullptr;
  int s = scratch_address(&scratch);
  if (s != MIE_OK) return s;
  cudaStream_t st = (cudaStream_t)stream;
  // the array keeps the previous call's contents; the ticket is the only word that must start at zero
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int), st);
  if (e != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  tiles_dilate_static_kernel<<<divup((int)ntiles, 256), 256, 0, st>>>(in_bits, N, Hin, Win, Hout, Wout, k, stride, pad,
                                                                      union_bits, out_bits, list, stale, counts, scratch);
  return check_launch();
}
