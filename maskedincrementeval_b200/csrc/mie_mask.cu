// Active-tile compaction: per-pixel masks as 64-bit tile words, ordered tile lists, and the
// dilated output-tile set of a convolution.
#include <stdio.h>
#include <string.h>
#include "mie_common.cuh"

namespace mie {
static thread_local char g_cuda_err[256] = "";
unsigned long long g_launch_count = 0;

void set_cuda_error(cudaError_t e) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
}
}  // namespace mie

using namespace mie;

extern "C" int mie_version(void) { return 1; }

extern "C" const char *mie_status_string(int s) {
  switch (s) {
    case MIE_OK: return "ok";
    case MIE_EINVAL: return "invalid argument";
    case MIE_EALIGN: return "misaligned pointer or stride";
    case MIE_EUNSUPPORTED: return "unsupported combination";
    case MIE_ECUDA: return "CUDA runtime error";
    case MIE_ETOOBIG: return "size beyond capacity";
    default: return "unknown status";
  }
}

extern "C" const char *mie_last_cuda_error(void) { return g_cuda_err; }

// ---------------------------------------------------------------------------------------------
// mask words from a delta tensor or an explicit mask tensor: one warp per 8x8 tile
// ---------------------------------------------------------------------------------------------
template <typename T, bool VEC4>
__global__ void __launch_bounds__(256) mask_words_kernel(const T *__restrict__ src, int64_t ps, int C, int N,
                                                         int H, int W, float thr, uint64_t *__restrict__ bits) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int TH = (H + 7) >> 3, TW = (W + 7) >> 3;
  const int ntiles = N * TH * TW;
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = (gridDim.x * blockDim.x) >> 5;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < ntiles; t += warps_per_grid) {
    const int tx = t % TW, ty = (t / TW) % TH, n = t / (TW * TH);
    const int rows = min(8, H - ty * 8), cols = min(8, W - tx * 8);
    unsigned lo = 0, hi = 0;
    if (VEC4) {
      // C % 4 == 0, ps % 4 == 0, base 16-byte aligned: each float4 lies inside one pixel
      const int c4 = C >> 2;
      const int per_row = cols * c4;
      const int total = rows * per_row;
#pragma unroll 4
      for (int i = lane; i < total; i += 32) {   // independent 16-byte loads: four in flight per lane
        const int r = i / per_row, rem = i - r * per_row;
        const int px = rem / c4, q = rem - px * c4;
        const float4 v = *reinterpret_cast<const float4 *>(
            reinterpret_cast<const float *>(src) + ((int64_t)(n * H + ty * 8 + r) * W + tx * 8 + px) * ps + q * 4);
        const bool a = fabsf(v.x) > thr || fabsf(v.y) > thr || fabsf(v.z) > thr || fabsf(v.w) > thr;
        const int b = r * 8 + px;
        if (a) { if (b < 32) lo |= 1u << b; else hi |= 1u << (b - 32); }
      }
    } else {
      const int per_row = cols * C;
      const int total = rows * per_row;
      for (int i = lane; i < total; i += 32) {
        const int r = i / per_row, rem = i - r * per_row;
        const int px = rem / C, c = rem - px * C;
        const T v = src[((int64_t)(n * H + ty * 8 + r) * W + tx * 8 + px) * ps + c];
        bool a;
        if (sizeof(T) == 4 && thr >= 0.0f) a = fabsf((float)v) > thr;  // float source
        else a = v != (T)0;                                           // explicit mask source
        const int b = r * 8 + px;
        if (a) { if (b < 32) lo |= 1u << b; else hi |= 1u << (b - 32); }
      }
    }
    lo = __reduce_or_sync(0xffffffffu, lo);
    hi = __reduce_or_sync(0xffffffffu, hi);
    if (lane == 0) bits[t] = ((uint64_t)hi << 32) | lo;
  }
}

// Few channels: one thread per pixel, one warp per half tile, the ballot is the half word.
template <typename T>
__global__ void __launch_bounds__(256) mask_words_px_kernel(const T *__restrict__ src, int64_t ps, int C, int N, int H,
                                                            int W, float thr, unsigned *__restrict__ bits32) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int TH = (H + 7) >> 3, TW = (W + 7) >> 3;
  const int ntiles = N * TH * TW;
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * 4 + (threadIdx.x >> 6); t < ntiles; t += gridDim.x * 4) {
    const int p = threadIdx.x & 63;
    const int tx = t % TW, ty = (t / TW) % TH, n = t / (TW * TH);
    const int y = ty * 8 + (p >> 3), x = tx * 8 + (p & 7);
    bool a = false;
    if (y < H && x < W) {
      const T *px = src + ((int64_t)(n * H + y) * W + x) * ps;
      for (int c = 0; c < C; ++c) {
        const T v = px[c];
        if (sizeof(T) == 4 && thr >= 0.0f) a |= fabsf((float)v) > thr;
        else a |= (v != (T)0);
      }
    }
    const unsigned half = __ballot_sync(0xffffffffu, a);
    if (lane == 0) bits32[2 * (size_t)t + ((p >> 5) & 1)] = half;
  }
}

static int mask_grid(int ntiles) {
  int blocks = divup(ntiles, 8);
  int cap = MIE_SM_COUNT * 8;
  return blocks < cap ? (blocks > 0 ? blocks : 1) : cap;
}

extern "C" int mie_mask_from_delta(const float *delta, int64_t ps, int N, int C, int H, int W, float thr,
                                   uint64_t *bits, void *stream) {
  if (!delta || !bits || N <= 0 || C <= 0 || H <= 0 || W <= 0 || ps < C || !(thr >= 0.0f)) return MIE_EINVAL;
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = (C % 4 == 0) && (ps % 4 == 0) && aligned16(delta);
  if (C <= 16) {
    int blocks = divup(ntiles, 4);
    if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
    launch_chained(mask_words_px_kernel<float>, dim3(blocks), dim3(256), 0, st, delta, ps, C, N, H, W, thr, reinterpret_cast<unsigned *>(bits));
    return check_launch();
  }
  if (vec) launch_chained(mask_words_kernel<float, true>, dim3(mask_grid(ntiles)), dim3(256), 0, st, delta, ps, C, N, H, W, thr, bits);
  else launch_chained(mask_words_kernel<float, false>, dim3(mask_grid(ntiles)), dim3(256), 0, st, delta, ps, C, N, H, W, thr, bits);
  return check_launch();
}

extern "C" int mie_mask_from_mask(const void *mask, int elem_size, int64_t mps, int cm, int N, int H, int W,
                                  uint64_t *bits, void *stream) {
  if (!mask || !bits || N <= 0 || cm <= 0 || H <= 0 || W <= 0 || mps < cm) return MIE_EINVAL;
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  cudaStream_t st = (cudaStream_t)stream;
  if (elem_size == 1)
    launch_chained(mask_words_kernel<uint8_t, false>, dim3(mask_grid(ntiles)), dim3(256), 0, st, (const uint8_t *)mask, mps, cm, N, H, W, -1.0f, bits);
  else if (elem_size == 4)
    launch_chained(mask_words_kernel<int32_t, false>, dim3(mask_grid(ntiles)), dim3(256), 0, st, (const int32_t *)mask, mps, cm, N, H, W, -1.0f, bits);
  else
    return MIE_EUNSUPPORTED;
  return check_launch();
}

// ---------------------------------------------------------------------------------------------
// ordered compaction of non-zero words (warp ballot + block prefix)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) tiles_compact_kernel(const uint64_t *__restrict__ bits, int ntiles,
                                                             int32_t *__restrict__ list, int32_t *__restrict__ counts) {
  grid_dependency_wait();
  grid_dependency_trigger();
  int n = block_ordered_compact([&](int i) { return bits[i] != 0ull; }, ntiles, list);
  if (threadIdx.x == 0) counts[0] = n;
}

extern "C" int mie_tiles_compact(const uint64_t *bits, int ntiles, int32_t *list, int32_t *counts, void *stream) {
  if (!bits || !list || !counts || ntiles <= 0) return MIE_EINVAL;
  launch_chained(tiles_compact_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream, bits, ntiles, list, counts);
  return check_launch();
}

__global__ void mask_expand_kernel(const uint64_t *__restrict__ bits, int N, int H, int W, uint8_t *__restrict__ out) {
  const int TH = (H + 7) >> 3, TW = (W + 7) >> 3;
  const int64_t total = (int64_t)N * H * W;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int x = (int)(i % W), y = (int)((i / W) % H), n = (int)(i / ((int64_t)W * H));
    const uint64_t w = bits[((int64_t)n * TH + (y >> 3)) * TW + (x >> 3)];
    out[i] = (uint8_t)((w >> ((y & 7) * 8 + (x & 7))) & 1ull);
  }
}

extern "C" int mie_mask_expand(const uint64_t *bits, int N, int H, int W, uint8_t *bytes, void *stream) {
  if (!bits || !bytes || N <= 0 || H <= 0 || W <= 0) return MIE_EINVAL;
  const int64_t total = (int64_t)N * H * W;
  int blocks = (int)((total + 255) / 256);
  if (blocks > MIE_SM_COUNT * 16) blocks = MIE_SM_COUNT * 16;
  mask_expand_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(bits, N, H, W, bytes);
  return check_launch();
}

// ---------------------------------------------------------------------------------------------
// dilated output-tile set of a convolution, plus the stale list, in one launch
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) tiles_dilate_kernel(
    const uint64_t *__restrict__ in_bits, int N, int Hin, int Win, int Hout, int Wout, int k, int stride, int pad,
    const uint64_t *__restrict__ union_bits, uint64_t *__restrict__ out_bits, int32_t *__restrict__ list,
    int32_t *__restrict__ stale, int32_t *__restrict__ counts, uint8_t *__restrict__ flags) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((Hout + 7) >> 3) * ((Wout + 7) >> 3);
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < ntiles) flags[t] = dilate_flag(t, in_bits, Hin, Win, Hout, Wout, k, stride, pad, union_bits, out_bits);
  // the block that finishes last compacts both lists in ascending order
  __shared__ bool s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&counts[2], 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  int na, ns;
  block_ordered_compact2([&](int i) { return (int)__ldcg(flags + i); }, ntiles, list, stale, &na, &ns);
  if (threadIdx.x == 0) {
    counts[0] = na;
    counts[1] = ns;
    counts[2] = 0;
  }
}

// Up to DILATE_SMALL_MAX tiles: one block keeps the flags in shared memory and compacts them itself -- no
// ticket, no fence, no round trip through global memory (the deeper levels of a UNet at batch 1 are this small;
// at 1452 tiles one block measured slower than the multi-block kernel).
constexpr int DILATE_SMALL_MAX = 512;

__global__ void __launch_bounds__(1024) tiles_dilate_small_kernel(
    const uint64_t *__restrict__ in_bits, int N, int Hin, int Win, int Hout, int Wout, int k, int stride, int pad,
    const uint64_t *__restrict__ union_bits, uint64_t *__restrict__ out_bits, int32_t *__restrict__ list,
    int32_t *__restrict__ stale, int32_t *__restrict__ counts) {
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ uint8_t s_flags[DILATE_SMALL_MAX];
  const int ntiles = N * ((Hout + 7) >> 3) * ((Wout + 7) >> 3);
  for (int t = threadIdx.x; t < ntiles; t += blockDim.x)
    s_flags[t] = dilate_flag(t, in_bits, Hin, Win, Hout, Wout, k, stride, pad, union_bits, out_bits);
  __syncthreads();
  int na, ns;
  block_ordered_compact2([&](int i) { return (int)s_flags[i]; }, ntiles, list, stale, &na, &ns);
  if (threadIdx.x == 0) {
    counts[0] = na;
    counts[1] = ns;
  }
}

extern "C" int mie_tiles_dilate(const uint64_t *in_bits, int N, int Hin, int Win, int Hout, int Wout, int k,
                                int stride, int pad, const uint64_t *union_bits, uint64_t *out_bits,
                                int32_t *list, int32_t *stale, int32_t *counts, uint8_t *flags, void *stream) {
  if (!in_bits || !list || !counts || !flags || N <= 0 || Hin <= 0 || Win <= 0 || Hout <= 0 || Wout <= 0)
    return MIE_EINVAL;
  if (k < 1 || k > 7 || stride < 1 || stride > 2 || pad < 0 || pad > k) return MIE_EUNSUPPORTED;
  if (out_bits && !stale) return MIE_EINVAL;
  const int ntiles = N * divup(Hout, 8) * divup(Wout, 8);
  if (ntiles <= DILATE_SMALL_MAX) {
    const int threads = ntiles <= 256 ? 256 : (ntiles <= 512 ? 512 : 1024);
    launch_chained(tiles_dilate_small_kernel, dim3(1), dim3(threads), 0, (cudaStream_t)stream, in_bits, N, Hin, Win, Hout, Wout, k, stride, pad,
                                                                       union_bits, out_bits, list, stale, counts);
    return check_launch();
  }
  launch_chained(tiles_dilate_kernel, dim3(divup(ntiles, 256)), dim3(256), 0, (cudaStream_t)stream, 
      in_bits, N, Hin, Win, Hout, Wout, k, stride, pad, union_bits, out_bits, list, stale, counts, flags);
  return check_launch();
}
