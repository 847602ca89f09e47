// Masked delta convolution over a compact list of active 8x8 output tiles, FP32 CUDA-core path,
// with the incremental activation fused into the epilogue.
//
// Work item  = WT output tiles x NB = 32*WN output channels, one thread block of 32*WT*WN threads.
// Warp       = one tile x 32 output channels.  Lane = (pc = lane & 7: pixel column of the tile,
//              nq = lane >> 3: which 8 of the warp's 32 channels) -> 8 pixels x 8 channels = 64 accumulators.
// Reduction  = input channels in chunks of 8; for each chunk the input tile plus halo is staged once in
//              shared memory as [channel quad][row][column][4 floats] (cp.async, 16 B each, zero-filled
//              outside the image, columns de-interleaved by parity for stride 2 so that the 8 lanes of
//              a warp always read 128 contiguous bytes); the filter rows of one ky are double-buffered.
// Epilogue   = d (+ addend) -> x = *res; dy = f(x + d) - f(x) (or - *emitted); *res = x + d; per-pixel
//              any(|dy| > thr) across all channels of the block -> tile word; withheld pixels written as 0.
#include <string.h>
#include "mie_common.cuh"

using namespace mie;

namespace mie {
bool tc_eligible(const mie_conv_args *a);
int launch_conv_tc(const mie_conv_args *a, cudaStream_t st);
}  // namespace mie

namespace {

struct ConvParams {
  const float *in; int64_t in_ps; int cin, hin, win;
  const float *w; int cin_pad, cout, cout_pad;
  int n, hout, wout, pad;
  const int32_t *list; const int32_t *stale; int32_t *counts; int max_tiles;
  float *out; int64_t out_ps; unsigned long long *out_bits;
  int act; float thr;
  float *res; int64_t res_ps;
  float *emitted; int64_t emitted_ps;
  const float *addend; int64_t addend_ps;
  int in_vec;   // input can be staged with 16-byte cp.async
  int io_vec;   // epilogue tensors can be accessed as float4
  const float *bias;   // per output channel, added before the activation (dense evaluation only)
  int refresh;         // dense evaluation: the reservoir is set instead of advanced, the output is f(conv + bias)
  mie_tail_job tail;   // the next convolution's tile dilation, run by the last block (list == nullptr: none)
  mie_tail_job head;   // this convolution's own tile dilation, run by block 0 while the others wait (list == nullptr: none)
  const float *in2; int64_t in2_ps;   // 1x1 head: second input, added on the fly
  float *accum; int64_t accum_ps;     // 1x1 head: accum += out at the sent pixels
};

constexpr int CC = 8;  // input channels per chunk
constexpr unsigned HEAD_SPIN_LIMIT = 1u << 22;   // polls (32 ns apart) a block waits for block 0's tile lists

template <int K, int S>
struct Geo {
  static constexpr int IN_T = 7 * S + K;            // input rows/cols feeding 8 outputs
  static constexpr int HALF = (IN_T + 1) / 2;
  static constexpr int PITCH = (S == 1) ? IN_T : 2 * HALF;  // float4 slots per staged row
  static constexpr int A_TILE_F4 = (CC / 4) * IN_T * PITCH; // float4 per tile per chunk
  __device__ static __forceinline__ int pos(int xi) { return (S == 1) ? xi : ((xi & 1) * HALF + (xi >> 1)); }
};

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// CPT = output channels per thread (8 or 4): a warp covers 4*CPT channels.  CPT = 4 doubles the warps per tile for
// 32-channel layers, which otherwise run one warp per scheduler.
template <int K, int S, int WT, int WN, int CPT>
__global__ void __launch_bounds__(32 * WT * WN, 512 / (32 * WT * WN)) conv_tiles_kernel(const ConvParams p) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const bool head_ok = run_head_job(p.head, HEAD_SPIN_LIMIT);
  if (threadIdx.x == blockDim.x - 1) count_head_job_passed(p.head);
  using G = Geo<K, S>;
  constexpr int NT = 32 * WT * WN;
  constexpr int NBW = 4 * CPT;          // channels per warp
  constexpr int NB = NBW * WN;
  constexpr int B_STAGE_F = K * CC * NB;  // floats per filter stage (one ky, one chunk)

  extern __shared__ float4 smem4[];
  float4 *As = smem4;                                             // [WT][CC/4][IN_T][PITCH]
  float *Bs = reinterpret_cast<float *>(smem4 + WT * G::A_TILE_F4);  // [2][K][CC][NB]
  __shared__ int s_tile[WT];
  __shared__ unsigned long long s_bits[WT];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ts = warp / WN, wn = warp % WN;
  const int pc = lane & 7, nq = lane >> 3;
  const int THo = (p.hout + 7) >> 3, TWo = (p.wout + 7) >> 3;
  const int ntiles_total = p.n * THo * TWo;

  // ---- zero the tiles that held data last step and are inactive now ----------------------------
  {
    const int n_stale = (p.stale && head_ok) ? min(p.counts[1], p.max_tiles) : 0;
    for (int s = blockIdx.x; s < n_stale; s += gridDim.x) {
      const int t = p.stale[s];
      if (t < 0 || t >= ntiles_total) { if (tid == 0) atomicOr(&p.counts[3], MIE_ERR_BAD_TILE); continue; }
      const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
      for (int i = tid; i < 64 * p.cout; i += NT) {
        const int px = i / p.cout, c = i - px * p.cout;
        const int oy = ty * 8 + (px >> 3), ox = tx * 8 + (px & 7);
        if (oy < p.hout && ox < p.wout) p.out[((int64_t)(n * p.hout + oy) * p.wout + ox) * p.out_ps + c] = 0.0f;
      }
    }
  }

  const int n_active = head_ok ? min(p.counts[0], p.max_tiles) : 0;
  const int n_groups = (n_active + WT - 1) / WT;
  const int n_cblk = p.cout_pad / NB;
  const int n_items = n_groups * n_cblk;
  const int n_chunks = p.cin_pad / CC;

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int grp = item / n_cblk, cb = item - grp * n_cblk;
    const int n0 = cb * NB;
    __syncthreads();  // previous item fully done with shared memory
    if (tid < WT) {
      const int li = grp * WT + tid;
      int t = (li < n_active) ? p.list[li] : -1;
      if (li < n_active && (t < 0 || t >= ntiles_total)) { atomicOr(&p.counts[3], MIE_ERR_BAD_TILE); t = -1; }
      s_tile[tid] = t;
      s_bits[tid] = 0ull;
    }
    __syncthreads();

    float acc[8][CPT];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int j = 0; j < CPT; ++j) acc[r][j] = 0.0f;

    for (int ch = 0; ch < n_chunks; ++ch) {
      const int c0 = ch * CC;
      __syncthreads();  // everyone finished computing on the previous chunk's input tile
      // ---- stage the input tiles (+halo) of this chunk -----------------------------------------
      if (p.in_vec) {
        constexpr int TOTAL = WT * G::IN_T * G::IN_T * (CC / 4);
        for (int i = tid; i < TOTAL; i += NT) {
          const int cq = i % (CC / 4);
          int rest = i / (CC / 4);
          const int xx = rest % G::IN_T; rest /= G::IN_T;
          const int yy = rest % G::IN_T;
          const int slot = rest / G::IN_T;
          float4 *dst = As + ((slot * (CC / 4) + cq) * G::IN_T + yy) * G::PITCH + G::pos(xx);
          const int t = s_tile[slot];
          bool ok = false;
          const float *src = nullptr;
          if (t >= 0 && c0 + cq * 4 < p.cin) {
            const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
            const int iy = ty * 8 * S - p.pad + yy, ix = tx * 8 * S - p.pad + xx;
            if (iy >= 0 && iy < p.hin && ix >= 0 && ix < p.win) {
              ok = true;
              src = p.in + ((int64_t)(n * p.hin + iy) * p.win + ix) * p.in_ps + c0 + cq * 4;
            }
          }
          if (ok) cp_async16(dst, src);
          else *dst = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      } else {
        constexpr int TOTAL = WT * G::IN_T * G::IN_T * CC;
        for (int i = tid; i < TOTAL; i += NT) {
          const int c = i % CC;
          int rest = i / CC;
          const int xx = rest % G::IN_T; rest /= G::IN_T;
          const int yy = rest % G::IN_T;
          const int slot = rest / G::IN_T;
          float *dst = reinterpret_cast<float *>(As + ((slot * (CC / 4) + (c >> 2)) * G::IN_T + yy) * G::PITCH + G::pos(xx)) + (c & 3);
          const int t = s_tile[slot];
          float v = 0.0f;
          if (t >= 0 && c0 + c < p.cin) {
            const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
            const int iy = ty * 8 * S - p.pad + yy, ix = tx * 8 * S - p.pad + xx;
            if (iy >= 0 && iy < p.hin && ix >= 0 && ix < p.win)
              v = p.in[((int64_t)(n * p.hin + iy) * p.win + ix) * p.in_ps + c0 + c];
          }
          *dst = v;
        }
      }
      // ---- filter rows: ky = 0 now, ky + 1 prefetched while ky is consumed -----------------------
      auto stage_b = [&](int ky, int buf) {
        constexpr int TOTAL = K * CC * (NB / 4);
        float *dstb = Bs + buf * B_STAGE_F;
        for (int i = tid; i < TOTAL; i += NT) {
          const int q = i % (NB / 4);
          const int rest = i / (NB / 4);
          const int c = rest % CC, kx = rest / CC;
          const float *src = p.w + ((int64_t)((ky * K + kx) * p.cin_pad + c0 + c)) * p.cout_pad + n0 + q * 4;
          cp_async16(dstb + (kx * CC + c) * NB + q * 4, src);
        }
      };
      stage_b(0, 0);
      cp_async_commit();
#pragma unroll 1
      for (int ky = 0; ky < K; ++ky) {
        if (ky + 1 < K) {
          stage_b(ky + 1, (ky + 1) & 1);
          cp_async_commit();
          cp_async_wait<1>();
        } else {
          cp_async_wait<0>();
        }
        __syncthreads();
        const float *B = Bs + (ky & 1) * B_STAGE_F + wn * NBW + nq * CPT;
        const float4 *A = As + (ts * (CC / 4)) * G::IN_T * G::PITCH + ky * G::PITCH;
        // the tap loop stays rolled: its body (2 channel quads x 272 instructions) fits the instruction
        // cache, the fully unrolled form (26 KB for k = 3, 43 KB for k = 5) did not
#pragma unroll 1
        for (int kx = 0; kx < K; ++kx) {
#pragma unroll
          for (int cq = 0; cq < CC / 4; ++cq) {
            float4 a[8];
#pragma unroll
            for (int r = 0; r < 8; ++r)
              a[r] = A[(cq * G::IN_T + r * S) * G::PITCH + G::pos(pc * S + kx)];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              // channels past Cin are zero padding (5 voxel bins in a chunk of 8): no FMAs for them
              if (c0 + cq * 4 + c >= p.cin) break;
              const float4 b0 = *reinterpret_cast<const float4 *>(B + (kx * CC + cq * 4 + c) * NB);
              float4 b1 = make_float4(0.f, 0.f, 0.f, 0.f);
              if (CPT == 8) b1 = *reinterpret_cast<const float4 *>(B + (kx * CC + cq * 4 + c) * NB + 4);
#pragma unroll
              for (int r = 0; r < 8; ++r) {
                const float av = (c == 0) ? a[r].x : (c == 1) ? a[r].y : (c == 2) ? a[r].z : a[r].w;
                acc[r][0] = fmaf(av, b0.x, acc[r][0]);
                acc[r][1] = fmaf(av, b0.y, acc[r][1]);
                acc[r][2] = fmaf(av, b0.z, acc[r][2]);
                acc[r][3] = fmaf(av, b0.w, acc[r][3]);
                if (CPT == 8) {
                  acc[r][CPT - 4] = fmaf(av, b1.x, acc[r][CPT - 4]);
                  acc[r][CPT - 3] = fmaf(av, b1.y, acc[r][CPT - 3]);
                  acc[r][CPT - 2] = fmaf(av, b1.z, acc[r][CPT - 2]);
                  acc[r][CPT - 1] = fmaf(av, b1.w, acc[r][CPT - 1]);
                }
              }
            }
          }
        }
        __syncthreads();  // filter buffer (ky & 1) may be overwritten by the next prefetch
      }
    }

    // ---- epilogue ---------------------------------------------------------------------------------
    const int t = s_tile[ts];
    const int tx = (t >= 0) ? t % TWo : 0, ty = (t >= 0) ? (t / TWo) % THo : 0, n = (t >= 0) ? t / (TWo * THo) : 0;
    const int co = n0 + wn * NBW + nq * CPT;
    const int ox = tx * 8 + pc;
    unsigned rowflags = 0;  // bit r: pixel (r, pc) has a channel with |dy| > thr
    if (t >= 0 && ox < p.wout) {
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int oy = ty * 8 + r;
        if (oy >= p.hout) continue;
        const int64_t pix = (int64_t)(n * p.hout + oy) * p.wout + ox;
        bool any_d = p.refresh != 0;
#pragma unroll
        for (int j = 0; j < CPT; ++j) any_d |= (acc[r][j] != 0.0f);
        if (p.bias) {
#pragma unroll
          for (int j = 0; j < CPT; ++j)
            if (co + j < p.cout) acc[r][j] += p.bias[co + j];
        }
        if (p.addend) {
#pragma unroll
          for (int j = 0; j < CPT; ++j)
            if (co + j < p.cout) {
              const float a = p.addend[pix * p.addend_ps + co + j];
              acc[r][j] += a;
              any_d |= (a != 0.0f);
            }
        }
        if (p.act != MIE_ACT_NONE) {
          // a pixel none of whose channels changed keeps its state: dy = 0 unless a carry is pending
          if (any_d || p.emitted) {
            if (p.io_vec) {
#pragma unroll
              for (int h = 0; h < CPT / 4; ++h) {
                if (co + h * 4 < p.cout) {
                  float4 *rp = reinterpret_cast<float4 *>(p.res + pix * p.res_ps + co + h * 4);
                  const float4 x = p.refresh ? make_float4(0.f, 0.f, 0.f, 0.f) : *rp;
                  const float4 xn = make_float4(x.x + acc[r][h * 4], x.y + acc[r][h * 4 + 1], x.z + acc[r][h * 4 + 2], x.w + acc[r][h * 4 + 3]);
                  if (any_d) *rp = xn;
                  float4 base;
                  if (p.refresh) base = make_float4(0.f, 0.f, 0.f, 0.f);
                  else if (p.emitted) base = *reinterpret_cast<const float4 *>(p.emitted + pix * p.emitted_ps + co + h * 4);
                  else base = make_float4(act_apply(p.act, x.x), act_apply(p.act, x.y), act_apply(p.act, x.z), act_apply(p.act, x.w));
                  acc[r][h * 4 + 0] = act_apply(p.act, xn.x) - base.x;
                  acc[r][h * 4 + 1] = act_apply(p.act, xn.y) - base.y;
                  acc[r][h * 4 + 2] = act_apply(p.act, xn.z) - base.z;
                  acc[r][h * 4 + 3] = act_apply(p.act, xn.w) - base.w;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < CPT; ++j)
                if (co + j < p.cout) {
                  float *rp = p.res + pix * p.res_ps + co + j;
                  const float x = p.refresh ? 0.0f : *rp, xn = x + acc[r][j];
                  if (any_d) *rp = xn;
                  const float base = p.refresh ? 0.0f : (p.emitted ? p.emitted[pix * p.emitted_ps + co + j] : act_apply(p.act, x));
                  acc[r][j] = act_apply(p.act, xn) - base;
                }
            }
          }
        }
        bool f = p.refresh != 0;   // a dense evaluation marks every pixel it wrote
#pragma unroll
        for (int j = 0; j < CPT; ++j) f |= (co + j < p.cout) && (fabsf(acc[r][j]) > p.thr);
        if (f) rowflags |= 1u << r;
      }
    }
    // combine the per-pixel flags of all channels handled by this block
    {
      unsigned lo = 0, hi = 0;
#pragma unroll
      for (int r = 0; r < 4; ++r) if ((rowflags >> r) & 1u) lo |= 1u << (r * 8 + pc);
#pragma unroll
      for (int r = 4; r < 8; ++r) if ((rowflags >> r) & 1u) hi |= 1u << ((r - 4) * 8 + pc);
      lo = __reduce_or_sync(0xffffffffu, lo);
      hi = __reduce_or_sync(0xffffffffu, hi);
      if (WN > 1) {
        if (lane == 0 && (lo | hi)) atomicOr(&s_bits[ts], ((unsigned long long)hi << 32) | lo);
        __syncthreads();
      } else {
        if (lane == 0) s_bits[ts] = ((unsigned long long)hi << 32) | lo;
        __syncwarp();
      }
    }
    const unsigned long long word = s_bits[ts];
    // Send decision of a thresholded layer: per pixel and per group of MIE_THR_GROUP = 16 consecutive output channels.
    // A thread holds CPT channels of 8 pixels (one tile column); the lanes that hold the other channels of the same
    // group and column are 8 (CPT = 8: two lanes per group) or 8, 16 and 24 (CPT = 4: the warp is one group) away.
    unsigned groupflags = rowflags | __shfl_xor_sync(0xffffffffu, rowflags, 8);
    if (CPT == 4) groupflags |= __shfl_xor_sync(0xffffffffu, groupflags, 16);
    if (t >= 0) {
      if (lane == 0 && wn == 0 && word) {
        if (n_cblk > 1) atomicOr(p.out_bits + t, word);
        else p.out_bits[t] = word;
      }
      if (ox < p.wout) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int oy = ty * 8 + r;
          if (oy >= p.hout) continue;
          const int64_t pix = (int64_t)(n * p.hout + oy) * p.wout + ox;
          const bool send = (groupflags >> r) & 1u;
          if (p.io_vec) {
#pragma unroll
            for (int h = 0; h < CPT / 4; ++h)
              if (co + h * 4 < p.cout) {
                const float4 v = send ? make_float4(acc[r][h * 4], acc[r][h * 4 + 1], acc[r][h * 4 + 2], acc[r][h * 4 + 3])
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(p.out + pix * p.out_ps + co + h * 4) = v;
                if (p.emitted && send) {
                  float4 *ep = reinterpret_cast<float4 *>(p.emitted + pix * p.emitted_ps + co + h * 4);
                  float4 e = *ep;
                  e.x += v.x; e.y += v.y; e.z += v.z; e.w += v.w;
                  *ep = e;
                }
              }
          } else {
#pragma unroll
            for (int j = 0; j < CPT; ++j)
              if (co + j < p.cout) {
                const float v = send ? acc[r][j] : 0.0f;
                p.out[pix * p.out_ps + co + j] = v;
                if (p.emitted && send) p.emitted[pix * p.emitted_ps + co + j] += v;
              }
          }
        }
      }
    }
  }
  run_tail_job(p.tail);
}


// ---------------------------------------------------------------------------------------------
// 1x1 convolution to a handful of output channels (prediction heads: 32 -> 1, 64 -> 2, ...).
// One thread per pixel, one 64-thread group per active tile; the filter sits in shared memory.
// ---------------------------------------------------------------------------------------------
constexpr int SMALL_COUT = 4;

__global__ void __launch_bounds__(256) conv1x1_small_kernel(const ConvParams p) {
  grid_dependency_wait();
  grid_dependency_trigger();
  extern __shared__ float s_w[];  // [cin][SMALL_COUT]
  const int tid = threadIdx.x, grp = tid >> 6, px = tid & 63, lane = tid & 31;
  for (int i = tid; i < p.cin * SMALL_COUT; i += blockDim.x) {
    const int ci = i / SMALL_COUT, co = i - ci * SMALL_COUT;
    s_w[i] = (co < p.cout) ? p.w[(int64_t)ci * p.cout_pad + co] : 0.0f;
  }
  __syncthreads();
  const int THo = (p.hout + 7) >> 3, TWo = (p.wout + 7) >> 3;
  const int ntiles_total = p.n * THo * TWo;
  unsigned *bits32 = reinterpret_cast<unsigned *>(p.out_bits);
  const bool head_ok = run_head_job(p.head, HEAD_SPIN_LIMIT);
  if (threadIdx.x == blockDim.x - 1) count_head_job_passed(p.head);
  const int n_stale = (p.stale && head_ok) ? min(p.counts[1], p.max_tiles) : 0;
  for (int s = blockIdx.x * 4 + grp; s < n_stale; s += gridDim.x * 4) {
    const int t = p.stale[s];
    if (t < 0 || t >= ntiles_total) { if (px == 0) atomicOr(&p.counts[3], MIE_ERR_BAD_TILE); continue; }
    const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
    const int oy = ty * 8 + (px >> 3), ox = tx * 8 + (px & 7);
    if (oy < p.hout && ox < p.wout)
      for (int c = 0; c < p.cout; ++c) p.out[((int64_t)(n * p.hout + oy) * p.wout + ox) * p.out_ps + c] = 0.0f;
  }
  const int n_active = head_ok ? min(p.counts[0], p.max_tiles) : 0;
  for (int li = blockIdx.x * 4 + grp; li < n_active; li += gridDim.x * 4) {
    const int t = p.list[li];
    if (t < 0 || t >= ntiles_total) { if (px == 0) atomicOr(&p.counts[3], MIE_ERR_BAD_TILE); continue; }
    const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
    const int oy = ty * 8 + (px >> 3), ox = tx * 8 + (px & 7);
    const bool valid = oy < p.hout && ox < p.wout;
    bool flag = false;
    if (valid) {
      const int64_t pix = (int64_t)(n * p.hout + oy) * p.wout + ox;  // 1x1, stride 1: input pixel == output pixel
      const float *ip = p.in + pix * p.in_ps;
      const float *ip2 = p.in2 ? p.in2 + pix * p.in2_ps : nullptr;
      float acc[SMALL_COUT] = {0.f, 0.f, 0.f, 0.f};
      if (p.in_vec) {
        for (int c = 0; c + 3 < p.cin; c += 4) {
          float4 v = *reinterpret_cast<const float4 *>(ip + c);
          if (ip2) {
            const float4 u = *reinterpret_cast<const float4 *>(ip2 + c);
            v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
          }
          const float *w = s_w + c * SMALL_COUT;
#pragma unroll
          for (int j = 0; j < SMALL_COUT; ++j)
            acc[j] += v.x * w[j] + v.y * w[SMALL_COUT + j] + v.z * w[2 * SMALL_COUT + j] + v.w * w[3 * SMALL_COUT + j];
        }
        for (int c = p.cin & ~3; c < p.cin; ++c) {
          const float v = ip[c] + (ip2 ? ip2[c] : 0.0f);
#pragma unroll
          for (int j = 0; j < SMALL_COUT; ++j) acc[j] += v * s_w[c * SMALL_COUT + j];
        }
      } else {
        for (int c = 0; c < p.cin; ++c) {
          const float v = ip[c] + (ip2 ? ip2[c] : 0.0f);
#pragma unroll
          for (int j = 0; j < SMALL_COUT; ++j) acc[j] += v * s_w[c * SMALL_COUT + j];
        }
      }
      bool any_d = p.refresh != 0;
#pragma unroll
      for (int j = 0; j < SMALL_COUT; ++j) {
        if (j < p.cout && p.bias) acc[j] += p.bias[j];
        if (j < p.cout && p.addend) acc[j] += p.addend[pix * p.addend_ps + j];
        any_d |= (j < p.cout) && (acc[j] != 0.0f);
      }
      float dy[SMALL_COUT];
#pragma unroll
      for (int j = 0; j < SMALL_COUT; ++j) {
        dy[j] = acc[j];
        if (j < p.cout && p.act != MIE_ACT_NONE) {
          if (any_d || p.emitted) {
            float *rp = p.res + pix * p.res_ps + j;
            const float x = p.refresh ? 0.0f : *rp, xn = x + acc[j];
            if (any_d) *rp = xn;
            const float base = p.refresh ? 0.0f : (p.emitted ? p.emitted[pix * p.emitted_ps + j] : act_apply(p.act, x));
            dy[j] = act_apply(p.act, xn) - base;
          } else {
            dy[j] = 0.0f;
          }
        }
        flag |= (j < p.cout) && fabsf(dy[j]) > p.thr;
      }
      flag |= p.refresh != 0;
#pragma unroll
      for (int j = 0; j < SMALL_COUT; ++j)
        if (j < p.cout) {
          const float v = flag ? dy[j] : 0.0f;
          p.out[pix * p.out_ps + j] = v;
          if (p.emitted && flag) p.emitted[pix * p.emitted_ps + j] += v;
          if (p.accum && flag) p.accum[pix * p.accum_ps + j] += v;
        }
    }
    const unsigned half = __ballot_sync(0xffffffffu, flag);
    if (lane == 0 && half) bits32[2 * (size_t)t + ((px >> 5) & 1)] = half;
  }
  run_tail_job(p.tail);
}

template <int K, int S, int WT, int WN, int CPT = 8>
int launch_conv(const ConvParams &p, int max_items, cudaStream_t st) {
  using G = Geo<K, S>;
  constexpr int NT = 32 * WT * WN;
  constexpr int NB = 4 * CPT * WN;
  const size_t smem = (size_t)WT * G::A_TILE_F4 * 16 + (size_t)2 * K * CC * NB * 4;
  // the attribute belongs to (kernel, device): remembered per instantiation and per device (a race between two host
  // threads sets the same value twice)
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MIE_ECUDA;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(conv_tiles_kernel<K, S, WT, WN, CPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
    attr_set[dev] = true;
  }
  // persistent grid: enough blocks to fill the machine, never more than the work that can exist
  int per_sm = (int)((200 * 1024) / (smem + 1024));
  const int by_threads = 2048 / NT;
  if (per_sm > by_threads) per_sm = by_threads;
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 4) per_sm = 4;
  int grid = MIE_SM_COUNT * per_sm;
  if (grid > max_items) grid = max_items;
  if (grid < 1) grid = 1;
  launch_chained(conv_tiles_kernel<K, S, WT, WN, CPT>, dim3(grid), dim3(NT), smem, st, p);
  return check_launch();
}

template <int K, int S>
int dispatch_w(const ConvParams &p, int wt, int wn, int max_items, cudaStream_t st) {
  if (wt == 4 && wn == 1) return launch_conv<K, S, 4, 2, 4>(p, max_items, st);  // 32 channels: 2 warps x 16 channels per tile
  if (wt == 4 && wn == 2) return launch_conv<K, S, 4, 2>(p, max_items, st);
  if (wt == 2 && wn == 4) return launch_conv<K, S, 2, 4>(p, max_items, st);
  if (wt == 1 && wn == 8) return launch_conv<K, S, 1, 8>(p, max_items, st);
  return MIE_EUNSUPPORTED;
}

}  // namespace

extern "C" int mie_conv_pack_dims(int cin, int cout, int k, int *cin_pad, int *cout_pad, int64_t *n_floats) {
  if (cin <= 0 || cout <= 0 || k <= 0) return MIE_EINVAL;
  const int cp = divup(cin, CC) * CC, op = divup(cout, 32) * 32;
  if (cin_pad) *cin_pad = cp;
  if (cout_pad) *cout_pad = op;
  if (n_floats) *n_floats = (int64_t)k * k * cp * op;
  return MIE_OK;
}

__global__ void pack_weights_kernel(const float *__restrict__ w, int cout, int cin, int k, int cin_pad, int cout_pad,
                                    float *__restrict__ wp, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int co = (int)(i % cout_pad);
    int64_t rest = i / cout_pad;
    const int ci = (int)(rest % cin_pad);
    const int tap = (int)(rest / cin_pad);
    float v = 0.0f;
    if (co < cout && ci < cin) v = w[((int64_t)co * cin + ci) * k * k + tap];
    wp[i] = v;
  }
}

extern "C" int mie_pack_conv_weights(const float *w_oihw, int cout, int cin, int k, float *wpacked, void *stream) {
  if (!w_oihw || !wpacked) return MIE_EINVAL;
  int cp, op;
  int64_t total;
  int s = mie_conv_pack_dims(cin, cout, k, &cp, &op, &total);
  if (s != MIE_OK) return s;
  int blocks = (int)((total + 255) / 256);
  if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
  pack_weights_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(w_oihw, cout, cin, k, cp, op, wpacked, total);
  return check_launch();
}

extern "C" int mie_conv_uses_tensor_cores(const mie_conv_args *a) { return (a && tc_eligible(a)) ? 1 : 0; }

extern "C" int mie_conv_tiles(const mie_conv_args *a, void *stream) {
  if (!a || !a->in || !a->wpacked || !a->list || !a->counts || !a->out || !a->out_bits) return MIE_EINVAL;
  if (a->cin <= 0 || a->cout <= 0 || a->n <= 0 || a->hin <= 0 || a->win <= 0 || a->hout <= 0 || a->wout <= 0) return MIE_EINVAL;
  if (a->in_ps < a->cin || a->out_ps < a->cout || a->max_tiles <= 0 || !(a->thr >= 0.0f)) return MIE_EINVAL;
  if (a->cin_pad % CC || a->cin_pad < a->cin || a->cout_pad % 32 || a->cout_pad < a->cout) return MIE_EINVAL;
  if (a->act != MIE_ACT_NONE && !a->res) return MIE_EINVAL;
  if (a->act < 0 || a->act > MIE_ACT_TANH) return MIE_EINVAL;
  if (a->act == MIE_ACT_NONE && a->emitted) return MIE_EINVAL;
  if (a->refresh && (a->thr != 0.0f || a->emitted)) return MIE_EINVAL;
  if (a->stride < 1 || a->stride > 2) return MIE_EUNSUPPORTED;
  if (!aligned16(a->wpacked)) return MIE_EALIGN;
  if (a->wpacked_tc && !aligned16(a->wpacked_tc)) return MIE_EALIGN;
  if (tail_check(a->tail, a->out_bits) != MIE_OK || head_check(a->head, a) != MIE_OK) return MIE_EINVAL;
  // Too many tiles for one block, or a cluster kernel (its blocks decide together, from the item count, whether to meet
  // at the closing cluster barrier: a block whose wait for the lists ran out would count differently): the separate
  // launch, then a plain convolution.
  if (a->own_tiles && (!a->head || !a->own_scratch || (reinterpret_cast<uintptr_t>(a->own_scratch) & 7))) return MIE_EINVAL;
  // own-tiles mode exists in the tensor-core kernels only; elsewhere it is the separate launch and a plain convolution
  if (a->head && (a->own_tiles ? !tc_eligible(a) : (!tail_fits(a->head) || mie_conv_cluster_size(a) > 1))) {
    const mie_tail_job *h = a->head;
    const int s = mie_tiles_dilate(h->in_bits, h->N, h->Hin, h->Win, h->Hout, h->Wout, h->k, h->stride, h->pad, h->union_bits,
                                   h->out_bits, h->list, h->stale, h->counts, h->flags, stream);
    if (s != MIE_OK) return s;
    mie_conv_args b = *a;
    b.head = nullptr;
    b.own_tiles = 0;
    return mie_conv_tiles(&b, stream);
  }
  if (tc_eligible(a)) return tail_after_launch(launch_conv_tc(a, (cudaStream_t)stream), a->tail, true, stream);

  ConvParams p;
  p.in = a->in; p.in_ps = a->in_ps; p.cin = a->cin; p.hin = a->hin; p.win = a->win;
  p.w = a->wpacked; p.cin_pad = a->cin_pad; p.cout = a->cout; p.cout_pad = a->cout_pad;
  p.n = a->n; p.hout = a->hout; p.wout = a->wout; p.pad = a->pad;
  p.list = a->list; p.stale = a->stale; p.counts = a->counts; p.max_tiles = a->max_tiles;
  p.out = a->out; p.out_ps = a->out_ps; p.out_bits = reinterpret_cast<unsigned long long *>(a->out_bits);
  p.act = a->act; p.thr = a->thr;
  p.res = a->res; p.res_ps = a->res_ps; p.emitted = a->emitted; p.emitted_ps = a->emitted_ps;
  p.addend = a->addend; p.addend_ps = a->addend_ps;
  p.bias = a->bias; p.refresh = a->refresh ? 1 : 0;
  p.tail = tail_for_kernel(a->tail);
  p.head = tail_for_kernel(a->head);
  p.in2 = a->in2; p.in2_ps = a->in2_ps; p.accum = a->accum; p.accum_ps = a->accum_ps;
  if (a->in2 && a->in2_ps < a->cin) return MIE_EINVAL;
  if (a->accum && (a->accum_ps < a->cout || a->refresh)) return MIE_EINVAL;
  // 16-byte staging reads whole channel quads: with cin % 4 != 0 the last quad reaches into the pixel's
  // padding channels (in_ps >= cin rounded up to 4), which meet zero filter rows and must be finite
  p.in_vec = (a->in_ps % 4 == 0) && aligned16(a->in) && (a->in_ps >= (a->cin + 3) / 4 * 4);
  p.io_vec = (a->cout % 4 == 0) && (a->out_ps % 4 == 0) && aligned16(a->out) &&
             (!a->res || ((a->res_ps % 4 == 0) && aligned16(a->res))) &&
             (!a->emitted || ((a->emitted_ps % 4 == 0) && aligned16(a->emitted)));

  if (a->k == 1 && a->stride == 1 && a->pad == 0 && a->cout <= SMALL_COUT && a->cin <= 2048) {
    int blocks = divup(a->max_tiles, 4);
    if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
    p.in_vec = p.in_vec && (a->cin % 4 == 0 || a->in_ps >= (a->cin + 3) / 4 * 4) &&
               (!a->in2 || (a->in2_ps % 4 == 0 && aligned16(a->in2) && a->in2_ps >= (a->cin + 3) / 4 * 4));
    launch_chained(conv1x1_small_kernel, dim3(blocks), dim3(256), (size_t)a->cin * SMALL_COUT * sizeof(float), (cudaStream_t)stream, p);
    return tail_after_launch(check_launch(), a->tail, true, stream);
  }

  if (a->in2 || a->accum) return MIE_EUNSUPPORTED;   // only the 1x1 head kernel above takes them
  // block shape: 32 channels -> 4 tiles x 1; otherwise 4 tiles x 64 channels.  (A thresholded fused activation
  // decides per 16-channel group, which both shapes hold inside one warp.)
  int wt = 4, wn = 2;
  if (a->cout_pad == 32 || a->cout_pad % 64) wn = 1;

  const int64_t max_items64 = (int64_t)divup(a->max_tiles, wt) * (a->cout_pad / (32 * wn));
  const int max_items = (int)(max_items64 > (1 << 30) ? (1 << 30) : max_items64);
  cudaStream_t st = (cudaStream_t)stream;
  const int k = a->k, s = a->stride;
#define MIE_CASE(KK, SS) if (k == KK && s == SS) return tail_after_launch(dispatch_w<KK, SS>(p, wt, wn, max_items, st), a->tail, true, stream)
  MIE_CASE(1, 1); MIE_CASE(1, 2); MIE_CASE(3, 1); MIE_CASE(3, 2);
  MIE_CASE(5, 1); MIE_CASE(5, 2); MIE_CASE(7, 1); MIE_CASE(7, 2);
#undef MIE_CASE
  return MIE_EUNSUPPORTED;
}

// ---------------------------------------------------------------------------------------------
// reference-shaped entry point: conv{k}x{k}_increment_ext(x_incr, mask, filter, out_incr, stride)
// ---------------------------------------------------------------------------------------------
namespace {
struct IncWs {
  size_t bits_in, bits_out, list, stale, counts, flags, wpacked, total;
};
IncWs inc_layout(int N, int cin, int H, int W, int cout, int k, int stride) {
  const int pad = k / 2;
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  const size_t nti = (size_t)N * divup(H, 8) * divup(W, 8), nto = (size_t)N * divup(Ho, 8) * divup(Wo, 8);
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  IncWs w;
  size_t o = 0;
  w.bits_in = o; o += up(nti * 8);
  w.bits_out = o; o += up(nto * 8);
  w.list = o; o += up(nto * 4);
  w.stale = o; o += up(nto * 4);
  w.counts = o; o += 256;
  w.flags = o; o += up(nto);
  int cp, op; int64_t nf;
  mie_conv_pack_dims(cin, cout, k, &cp, &op, &nf);
  w.wpacked = o; o += up((size_t)nf * 4);
  w.total = o;
  return w;
}
__global__ void pack_weights_ihwo_kernel(const float *__restrict__ f, int cout, int cin, int k, int cin_pad, int cout_pad,
                                         float *__restrict__ wp, int64_t total) {
  // f[ci][ky][kx][co]  ->  wp[ky*k+kx][ci][co]
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int co = (int)(i % cout_pad);
    int64_t rest = i / cout_pad;
    const int ci = (int)(rest % cin_pad);
    const int tap = (int)(rest / cin_pad);
    float v = 0.0f;
    if (co < cout && ci < cin) v = f[((int64_t)ci * k * k + tap) * cout + co];
    wp[i] = v;
  }
}
}  // namespace

extern "C" int64_t mie_conv_increment_workspace_bytes(int N, int cin, int H, int W, int cout, int k, int stride) {
  if (N <= 0 || cin <= 0 || H <= 0 || W <= 0 || cout <= 0 || k <= 0 || stride <= 0) return MIE_EINVAL;
  return (int64_t)inc_layout(N, cin, H, W, cout, k, stride).total;
}

extern "C" int mie_conv_increment_ext(const float *x_incr, const void *mask, int mask_elem_size, const float *filter,
                                      float *out_incr, int N, int cin, int H, int W, int cout, int k, int stride,
                                      void *workspace, int64_t workspace_bytes, void *stream) {
  if (!x_incr || !filter || !out_incr || !workspace) return MIE_EINVAL;
  if (N <= 0 || cin <= 0 || H <= 0 || W <= 0 || cout <= 0) return MIE_EINVAL;
  if (!(k == 1 || k == 3 || k == 5 || k == 7) || stride < 1 || stride > 2) return MIE_EUNSUPPORTED;
  if (mask && mask_elem_size != 1 && mask_elem_size != 4) return MIE_EUNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return MIE_EALIGN;
  const IncWs L = inc_layout(N, cin, H, W, cout, k, stride);
  if (workspace_bytes < (int64_t)L.total) return MIE_ETOOBIG;
  const int pad = k / 2;
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  const int nto = N * divup(Ho, 8) * divup(Wo, 8);
  char *ws = static_cast<char *>(workspace);
  uint64_t *bits_in = reinterpret_cast<uint64_t *>(ws + L.bits_in);
  uint64_t *bits_out = reinterpret_cast<uint64_t *>(ws + L.bits_out);
  int32_t *list = reinterpret_cast<int32_t *>(ws + L.list), *stale = reinterpret_cast<int32_t *>(ws + L.stale);
  int32_t *counts = reinterpret_cast<int32_t *>(ws + L.counts);
  uint8_t *flags = reinterpret_cast<uint8_t *>(ws + L.flags);
  float *wp = reinterpret_cast<float *>(ws + L.wpacked);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e;
  if ((e = cudaMemsetAsync(counts, 0, 16, st)) != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  if ((e = cudaMemsetAsync(bits_out, 0, (size_t)nto * 8, st)) != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  // the caller hands in uninitialised memory: inactive tiles must read as zero
  if ((e = cudaMemsetAsync(out_incr, 0, (size_t)N * Ho * Wo * cout * 4, st)) != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  int s;
  if (mask) s = mie_mask_from_mask(mask, mask_elem_size, cin, cin, N, H, W, bits_in, stream);
  else s = mie_mask_from_delta(x_incr, cin, N, cin, H, W, 0.0f, bits_in, stream);
  if (s != MIE_OK) return s;
  int cp, op; int64_t nf;
  mie_conv_pack_dims(cin, cout, k, &cp, &op, &nf);
  {
    int blocks = (int)((nf + 255) / 256);
    if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
    pack_weights_ihwo_kernel<<<blocks, 256, 0, st>>>(filter, cout, cin, k, cp, op, wp, nf);
    if ((s = check_launch()) != MIE_OK) return s;
  }
  s = mie_tiles_dilate(bits_in, N, H, W, Ho, Wo, k, stride, pad, nullptr, nullptr, list, nullptr, counts, flags, stream);
  if (s != MIE_OK) return s;
  mie_conv_args a;
  memset(&a, 0, sizeof(a));
  a.in = x_incr; a.in_ps = cin; a.cin = cin; a.hin = H; a.win = W;
  a.wpacked = wp; a.cin_pad = cp; a.cout = cout; a.cout_pad = op;
  a.n = N; a.hout = Ho; a.wout = Wo; a.k = k; a.stride = stride; a.pad = pad;
  a.list = list; a.stale = nullptr; a.counts = counts; a.max_tiles = nto;
  a.out = out_incr; a.out_ps = cout; a.out_bits = bits_out;
  a.act = MIE_ACT_NONE; a.thr = 0.0f;
  return mie_conv_tiles(&a, stream);
}
