// Fused incremental point operations over delta fields.
//
// Every kernel walks all 8x8 tiles with a grid-stride loop, one thread block per tile at a time.
// A tile whose input words are all zero costs one 8-byte read (plus clearing stale output if the
// output tile held data from the previous step).  Inside an active tile only the active pixels touch
// the persistent state, so reservoir traffic follows the pixel mask, not the tile mask.
#include "mie_common.cuh"

using namespace mie;

namespace {

constexpr int PW_THREADS = 128;

static int tile_grid(int ntiles) {
  const int cap = MIE_SM_COUNT * 8;
  return ntiles < cap ? (ntiles > 0 ? ntiles : 1) : cap;
}

struct TileGeom {
  int n, ty, tx, rows, cols;
};

__device__ __forceinline__ TileGeom tile_geom(int t, int H, int W) {
  const int TH = (H + 7) >> 3, TW = (W + 7) >> 3;
  TileGeom g;
  g.tx = t % TW;
  g.ty = (t / TW) % TH;
  g.n = t / (TW * TH);
  g.rows = min(8, H - g.ty * 8);
  g.cols = min(8, W - g.tx * 8);
  return g;
}

__device__ __forceinline__ int64_t pix_index(const TileGeom &g, int p, int H, int W) {
  return (int64_t)(g.n * H + g.ty * 8 + (p >> 3)) * W + g.tx * 8 + (p & 7);
}

__device__ __forceinline__ bool pix_valid(const TileGeom &g, int p) { return (p >> 3) < g.rows && (p & 7) < g.cols; }

// zero every channel of every valid pixel of a tile
__device__ __forceinline__ void zero_tile(float *out, int64_t ps, int C, const TileGeom &g, int H, int W) {
  for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
    const int p = e / C, c = e - p * C;
    if (pix_valid(g, p)) out[pix_index(g, p, H, W) * ps + c] = 0.0f;
  }
}

__device__ __forceinline__ void or_word(unsigned *s_lo_hi, int p) {
  atomicOr(&s_lo_hi[p >> 5], 1u << (p & 31));
}

// ---------------------------------------------------------------------------------------------
// incremental activation
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) act_incr_kernel(
    const float *in, int64_t in_ps, const uint64_t *__restrict__ in_bits, float *__restrict__ res,
    int64_t res_ps, float *__restrict__ emitted, int64_t em_ps, float *out, int64_t out_ps, uint64_t *out_bits,
    int N, int C, int H, int W, int op, float thr, int accumulate) {
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ unsigned long long s_g[64];   // per pixel: which groups of 16 channels have a change above the threshold
  __shared__ unsigned s_w[2];
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t win = in_bits[t];
    const TileGeom g = tile_geom(t, H, W);
    if (win == 0ull) {
      if (out_bits[t] != 0ull) {  // uniform across the block
        __syncthreads();
        zero_tile(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    if (threadIdx.x < 64) s_g[threadIdx.x] = 0ull;
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
      const int p = e / C, c = e - p * C;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float dy = 0.0f;
      if ((win >> p) & 1ull) {
        const float d = in[pix * in_ps + c];
        const float x = res[pix * res_ps + c];
        const float xn = x + d;
        if (accumulate) res[pix * res_ps + c] = xn;
        const float base = emitted ? emitted[pix * em_ps + c] : act_apply(op, x);
        dy = act_apply(op, xn) - base;
        if (fabsf(dy) > thr) atomicOr(&s_g[p], 1ull << (c >> 4));
      }
      out[pix * out_ps + c] = dy;
    }
    __syncthreads();
    if (threadIdx.x < 64) {   // the tile word: a pixel is active when one of its groups is sent
      const unsigned bal = __ballot_sync(0xffffffffu, s_g[threadIdx.x] != 0ull);
      if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = bal;
    }
    if (thr > 0.0f || emitted) {
      // second pass: withheld groups are written as zero; sent groups are added to the carry
      for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
        const int p = e / C, c = e - p * C;
        if (!pix_valid(g, p) || !((win >> p) & 1ull)) continue;
        const int64_t pix = pix_index(g, p, H, W);
        if ((s_g[p] >> (c >> 4)) & 1ull) {
          if (emitted) emitted[pix * em_ps + c] += out[pix * out_ps + c];
        } else {
          out[pix * out_ps + c] = 0.0f;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) out_bits[t] = ((uint64_t)s_w[1] << 32) | s_w[0];
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// incremental product
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) mul_incr_kernel(
    const float *__restrict__ d1, int64_t d1_ps, const uint64_t *__restrict__ bits1, float *__restrict__ x1, int64_t x1_ps,
    const float *__restrict__ d2, int64_t d2_ps, const uint64_t *__restrict__ bits2, float *__restrict__ x2, int64_t x2_ps,
    float *__restrict__ out, int64_t out_ps, uint64_t *__restrict__ out_bits, int N, int C, int H, int W, float thr,
    int accumulate) {
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ unsigned s_w[2];
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t w1 = (d1 && bits1) ? bits1[t] : 0ull, w2 = (d2 && bits2) ? bits2[t] : 0ull;
    const uint64_t win = w1 | w2;
    const TileGeom g = tile_geom(t, H, W);
    if (win == 0ull) {
      if (out_bits[t] != 0ull) {
        __syncthreads();
        zero_tile(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    if (threadIdx.x < 2) s_w[threadIdx.x] = 0u;
    __syncthreads();
    for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
      const int p = e / C, c = e - p * C;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float d = 0.0f;
      if ((win >> p) & 1ull) {
        const float a = ((w1 >> p) & 1ull) ? d1[pix * d1_ps + c] : 0.0f;
        const float b = ((w2 >> p) & 1ull) ? d2[pix * d2_ps + c] : 0.0f;
        const float v1 = x1[pix * x1_ps + c], v2 = x2[pix * x2_ps + c];
        d = (b + v2) * a + v1 * b;
        if (accumulate && a != 0.0f) x1[pix * x1_ps + c] = v1 + a;
        if (accumulate && b != 0.0f) x2[pix * x2_ps + c] = v2 + b;
        if (fabsf(d) > thr) or_word(s_w, p);
      }
      out[pix * out_ps + c] = d;
    }
    __syncthreads();
    const uint64_t wout = ((uint64_t)s_w[1] << 32) | s_w[0];
    if (thr > 0.0f) {
      for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
        const int p = e / C, c = e - p * C;
        if (pix_valid(g, p) && ((win >> p) & 1ull) && !((wout >> p) & 1ull)) out[pix_index(g, p, H, W) * out_ps + c] = 0.0f;
      }
    }
    if (threadIdx.x == 0) out_bits[t] = wout;
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// ConvLSTM point-wise block
// ---------------------------------------------------------------------------------------------
// Sigmoid and tanh of the ConvLSTM point kernels: one ex2.approx and one rcp.approx each instead of libm's expf / tanhf
// and an IEEE division -- a third of the instructions; with ten of them per element the kernel was bound by
// instruction issue, not by memory.  Relative error below 1e-6 (tanh switches to its odd Taylor polynomial below 0.4,
// where the exponential form would lose relative accuracy; small gate and cell values keep theirs), two orders of
// magnitude inside the 1e-4 parity bar.  The same function evaluates f(x) and f(x + dx): an unchanged input still
// gives an exactly zero delta, and the deltas of successive steps still telescope.
__device__ __forceinline__ float sigmoidf_acc(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float tanhf_acc(float x) {
  const float ax = fabsf(x);
  if (ax < 0.4f) {
    const float x2 = x * x;
    float p = -1382.0f / 155925.0f;
    p = fmaf(p, x2, 62.0f / 2835.0f);
    p = fmaf(p, x2, -17.0f / 315.0f);
    p = fmaf(p, x2, 2.0f / 15.0f);
    p = fmaf(p, x2, -1.0f / 3.0f);
    p = fmaf(p, x2, 1.0f);
    return x * p;
  }
  const float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * ax));   // exp overflows to inf beyond 44: t = 1
  return copysignf(t, x);
}

__global__ void __launch_bounds__(PW_THREADS) convlstm_point_kernel(
    const float *__restrict__ dg, int64_t dg_ps, const uint64_t *__restrict__ dg_bits, float *__restrict__ gres, int64_t g_ps,
    const float *__restrict__ dcp, int64_t dcp_ps, const uint64_t *__restrict__ dcp_bits, float *__restrict__ cprev,
    int64_t cprev_ps, float *__restrict__ cell, int64_t cell_ps, float *__restrict__ dh, int64_t dh_ps,
    uint64_t *__restrict__ dh_bits, float *__restrict__ dc, int64_t dc_ps, uint64_t *__restrict__ dc_bits, int N, int C,
    int H, int W, int sum_m2, float thr) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t wg = dg_bits[t];
    const uint64_t wc = (dcp && dcp_bits) ? dcp_bits[t] : 0ull;
    const uint64_t win = wg | wc;
    const TileGeom g = tile_geom(t, H, W);
    if (win == 0ull) {
      const bool sh = dh_bits[t] != 0ull, sc = dc_bits[t] != 0ull;
      if (sh || sc) {
        __syncthreads();
        if (sh) zero_tile(dh, dh_ps, C, g, H, W);
        if (sc) zero_tile(dc, dc_ps, C, g, H, W);
        if (threadIdx.x == 0) { dh_bits[t] = 0ull; dc_bits[t] = 0ull; }
      }
      continue;
    }
    for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
      const int p = e / C, c = e - p * C;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float o_h = 0.0f, o_c = 0.0f;
      if ((win >> p) & 1ull) {
        const bool hg = (wg >> p) & 1ull;
        float *gp = gres + pix * g_ps + c;
        const float gi = gp[0], gf = gp[C], go = gp[2 * C], gc = gp[3 * C];
        float di = 0.f, df = 0.f, dob = 0.f, dcg = 0.f;
        if (hg) {
          const float *dp = dg + pix * dg_ps + c;
          di = dp[0]; df = dp[C]; dob = dp[2 * C]; dcg = dp[3 * C];
          gp[0] = gi + di; gp[C] = gf + df; gp[2 * C] = go + dob; gp[3 * C] = gc + dcg;
        }
        const float i_o = sigmoidf_acc(gi), f_o = sigmoidf_acc(gf), o_o = sigmoidf_acc(go), g_o = tanhf_acc(gc);
        const float Di = sigmoidf_acc(gi + di) - i_o, Df = sigmoidf_acc(gf + df) - f_o;
        const float Do = sigmoidf_acc(go + dob) - o_o, Dg = tanhf_acc(gc + dcg) - g_o;
        const float m1 = (Dg + g_o) * Di + i_o * Dg;
        float m2 = 0.0f;
        if (cprev) {
          const float cp_o = cprev[pix * cprev_ps + c];
          const float Dcp = ((wc >> p) & 1ull) ? dcp[pix * dcp_ps + c] : 0.0f;
          m2 = (Dcp + cp_o) * Df + f_o * Dcp;
          if (Dcp != 0.0f) cprev[pix * cprev_ps + c] = cp_o + Dcp;
        }
        const float Dc = sum_m2 ? (m1 + m2) : m1;
        const float c_o = cell[pix * cell_ps + c];
        const float tc_o = tanhf_acc(c_o);
        const float Dtc = tanhf_acc(c_o + Dc) - tc_o;
        if (Dc != 0.0f) cell[pix * cell_ps + c] = c_o + Dc;
        o_h = (Dtc + tc_o) * Do + o_o * Dtc;
        o_c = Dc;
      }
      dh[pix * dh_ps + c] = o_h;
      dc[pix * dc_ps + c] = o_c;
    }
    __syncthreads();
    if (threadIdx.x == 0) { dh_bits[t] = win; dc_bits[t] = win; }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// x2 upsample of (a + b)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool bit_at(const uint64_t *bits, int n, int y, int x, int TH, int TW) {
  return (bits[((int64_t)n * TH + (y >> 3)) * TW + (x >> 3)] >> ((y & 7) * 8 + (x & 7))) & 1ull;
}

// source rows/cols and weights of output coordinate o for a x`scale` upsample of extent L (rs = 1 / scale):
// the index arithmetic of torch's bilinear interpolation with align_corners=False
__device__ __forceinline__ void up_src(int o, int L, int mode, int scale, float rs, int &i0, int &i1, float &w1) {
  if (mode == MIE_UP_NEAREST) { i0 = i1 = o / scale; w1 = 0.0f; return; }
  if (scale == 2) {
    // closed form of the lines below for scale 2 (0.5 * (o + 0.5) - 0.5 = o / 2 - 0.25 is exact in fp32): the same
    // indices and the same weights 0.75 / 0.25, without the conversions
    const int i = o >> 1;
    if (o & 1) { i0 = i; i1 = min(i + 1, L - 1); w1 = 0.25f; }
    else if (i == 0) { i0 = i1 = 0; w1 = 0.0f; }
    else { i0 = i - 1; i1 = i; w1 = 0.75f; }
    return;
  }
  float s = rs * (o + 0.5f) - 0.5f;
  if (s < 0.0f) s = 0.0f;
  i0 = (int)s;
  i1 = min(i0 + 1, L - 1);
  w1 = s - (float)i0;
  if (w1 == 0.0f) i1 = i0;
}

__global__ void __launch_bounds__(PW_THREADS) upsample2x_kernel(
    const float *__restrict__ a, int64_t a_ps, const uint64_t *__restrict__ a_bits, const float *__restrict__ b,
    int64_t b_ps, const uint64_t *__restrict__ b_bits, float *__restrict__ out, int64_t out_ps,
    uint64_t *__restrict__ out_bits, int N, int C, int H, int W, int mode, int scale) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int Ho = scale * H, Wo = scale * W;
  const float rs = 1.0f / (float)scale;
  const int THi = (H + 7) >> 3, TWi = (W + 7) >> 3;
  const int ntiles = N * ((Ho + 7) >> 3) * ((Wo + 7) >> 3);
  __shared__ unsigned s_w[2];
  __shared__ unsigned char s_fa[64], s_fb[64];  // per output pixel: 4 source-activity bits for a and b
  const int ncb = (C + 63) / 64;   // work item = (tile, block of 64 channels)
  const int n_items = ntiles * ncb;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int t = item / ncb, blk = item - t * ncb;
    const TileGeom g = tile_geom(t, Ho, Wo);
    __syncthreads();
    if (threadIdx.x < 64) {
      const int p = threadIdx.x;
      unsigned fa = 0, fb = 0;
      if (pix_valid(g, p)) {
        int y0, y1, x0, x1; float wy, wx;
        up_src(g.ty * 8 + (p >> 3), H, mode, scale, rs, y0, y1, wy);
        up_src(g.tx * 8 + (p & 7), W, mode, scale, rs, x0, x1, wx);
        fa = (bit_at(a_bits, g.n, y0, x0, THi, TWi) ? 1u : 0u) | (bit_at(a_bits, g.n, y0, x1, THi, TWi) ? 2u : 0u) |
             (bit_at(a_bits, g.n, y1, x0, THi, TWi) ? 4u : 0u) | (bit_at(a_bits, g.n, y1, x1, THi, TWi) ? 8u : 0u);
        if (b)
          fb = (bit_at(b_bits, g.n, y0, x0, THi, TWi) ? 1u : 0u) | (bit_at(b_bits, g.n, y0, x1, THi, TWi) ? 2u : 0u) |
               (bit_at(b_bits, g.n, y1, x0, THi, TWi) ? 4u : 0u) | (bit_at(b_bits, g.n, y1, x1, THi, TWi) ? 8u : 0u);
      }
      s_fa[p] = (unsigned char)fa;
      s_fb[p] = (unsigned char)fb;
      const unsigned bal = __ballot_sync(0xffffffffu, (fa | fb) != 0);
      if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = bal;
    }
    __syncthreads();
    const uint64_t wout = ((uint64_t)s_w[1] << 32) | s_w[0];
    if (wout == 0ull) {
      if (blk == 0 && out_bits[t] != 0ull) {   // only this block reads or writes the word
        zero_tile(out, out_ps, C, g, Ho, Wo);
        __syncthreads();
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    const int c_lo = blk * 64, cw = min(C, c_lo + 64) - c_lo;
    for (int e = threadIdx.x; e < 64 * cw; e += blockDim.x) {
      const int p = e / cw, c = c_lo + (e - p * cw);
      if (!pix_valid(g, p)) continue;
      float v = 0.0f;
      const unsigned fa = s_fa[p], fb = s_fb[p];
      if (fa | fb) {
        int y0, y1, x0, x1; float wy, wx;
        up_src(g.ty * 8 + (p >> 3), H, mode, scale, rs, y0, y1, wy);
        up_src(g.tx * 8 + (p & 7), W, mode, scale, rs, x0, x1, wx);
        const int64_t r0 = (int64_t)(g.n * H + y0) * W, r1 = (int64_t)(g.n * H + y1) * W;
        float v00 = 0.f, v01 = 0.f, v10 = 0.f, v11 = 0.f;
        if (fa & 1u) v00 += a[(r0 + x0) * a_ps + c];
        if (fa & 2u) v01 += a[(r0 + x1) * a_ps + c];
        if (fa & 4u) v10 += a[(r1 + x0) * a_ps + c];
        if (fa & 8u) v11 += a[(r1 + x1) * a_ps + c];
        if (fb & 1u) v00 += b[(r0 + x0) * b_ps + c];
        if (fb & 2u) v01 += b[(r0 + x1) * b_ps + c];
        if (fb & 4u) v10 += b[(r1 + x0) * b_ps + c];
        if (fb & 8u) v11 += b[(r1 + x1) * b_ps + c];
        if (mode == MIE_UP_NEAREST) v = v00;
        else v = (1.0f - wy) * ((1.0f - wx) * v00 + wx * v01) + wy * ((1.0f - wx) * v10 + wx * v11);
      }
      out[pix_index(g, p, Ho, Wo) * out_ps + c] = v;
    }
    if (blk == 0 && threadIdx.x == 0) out_bits[t] = wout;
  }
}


// ---------------------------------------------------------------------------------------------
// vectorised variants: work item = (tile, block of CB channels), float4 over channels.
// The output mask of these operators is a function of the input masks alone (no value test), so blocks
// that share a tile need no reduction: block 0 of a tile owns the tile word and the stale clean-up.
// ---------------------------------------------------------------------------------------------
constexpr int CB = 32;  // channels per work item

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ float4 f4add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

__device__ __forceinline__ void zero_tile4(float *out, int64_t ps, int C, const TileGeom &g, int H, int W) {
  const int q4 = C >> 2;
  for (int e = threadIdx.x; e < 64 * q4; e += blockDim.x) {
    const int p = e / q4, q = e - p * q4;
    if (pix_valid(g, p)) st4(out + pix_index(g, p, H, W) * ps + q * 4, make_float4(0.f, 0.f, 0.f, 0.f));
  }
}

__device__ __forceinline__ void lstm_elem(float gi, float gf, float go, float gc, float di, float df, float dob, float dcg,
                                          float cp_o, float Dcp, bool use_cp, float c_o, int sum_m2, float &o_h, float &o_c,
                                          float &h_new) {
  const float i_o = sigmoidf_acc(gi), f_o = sigmoidf_acc(gf), o_o = sigmoidf_acc(go), g_o = tanhf_acc(gc);
  const float Di = sigmoidf_acc(gi + di) - i_o, Df = sigmoidf_acc(gf + df) - f_o;
  const float Do = sigmoidf_acc(go + dob) - o_o, Dg = tanhf_acc(gc + dcg) - g_o;
  const float m1 = (Dg + g_o) * Di + i_o * Dg;
  const float m2 = use_cp ? ((Dcp + cp_o) * Df + f_o * Dcp) : 0.0f;
  const float Dc = sum_m2 ? (m1 + m2) : m1;
  const float tc_o = tanhf_acc(c_o);
  const float Dtc = tanhf_acc(c_o + Dc) - tc_o;
  o_h = (Dtc + tc_o) * Do + o_o * Dtc;
  o_c = Dc;
  h_new = (o_o + Do) * (tc_o + Dtc);   // the hidden value itself: what a thresholded cell differences against what it sent
}

__global__ void __launch_bounds__(PW_THREADS, 6) convlstm_point_vec_kernel(
    const float *__restrict__ dg, int64_t dg_ps, const uint64_t *__restrict__ dg_bits, float *__restrict__ gres, int64_t g_ps,
    const float *__restrict__ dcp, int64_t dcp_ps, const uint64_t *__restrict__ dcp_bits, float *__restrict__ cprev,
    int64_t cprev_ps, float *__restrict__ cell, int64_t cell_ps, float *__restrict__ dh, int64_t dh_ps,
    uint64_t *dh_bits, float *__restrict__ dc, int64_t dc_ps, uint64_t *dc_bits, int N, int C, int H, int W, int sum_m2,
    int cbw /* channels per work item: 32, or fewer on small fields so that every SM gets several blocks */,
    float *__restrict__ hsent, int64_t hs_ps, float thr, unsigned long long *__restrict__ acc_words,
    int *__restrict__ tickets, const mie_tail_job tail) {
  // Thresholded mode (hsent != null, C and cbw multiples of 16): the hidden delta is taken against what has been sent
  // so far, dh = h_new - hsent, and a pixel's group of 16 channels is sent (and added to hsent) when one of its |dh|
  // exceeds thr, else written as zero; the hidden mask is then the set of pixels with a sent group.  The channel blocks
  // of a tile OR their pixels into acc_words[t] and draw a ticket; the block that draws the last one publishes the word
  // and leaves both scratch entries zero for the next launch.  The cell delta and its mask stay lossless.
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ unsigned s_w[2];
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int ncb = (C + cbw - 1) / cbw;
  const int n_items = ntiles * ncb;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int t = item / ncb, cb = item - t * ncb;
    const uint64_t wg = dg_bits[t];
    const uint64_t wc = (dcp && dcp_bits) ? dcp_bits[t] : 0ull;
    const uint64_t win = wg | wc;
    const TileGeom g = tile_geom(t, H, W);
    if (win == 0ull) {
      if (cb == 0) {
        const bool sh = dh_bits[t] != 0ull, sc = dc_bits[t] != 0ull;  // only this block reads or writes them
        if (sh || sc) {
          __syncthreads();
          if (sh) zero_tile4(dh, dh_ps, C, g, H, W);
          if (sc) zero_tile4(dc, dc_ps, C, g, H, W);
          if (threadIdx.x == 0) { dh_bits[t] = 0ull; dc_bits[t] = 0ull; }
        }
      }
      continue;
    }
    if (hsent) {
      __syncthreads();
      if (threadIdx.x < 2) s_w[threadIdx.x] = 0u;
      __syncthreads();
    }
    const int c_lo = cb * cbw, q4 = (min(C, c_lo + cbw) - c_lo) >> 2;
    // thresholded mode: q4 is a multiple of 4, so 64 * q4 is a multiple of the block size and a warp's lanes 4k..4k+3
    // hold the four quads of one 16-channel group of one pixel: no lane leaves the loop before the shuffles below
    const int q4_shift = (q4 & (q4 - 1)) == 0 ? __ffs(q4) - 1 : -1;   // whole blocks: a shift instead of a division
    // (unrolled by two with registers for both elements' loads the kernel ran 18 % slower: four resident blocks instead of six)
    for (int e = threadIdx.x; e < 64 * q4; e += blockDim.x) {
      const int p = q4_shift >= 0 ? (e >> q4_shift) : e / q4, c = c_lo + (e - p * q4) * 4;
      const bool ok = pix_valid(g, p);
      const int64_t pix = ok ? pix_index(g, p, H, W) : 0;
      float4 oh = make_float4(0.f, 0.f, 0.f, 0.f), oc = oh, hn = oh;
      const bool on = ok && ((win >> p) & 1ull);
      if (on) {
        const bool hg = (wg >> p) & 1ull;
        float *gp = gres + pix * g_ps + c;
        const float4 gi = ld4(gp), gf = ld4(gp + C), go = ld4(gp + 2 * C), gc = ld4(gp + 3 * C);
        float4 di = oh, df = oh, dob = oh, dcg = oh;
        if (hg) {
          const float *dp = dg + pix * dg_ps + c;
          di = ld4(dp); df = ld4(dp + C); dob = ld4(dp + 2 * C); dcg = ld4(dp + 3 * C);
          st4(gp, f4add(gi, di)); st4(gp + C, f4add(gf, df)); st4(gp + 2 * C, f4add(go, dob)); st4(gp + 3 * C, f4add(gc, dcg));
        }
        float4 cpo = oh, Dcp = oh;
        if (cprev) {
          cpo = ld4(cprev + pix * cprev_ps + c);
          if ((wc >> p) & 1ull) {
            Dcp = ld4(dcp + pix * dcp_ps + c);
            st4(cprev + pix * cprev_ps + c, f4add(cpo, Dcp));
          }
        }
        const float4 co = ld4(cell + pix * cell_ps + c);
        lstm_elem(gi.x, gf.x, go.x, gc.x, di.x, df.x, dob.x, dcg.x, cpo.x, Dcp.x, cprev != nullptr, co.x, sum_m2, oh.x, oc.x, hn.x);
        lstm_elem(gi.y, gf.y, go.y, gc.y, di.y, df.y, dob.y, dcg.y, cpo.y, Dcp.y, cprev != nullptr, co.y, sum_m2, oh.y, oc.y, hn.y);
        lstm_elem(gi.z, gf.z, go.z, gc.z, di.z, df.z, dob.z, dcg.z, cpo.z, Dcp.z, cprev != nullptr, co.z, sum_m2, oh.z, oc.z, hn.z);
        lstm_elem(gi.w, gf.w, go.w, gc.w, di.w, df.w, dob.w, dcg.w, cpo.w, Dcp.w, cprev != nullptr, co.w, sum_m2, oh.w, oc.w, hn.w);
        st4(cell + pix * cell_ps + c, f4add(co, oc));
      }
      if (hsent) {
        float4 sent = make_float4(0.f, 0.f, 0.f, 0.f);
        bool over = false;
        if (on) {
          sent = ld4(hsent + pix * hs_ps + c);
          oh = make_float4(hn.x - sent.x, hn.y - sent.y, hn.z - sent.z, hn.w - sent.w);
          over = fabsf(oh.x) > thr || fabsf(oh.y) > thr || fabsf(oh.z) > thr || fabsf(oh.w) > thr;
        }
        unsigned bal = __ballot_sync(0xffffffffu, over);
        const bool send = (bal >> ((threadIdx.x & 31) & ~3)) & 0xFu;   // any of the four lanes of this pixel's group
        if (on) {
          if (send) { st4(hsent + pix * hs_ps + c, hn); or_word(s_w, p); }
          else oh = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      if (ok) {
        st4(dh + pix * dh_ps + c, oh);
        st4(dc + pix * dc_ps + c, oc);
      }
    }
    if (hsent) {
      __syncthreads();
      if (threadIdx.x == 0) {
        const unsigned long long mine = ((unsigned long long)s_w[1] << 32) | s_w[0];
        if (ncb == 1) {
          dh_bits[t] = mine;
          dc_bits[t] = win;
        } else {
          if (mine) atomicOr(&acc_words[t], mine);
          __threadfence();
          if (atomicAdd(&tickets[t], 1) == ncb - 1) {      // every other block of this tile has contributed
            dh_bits[t] = atomicExch(&acc_words[t], 0ull);
            dc_bits[t] = win;
            tickets[t] = 0;
          }
        }
      }
    } else if (cb == 0 && threadIdx.x == 0) {
      dh_bits[t] = win;
      dc_bits[t] = win;
    }
  }
  run_tail_job(tail);
}

// Incremental activation, float4 over channels, one block per tile (the output mask needs every channel of a pixel).
// All loads of a thread's elements are issued before the first dependent store, so that a thread has up to
// 2 x (2..3) 16-byte loads in flight instead of one scalar load at a time.
template <int OP>
__global__ void __launch_bounds__(256) act_incr_vec_kernel(
    const float *in, int64_t in_ps, const uint64_t *__restrict__ in_bits, float *__restrict__ res, int64_t res_ps,
    float *__restrict__ emitted, int64_t em_ps, float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H, int W,
    float thr, int accumulate) {
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ unsigned long long s_g[64];   // per pixel: which groups of 16 channels have a change above the threshold
  __shared__ unsigned s_w[2];
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int q4 = C >> 2, total = 64 * q4;
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t win = in_bits[t];
    const TileGeom g = tile_geom(t, H, W);
    if (win == 0ull) {
      if (out_bits[t] != 0ull) {  // uniform across the block
        __syncthreads();
        zero_tile4(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    if (threadIdx.x < 64) s_g[threadIdx.x] = 0ull;
    __syncthreads();
    for (int e0 = threadIdx.x; e0 < total; e0 += 2 * blockDim.x) {
      int p[2], c[2];
      bool ok[2], on[2];
      int64_t pix[2];
      float4 d[2], x[2], b[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int e = e0 + u * blockDim.x;
        p[u] = e / q4;
        c[u] = (e - p[u] * q4) * 4;
        ok[u] = e < total && pix_valid(g, p[u]);
        on[u] = ok[u] && ((win >> p[u]) & 1ull);
        pix[u] = ok[u] ? pix_index(g, p[u], H, W) : 0;
        if (on[u]) {
          d[u] = ld4(in + pix[u] * in_ps + c[u]);
          x[u] = ld4(res + pix[u] * res_ps + c[u]);
          if (emitted) b[u] = ld4(emitted + pix[u] * em_ps + c[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!ok[u]) continue;
        float4 dy = make_float4(0.f, 0.f, 0.f, 0.f);
        if (on[u]) {
          const float4 xn = f4add(x[u], d[u]);
          if (accumulate) st4(res + pix[u] * res_ps + c[u], xn);
          if (!emitted) b[u] = make_float4(act_t<OP>(x[u].x), act_t<OP>(x[u].y), act_t<OP>(x[u].z), act_t<OP>(x[u].w));
          dy = make_float4(act_t<OP>(xn.x) - b[u].x, act_t<OP>(xn.y) - b[u].y, act_t<OP>(xn.z) - b[u].z, act_t<OP>(xn.w) - b[u].w);
          if (fabsf(dy.x) > thr || fabsf(dy.y) > thr || fabsf(dy.z) > thr || fabsf(dy.w) > thr)
            atomicOr(&s_g[p[u]], 1ull << (c[u] >> 4));
        }
        st4(out + pix[u] * out_ps + c[u], dy);
      }
    }
    __syncthreads();
    if (threadIdx.x < 64) {   // the tile word: a pixel is active when one of its groups is sent
      const unsigned bal = __ballot_sync(0xffffffffu, s_g[threadIdx.x] != 0ull);
      if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = bal;
    }
    if (thr > 0.0f || emitted) {
      // second pass: withheld groups are written as zero; sent groups are added to the carry
      for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const int pp = e / q4, cc = (e - pp * q4) * 4;
        if (!pix_valid(g, pp) || !((win >> pp) & 1ull)) continue;
        const int64_t px = pix_index(g, pp, H, W);
        if ((s_g[pp] >> (cc >> 4)) & 1ull) {
          if (emitted) st4(emitted + px * em_ps + cc, f4add(ld4(emitted + px * em_ps + cc), ld4(out + px * out_ps + cc)));
        } else {
          st4(out + px * out_ps + cc, make_float4(0.f, 0.f, 0.f, 0.f));
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) out_bits[t] = ((uint64_t)s_w[1] << 32) | s_w[0];
    __syncthreads();
  }
}

// Incremental product, float4 over channels, one block per tile; the loads of two elements per thread are issued
// before the first dependent store (the scalar kernel above ran one 4-byte load chain at a time).
__global__ void __launch_bounds__(256) mul_incr_vec_kernel(
    const float *__restrict__ d1, int64_t d1_ps, const uint64_t *__restrict__ bits1, float *__restrict__ x1, int64_t x1_ps,
    const float *__restrict__ d2, int64_t d2_ps, const uint64_t *__restrict__ bits2, float *__restrict__ x2, int64_t x2_ps,
    float *__restrict__ out, int64_t out_ps, uint64_t *__restrict__ out_bits, int N, int C, int H, int W, float thr,
    int accumulate) {
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ unsigned s_w[2];
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int q4 = C >> 2, total = 64 * q4;
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t w1 = (d1 && bits1) ? bits1[t] : 0ull, w2 = (d2 && bits2) ? bits2[t] : 0ull;
    const uint64_t win = w1 | w2;
    const TileGeom g = tile_geom(t, H, W);
    if (win == 0ull) {
      if (out_bits[t] != 0ull) {
        __syncthreads();
        zero_tile4(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    if (threadIdx.x < 2) s_w[threadIdx.x] = 0u;
    __syncthreads();
    for (int e0 = threadIdx.x; e0 < total; e0 += 2 * blockDim.x) {
      int p[2], c[2];
      bool ok[2], on[2];
      int64_t pix[2];
      float4 a[2], b[2], v1[2], v2[2];
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int e = e0 + u * blockDim.x;
        p[u] = e / q4;
        c[u] = (e - p[u] * q4) * 4;
        ok[u] = e < total && pix_valid(g, p[u]);
        on[u] = ok[u] && ((win >> p[u]) & 1ull);
        pix[u] = ok[u] ? pix_index(g, p[u], H, W) : 0;
        a[u] = b[u] = zero;
        if (on[u]) {
          if ((w1 >> p[u]) & 1ull) a[u] = ld4(d1 + pix[u] * d1_ps + c[u]);
          if ((w2 >> p[u]) & 1ull) b[u] = ld4(d2 + pix[u] * d2_ps + c[u]);
          v1[u] = ld4(x1 + pix[u] * x1_ps + c[u]);
          v2[u] = ld4(x2 + pix[u] * x2_ps + c[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (!ok[u]) continue;
        float4 d = zero;
        if (on[u]) {
          d = make_float4((b[u].x + v2[u].x) * a[u].x + v1[u].x * b[u].x, (b[u].y + v2[u].y) * a[u].y + v1[u].y * b[u].y,
                          (b[u].z + v2[u].z) * a[u].z + v1[u].z * b[u].z, (b[u].w + v2[u].w) * a[u].w + v1[u].w * b[u].w);
          if (accumulate) {
            if (a[u].x != 0.0f || a[u].y != 0.0f || a[u].z != 0.0f || a[u].w != 0.0f) st4(x1 + pix[u] * x1_ps + c[u], f4add(v1[u], a[u]));
            if (b[u].x != 0.0f || b[u].y != 0.0f || b[u].z != 0.0f || b[u].w != 0.0f) st4(x2 + pix[u] * x2_ps + c[u], f4add(v2[u], b[u]));
          }
          if (fabsf(d.x) > thr || fabsf(d.y) > thr || fabsf(d.z) > thr || fabsf(d.w) > thr) or_word(s_w, p[u]);
        }
        st4(out + pix[u] * out_ps + c[u], d);
      }
    }
    __syncthreads();
    const uint64_t wout = ((uint64_t)s_w[1] << 32) | s_w[0];
    if (thr > 0.0f) {
      for (int e = threadIdx.x; e < total; e += blockDim.x) {
        const int pp = e / q4, cc = (e - pp * q4) * 4;
        if (pix_valid(g, pp) && ((win >> pp) & 1ull) && !((wout >> pp) & 1ull))
          st4(out + pix_index(g, pp, H, W) * out_ps + cc, make_float4(0.f, 0.f, 0.f, 0.f));
      }
    }
    if (threadIdx.x == 0) out_bits[t] = wout;
    __syncthreads();
  }
}

// Channel concatenation, float4 over channels: work item = (tile, block of 64 output channels).
__global__ void __launch_bounds__(PW_THREADS) cat2_vec_kernel(
    const float *__restrict__ a, int64_t a_ps, const uint64_t *__restrict__ a_bits, int ca, const float *__restrict__ b,
    int64_t b_ps, const uint64_t *__restrict__ b_bits, int cb, float *__restrict__ out, int64_t out_ps,
    uint64_t *out_bits, int N, int H, int W, const mie_tail_job tail) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int C = ca + cb;
  const int ncb = (C + 63) / 64;
  const int n_items = ntiles * ncb;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int t = item / ncb, blk = item - t * ncb;
    const uint64_t wa = a_bits[t], wb = b_bits[t], w = wa | wb;
    const TileGeom g = tile_geom(t, H, W);
    if (w == 0ull) {
      if (blk == 0 && out_bits[t] != 0ull) {   // only this block reads or writes the word
        __syncthreads();
        zero_tile4(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    const int c_lo = blk * 64, q4 = (min(C, c_lo + 64) - c_lo) >> 2;
#pragma unroll 4
    for (int e = threadIdx.x; e < 64 * q4; e += blockDim.x) {   // independent copies: four loads in flight per thread
      const int p = e / q4, c = c_lo + (e - p * q4) * 4;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < ca) { if ((wa >> p) & 1ull) v = ld4(a + pix * a_ps + c); }
      else { if ((wb >> p) & 1ull) v = ld4(b + pix * b_ps + (c - ca)); }
      st4(out + pix * out_ps + c, v);
    }
    if (blk == 0 && threadIdx.x == 0) out_bits[t] = w;
  }
  run_tail_job(tail);
}

__global__ void __launch_bounds__(PW_THREADS) upsample2x_vec_kernel(
    const float *__restrict__ a, int64_t a_ps, const uint64_t *__restrict__ a_bits, const float *__restrict__ b,
    int64_t b_ps, const uint64_t *__restrict__ b_bits, float *__restrict__ out, int64_t out_ps, uint64_t *out_bits, int N,
    int C, int H, int W, int mode, int scale) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int Ho = scale * H, Wo = scale * W;
  const float rs = 1.0f / (float)scale;
  const int THi = (H + 7) >> 3, TWi = (W + 7) >> 3;
  const int ntiles = N * ((Ho + 7) >> 3) * ((Wo + 7) >> 3);
  const int ncb = (C + CB - 1) / CB;
  const int n_items = ntiles * ncb;
  __shared__ unsigned s_w[2];
  __shared__ unsigned char s_fa[64], s_fb[64];
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int t = item / ncb, cb = item - t * ncb;
    const TileGeom g = tile_geom(t, Ho, Wo);
    __syncthreads();
    if (threadIdx.x < 64) {
      const int p = threadIdx.x;
      unsigned fa = 0, fb = 0;
      if (pix_valid(g, p)) {
        int y0, y1, x0, x1; float wy, wx;
        up_src(g.ty * 8 + (p >> 3), H, mode, scale, rs, y0, y1, wy);
        up_src(g.tx * 8 + (p & 7), W, mode, scale, rs, x0, x1, wx);
        fa = (bit_at(a_bits, g.n, y0, x0, THi, TWi) ? 1u : 0u) | (bit_at(a_bits, g.n, y0, x1, THi, TWi) ? 2u : 0u) |
             (bit_at(a_bits, g.n, y1, x0, THi, TWi) ? 4u : 0u) | (bit_at(a_bits, g.n, y1, x1, THi, TWi) ? 8u : 0u);
        if (b)
          fb = (bit_at(b_bits, g.n, y0, x0, THi, TWi) ? 1u : 0u) | (bit_at(b_bits, g.n, y0, x1, THi, TWi) ? 2u : 0u) |
               (bit_at(b_bits, g.n, y1, x0, THi, TWi) ? 4u : 0u) | (bit_at(b_bits, g.n, y1, x1, THi, TWi) ? 8u : 0u);
      }
      s_fa[p] = (unsigned char)fa;
      s_fb[p] = (unsigned char)fb;
      const unsigned bal = __ballot_sync(0xffffffffu, (fa | fb) != 0);
      if ((threadIdx.x & 31) == 0) s_w[threadIdx.x >> 5] = bal;
    }
    __syncthreads();
    const uint64_t wout = ((uint64_t)s_w[1] << 32) | s_w[0];
    if (wout == 0ull) {
      if (cb == 0 && out_bits[t] != 0ull) {
        if (C & 3) zero_tile(out, out_ps, C, g, Ho, Wo);
        else zero_tile4(out, out_ps, C, g, Ho, Wo);
        __syncthreads();
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    const int c_lo = cb * CB, q4 = (min(C, c_lo + CB) - c_lo) >> 2;
    for (int e = threadIdx.x; e < 64 * q4; e += blockDim.x) {
      const int p = e / q4, c = c_lo + (e - p * q4) * 4;
      if (!pix_valid(g, p)) continue;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      const unsigned fa = s_fa[p], fb = s_fb[p];
      if (fa | fb) {
        int y0, y1, x0, x1; float wy, wx;
        up_src(g.ty * 8 + (p >> 3), H, mode, scale, rs, y0, y1, wy);
        up_src(g.tx * 8 + (p & 7), W, mode, scale, rs, x0, x1, wx);
        const int64_t r0 = (int64_t)(g.n * H + y0) * W, r1 = (int64_t)(g.n * H + y1) * W;
        float4 v00 = v, v01 = v, v10 = v, v11 = v;
        if (fa & 1u) v00 = ld4(a + (r0 + x0) * a_ps + c);
        if (fa & 2u) v01 = ld4(a + (r0 + x1) * a_ps + c);
        if (fa & 4u) v10 = ld4(a + (r1 + x0) * a_ps + c);
        if (fa & 8u) v11 = ld4(a + (r1 + x1) * a_ps + c);
        if (fb & 1u) v00 = f4add(v00, ld4(b + (r0 + x0) * b_ps + c));
        if (fb & 2u) v01 = f4add(v01, ld4(b + (r0 + x1) * b_ps + c));
        if (fb & 4u) v10 = f4add(v10, ld4(b + (r1 + x0) * b_ps + c));
        if (fb & 8u) v11 = f4add(v11, ld4(b + (r1 + x1) * b_ps + c));
        if (mode == MIE_UP_NEAREST) {
          v = v00;
        } else {
          const float ax = 1.0f - wx, ay = 1.0f - wy;
          v.x = ay * (ax * v00.x + wx * v01.x) + wy * (ax * v10.x + wx * v11.x);
          v.y = ay * (ax * v00.y + wx * v01.y) + wy * (ax * v10.y + wx * v11.y);
          v.z = ay * (ax * v00.z + wx * v01.z) + wy * (ax * v10.z + wx * v11.z);
          v.w = ay * (ax * v00.w + wx * v01.w) + wy * (ax * v10.w + wx * v11.w);
        }
      }
      st4(out + pix_index(g, p, Ho, Wo) * out_ps + c, v);
    }
    // channel counts off 4 (2·C + 2 in the flow decoders): the last block takes the 1..3 remaining channels one by one
    const int ct = C & 3;
    if (ct && cb == ncb - 1) {
      const int c_tail = C - ct;
      for (int e = threadIdx.x; e < 64 * ct; e += blockDim.x) {
        const int p = e / ct, c = c_tail + (e - p * ct);
        if (!pix_valid(g, p)) continue;
        float v = 0.0f;
        const unsigned fa = s_fa[p], fb = s_fb[p];
        if (fa | fb) {
          int y0, y1, x0, x1; float wy, wx;
          up_src(g.ty * 8 + (p >> 3), H, mode, scale, rs, y0, y1, wy);
          up_src(g.tx * 8 + (p & 7), W, mode, scale, rs, x0, x1, wx);
          const int64_t r0 = (int64_t)(g.n * H + y0) * W, r1 = (int64_t)(g.n * H + y1) * W;
          float v00 = 0.f, v01 = 0.f, v10 = 0.f, v11 = 0.f;
          if (fa & 1u) v00 += a[(r0 + x0) * a_ps + c];
          if (fa & 2u) v01 += a[(r0 + x1) * a_ps + c];
          if (fa & 4u) v10 += a[(r1 + x0) * a_ps + c];
          if (fa & 8u) v11 += a[(r1 + x1) * a_ps + c];
          if (fb & 1u) v00 += b[(r0 + x0) * b_ps + c];
          if (fb & 2u) v01 += b[(r0 + x1) * b_ps + c];
          if (fb & 4u) v10 += b[(r1 + x0) * b_ps + c];
          if (fb & 8u) v11 += b[(r1 + x1) * b_ps + c];
          if (mode == MIE_UP_NEAREST) v = v00;
          else v = (1.0f - wy) * ((1.0f - wx) * v00 + wx * v01) + wy * ((1.0f - wx) * v10 + wx * v11);
        }
        out[pix_index(g, p, Ho, Wo) * out_ps + c] = v;
      }
    }
    if (cb == 0 && threadIdx.x == 0) out_bits[t] = wout;
  }
}

// x2 upsample of (a [+ b]), sources staged in shared memory.  Work item = (8x8 output tile, block of 32 channels).
// An output tile reads a 6x6 window of source pixels (rows 4*ty-1 .. 4*ty+4, clamped at the border).  The kernel above
// fetches the four sources of every output element separately and recomputes their addresses each time -- more than
// 400 instructions per 16-byte store, which made it instruction-bound at a quarter of the memory bandwidth.  Here the
// window is loaded once (36 address computations per item instead of 512, one round trip, inactive source pixels not
// loaded at all) and the 64 outputs are blended from shared memory.  Same interpolation arithmetic (up_src).
constexpr int UP_WIN = 6;

__global__ void __launch_bounds__(PW_THREADS, 8) upsample2x_tile_kernel(
    const float *__restrict__ a, int64_t a_ps, const uint64_t *__restrict__ a_bits, const float *__restrict__ b,
    int64_t b_ps, const uint64_t *__restrict__ b_bits, float *__restrict__ out, int64_t out_ps, uint64_t *out_bits, int N,
    int C, int H, int W, int mode, const mie_tail_job tail) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int Ho = 2 * H, Wo = 2 * W;
  const int THi = (H + 7) >> 3, TWi = (W + 7) >> 3;
  const int ntiles = N * ((Ho + 7) >> 3) * ((Wo + 7) >> 3);
  const int ncb = (C + CB - 1) / CB;
  const int n_items = ntiles * ncb;
  __shared__ float4 s_src[UP_WIN * UP_WIN][CB / 4];
  __shared__ unsigned s_on[4], s_out[2];   // s_on: window activity of a (words 0, 1) and of b (words 2, 3)
  const int tid = threadIdx.x;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int t = item / ncb, cb = item - t * ncb;
    const TileGeom g = tile_geom(t, Ho, Wo);
    const int r0 = 4 * g.ty - 1, c0 = 4 * g.tx - 1;
    __syncthreads();   // the previous item's reads of shared memory are done
    // which source pixels of the window are active (threads 0..35: warp 0 whole, first four lanes of warp 1)
    if (tid < 64) {
      bool on_a = false, on_b = false;
      if (tid < UP_WIN * UP_WIN) {
        const int sy = min(max(r0 + tid / UP_WIN, 0), H - 1), sx = min(max(c0 + tid % UP_WIN, 0), W - 1);
        on_a = bit_at(a_bits, g.n, sy, sx, THi, TWi);
        on_b = b && bit_at(b_bits, g.n, sy, sx, THi, TWi);
      }
      const unsigned bal_a = __ballot_sync(0xffffffffu, on_a), bal_b = __ballot_sync(0xffffffffu, on_b);
      if ((tid & 31) == 0) { s_on[tid >> 5] = bal_a; s_on[2 + (tid >> 5)] = bal_b; }
    }
    __syncthreads();
    const uint64_t mask_a = ((uint64_t)s_on[1] << 32) | s_on[0], mask_b = ((uint64_t)s_on[3] << 32) | s_on[2];
    const uint64_t on_mask = mask_a | mask_b;
    // output word: a pixel is active when one of its sources is
    if (tid < 64) {
      bool act = false;
      if (pix_valid(g, tid)) {
        int y0, y1, x0, x1; float wy, wx;
        up_src(g.ty * 8 + (tid >> 3), H, mode, 2, 0.5f, y0, y1, wy);
        up_src(g.tx * 8 + (tid & 7), W, mode, 2, 0.5f, x0, x1, wx);
        const uint64_t m = (1ull << ((y0 - r0) * UP_WIN + (x0 - c0))) | (1ull << ((y0 - r0) * UP_WIN + (x1 - c0))) |
                           (1ull << ((y1 - r0) * UP_WIN + (x0 - c0))) | (1ull << ((y1 - r0) * UP_WIN + (x1 - c0)));
        act = (on_mask & m) != 0ull;
      }
      const unsigned bal = __ballot_sync(0xffffffffu, act);
      if ((tid & 31) == 0) s_out[tid >> 5] = bal;
    }
    __syncthreads();
    const uint64_t wout = ((uint64_t)s_out[1] << 32) | s_out[0];
    if (wout == 0ull) {
      if (cb == 0 && out_bits[t] != 0ull) {      // only this block reads or writes the word
        zero_tile4(out, out_ps, C, g, Ho, Wo);
        __syncthreads();
        if (tid == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    const int c_lo = cb * CB, q4 = (min(C, c_lo + CB) - c_lo) >> 2;
    if (q4 == CB / 4) {
      // ---- whole 32-channel blocks: every index is a shift or a per-thread constant.  (The general loops below spend
      // more than 200 instructions per 16-byte store on divisions, up_src and 64-bit pixel indices, and the kernel was
      // bound by instruction issue at a third of the memory bandwidth.)
      const int q = tid & 7;
#pragma unroll
      for (int it = 0; it < 3; ++it) {
        const int sp = (tid >> 3) + 16 * it;
        if (sp < UP_WIN * UP_WIN) {
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if ((on_mask >> sp) & 1ull) {
            const int sy = min(max(r0 + sp / UP_WIN, 0), H - 1), sx = min(max(c0 + sp % UP_WIN, 0), W - 1);
            const int64_t pix = (int64_t)(g.n * H + sy) * W + sx;
            if ((mask_a >> sp) & 1ull) v = ld4(a + pix * a_ps + c_lo + q * 4);
            if ((mask_b >> sp) & 1ull) v = f4add(v, ld4(b + pix * b_ps + c_lo + q * 4));
          }
          s_src[sp][q] = v;
        }
      }
      __syncthreads();
      // Output pixel (row pr, column pc) of the tile.  Window entries are loaded from clamped coordinates, so a clamped
      // neighbour is a duplicate of the pixel itself: the even output coordinate 2i always blends window entries
      // (i', i'+1) with weight 0.75 on the second (0 at the field's first row / column, where up_src gives both sources
      // as pixel 0), the odd one (i'+1, i'+2) with weight 0.25 -- up_src's sources and weights without its branches.
      const int pc = (tid >> 3) & 7, prb = tid >> 6;
      const int ox = g.tx * 8 + pc;
      const bool nearest = mode == MIE_UP_NEAREST;
      const int kx = nearest ? (pc >> 1) + 1 : (pc >> 1) + (pc & 1);
      const float wx = (pc & 1) ? 0.25f : (ox == 0 ? 0.0f : 0.75f), ax = 1.0f - wx;
      if (ox < Wo) {
        float *op = out + ((int64_t)(g.n * Ho + g.ty * 8 + prb) * Wo + ox) * out_ps + c_lo + q * 4;
        const int64_t row_step = 2 * (int64_t)Wo * out_ps;
#pragma unroll
        for (int it = 0; it < 4; ++it, op += row_step) {
          const int pr = prb + 2 * it, oy = g.ty * 8 + pr;
          if (oy >= Ho) break;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if ((wout >> (pr * 8 + pc)) & 1ull) {
            if (nearest) {
              v = s_src[((pr >> 1) + 1) * UP_WIN + kx][q];
            } else {
              const int ky = (pr >> 1) + (pr & 1);
              const float wy = (pr & 1) ? 0.25f : (oy == 0 ? 0.0f : 0.75f), ay = 1.0f - wy;
              const float4 v00 = s_src[ky * UP_WIN + kx][q], v01 = s_src[ky * UP_WIN + kx + 1][q];
              const float4 v10 = s_src[(ky + 1) * UP_WIN + kx][q], v11 = s_src[(ky + 1) * UP_WIN + kx + 1][q];
              v.x = ay * (ax * v00.x + wx * v01.x) + wy * (ax * v10.x + wx * v11.x);
              v.y = ay * (ax * v00.y + wx * v01.y) + wy * (ax * v10.y + wx * v11.y);
              v.z = ay * (ax * v00.z + wx * v01.z) + wy * (ax * v10.z + wx * v11.z);
              v.w = ay * (ax * v00.w + wx * v01.w) + wy * (ax * v10.w + wx * v11.w);
            }
          }
          st4(op, v);
        }
      }
      if (cb == 0 && tid == 0) out_bits[t] = wout;
      continue;
    }
    // stage the window: one 16-byte load per (source pixel, channel quad), all independent
    for (int i = tid; i < UP_WIN * UP_WIN * q4; i += blockDim.x) {
      const int sp = i / q4, q = i - sp * q4;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((on_mask >> sp) & 1ull) {
        const int sy = min(max(r0 + sp / UP_WIN, 0), H - 1), sx = min(max(c0 + sp % UP_WIN, 0), W - 1);
        const int64_t pix = (int64_t)(g.n * H + sy) * W + sx;
        if ((mask_a >> sp) & 1ull) v = ld4(a + pix * a_ps + c_lo + q * 4);
        if ((mask_b >> sp) & 1ull) v = f4add(v, ld4(b + pix * b_ps + c_lo + q * 4));
      }
      s_src[sp][q] = v;
    }
    __syncthreads();
    for (int e = tid; e < 64 * q4; e += blockDim.x) {
      const int p = (q4 == 8) ? (e >> 3) : e / q4, q = e - p * q4;   // full 32-channel blocks: no division
      if (!pix_valid(g, p)) continue;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((wout >> p) & 1ull) {
        int y0, y1, x0, x1; float wy, wx;
        up_src(g.ty * 8 + (p >> 3), H, mode, 2, 0.5f, y0, y1, wy);
        up_src(g.tx * 8 + (p & 7), W, mode, 2, 0.5f, x0, x1, wx);
        const float4 v00 = s_src[(y0 - r0) * UP_WIN + (x0 - c0)][q];
        if (mode == MIE_UP_NEAREST) {
          v = v00;
        } else {
          const float4 v01 = s_src[(y0 - r0) * UP_WIN + (x1 - c0)][q];
          const float4 v10 = s_src[(y1 - r0) * UP_WIN + (x0 - c0)][q];
          const float4 v11 = s_src[(y1 - r0) * UP_WIN + (x1 - c0)][q];
          const float ax = 1.0f - wx, ay = 1.0f - wy;
          v.x = ay * (ax * v00.x + wx * v01.x) + wy * (ax * v10.x + wx * v11.x);
          v.y = ay * (ax * v00.y + wx * v01.y) + wy * (ax * v10.y + wx * v11.y);
          v.z = ay * (ax * v00.z + wx * v01.z) + wy * (ax * v10.z + wx * v11.z);
          v.w = ay * (ax * v00.w + wx * v01.w) + wy * (ax * v10.w + wx * v11.w);
        }
      }
      st4(out + pix_index(g, p, Ho, Wo) * out_ps + c_lo + q * 4, v);
    }
    if (cb == 0 && tid == 0) out_bits[t] = wout;
  }
  run_tail_job(tail);
}

__global__ void __launch_bounds__(PW_THREADS) add_vec_kernel(
    const float *__restrict__ a, int64_t a_ps, const uint64_t *__restrict__ a_bits, const float *__restrict__ b,
    int64_t b_ps, const uint64_t *__restrict__ b_bits, float *__restrict__ out, int64_t out_ps, uint64_t *out_bits, int N,
    int C, int H, int W, const mie_tail_job tail) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int ncb = (C + CB - 1) / CB;
  const int n_items = ntiles * ncb;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int t = item / ncb, cb = item - t * ncb;
    const uint64_t wa = a_bits[t], wb = b_bits[t], w = wa | wb;
    const TileGeom g = tile_geom(t, H, W);
    if (w == 0ull) {
      if (cb == 0 && out_bits[t] != 0ull) {
        __syncthreads();
        zero_tile4(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    const int c_lo = cb * CB, q4 = (min(C, c_lo + CB) - c_lo) >> 2;
    for (int e = threadIdx.x; e < 64 * q4; e += blockDim.x) {
      const int p = e / q4, c = c_lo + (e - p * q4) * 4;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((wa >> p) & 1ull) v = ld4(a + pix * a_ps + c);
      if ((wb >> p) & 1ull) v = f4add(v, ld4(b + pix * b_ps + c));
      st4(out + pix * out_ps + c, v);
    }
    if (cb == 0 && threadIdx.x == 0) out_bits[t] = w;
  }
  run_tail_job(tail);
}

// Block size of the kernels that keep one block per tile (their output mask needs every channel of a pixel):
// few tiles with many channels get wide blocks, so that a deep UNet level does not run on six small blocks.
static int wide_threads(int ntiles, int C) {
  int th = PW_THREADS;
  while (th < 1024 && (int64_t)ntiles * th < (int64_t)MIE_SM_COUNT * 1024 && th * 8 <= 64 * C) th <<= 1;
  return th;
}

static int item_grid(int64_t items) {
  const int64_t cap = (int64_t)MIE_SM_COUNT * 16;
  return (int)(items < cap ? (items > 0 ? items : 1) : cap);
}

// ---------------------------------------------------------------------------------------------
// add, concatenate, accumulate
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(PW_THREADS) add_kernel(
    const float *__restrict__ a, int64_t a_ps, const uint64_t *__restrict__ a_bits, const float *__restrict__ b,
    int64_t b_ps, const uint64_t *__restrict__ b_bits, float *__restrict__ out, int64_t out_ps,
    uint64_t *__restrict__ out_bits, int N, int C, int H, int W) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t wa = a_bits[t], wb = b_bits[t], w = wa | wb;
    const TileGeom g = tile_geom(t, H, W);
    if (w == 0ull) {
      if (out_bits[t] != 0ull) {
        __syncthreads();
        zero_tile(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
      const int p = e / C, c = e - p * C;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float v = 0.0f;
      if ((wa >> p) & 1ull) v += a[pix * a_ps + c];
      if ((wb >> p) & 1ull) v += b[pix * b_ps + c];
      out[pix * out_ps + c] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) out_bits[t] = w;
  }
}

constexpr int CBS = 64;  // channels per work item of the scalar channel-split kernels

// work item = (tile, block of CBS channels): the deep levels of a UNet have a handful of tiles but a thousand channels
__global__ void __launch_bounds__(PW_THREADS) cat2_kernel(
    const float *__restrict__ a, int64_t a_ps, const uint64_t *__restrict__ a_bits, int ca, const float *__restrict__ b,
    int64_t b_ps, const uint64_t *__restrict__ b_bits, int cb, float *__restrict__ out, int64_t out_ps,
    uint64_t *__restrict__ out_bits, int N, int H, int W) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int C = ca + cb;
  const int ncb = (C + CBS - 1) / CBS;
  const int n_items = ntiles * ncb;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int t = item / ncb, blk = item - t * ncb;
    const uint64_t wa = a_bits[t], wb = b_bits[t], w = wa | wb;
    const TileGeom g = tile_geom(t, H, W);
    if (w == 0ull) {
      if (blk == 0 && out_bits[t] != 0ull) {   // only this block reads or writes the word
        __syncthreads();
        zero_tile(out, out_ps, C, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    const int c_lo = blk * CBS, cw = min(C, c_lo + CBS) - c_lo;
    for (int e = threadIdx.x; e < 64 * cw; e += blockDim.x) {
      const int p = e / cw, c = c_lo + (e - p * cw);
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float v = 0.0f;
      if (c < ca) { if ((wa >> p) & 1ull) v = a[pix * a_ps + c]; }
      else { if ((wb >> p) & 1ull) v = b[pix * b_ps + (c - ca)]; }
      out[pix * out_ps + c] = v;
    }
    if (blk == 0 && threadIdx.x == 0) out_bits[t] = w;
  }
}

__global__ void __launch_bounds__(PW_THREADS) accumulate_kernel(float *__restrict__ y, int64_t y_ps,
                                                                const float *__restrict__ d, int64_t d_ps,
                                                                const uint64_t *__restrict__ d_bits, int N, int C, int H,
                                                                int W) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t w = d_bits[t];
    if (w == 0ull) continue;
    const TileGeom g = tile_geom(t, H, W);
    for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
      const int p = e / C, c = e - p * C;
      if (!pix_valid(g, p) || !((w >> p) & 1ull)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      y[pix * y_ps + c] += d[pix * d_ps + c];
    }
  }
}

// ---------------------------------------------------------------------------------------------
// dense activation increment over n contiguous floats (the reference's native entry point)
// ---------------------------------------------------------------------------------------------
template <int OP, bool VEC>
__global__ void __launch_bounds__(256) activation_increment_kernel(float *__restrict__ X, const float *__restrict__ in,
                                                                   float *__restrict__ out, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    const int64_t n4 = n >> 2;
    float4 *X4 = reinterpret_cast<float4 *>(X);
    const float4 *I4 = reinterpret_cast<const float4 *>(in);
    float4 *O4 = reinterpret_cast<float4 *>(out);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
      const float4 x = X4[i], d = __ldcs(I4 + i);
      const float4 xn = make_float4(x.x + d.x, x.y + d.y, x.z + d.z, x.w + d.w);
      const float4 o = make_float4(act_t<OP>(xn.x) - act_t<OP>(x.x), act_t<OP>(xn.y) - act_t<OP>(x.y),
                                   act_t<OP>(xn.z) - act_t<OP>(x.z), act_t<OP>(xn.w) - act_t<OP>(x.w));
      X4[i] = xn;
      __stcs(O4 + i, o);
    }
    for (int64_t i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const float x = X[i], xn = x + in[i];
      out[i] = act_t<OP>(xn) - act_t<OP>(x);
      X[i] = xn;
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const float x = X[i], xn = x + in[i];
      out[i] = act_t<OP>(xn) - act_t<OP>(x);
      X[i] = xn;
    }
  }
}

template <int OP>
int launch_act_dense(float *X, const float *in, float *out, int64_t n, cudaStream_t st) {
  const bool vec = aligned16(X) && aligned16(in) && aligned16(out);
  const int64_t work = vec ? (n >> 2) : n;
  int64_t blocks = divup64(work > 0 ? work : 1, 256);
  const int64_t cap = (int64_t)MIE_SM_COUNT * 8;  // 8 resident blocks of 256 threads per SM
  if (blocks > cap) blocks = cap;
  if (vec) activation_increment_kernel<OP, true><<<(int)blocks, 256, 0, st>>>(X, in, out, n);
  else activation_increment_kernel<OP, false><<<(int)blocks, 256, 0, st>>>(X, in, out, n);
  return check_launch();
}


// ---------------------------------------------------------------------------------------------
// input side: delta against the previous frame + mask, event binning, quantiser
// ---------------------------------------------------------------------------------------------
// one thread per pixel, 64 threads per tile, 4 tiles per block; the ballot of a warp is half a tile word
__global__ void __launch_bounds__(256) delta_mask_kernel(const float *__restrict__ x, int64_t x_ps, float *__restrict__ xp,
                                                         int64_t xp_ps, float *__restrict__ dx, int64_t dx_ps,
                                                         unsigned *__restrict__ bits32, int N, int C, int H, int W, float thr,
                                                         float *__restrict__ split, int64_t split_ps, int shalf,
                                                         unsigned *__restrict__ split_bits32, const mie_tail_job tail) {
  // `split` (optional): the split-precision copy [d, d - tf32(d), d] of the delta (what mie_split_tf32 would make of it),
  // written in the same pass; a half tile (32 pixels = one warp) that is inactive now and was inactive in the copy's
  // last state is skipped, so the copy keeps the zero invariant at the cost of the active half tiles only.
  grid_dependency_wait();
  grid_dependency_trigger();
  const int TH = (H + 7) >> 3, TW = (W + 7) >> 3;
  const int ntiles = N * TH * TW;
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * 4 + (threadIdx.x >> 6); t < ntiles; t += gridDim.x * 4) {
    const int p = threadIdx.x & 63;
    const int tx = t % TW, ty = (t / TW) % TH, n = t / (TW * TH);
    const int y = ty * 8 + (p >> 3), xx = tx * 8 + (p & 7);
    const bool inside = y < H && xx < W;
    const int64_t pix = inside ? (int64_t)(n * H + y) * W + xx : 0;
    bool a = false;
    if (inside)
      for (int c = 0; c < C; ++c) a |= fabsf(x[pix * x_ps + c] - xp[pix * xp_ps + c]) > thr;
    const unsigned half = __ballot_sync(0xffffffffu, a);
    const size_t wi = 2 * (size_t)t + ((p >> 5) & 1);
    const bool copy = split && (half | split_bits32[wi]) != 0u;
    if (inside) {
      for (int c = 0; c < C; ++c) {
        const float v = x[pix * x_ps + c];
        const float d = a ? v - xp[pix * xp_ps + c] : 0.0f;
        dx[pix * dx_ps + c] = d;
        if (a) xp[pix * xp_ps + c] = v;
        if (copy) {
          float *o = split + pix * split_ps + c;
          o[0] = d;
          o[shalf] = d - __uint_as_float(__float_as_uint(d) & 0xFFFFE000u);
          o[2 * shalf] = d;
        }
      }
    }
    __syncwarp();      // every lane has read the copy's old word before lane 0 replaces it
    if (lane == 0) {
      bits32[wi] = half;
      if (split) split_bits32[wi] = half;
    }
  }
  run_tail_job(tail);
}

__global__ void __launch_bounds__(256) events_to_voxel_kernel(const float *__restrict__ ev, int n_events, int bins, int sh,
                                                              int sw, float *__restrict__ vox, int64_t ps, int H, int W,
                                                              int pl, int pt) {
  grid_dependency_wait();
  grid_dependency_trigger();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_events; i += gridDim.x * blockDim.x) {
    const float4 e = *reinterpret_cast<const float4 *>(ev + 4 * (size_t)i);
    const float ts = (float)(bins - 1) * e.x;
    const int xi = (int)e.y, yi = (int)e.z;
    if (xi < 0 || xi >= sw || yi < 0 || yi >= sh) continue;
    const float pol = (e.w == 0.0f) ? -1.0f : e.w;
    const int ti = (int)ts;
    const float dt = ts - (float)ti;
    const int64_t pix = (int64_t)(yi + pt) * W + (xi + pl);
    if (ti >= 0 && ti < bins) atomicAdd(vox + pix * ps + ti, pol * (1.0f - dt));
    if (ti + 1 >= 0 && ti + 1 < bins) atomicAdd(vox + pix * ps + ti + 1, pol * dt);
  }
}

// Signed event counts: channel 0 counts the events of polarity -1, channel 1 those of polarity +1 (any other
// polarity value is dropped, as the reference's two boolean selections do).  Counts are small integers, exact in
// fp32, so the atomic summation order does not show.
__global__ void __launch_bounds__(256) events_to_counts_kernel(const float *__restrict__ ev, int n_events, int sh, int sw,
                                                               float *__restrict__ img, int64_t ps, int W, int pl, int pt) {
  grid_dependency_wait();
  grid_dependency_trigger();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_events; i += gridDim.x * blockDim.x) {
    const float4 e = *reinterpret_cast<const float4 *>(ev + 4 * (size_t)i);
    const int xi = (int)e.y, yi = (int)e.z;
    if (xi < 0 || xi >= sw || yi < 0 || yi >= sh) continue;
    const int ch = (e.w == 1.0f) ? 1 : ((e.w == -1.0f) ? 0 : -1);
    if (ch < 0) continue;
    atomicAdd(img + ((int64_t)(yi + pt) * W + (xi + pl)) * ps + ch, 1.0f);
  }
}

__global__ void __launch_bounds__(256) kfenced_kernel(const float *__restrict__ dx, int64_t dx_ps, float *__restrict__ carry,
                                                      int64_t c_ps, float k, float *__restrict__ q, int64_t q_ps,
                                                      unsigned *__restrict__ bits32, int N, int C, int H, int W) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int TH = (H + 7) >> 3, TW = (W + 7) >> 3;
  const int ntiles = N * TH * TW;
  const int lane = threadIdx.x & 31;
  for (int t = blockIdx.x * 4 + (threadIdx.x >> 6); t < ntiles; t += gridDim.x * 4) {
    const int p = threadIdx.x & 63;
    const int tx = t % TW, ty = (t / TW) % TH, n = t / (TW * TH);
    const int y = ty * 8 + (p >> 3), xx = tx * 8 + (p & 7);
    bool a = false;
    if (y < H && xx < W) {
      const int64_t pix = (int64_t)(n * H + y) * W + xx;
      for (int c = 0; c < C; ++c) {
        const float T = carry[pix * c_ps + c] + dx[pix * dx_ps + c];
        const float f = k * floorf(0.5f + T / k);
        carry[pix * c_ps + c] = T - f;
        q[pix * q_ps + c] = f;
        a |= (f != 0.0f);
      }
    }
    const unsigned half = __ballot_sync(0xffffffffu, a);
    if (lane == 0) bits32[2 * (size_t)t + ((p >> 5) & 1)] = half;
  }
}

// The quantiser with float4 over channels, one block per tile: a thread-per-pixel loop over several hundred channels
// (the deep layers of a UNet) runs at a few per cent of the memory bandwidth.
__global__ void __launch_bounds__(256) kfenced_vec_kernel(const float *__restrict__ dx, int64_t dx_ps, float *__restrict__ carry,
                                                          int64_t c_ps, float k, float *__restrict__ q, int64_t q_ps,
                                                          uint64_t *__restrict__ bits, int N, int C, int H, int W) {
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ unsigned s_w[2];
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int q4 = C >> 2, total = 64 * q4;
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const TileGeom g = tile_geom(t, H, W);
    __syncthreads();
    if (threadIdx.x < 2) s_w[threadIdx.x] = 0u;
    __syncthreads();
    for (int e = threadIdx.x; e < total; e += blockDim.x) {
      const int p = e / q4, c = (e - p * q4) * 4;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      const float4 T = f4add(ld4(carry + pix * c_ps + c), ld4(dx + pix * dx_ps + c));
      const float4 f = make_float4(k * floorf(0.5f + T.x / k), k * floorf(0.5f + T.y / k), k * floorf(0.5f + T.z / k),
                                   k * floorf(0.5f + T.w / k));
      st4(carry + pix * c_ps + c, make_float4(T.x - f.x, T.y - f.y, T.z - f.z, T.w - f.w));
      st4(q + pix * q_ps + c, f);
      if (f.x != 0.0f || f.y != 0.0f || f.z != 0.0f || f.w != 0.0f) or_word(s_w, p);
    }
    __syncthreads();
    if (threadIdx.x == 0) bits[t] = ((uint64_t)s_w[1] << 32) | s_w[0];
  }
}

}  // namespace

extern "C" int mie_activation_increment(float *X, const float *in_incr, float *out_incr, int64_t n, int op, void *stream) {
  if (!X || !in_incr || !out_incr || n < 0) return MIE_EINVAL;
  if (n == 0) return MIE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  switch (op) {
    case MIE_ACT_RELU: return launch_act_dense<MIE_ACT_RELU>(X, in_incr, out_incr, n, st);
    case MIE_ACT_SIGMOID: return launch_act_dense<MIE_ACT_SIGMOID>(X, in_incr, out_incr, n, st);
    case MIE_ACT_TANH: return launch_act_dense<MIE_ACT_TANH>(X, in_incr, out_incr, n, st);
    case MIE_ACT_NONE: return launch_act_dense<MIE_ACT_NONE>(X, in_incr, out_incr, n, st);
    default: return MIE_EINVAL;
  }
}

// Split-precision copy of a narrow delta field for the tensor cores:
//   out[c] = d, out[half + c] = d - tf32_trunc(d), out[2*half + c] = d.
// The MMA truncates all three to TF32.  Against the filter blocks [W_hi, W_hi, W_lo] (W_hi = tf32(W), W_lo =
// tf32(W - W_hi)) the convolution over the 3*half channels is d_hi*W_hi + d_lo*W_hi + d_hi*W_lo: the fp32
// convolution of d with W up to the dropped d_lo*W_lo term (~2^-21 relative).
__global__ void __launch_bounds__(256) split_tf32_kernel(const float *__restrict__ in, int64_t in_ps,
                                                         const uint64_t *__restrict__ in_bits, int C, int half,
                                                         float *__restrict__ out, int64_t out_ps,
                                                         uint64_t *__restrict__ out_bits, int N, int H, int W,
                                                         const mie_tail_job tail) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t w = in_bits[t];
    const TileGeom g = tile_geom(t, H, W);
    if (w == 0ull) {
      if (out_bits[t] != 0ull) {   // held data last step: back to zero
        __syncthreads();
        zero_tile(out, out_ps, 3 * half, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
      const int p = e / C, c = e - p * C;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      const float v = ((w >> p) & 1ull) ? in[pix * in_ps + c] : 0.0f;
      const float hi = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
      out[pix * out_ps + c] = v;
      out[pix * out_ps + half + c] = v - hi;
      out[pix * out_ps + 2 * half + c] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) out_bits[t] = w;
  }
  run_tail_job(tail);
}

// The same with float4 over channels (C and half multiples of 4): four independent 16-byte loads in flight per thread.
__global__ void __launch_bounds__(256) split_tf32_vec_kernel(const float *__restrict__ in, int64_t in_ps,
                                                             const uint64_t *__restrict__ in_bits, int C, int half,
                                                             float *__restrict__ out, int64_t out_ps,
                                                             uint64_t *__restrict__ out_bits, int N, int H, int W,
                                                             const mie_tail_job tail) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int ntiles = N * ((H + 7) >> 3) * ((W + 7) >> 3);
  const int q4 = C >> 2;
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const uint64_t w = in_bits[t];
    const TileGeom g = tile_geom(t, H, W);
    if (w == 0ull) {
      if (out_bits[t] != 0ull) {   // held data last step: back to zero
        __syncthreads();
        zero_tile4(out, out_ps, 3 * half, g, H, W);
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
#pragma unroll 4
    for (int e = threadIdx.x; e < 64 * q4; e += blockDim.x) {
      const int p = e / q4, c = (e - p * q4) * 4;
      if (!pix_valid(g, p)) continue;
      const int64_t pix = pix_index(g, p, H, W);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if ((w >> p) & 1ull) v = ld4(in + pix * in_ps + c);
      const float4 lo = make_float4(v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u),
                                    v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u),
                                    v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u),
                                    v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u));
      float *o = out + pix * out_ps + c;
      st4(o, v);
      st4(o + half, lo);
      st4(o + 2 * half, v);
    }
    __syncthreads();
    if (threadIdx.x == 0) out_bits[t] = w;
  }
  run_tail_job(tail);
}

#define MIE_CHECK_FIELD(ptr, ps, C) if (!(ptr) || (ps) < (C)) return MIE_EINVAL

extern "C" int mie_act_incr(const float *in, int64_t in_ps, const uint64_t *in_bits, float *res, int64_t res_ps,
                            float *emitted, int64_t emitted_ps, float *out, int64_t out_ps, uint64_t *out_bits, int N,
                            int C, int H, int W, int op, float thr, int accumulate, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !in_bits || !out_bits || !(thr >= 0.0f)) return MIE_EINVAL;
  if (!accumulate && emitted) return MIE_EINVAL;   // a carry without an advancing reservoir would send the same change again
  if (C > 1024) return MIE_ETOOBIG;                // 64 channel groups per pixel in the kernels' flag words
  if (op < MIE_ACT_NONE || op > MIE_ACT_TANH) return MIE_EINVAL;
  MIE_CHECK_FIELD(in, in_ps, C); MIE_CHECK_FIELD(res, res_ps, C); MIE_CHECK_FIELD(out, out_ps, C);
  if (emitted && emitted_ps < C) return MIE_EINVAL;
  if (in == out && in_ps != out_ps) return MIE_EINVAL;
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  const bool vec = C % 4 == 0 && in_ps % 4 == 0 && res_ps % 4 == 0 && out_ps % 4 == 0 && aligned16(in) && aligned16(res) &&
                   aligned16(out) && (!emitted || (emitted_ps % 4 == 0 && aligned16(emitted)));
  if (vec) {
    const dim3 grid(tile_grid(ntiles)), block(256);
    cudaStream_t st = (cudaStream_t)stream;
#define MIE_ACT_VEC(OP) launch_chained(act_incr_vec_kernel<OP>, grid, block, 0, st, in, in_ps, in_bits, res, res_ps, emitted, \
                                       emitted_ps, out, out_ps, out_bits, N, C, H, W, thr, accumulate ? 1 : 0)
    switch (op) {
      case MIE_ACT_RELU: MIE_ACT_VEC(MIE_ACT_RELU); break;
      case MIE_ACT_SIGMOID: MIE_ACT_VEC(MIE_ACT_SIGMOID); break;
      case MIE_ACT_TANH: MIE_ACT_VEC(MIE_ACT_TANH); break;
      default: MIE_ACT_VEC(MIE_ACT_NONE); break;
    }
#undef MIE_ACT_VEC
    return check_launch();
  }
  launch_chained(act_incr_kernel, dim3(tile_grid(ntiles)), dim3(wide_threads(ntiles, C)), 0, (cudaStream_t)stream, 
      in, in_ps, in_bits, res, res_ps, emitted, emitted_ps, out, out_ps, out_bits, N, C, H, W, op, thr, accumulate ? 1 : 0);
  return check_launch();
}

extern "C" int mie_mul_incr(const float *d1, int64_t d1_ps, const uint64_t *bits1, float *x1, int64_t x1_ps,
                            const float *d2, int64_t d2_ps, const uint64_t *bits2, float *x2, int64_t x2_ps, float *out,
                            int64_t out_ps, uint64_t *out_bits, int N, int C, int H, int W, float thr, int accumulate,
                            void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !out_bits || !(thr >= 0.0f)) return MIE_EINVAL;
  MIE_CHECK_FIELD(x1, x1_ps, C); MIE_CHECK_FIELD(x2, x2_ps, C); MIE_CHECK_FIELD(out, out_ps, C);
  if (d1 && (!bits1 || d1_ps < C)) return MIE_EINVAL;
  if (d2 && (!bits2 || d2_ps < C)) return MIE_EINVAL;
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  if (C % 4 == 0 && x1_ps % 4 == 0 && x2_ps % 4 == 0 && out_ps % 4 == 0 && aligned16(x1) && aligned16(x2) && aligned16(out) &&
      (!d1 || (d1_ps % 4 == 0 && aligned16(d1))) && (!d2 || (d2_ps % 4 == 0 && aligned16(d2)))) {
    launch_chained(mul_incr_vec_kernel, dim3(tile_grid(ntiles)), dim3(256), 0, (cudaStream_t)stream,
        d1, d1_ps, bits1, x1, x1_ps, d2, d2_ps, bits2, x2, x2_ps, out, out_ps, out_bits, N, C, H, W, thr, accumulate ? 1 : 0);
    return check_launch();
  }
  launch_chained(mul_incr_kernel, dim3(tile_grid(ntiles)), dim3(wide_threads(ntiles, C)), 0, (cudaStream_t)stream, 
      d1, d1_ps, bits1, x1, x1_ps, d2, d2_ps, bits2, x2, x2_ps, out, out_ps, out_bits, N, C, H, W, thr, accumulate ? 1 : 0);
  return check_launch();
}

extern "C" int mie_convlstm_point(const float *dg, int64_t dg_ps, const uint64_t *dg_bits, float *g, int64_t g_ps,
                                  const float *dc_prev, int64_t dcp_ps, const uint64_t *dcp_bits, float *cprev,
                                  int64_t cprev_ps, float *cell, int64_t cell_ps, float *dh, int64_t dh_ps,
                                  uint64_t *dh_bits, float *dc, int64_t dc_ps, uint64_t *dc_bits, int N, int C, int H,
                                  int W, int sum_m2, float thr, float *h_sent, int64_t hs_ps, void *thr_scratch,
                                  const mie_tail_job *tail, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !dg_bits || !dh_bits || !dc_bits || !(thr >= 0.0f)) return MIE_EINVAL;
  if (tail_check(tail, dh_bits) != MIE_OK) return MIE_EINVAL;
  if (h_sent && (hs_ps < C || !thr_scratch)) return MIE_EINVAL;
  if (thr_scratch && (reinterpret_cast<uintptr_t>(thr_scratch) & 7)) return MIE_EALIGN;
  if (thr > 0.0f && !h_sent) return MIE_EINVAL;     // withholding without a record of what was sent would lose it
  MIE_CHECK_FIELD(dg, dg_ps, 4 * C); MIE_CHECK_FIELD(g, g_ps, 4 * C); MIE_CHECK_FIELD(cell, cell_ps, C);
  MIE_CHECK_FIELD(dh, dh_ps, C); MIE_CHECK_FIELD(dc, dc_ps, C);
  if (dc_prev && (!dcp_bits || dcp_ps < C || !cprev)) return MIE_EINVAL;
  if (cprev && cprev_ps < C) return MIE_EINVAL;
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  const bool vec = C % 4 == 0 && dg_ps % 4 == 0 && g_ps % 4 == 0 && cell_ps % 4 == 0 && dh_ps % 4 == 0 &&
                   dc_ps % 4 == 0 && aligned16(dg) && aligned16(g) && aligned16(cell) && aligned16(dh) && aligned16(dc) &&
                   (!dc_prev || (dcp_ps % 4 == 0 && aligned16(dc_prev))) && (!cprev || (cprev_ps % 4 == 0 && aligned16(cprev)));
  if (h_sent && !(vec && C % 16 == 0 && hs_ps % 4 == 0 && aligned16(h_sent))) return MIE_EUNSUPPORTED;
  if (vec) {
    // each element costs ~11 vector loads and 10 transcendentals: on the small fields of a UNet's deep levels a
    // block of 64 px x 32 ch leaves most SMs with one block of four sequential rounds; narrower items fix that.
    int cbw = CB;
    while (cbw > 8 && (int64_t)ntiles * divup(C, cbw) < (int64_t)MIE_SM_COUNT * 8) cbw >>= 1;
    if (h_sent && cbw < 16) cbw = 16;     // a work item holds whole 16-channel groups
    unsigned long long *acc_words = static_cast<unsigned long long *>(thr_scratch);
    int *tickets = thr_scratch ? reinterpret_cast<int *>(acc_words + ntiles) : nullptr;
    launch_chained(convlstm_point_vec_kernel, dim3(item_grid((int64_t)ntiles * divup(C, cbw))), dim3(PW_THREADS), 0, (cudaStream_t)stream, 
        dg, dg_ps, dg_bits, g, g_ps, dc_prev, dcp_ps, dcp_bits, cprev, cprev_ps, cell, cell_ps, dh, dh_ps, dh_bits, dc,
        dc_ps, dc_bits, N, C, H, W, sum_m2, cbw, h_sent, hs_ps, thr, acc_words, tickets, tail_for_kernel(tail));
    return tail_after_launch(check_launch(), tail, true, stream);
  }
  launch_chained(convlstm_point_kernel, dim3(tile_grid(ntiles)), dim3(PW_THREADS), 0, (cudaStream_t)stream, 
      dg, dg_ps, dg_bits, g, g_ps, dc_prev, dcp_ps, dcp_bits, cprev, cprev_ps, cell, cell_ps, dh, dh_ps, dh_bits, dc,
      dc_ps, dc_bits, N, C, H, W, sum_m2, thr);
  return tail_after_launch(check_launch(), tail, false, stream);
}

extern "C" int mie_upsample(const float *a, int64_t a_ps, const uint64_t *a_bits, const float *b, int64_t b_ps,
                              const uint64_t *b_bits, float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H,
                              int W, int scale, int mode, const mie_tail_job *tail, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !a_bits || !out_bits) return MIE_EINVAL;
  if (tail_check(tail, out_bits) != MIE_OK) return MIE_EINVAL;
  if (mode != MIE_UP_BILINEAR && mode != MIE_UP_NEAREST) return MIE_EINVAL;
  if (scale < 1 || scale > 16 || (scale & (scale - 1))) return MIE_EUNSUPPORTED;   // powers of two: 1/scale is exact (1 copies)
  MIE_CHECK_FIELD(a, a_ps, C); MIE_CHECK_FIELD(out, out_ps, C);
  if (b && (!b_bits || b_ps < C)) return MIE_EINVAL;
  const int ntiles = N * divup(scale * H, 8) * divup(scale * W, 8);
  if (scale == 2 && C % 4 == 0 && a_ps % 4 == 0 && out_ps % 4 == 0 && aligned16(a) && aligned16(out) &&
      (!b || (b_ps % 4 == 0 && aligned16(b)))) {
    launch_chained(upsample2x_tile_kernel, dim3(item_grid((int64_t)ntiles * divup(C, CB))), dim3(PW_THREADS), 0, (cudaStream_t)stream,
        a, a_ps, a_bits, b, b_ps, b_bits, out, out_ps, out_bits, N, C, H, W, mode, tail_for_kernel(tail));
    return tail_after_launch(check_launch(), tail, true, stream);
  }
  if (C >= 4 && a_ps % 4 == 0 && out_ps % 4 == 0 && aligned16(a) && aligned16(out) && (!b || (b_ps % 4 == 0 && aligned16(b)))) {
    launch_chained(upsample2x_vec_kernel, dim3(item_grid((int64_t)ntiles * divup(C, CB))), dim3(PW_THREADS), 0, (cudaStream_t)stream, 
        a, a_ps, a_bits, b, b_ps, b_bits, out, out_ps, out_bits, N, C, H, W, mode, scale);
    return tail_after_launch(check_launch(), tail, false, stream);
  }
  launch_chained(upsample2x_kernel, dim3(item_grid((int64_t)ntiles * divup(C, 64))), dim3(PW_THREADS), 0, (cudaStream_t)stream, a, a_ps, a_bits, b, b_ps, b_bits, out,
                                                                                out_ps, out_bits, N, C, H, W, mode, scale);
  return tail_after_launch(check_launch(), tail, false, stream);
}

extern "C" int mie_upsample2x(const float *a, int64_t a_ps, const uint64_t *a_bits, const float *b, int64_t b_ps,
                              const uint64_t *b_bits, float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H,
                              int W, int mode, const mie_tail_job *tail, void *stream) {
  return mie_upsample(a, a_ps, a_bits, b, b_ps, b_bits, out, out_ps, out_bits, N, C, H, W, 2, mode, tail, stream);
}

extern "C" int mie_add(const float *a, int64_t a_ps, const uint64_t *a_bits, const float *b, int64_t b_ps,
                       const uint64_t *b_bits, float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H, int W,
                       const mie_tail_job *tail, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !a_bits || !b_bits || !out_bits) return MIE_EINVAL;
  if (tail_check(tail, out_bits) != MIE_OK) return MIE_EINVAL;
  MIE_CHECK_FIELD(a, a_ps, C); MIE_CHECK_FIELD(b, b_ps, C); MIE_CHECK_FIELD(out, out_ps, C);
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  if (C % 4 == 0 && a_ps % 4 == 0 && b_ps % 4 == 0 && out_ps % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(out)) {
    launch_chained(add_vec_kernel, dim3(item_grid((int64_t)ntiles * divup(C, CB))), dim3(PW_THREADS), 0, (cudaStream_t)stream, 
        a, a_ps, a_bits, b, b_ps, b_bits, out, out_ps, out_bits, N, C, H, W, tail_for_kernel(tail));
    return tail_after_launch(check_launch(), tail, true, stream);
  }
  launch_chained(add_kernel, dim3(tile_grid(ntiles)), dim3(PW_THREADS), 0, (cudaStream_t)stream, a, a_ps, a_bits, b, b_ps, b_bits, out, out_ps,
                                                                         out_bits, N, C, H, W);
  return tail_after_launch(check_launch(), tail, false, stream);
}

extern "C" int mie_cat2(const float *a, int64_t a_ps, const uint64_t *a_bits, int ca, const float *b, int64_t b_ps,
                        const uint64_t *b_bits, int cb, float *out, int64_t out_ps, uint64_t *out_bits, int N, int H,
                        int W, const mie_tail_job *tail, void *stream) {
  if (N <= 0 || ca <= 0 || cb <= 0 || H <= 0 || W <= 0 || !a_bits || !b_bits || !out_bits) return MIE_EINVAL;
  if (tail_check(tail, out_bits) != MIE_OK) return MIE_EINVAL;
  MIE_CHECK_FIELD(a, a_ps, ca); MIE_CHECK_FIELD(b, b_ps, cb); MIE_CHECK_FIELD(out, out_ps, ca + cb);
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  if (ca % 4 == 0 && cb % 4 == 0 && a_ps % 4 == 0 && b_ps % 4 == 0 && out_ps % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(out)) {
    launch_chained(cat2_vec_kernel, dim3(item_grid((int64_t)ntiles * divup(ca + cb, 64))), dim3(PW_THREADS), 0, (cudaStream_t)stream,
                   a, a_ps, a_bits, ca, b, b_ps, b_bits, cb, out, out_ps, out_bits, N, H, W, tail_for_kernel(tail));
    return tail_after_launch(check_launch(), tail, true, stream);
  }
  launch_chained(cat2_kernel, dim3(item_grid((int64_t)ntiles * divup(ca + cb, CBS))), dim3(PW_THREADS), 0, (cudaStream_t)stream, a, a_ps, a_bits, ca, b, b_ps, b_bits, cb, out,
                                                                          out_ps, out_bits, N, H, W);
  return tail_after_launch(check_launch(), tail, false, stream);
}

extern "C" int mie_accumulate(float *y, int64_t y_ps, const float *d, int64_t d_ps, const uint64_t *d_bits, int N, int C,
                              int H, int W, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !d_bits) return MIE_EINVAL;
  MIE_CHECK_FIELD(y, y_ps, C); MIE_CHECK_FIELD(d, d_ps, C);
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  launch_chained(accumulate_kernel, dim3(tile_grid(ntiles)), dim3(PW_THREADS), 0, (cudaStream_t)stream, y, y_ps, d, d_ps, d_bits, N, C, H, W);
  return check_launch();
}

extern "C" int mie_delta_mask(const float *x, int64_t x_ps, float *x_prev, int64_t xp_ps, float *dx, int64_t dx_ps,
                              uint64_t *bits, int N, int C, int H, int W, float thr, float *split, int64_t split_ps,
                              uint64_t *split_bits, const mie_tail_job *tail, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !bits || !(thr >= 0.0f)) return MIE_EINVAL;
  if (tail_check(tail, bits) != MIE_OK) return MIE_EINVAL;
  const int shalf = divup(C, 8) * 8;
  if (split && (!split_bits || split_ps < 3 * shalf)) return MIE_EINVAL;
  MIE_CHECK_FIELD(x, x_ps, C); MIE_CHECK_FIELD(x_prev, xp_ps, C); MIE_CHECK_FIELD(dx, dx_ps, C);
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  int blocks = divup(ntiles, 4);
  if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
  launch_chained(delta_mask_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, x, x_ps, x_prev, xp_ps, dx, dx_ps,
                                                              reinterpret_cast<unsigned *>(bits), N, C, H, W, thr, split, split_ps,
                                                              shalf, reinterpret_cast<unsigned *>(split_bits), tail_for_kernel(tail));
  return tail_after_launch(check_launch(), tail, true, stream);
}

extern "C" int mie_events_to_voxel(const float *events, int n_events, int num_bins, int sensor_h, int sensor_w, float *voxel,
                                   int64_t v_ps, int H, int W, int pad_left, int pad_top, void *stream) {
  if (!voxel || n_events < 0 || num_bins <= 0 || sensor_h <= 0 || sensor_w <= 0 || H <= 0 || W <= 0 || v_ps < num_bins)
    return MIE_EINVAL;
  if (pad_left < 0 || pad_top < 0 || sensor_h + pad_top > H || sensor_w + pad_left > W) return MIE_EINVAL;
  if (n_events > 0 && (!events || !aligned16(events))) return events ? MIE_EALIGN : MIE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(voxel, 0, (size_t)H * W * v_ps * sizeof(float), st);
  if (e != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  if (n_events == 0) return MIE_OK;
  int blocks = divup(n_events, 256);
  if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
  launch_chained(events_to_voxel_kernel, dim3(blocks), dim3(256), 0, st, events, n_events, num_bins, sensor_h, sensor_w, voxel, v_ps, H, W, pad_left,
                                                 pad_top);
  return check_launch();
}

extern "C" int mie_events_to_count_image(const float *events, int n_events, int sensor_h, int sensor_w, float *image,
                                         int64_t i_ps, int H, int W, int pad_left, int pad_top, void *stream) {
  if (!image || n_events < 0 || sensor_h <= 0 || sensor_w <= 0 || H <= 0 || W <= 0 || i_ps < 2) return MIE_EINVAL;
  if (pad_left < 0 || pad_top < 0 || sensor_h + pad_top > H || sensor_w + pad_left > W) return MIE_EINVAL;
  if (n_events > 0 && (!events || !aligned16(events))) return events ? MIE_EALIGN : MIE_EINVAL;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(image, 0, (size_t)H * W * i_ps * sizeof(float), st);
  if (e != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  if (n_events == 0) return MIE_OK;
  int blocks = divup(n_events, 256);
  if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
  launch_chained(events_to_counts_kernel, dim3(blocks), dim3(256), 0, st, events, n_events, sensor_h, sensor_w, image, i_ps, W, pad_left, pad_top);
  return check_launch();
}

// Max-pool of a delta field against its reservoir: out = maxpool(res + d) - maxpool(res) on the output tiles whose
// windows touch an active input pixel; windows are clipped to the image (torch pads with -inf).  The reservoir is
// only read here: neighbouring windows overlap, so it is advanced afterwards (mie_accumulate on the same delta).
__global__ void __launch_bounds__(1024) maxpool_incr_kernel(
    const float *__restrict__ d, int64_t d_ps, const uint64_t *__restrict__ d_bits, const float *__restrict__ res,
    int64_t res_ps, float *__restrict__ out, int64_t out_ps, uint64_t *__restrict__ out_bits, int N, int C, int H, int W,
    int Ho, int Wo, int k, int stride, int pad) {
  grid_dependency_wait();
  grid_dependency_trigger();
  __shared__ unsigned s_w[2], s_any[2];
  const int THi = (H + 7) >> 3, TWi = (W + 7) >> 3;
  const int ntiles = N * ((Ho + 7) >> 3) * ((Wo + 7) >> 3);
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const TileGeom g = tile_geom(t, Ho, Wo);
    __syncthreads();
    if (threadIdx.x < 2) { s_w[threadIdx.x] = 0u; s_any[threadIdx.x] = 0u; }
    __syncthreads();
    // which output pixels of the tile have an active input pixel in their window
    if (threadIdx.x < 64 && pix_valid(g, threadIdx.x)) {
      const int oy = g.ty * 8 + (threadIdx.x >> 3), ox = g.tx * 8 + (threadIdx.x & 7);
      bool a = false;
      for (int ky = 0; ky < k && !a; ++ky) {
        const int iy = oy * stride - pad + ky;
        if (iy < 0 || iy >= H) continue;
        for (int kx = 0; kx < k; ++kx) {
          const int ix = ox * stride - pad + kx;
          if (ix >= 0 && ix < W && bit_at(d_bits, g.n, iy, ix, THi, TWi)) { a = true; break; }
        }
      }
      if (a) or_word(s_any, threadIdx.x);
    }
    __syncthreads();
    const uint64_t touched = ((uint64_t)s_any[1] << 32) | s_any[0];
    if (touched == 0ull) {
      if (out_bits[t] != 0ull) {
        zero_tile(out, out_ps, C, g, Ho, Wo);
        __syncthreads();
        if (threadIdx.x == 0) out_bits[t] = 0ull;
      }
      continue;
    }
    for (int e = threadIdx.x; e < 64 * C; e += blockDim.x) {
      const int p = e / C, c = e - p * C;
      if (!pix_valid(g, p)) continue;
      const int oy = g.ty * 8 + (p >> 3), ox = g.tx * 8 + (p & 7);
      float v = 0.0f;
      if ((touched >> p) & 1ull) {
        float m_new = -INFINITY, m_old = -INFINITY;
        for (int ky = 0; ky < k; ++ky) {
          const int iy = oy * stride - pad + ky;
          if (iy < 0 || iy >= H) continue;
          for (int kx = 0; kx < k; ++kx) {
            const int ix = ox * stride - pad + kx;
            if (ix < 0 || ix >= W) continue;
            const int64_t pix = (int64_t)(g.n * H + iy) * W + ix;
            const float r = res[pix * res_ps + c];
            const float dv = bit_at(d_bits, g.n, iy, ix, THi, TWi) ? d[pix * d_ps + c] : 0.0f;
            m_old = fmaxf(m_old, r);
            m_new = fmaxf(m_new, r + dv);
          }
        }
        v = m_new - m_old;
        if (v != 0.0f) or_word(s_w, p);
      }
      out[((int64_t)(g.n * Ho + oy) * Wo + ox) * out_ps + c] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) out_bits[t] = ((uint64_t)s_w[1] << 32) | s_w[0];
  }
}

// Border of a [1,C,H,W] field filled by reflection of its interior (sensor image of sh x sw placed at (pt, pl)),
// index arithmetic of torch.nn.ReflectionPad2d: the edge pixel is not repeated.
__global__ void __launch_bounds__(256) reflect_border_kernel(float *__restrict__ f, int64_t ps, int C, int H, int W, int sh,
                                                             int sw, int pl, int pt) {
  grid_dependency_wait();
  grid_dependency_trigger();
  const int64_t total = (int64_t)H * W;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int y = (int)(i / W), x = (int)(i - (int64_t)y * W);
    int sy = y - pt, sx = x - pl;
    if (sy >= 0 && sy < sh && sx >= 0 && sx < sw) continue;   // interior
    if (sy < 0) sy = -sy; else if (sy >= sh) sy = 2 * (sh - 1) - sy;
    if (sx < 0) sx = -sx; else if (sx >= sw) sx = 2 * (sw - 1) - sx;
    const float *src = f + ((int64_t)(sy + pt) * W + (sx + pl)) * ps;
    float *dst = f + i * ps;
    for (int c = 0; c < C; ++c) dst[c] = src[c];
  }
}

extern "C" int mie_reflect_border(float *field, int64_t ps, int C, int H, int W, int sensor_h, int sensor_w, int pad_left,
                                  int pad_top, void *stream) {
  if (!field || C <= 0 || ps < C || H <= 0 || W <= 0 || sensor_h <= 0 || sensor_w <= 0) return MIE_EINVAL;
  if (pad_left < 0 || pad_top < 0 || sensor_h + pad_top > H || sensor_w + pad_left > W) return MIE_EINVAL;
  // a reflected index must land inside the sensor image
  if (pad_left >= sensor_w || W - sensor_w - pad_left >= sensor_w || pad_top >= sensor_h || H - sensor_h - pad_top >= sensor_h)
    return MIE_EINVAL;
  int blocks = divup(H * W, 256);
  if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
  launch_chained(reflect_border_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, field, ps, C, H, W, sensor_h, sensor_w, pad_left, pad_top);
  return check_launch();
}

extern "C" int mie_kfenced(const float *dx, int64_t dx_ps, float *carry, int64_t c_ps, float k, float *q, int64_t q_ps,
                           uint64_t *bits, int N, int C, int H, int W, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !bits || !(k > 0.0f)) return MIE_EINVAL;
  MIE_CHECK_FIELD(dx, dx_ps, C); MIE_CHECK_FIELD(carry, c_ps, C); MIE_CHECK_FIELD(q, q_ps, C);
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  if (C >= 16 && C % 4 == 0 && dx_ps % 4 == 0 && c_ps % 4 == 0 && q_ps % 4 == 0 && aligned16(dx) && aligned16(carry) && aligned16(q)) {
    launch_chained(kfenced_vec_kernel, dim3(tile_grid(ntiles)), dim3(256), 0, (cudaStream_t)stream, dx, dx_ps, carry, c_ps, k, q, q_ps,
                   bits, N, C, H, W);
    return check_launch();
  }
  int blocks = divup(ntiles, 4);
  if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
  launch_chained(kfenced_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, dx, dx_ps, carry, c_ps, k, q, q_ps,
                                                           reinterpret_cast<unsigned *>(bits), N, C, H, W);
  return check_launch();
}

extern "C" int mie_split_tf32(const float *in, int64_t in_ps, const uint64_t *in_bits, int C, float *out, int64_t out_ps,
                              uint64_t *out_bits, int N, int H, int W, const mie_tail_job *tail, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !in_bits || !out_bits) return MIE_EINVAL;
  if (tail_check(tail, out_bits) != MIE_OK) return MIE_EINVAL;
  const int half = divup(C, 8) * 8;
  MIE_CHECK_FIELD(in, in_ps, C); MIE_CHECK_FIELD(out, out_ps, 3 * half);
  const int ntiles = N * divup(H, 8) * divup(W, 8);
  if (C % 4 == 0 && in_ps % 4 == 0 && out_ps % 4 == 0 && aligned16(in) && aligned16(out)) {
    launch_chained(split_tf32_vec_kernel, dim3(tile_grid(ntiles)), dim3(256), 0, (cudaStream_t)stream, in, in_ps, in_bits, C, half, out,
                   out_ps, out_bits, N, H, W, tail_for_kernel(tail));
    return tail_after_launch(check_launch(), tail, true, stream);
  }
  launch_chained(split_tf32_kernel, dim3(tile_grid(ntiles)), dim3(256), 0, (cudaStream_t)stream, in, in_ps, in_bits, C, half, out, out_ps, out_bits,
                                                                        N, H, W, tail_for_kernel(tail));
  return tail_after_launch(check_launch(), tail, true, stream);
}

extern "C" int mie_maxpool_incr(const float *d, int64_t d_ps, const uint64_t *d_bits, const float *res, int64_t res_ps,
                                float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H, int W, int k, int stride,
                                int pad, void *stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !d_bits || !out_bits) return MIE_EINVAL;
  if (k < 1 || k > 7 || stride < 1 || stride > 4 || pad < 0 || 2 * pad > k) return MIE_EUNSUPPORTED;
  MIE_CHECK_FIELD(d, d_ps, C); MIE_CHECK_FIELD(res, res_ps, C);
  const int Ho = (H + 2 * pad - k) / stride + 1, Wo = (W + 2 * pad - k) / stride + 1;
  if (Ho <= 0 || Wo <= 0) return MIE_EINVAL;
  MIE_CHECK_FIELD(out, out_ps, C);
  const int ntiles = N * divup(Ho, 8) * divup(Wo, 8);
  launch_chained(maxpool_incr_kernel, dim3(tile_grid(ntiles)), dim3(wide_threads(ntiles, C)), 0, (cudaStream_t)stream, 
      d, d_ps, d_bits, res, res_ps, out, out_ps, out_bits, N, C, H, W, Ho, Wo, k, stride, pad);
  return check_launch();
}
