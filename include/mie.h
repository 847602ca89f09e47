/*
 * libmie -- masked incremental inference kernels for NVIDIA B200 (sm_100a), C ABI.
 *
 * This is the native boundary of the library.  It replaces the reference's pybind11 module
 * `pointops_ext` (ext/pointops/_C_ext/pointops/ops.cpp:117-123) and the elementwise PyTorch code the
 * reference runs around it (incr_modules/mask_incr_functional.py, incr_modules/mask_incr_modules.py).
 *
 * Conventions shared by every entry point
 *  - every pointer is a DEVICE pointer unless its comment says "host"; the library allocates no device
 *    memory and owns none (one exception is declared as such); what it keeps between calls never shows in a
 *    result: the process-wide options of mie_set_option, a launch counter, a per-thread cache of encoded tensor
 *    maps, and which devices have had a kernel's shared-memory limit raised;
 *  - tensors are fp32, NCHW-logical and channels-last in memory: element (n,y,x,c) of a field lives
 *    at base[((n*H + y)*W + x)*ps + c]; `ps` (pixel stride, in floats) >= C lets a field be a channel
 *    slice of a wider buffer;
 *  - a *delta field* is such a tensor plus one 64-bit word per 8x8 tile (`bits`, N*TH*TW words,
 *    TH=ceil(H/8), TW=ceil(W/8), tile index (n*TH+ty)*TW+tx): bit (py*8+px) is set when pixel
 *    (ty*8+py, tx*8+px) is active.  Invariant kept by every kernel: the tensor is exactly 0 at
 *    every pixel whose bit is clear;
 *  - `stream` is a cudaStream_t passed as void*; kernels are enqueued, never synchronised;
 *  - the return value is MIE_OK or a negative MIE_E* code; nothing ever calls exit() or traps
 *    the device (the reference's CUDA_CHECK_ERRORS does, include/checks.h:12-21).
 */
#ifndef MIE_H
#define MIE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MIE_OK = 0,
  MIE_EINVAL = -1,      /* bad argument (null pointer, non-positive size, unsupported k/stride) */
  MIE_EALIGN = -2,      /* pointer or stride not aligned as the entry point requires */
  MIE_EUNSUPPORTED = -3,/* valid but not implemented combination */
  MIE_ECUDA = -4,       /* a CUDA runtime call failed; see mie_last_cuda_error() */
  MIE_ETOOBIG = -5      /* size beyond a fixed capacity */
};

/* Bits of the device-side error word counts[3] of a convolution's work lists (see mie_tiles_dilate).  The kernels
 * never trap: a bad list entry is skipped, an expired wait makes the block leave its loops, free what it holds and
 * return; the word tells the host afterwards.  The reference's answer to any CUDA error is exit(-1)
 * (include/checks.h:12-21). */
enum {
  MIE_ERR_BAD_TILE = 1,     /* a tile-list entry was outside the field: skipped, its output left untouched */
  MIE_ERR_WAIT_EXPIRED = 2  /* a bounded barrier wait ran out inside a tensor-core kernel: that launch's output is invalid */
};

/* Process-wide options (host).  No counterpart in the reference. */
enum {
  /* 1 (default): thresholded convolutions (thr > 0 or a carry buffer) may run on the tensor cores; 0: they run on
   *    the FP32 kernel. */
  MIE_OPT_TC_THRESHOLDED = 1,
  /* iterations after which a barrier wait of the tensor-core kernels gives up; 0 restores the default (2^20) */
  MIE_OPT_TC_SPIN_LIMIT = 2,
  /* self-test of the expiry path: 1 makes the tensor-core kernels' producers issue no loads, so that the first wait
   * of every block with work runs out and MIE_ERR_WAIT_EXPIRED is raised; the launch writes no output */
  MIE_OPT_TC_WITHHOLD_LOADS = 3,
  /* counter of the kernels this library has enqueued for the step path (every launch of the kernels behind the entry
   * points below except the one-off packing kernels); mie_set_option stores a value (0 resets), mie_get_option reads
   * it modulo 2^31 */
  MIE_OPT_LAUNCH_COUNT = 4,
  /* 1 (default): small-image layers with long reductions run the tensor-core kernel as clusters of 2 or 4 thread
   * blocks that split the input channels of a work item and exchange partial sums through distributed shared
   * memory; 0: one thread block per work item */
  MIE_OPT_TC_KSPLIT = 5,
  /* which tensor-core kernels honour mie_conv_args.own_tiles, as a bit mask: 1 the per-tap kernel, 2 the per-tap kernel as
   * clusters, 4 the halo kernel, 8 the halo kernel as clusters; the others get the separate dilation launch from the
   * entry point.  Default 7: the clustered halo kernel measured slower with the mode than without */
  MIE_OPT_TC_OWN_KERNELS = 6
};
int mie_set_option(int option, int value);
int mie_get_option(int option, int *value /* host */);

enum { MIE_ACT_NONE = 0, MIE_ACT_RELU = 1, MIE_ACT_SIGMOID = 2, MIE_ACT_TANH = 3 };
/* Thresholded layers send or withhold a pixel's output channels in groups of this many consecutive channels (a layer of
 * up to 16 channels decides per pixel).  It is the unit the convolution epilogues work in, so a group is decided by the
 * thread that computed it, in one pass, and a convolution's channel blocks stay as narrow as in lossless mode -- a
 * whole-pixel decision would force one thread block to hold every channel of a pixel. */
#define MIE_THR_GROUP 16
enum { MIE_UP_BILINEAR = 0, MIE_UP_NEAREST = 1 };

int mie_version(void);
const char *mie_status_string(int status);
/* host: text of the last CUDA error seen by this thread inside the library */
const char *mie_last_cuda_error(void);

/* ---------------------------------------------------------------------------------------------
 * Active-tile compaction.
 * No counterpart runs in the reference: it returns None for every mask
 * (incr_modules/mask_incr_modules.py:178) and discards the caller's (pointops_functional.py:22);
 * the expression this follows is compute_mask (incr_modules/utils.py:22-25) with a 1x1 field.
 * ------------------------------------------------------------------------------------------- */

/* bits <- per-pixel any_c(|delta| > thr), strict.  Writes all N*TH*TW words. */
int mie_mask_from_delta(const float *delta, int64_t ps, int N, int C, int H, int W, float thr,
                        uint64_t *bits, void *stream);

/* bits <- per-pixel any_c(mask != 0) from an explicit mask tensor with `cm` channels per pixel
 * (1 for an [N,1,H,W] mask), channels-last, elements of `elem_size` bytes (1: bool/uint8, 4: int32 as
 * the reference's kernels take, ext_conv.cu:238).  `mps` = pixel stride in elements. */
int mie_mask_from_mask(const void *mask, int elem_size, int64_t mps, int cm, int N, int H, int W,
                       uint64_t *bits, void *stream);

/* list[0..count) <- ascending indices of tiles whose word is non-zero; counts[0] <- count. */
int mie_tiles_compact(const uint64_t *bits, int ntiles, int32_t *list, int32_t *counts, void *stream);

/* bytes[N*H*W] <- 0/1 per pixel, expanded from the tile words. */
int mie_mask_expand(const uint64_t *bits, int N, int H, int W, uint8_t *bytes, void *stream);

/* Output-tile set of a k x k / stride / pad convolution: an output tile is active when the
 * receptive field of one of its pixels holds an active input pixel, or when its word in
 * `union_bits` (output geometry, may be null) is non-zero.
 *   list[0..counts[0])   ascending active output tiles
 *   stale[0..counts[1])  tiles whose word in `out_bits` was non-zero (they hold data from the
 *                        previous step) but are not active now: the consumer must zero them
 *   out_bits             every word cleared to 0 (the convolution then sets the active ones)
 * counts is int32[4]: {n_active, n_stale, ticket (must be 0 on entry, is 0 on exit), error word (MIE_ERR_* bits,
 * only ever OR-ed into by the convolution kernels; the host clears it)}.
 * flags is scratch of N*THo*TWo bytes. */
int mie_tiles_dilate(const uint64_t *in_bits, int N, int Hin, int Win, int Hout, int Wout, int k,
                     int stride, int pad, const uint64_t *union_bits, uint64_t *out_bits,
                     int32_t *list, int32_t *stale, int32_t *counts, uint8_t *flags, void *stream);

/* Same result as mie_tiles_dilate, for hosts that are not allowed to allocate device memory.
 * It has no counterpart in the reference.
 * mie_tiles_dilate borrows a flag byte per output tile and a ticket word from its caller.  A program that
 * embeds this library in a camera / inference pipeline whose device memory was partitioned at start-up
 * (allocation afterwards is forbidden there: cudaMalloc synchronises the device, may fail under fragmentation
 * late in a recording, and is not permitted while a stream is being captured) has nowhere to take them from.
 * This variant keeps that scratch inside the library, in a fixed array of MIE_STATIC_MAX_TILES + 256 bytes of
 * device memory that every GPU loading the library holds until the process ends, and calls no allocating
 * routine.  Inputs and outputs are still the caller's; counts is at least int32[2] =
 * {n_active, n_stale}: only these two words are written, so the int32[4] block of mie_tiles_dilate can be passed as is.
 *  - more than MIE_STATIC_MAX_TILES output tiles -> MIE_ETOOBIG;
 *  - the array is shared by all calls on a device and keeps the last call's contents (the word that must be
 *    zero is cleared on `stream` before the launch): calls that overlap on the GPU race -- serialise them;
 *  - the first call on a device resolves the array's address; make it before any stream capture starts. */
#define MIE_STATIC_MAX_TILES 262144
int mie_tiles_dilate_static(const uint64_t *in_bits, int N, int Hin, int Win, int Hout, int Wout, int k,
                            int stride, int pad, const uint64_t *union_bits, uint64_t *out_bits,
                            int32_t *list, int32_t *stale, int32_t *counts, void *stream);

/* A tile dilation carried by the kernel that produces its input ("tail job").  No counterpart in the reference.
 * mie_tiles_dilate depends on nothing but tile words that the launch before it has just written, and at the sizes of
 * one camera stream it is a single thread block: a launch per convolution spent on a few hundred words.  An entry
 * point that takes a `tail` argument (host pointer, may be null) has the last thread block of its kernel to finish
 * run the job after the grid's own work: same arguments as mie_tiles_dilate, same results as a mie_tiles_dilate
 * launch placed directly after that kernel in the stream -- which the caller then leaves out.
 *  - in_bits must be the tile words that entry point writes (its out_bits / dh_bits); union_bits, if any, must be
 *    complete before the launch;
 *  - counts[2] (the ticket) must be 0 on entry and is 0 on exit; flags is scratch of N*THo*TWo bytes;
 *  - a job of more than MIE_TAIL_MAX_TILES output tiles, or one given to a call whose kernel variant cannot carry
 *    it, is enqueued as a separate mie_tiles_dilate launch by the entry point itself: on return the dilation is in the
 *    stream either way. */
#define MIE_TAIL_MAX_TILES 2048
typedef struct mie_tail_job {
  const uint64_t *in_bits; int N, Hin, Win, Hout, Wout, k, stride, pad;
  const uint64_t *union_bits; uint64_t *out_bits;
  int32_t *list; int32_t *stale; int32_t *counts; uint8_t *flags;
} mie_tail_job;

/* ---------------------------------------------------------------------------------------------
 * Masked delta convolution with fused incremental activation.
 * Replaces conv{1x1,3x3,5x5,7x7}_increment_ext (ops.cpp:51-114 -> ext_conv.cu:28-417) and, when
 * act != NONE, the nnReservedActivation that follows every convolution in the networks
 * (incr_modules/mask_incr_modules.py:101-103, 248-251).
 * ------------------------------------------------------------------------------------------- */
typedef struct mie_conv_args {
  /* input delta field */
  const float *in; int64_t in_ps; int cin; int hin; int win;
  /* weights packed by mie_pack_conv_weights: [k*k][cin_pad][cout_pad] */
  const float *wpacked; int cin_pad; int cout; int cout_pad;
  int n; int hout; int wout; int k; int stride; int pad;
  /* work lists from mie_tiles_dilate */
  const int32_t *list; const int32_t *stale; int32_t *counts; int max_tiles;
  /* output delta field; the tile words of the listed tiles must be 0 on entry (mie_tiles_dilate clears them):
   * the kernels OR the sent pixels in */
  float *out; int64_t out_ps; uint64_t *out_bits;
  /* fused epilogue: d = conv (+ addend); act==NONE: dy = d; else with x = *res:
   *   dy = f(x + d) - (emitted ? *emitted : f(x));  *res = x + d;
   * thr > 0: the decision unit is a pixel's group of MIE_THR_GROUP consecutive output channels: a group is sent when
   * one of its channels has |dy| > thr, a withheld group is written as 0; the pixel's mask bit is set when one of its
   * groups is sent; when `emitted` is given it accumulates what was sent. */
  int act; float thr;
  float *res; int64_t res_ps;
  float *emitted; int64_t emitted_ps;
  const float *addend; int64_t addend_ps;
  /* optional second copy of the filter packed by mie_pack_conv_weights_tc ([k*k][cin_pad/32][cout_pad][32], TF32
   * rounded).  When given, and the layer qualifies (Cin*k*k >= 256, 16-byte aligned channel strides, ...), the
   * convolution runs on the tensor cores (tcgen05, TF32 inputs, FP32 accumulation); otherwise on the FP32 path. */
  const float *wpacked_tc;
  /* Dense evaluation (the refresh pass, nnConvIncr.forward_refresh_reservoirs + the activation's,
   * incr_modules/mask_incr_modules.py:182-196, 253-256): with `refresh` non-zero the input is a dense tensor, not a
   * delta: d = conv + bias (+ addend); *res = d (set, not advanced); out = f(d) (act == NONE: out = d); every pixel of
   * every listed tile is written and marked in the tile words.  Needs thr == 0 and no carry buffer; always runs on the
   * FP32 kernel.  `bias` (cout floats, may be null) is only read in this mode or when given. */
  const float *bias;
  int refresh;
  /* optional tile dilation of the next convolution, run in this kernel's tail (in_bits == out_bits of this call) */
  const mie_tail_job *tail;
  /* optional: THIS convolution's own tile dilation (the mie_tiles_dilate call that would precede it: same geometry,
   * list / stale / counts / out_bits of this call), run by the first thread block of the convolution kernel while the
   * others wait for its lists -- one launch instead of two.  counts[2] must be 0 on entry and is 0 on exit.  More than
   * MIE_TAIL_MAX_TILES output tiles: the entry point enqueues the separate launch itself. */
  const mie_tail_job *head;
  /* 1x1 prediction heads only (k == 1, stride 1, pad 0, cout <= 4; MIE_EUNSUPPORTED elsewhere):
   * `in2` -- a second input field of the same shape, added to `in` as it is read (the skip sum in front of the
   *          prediction layer, incr_modules/e2depth_incr.py:430-434, without materialising it); its tile words go to
   *          mie_tiles_dilate as `union_bits`, which for a 1x1 convolution has the input's geometry;
   * `accum` -- a [N,cout,H,W] field that receives `accum += out` at the pixels this call sends (the driver's
   *          `c += c_incr[0]`, run_e2depth_continuous_dataset.py:74, without a separate pass); not in dense evaluation. */
  const float *in2; int64_t in2_ps;
  float *accum; int64_t accum_ps;
  /* `own_tiles` non-zero, together with `head`: no global tile list is made at all.  The thread blocks of the
   * convolution kernel share out the output tiles statically (tile pairs dealt round-robin); each block tests the
   * tiles it owns against the input words itself (the same test as mie_tiles_dilate), compacts the active ones into a
   * list in its shared memory and works through that; the block that owns a tile zeroes it when it is stale.  One
   * launch instead of two and no hand-over between blocks; at full activity the work is spread exactly as with the
   * global list.  `list`, `stale` and counts[0..2] are neither read nor written (counts[3] still collects errors).
   * A tile that several blocks work on (column blocks, clusters) gets its word through `own_scratch`: 12 bytes per output
   * tile, 8-byte aligned, zero on entry and zero again on exit (8 bytes in which the blocks OR their pixels + a ticket;
   * the last block to contribute stores the word).  Convolutions that run on the FP32 kernels or on a kernel that
   * MIE_OPT_TC_OWN_KERNELS leaves out, and fields with more than 256 tiles per thread block, get the separate
   * mie_tiles_dilate launch from the entry point instead. */
  int own_tiles;
  void *own_scratch;
} mie_conv_args;

int mie_conv_tiles(const mie_conv_args *args /* host */, void *stream);

/* Host only, no device work: 1 if mie_conv_tiles would run these arguments on the tensor cores, else 0. */
int mie_conv_uses_tensor_cores(const mie_conv_args *args /* host */);

/* Host only, no device work: the number of thread blocks per cluster mie_conv_tiles would use for these arguments on the
 * tensor cores (2 or 4: the blocks of a cluster split a work item's input channels, see MIE_OPT_TC_KSPLIT; 1: no
 * cluster), 0 when the layer does not run on the tensor cores.  No counterpart in the reference. */
int mie_conv_cluster_size(const mie_conv_args *args /* host */);

/* Host helper (no device work): floats needed for the packed copy of a [cout,cin,k,k] filter, and
 * the padded extents the kernels assume. */
int mie_conv_pack_dims(int cin, int cout, int k, int *cin_pad, int *cout_pad, int64_t *n_floats);

/* Same for the tensor-core copy: cin padded to 32, layout [k*k][cin_pad/32][cout_pad][32]. */
int mie_conv_pack_dims_tc(int cin, int cout, int k, int *cin_pad, int *cout_pad, int64_t *n_floats);
int mie_pack_conv_weights_tc(const float *w_oihw, int cout, int cin, int k, float *wpacked, void *stream);

/* wpacked[(ky*k+kx)][ci][co] <- w[co][ci][ky][kx] (PyTorch OIHW, contiguous), zero padded.
 * The reference keeps a [Cin,kH,kW,Cout] copy for the same purpose
 * (ext/pointops/pointops_functional.py:13-14). */
int mie_pack_conv_weights(const float *w_oihw, int cout, int cin, int k, float *wpacked, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Reference-shaped entry points (same argument meaning as the pybind functions they replace).
 * ------------------------------------------------------------------------------------------- */

/* out = relu(X + in) - relu(X); X += in, over n contiguous floats.
 * activation_increment(X, in_incr, out_incr), ops.cpp:8-23 -> pointop_cuda.cu:17-96 (ReLU only
 * there; `op` selects MIE_ACT_* here). */
int mie_activation_increment(float *X, const float *in_incr, float *out_incr, int64_t n, int op,
                             void *stream);

/* conv{k}x{k}_increment_ext(x_incr, mask, filter, out_incr, stride), ops.cpp:51-114.
 * x_incr [N,Cin,H,W] channels-last; mask: same shape as x_incr, `mask_elem_size` bytes per element
 * (0 = no mask given: derive it from x_incr != 0); filter [Cin,k,k,Cout] contiguous
 * (pointops_functional.py:13-14); out_incr [N,Cout,Hout,Wout] channels-last, every element is
 * written (the reference hands in torch.empty, pointops_functional.py:29).  pad = k/2.
 * workspace: device scratch of mie_conv_increment_workspace_bytes(...) bytes, 256-byte aligned. */
int64_t mie_conv_increment_workspace_bytes(int N, int cin, int H, int W, int cout, int k, int stride);
int mie_conv_increment_ext(const float *x_incr, const void *mask, int mask_elem_size, const float *filter,
                           float *out_incr, int N, int cin, int H, int W, int cout, int k, int stride,
                           void *workspace, int64_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Fused incremental point operations over delta fields.  All of them walk every tile, skip tiles
 * whose input words are all zero (clearing stale output there) and keep the zero invariant.
 * ------------------------------------------------------------------------------------------- */

/* dy = f(res + dx) - (emitted ? emitted : f(res)); res += dx when `accumulate` is non-zero; send decision per pixel and
 * group of MIE_THR_GROUP channels as in mie_conv_tiles; out mask = a group of the pixel was sent.  C <= 1024.
 * accumulate = 1: nnReservedActivation.forward, incr_modules/mask_incr_modules.py:248-251;
 * accumulate = 0: NonlinearPointOpIncr.forward against a reservoir some other module advances, :101-103 (no carry then).
 * in/out may alias (in place) when in_ps == out_ps. */
int mie_act_incr(const float *in, int64_t in_ps, const uint64_t *in_bits, float *res, int64_t res_ps,
                 float *emitted, int64_t emitted_ps, float *out, int64_t out_ps, uint64_t *out_bits,
                 int N, int C, int H, int W, int op, float thr, int accumulate, void *stream);

/* out = (d2 + x2)*d1 + x1*d2; with `accumulate` non-zero also x1 += d1; x2 += d2.  Either delta may be null (all zero).
 * accumulate = 0: IncrPointwiseMultiply, incr_modules/mask_incr_functional.py:52-54 (reservoirs only read);
 * accumulate = 1: nnReservedMultiplication.forward, incr_modules/mask_incr_modules.py:71-75. */
int mie_mul_incr(const float *d1, int64_t d1_ps, const uint64_t *bits1, float *x1, int64_t x1_ps,
                 const float *d2, int64_t d2_ps, const uint64_t *bits2, float *x2, int64_t x2_ps,
                 float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H, int W, float thr,
                 int accumulate, void *stream);

/* The point-wise part of ConvLSTMIncr.forward (incr_modules/e2depth_incr.py:103-120) in one pass:
 * gate pre-activation deltas dg [N,4C,H,W] (order in, remember, out, cell) are folded into the
 * pre-activation reservoir g; the three products and tanh of the cell follow.
 *   g      [N,4C,H,W]  gate pre-activations (the four activation reservoirs side by side)
 *   cprev  [N,C,H,W]   accumulated previous-cell input of product m2 (only touched if dc_prev given)
 *   cell   [N,C,H,W]   accumulated cell (reservoir of the second tanh)
 *   dc_prev/dcp_bits   incoming previous-cell delta, may be null
 *   dh, dc             outgoing hidden and cell deltas; their masks are the union of the incoming masks
 *                      (gate delta | previous-cell delta), pixel for pixel
 *   h_sent / thr       thresholded hidden output (no counterpart in the reference): with h_sent given ([N,C,H,W], what
 *                      has been sent so far; the dense hidden state right after a refresh) the hidden delta is
 *                      dh = h_new - h_sent, a pixel's group of MIE_THR_GROUP channels is sent (and h_sent advanced)
 *                      when one of its |dh| exceeds thr and written as 0 otherwise, and the hidden mask is the set of
 *                      pixels with a sent group.  Needs C % 16 == 0 and 16-byte aligned strides.  thr > 0 needs h_sent
 *   thr_scratch        with h_sent: 12 bytes per tile (N*TH*TW tiles), 8-byte aligned, zero before the first call; the
 *                      kernel leaves it zero (the channel blocks of a tile combine their mask bits through it)
 *   sum_m2             1: cell delta = m1 + m2 (dense-exact); 0: m1 only, as the reference computes
 *                      (its `+` concatenates two lists, e2depth_incr.py:113) */
int mie_convlstm_point(const float *dg, int64_t dg_ps, const uint64_t *dg_bits, float *g, int64_t g_ps,
                       const float *dc_prev, int64_t dcp_ps, const uint64_t *dcp_bits,
                       float *cprev, int64_t cprev_ps, float *cell, int64_t cell_ps,
                       float *dh, int64_t dh_ps, uint64_t *dh_bits, float *dc, int64_t dc_ps,
                       uint64_t *dc_bits, int N, int C, int H, int W, int sum_m2, float thr, float *h_sent,
                       int64_t hs_ps, void *thr_scratch, const mie_tail_job *tail /* reads dh_bits; may be null */,
                       void *stream);

/* out[N,C,2H,2W] = up2(a (+ b)); bilinear (align_corners=False) or nearest.  b may be null.
 * interpolate_from_module, incr_modules/mask_incr_functional.py:76-78; the sum is the skip
 * connection the networks apply just before (incr_modules/e2depth_incr.py:430). */
int mie_upsample2x(const float *a, int64_t a_ps, const uint64_t *a_bits, const float *b, int64_t b_ps,
                   const uint64_t *b_bits, float *out, int64_t out_ps, uint64_t *out_bits, int N, int C,
                   int H, int W, int mode, const mie_tail_job *tail /* reads out_bits; may be null */, void *stream);

/* The same for a scale of 1 (a masked copy), 2, 4, 8 or 16: out[N,C,scale*H,scale*W].  F.interpolate(delta, size=highest_resolution,
 * mode="bilinear", align_corners=False) on the multi-resolution predictions and decoder outputs,
 * incr_modules/delayedevflownet_incr.py:260-268. */
int mie_upsample(const float *a, int64_t a_ps, const uint64_t *a_bits, const float *b, int64_t b_ps,
                 const uint64_t *b_bits, float *out, int64_t out_ps, uint64_t *out_bits, int N, int C,
                 int H, int W, int scale, int mode, const mie_tail_job *tail /* reads out_bits; may be null */,
                 void *stream);

/* out = a + b, out mask = mask_a | mask_b.  Skip / residual sum of two delta fields. */
int mie_add(const float *a, int64_t a_ps, const uint64_t *a_bits, const float *b, int64_t b_ps,
            const uint64_t *b_bits, float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H,
            int W, const mie_tail_job *tail /* reads out_bits; may be null */, void *stream);

/* out[..., 0:ca] = a, out[..., ca:ca+cb] = b; out mask = mask_a | mask_b.  Channel concatenation
 * (torch.cat in incr_modules/e2depth_incr.py:100 and skip_concat, incr_modules/evflownet_incr.py:9-14). */
int mie_cat2(const float *a, int64_t a_ps, const uint64_t *a_bits, int ca, const float *b, int64_t b_ps,
             const uint64_t *b_bits, int cb, float *out, int64_t out_ps, uint64_t *out_bits, int N, int H,
             int W, const mie_tail_job *tail /* reads out_bits; may be null */, void *stream);

/* y += d over the active tiles of d.  The caller-side accumulation of the driver loop
 * (run_e2depth_continuous_dataset.py:74) and IncrementReserve.accumulate
 * (incr_modules/mask_incr_functional.py:41-42). */
int mie_accumulate(float *y, int64_t y_ps, const float *d, int64_t d_ps, const uint64_t *d_bits, int N,
                   int C, int H, int W, void *stream);

/* ---------------------------------------------------------------------------------------------
 * The steps either side of the network in the reference's driver loop.
 * ------------------------------------------------------------------------------------------- */

/* dx = x - x_prev; x_prev = x; bits = per-pixel any_c(|dx| > thr), one pass.  Withheld pixels (all |dx| <= thr)
 * are written as 0 and keep their x_prev, so nothing is lost, only deferred.
 * The driver's `x = event_tensor - event_tensor_prev` (run_e2depth_continuous_dataset.py:66) plus the mask.
 * `split` (may be null): also write what mie_split_tf32 would make of dx -- [dx, dx - tf32(dx), dx] as three blocks of
 * C rounded up to 8 channels, pixel stride split_ps, tile words split_bits (which must describe the copy's previous
 * contents: half tiles that are and were inactive are skipped) -- for a first layer that runs in split precision. */
int mie_delta_mask(const float *x, int64_t x_ps, float *x_prev, int64_t xp_ps, float *dx, int64_t dx_ps,
                   uint64_t *bits, int N, int C, int H, int W, float thr,
                   float *split /* may be null */, int64_t split_ps, uint64_t *split_bits,
                   const mie_tail_job *tail /* reads bits; may be null */, void *stream);

/* Voxel grid of one window of events: temporal-bilinear, spatial-nearest accumulation, as
 * events_to_voxel_grid_absT (data_fetchers/utils/util.py:78-110).  events: [n_events][4] floats
 * (t in [0,1), x, y, polarity; polarity 0 counts as -1).  voxel: [1, num_bins, H, W] channels-last with pixel
 * stride v_ps, zeroed by this call; (pad_left, pad_top) shift the sensor image inside a larger grid
 * (reflection padding itself is left to the caller). */
int mie_events_to_voxel(const float *events, int n_events, int num_bins, int sensor_h, int sensor_w,
                        float *voxel, int64_t v_ps, int H, int W, int pad_left, int pad_top, void *stream);

/* Two-channel image of signed event counts of one window: channel 0 = number of events with polarity -1, channel 1 =
 * with polarity +1, per pixel, as event_histogram (data_fetchers/utils/util.py:62-75) builds on the host with
 * np.add.at -- the input representation of the flow networks.  events as for mie_events_to_voxel (the time stamp is
 * not used); image: [1, 2, H, W] channels-last with pixel stride i_ps >= 2, zeroed by this call; (pad_left, pad_top)
 * place the sensor image inside a larger field. */
int mie_events_to_count_image(const float *events, int n_events, int sensor_h, int sensor_w, float *image,
                              int64_t i_ps, int H, int W, int pad_left, int pad_top, void *stream);

/* Split-precision copy of a delta field for the tensor-core convolution, which
 * truncates its inputs to TF32: with half = C rounded up to 8,
 *   out[c] = d[c],  out[half + c] = d[c] - tf32_trunc(d[c]),  out[2*half + c] = d[c];
 * the other channels of `out` (pixel stride out_ps >= 3*half, zero-initialised by the caller) are not written.
 * Convolving `out` with the filter blocks [W, W, W - tf32(W)] at channel offsets 0, half, 2*half gives the fp32
 * convolution of d with W (the dropped term is ~2^-21 relative).  out_bits (one word per tile, zero before the
 * first call) remembers which tiles of `out` hold data so that they are zeroed again when their input tile goes
 * inactive.  No counterpart in the reference. */
int mie_split_tf32(const float *in, int64_t in_ps, const uint64_t *in_bits, int C, float *out, int64_t out_ps,
                   uint64_t *out_bits, int N, int H, int W, const mie_tail_job *tail /* reads out_bits; may be null */,
                   void *stream);

/* Fills the border of a [1,C,H,W] channels-last field by reflection of the sensor_h x sensor_w image that sits at
 * (pad_top, pad_left) inside it -- the index arithmetic of torch.nn.ReflectionPad2d, which the reference's driver
 * applies to the voxel grid before the network (run_e2depth_continuous_dataset.py:49). */
int mie_reflect_border(float *field, int64_t ps, int C, int H, int W, int sensor_h, int sensor_w, int pad_left,
                       int pad_top, void *stream);

/* out = maxpool(res + d) - maxpool(res) for a k x k window (stride, pad as torch.nn.MaxPool2d, floor mode);
 * out is [N,C,Ho,Wo] with Ho = (H + 2*pad - k)/stride + 1.  The reservoir is only read: advance it afterwards with
 * mie_accumulate(res, d).  nnMaxPool2dIncr.forward, incr_modules/mask_incr_modules.py:217-220. */
int mie_maxpool_incr(const float *d, int64_t d_ps, const uint64_t *d_bits, const float *res, int64_t res_ps,
                     float *out, int64_t out_ps, uint64_t *out_bits, int N, int C, int H, int W, int k, int stride,
                     int pad, void *stream);

/* Sigma-delta quantiser with carry: T = carry + dx; q = k * floor(0.5 + T / k); carry = T - q; bits = q != 0.
 * KFencedMaskModule.forward, incr_modules/mask_incr_modules.py:31-41. */
int mie_kfenced(const float *dx, int64_t dx_ps, float *carry, int64_t c_ps, float k, float *q, int64_t q_ps,
                uint64_t *bits, int N, int C, int H, int W, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MIE_H */
