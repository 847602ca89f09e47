// Masked delta convolution on the 5th-generation tensor cores (tcgen05, TF32 inputs, FP32 accumulation in
// tensor memory) for layers whose reduction depth Cin*k*k makes a dense contraction pay off.
//
// Implicit GEMM over the compact list of active 8x8 output tiles:
//   M = 128 rows   = 2 active tiles x 64 pixels (one tensor-memory lane per pixel)
//   N = NB columns = up to 256 output channels (one tensor-memory column per channel)
//   K              = Cin * k * k, walked as (32-channel chunk, filter tap).
// Two kernels share the epilogue (tcgen05.ld, fused incremental activation, tile words):
//
// conv_tc_kernel (per-tap): one pipeline stage per (chunk, tap), both operands moved by TMA (tiled mode,
// 128-byte swizzle; every copy is issued by one thread block for its own shared memory, also in the cluster variants):
//   A: for each of the two tiles a box [1 image][8 rows][8 cols][32 channels] of the input field, shifted by
//      the tap; out-of-image elements are zero-filled by the TMA unit, which is the convolution padding.
//      The box lands as 64 rows of 128 bytes in pixel order = the K-major operand layout tcgen05.mma reads.
//      Stride-2 layers read from four parity views of the input (one tensor map per row/column parity).
//   B: box [1 tap][NB output channels][32 input channels] of the filter, stored [tap][cout][cin].
//   Roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = MMA issuer (one lane) and owner of the
//   tensor-memory allocation, warps 2..5 = epilogue.  Takes stride 2, k = 1 and blocks of 256 channels.
//
// conv_tc_halo_kernel (halo-resident): stride 1, k in {3,5,7}.  The input halo of both tiles stays in shared
// memory for a whole channel chunk, a filter tap is an address shift of the operand descriptor, and only filter
// slices stream through the ring -- several taps per stage, two MMA-issuing warps.  See the comment at the kernel.
//
// Every mbarrier wait is bounded; on expiry the block raises counts[3], leaves its loops, frees its tensor
// memory and returns.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include "mie_common.cuh"

using namespace mie;

namespace mie {

struct TcParams {
  int cin, cout, cout_pad, cin_pad;   // cin_pad: multiple of 32 (filter K extent)
  int n, hin, win, hout, wout, k, stride, pad;
  const int32_t *list; const int32_t *stale; int32_t *counts; int max_tiles;
  float *out; int64_t out_ps; unsigned int *out_bits32;
  int act; float thr;
  float *res; int64_t res_ps;
  float *emitted; int64_t emitted_ps;
  const float *addend; int64_t addend_ps;
  int nb;        // output channels per block (multiple of 16, <= 256)
  int stages;    // pipeline depth
  int tps;       // halo kernel: filter taps per pipeline stage (divides k*k)
  int issuers;   // halo kernel: 1 or 2 MMA-issuing warps (2: stages alternate, one accumulator each)
  unsigned spin_limit;   // iterations after which a barrier wait gives up (MIE_OPT_TC_SPIN_LIMIT)
  int withhold_loads;    // self-test: the producers issue nothing, so the first wait runs out (MIE_OPT_TC_WITHHOLD_LOADS)
  mie_tail_job tail;     // the next convolution's tile dilation, run by the last block (list == nullptr: none)
  mie_tail_job head;     // this convolution's own tile dilation, run by block 0 while the others wait (list == nullptr: none)
  int ksplit;            // halo kernel: CTAs of a cluster that share one work item, each reducing 1/ksplit of the
                         // input-channel chunks (1: no cluster)
  int own;               // every block finds the active tiles among those it owns itself (`head` describes the test);
                         // no global list is read
  unsigned long long *own_words;   // own mode, tiles that several blocks finish: the word under construction ...
  int *own_tickets;                // ... and how many epilogue warps have contributed to it (both zero between launches)
};

namespace {

// -DMIE_TC_TRACE (debug builds only): conv_tc_kernel records SM-clock timestamps of its phases per block, read back
// through mie_debug_trace().  Compiled out of the product build.
#ifdef MIE_TC_TRACE
__device__ long long g_tc_trace[1024 * 16];
__device__ __forceinline__ long long trace_gtime() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define TC_TRACE(slot) do { if (blockIdx.x < 1024) g_tc_trace[blockIdx.x * 16 + (slot)] = clock64(); } while (0)
#define TC_TRACE_G(slot) do { if (blockIdx.x < 1024) g_tc_trace[blockIdx.x * 16 + (slot)] = trace_gtime(); } while (0)
#define TC_TRACE_V(slot, v) do { if (blockIdx.x < 1024) g_tc_trace[blockIdx.x * 16 + (slot)] = (v); } while (0)
#else
#define TC_TRACE(slot) do { } while (0)
#define TC_TRACE_G(slot) do { } while (0)
#define TC_TRACE_V(slot, v) do { } while (0)
#endif

constexpr int TC_THREADS = 192;
constexpr int A_STAGE_BYTES = 128 * 128;  // 128 pixels x 32 channels x 4 B
constexpr unsigned SPIN_LIMIT = 1u << 20;   // default of TcParams::spin_limit

__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait on a phase parity.  Returns false when the limit ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity, volatile int *abort_flag, unsigned limit) {
  const unsigned addr = smem_u32(bar);
  for (unsigned it = 0; it < limit; ++it) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_4d_raw(unsigned smem_addr, const CUtensorMap *map, unsigned bar_addr, int c0, int c1,
                                                int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_addr), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_load_5d_raw(unsigned smem_addr, const CUtensorMap *map, unsigned bar_addr, int c0, int c1,
                                                int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_addr), "l"(reinterpret_cast<unsigned long long>(map)), "r"(bar_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes,
// 8-row groups 1024 bytes apart.  Bits: [0,14) address>>4, [16,30) leading offset>>4 (unused for swizzled
// K-major), [32,46) stride offset>>4, [46,48) version = 1, [61,64) layout = 2 (128-byte swizzle).
__device__ __forceinline__ unsigned long long make_smem_desc(unsigned smem_addr, unsigned sbo_bytes = 1024) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(sbo_bytes >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}

// Descriptor of a K-major operand stored WITHOUT swizzle: 8 rows x 16 bytes form one contiguous 128-byte core
// matrix; `lbo_bytes` is the distance between the two core matrices an MMA reads along K, `sbo_bytes` the distance
// between consecutive 8-row groups.  The start address only needs 16-byte alignment, which is what lets a filter
// tap be expressed as an address shift inside a resident halo tile.
__device__ __forceinline__ unsigned long long make_smem_desc_plain(unsigned smem_addr, unsigned lbo_bytes, unsigned sbo_bytes) {
  unsigned long long d = 0;
  d |= (unsigned long long)((smem_addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)(lbo_bytes >> 4) << 16;
  d |= (unsigned long long)(sbo_bytes >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  return d;
}

// Instruction descriptor for kind::tf32, FP32 accumulator, both operands K-major, M = 128.
__device__ __forceinline__ unsigned make_idesc_tf32(int n) {
  unsigned d = 0;
  d |= 1u << 4;                 // accumulator format F32
  d |= 2u << 7;                 // A format TF32
  d |= 2u << 10;                // B format TF32
  d |= (unsigned)(n >> 3) << 17;
  d |= (unsigned)(128 >> 4) << 24;
  return d;
}

// The four K-slices of one stage (descriptor low words advance by 2 = 32 bytes), one predicate set-up.
__device__ __forceinline__ void umma_tf32_x4(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                             unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "add.u64 a1, %1, 2;\n\tadd.u64 a2, %1, 4;\n\tadd.u64 a3, %1, 6;\n\t"
      "add.u64 b1, %2, 2;\n\tadd.u64 b2, %2, 4;\n\tadd.u64 b3, %2, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], a1, b1, %3, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], a2, b2, %3, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], a3, b3, %3, q;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with a caller-given advance of the A descriptor per K-slice (in 16-byte units) and only the first `nks`
// (1..4) slices issued: a chunk that holds fewer than 32 real channels needs no MMA on its zero padding.
__device__ __forceinline__ void umma_tf32_step(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                               unsigned idesc, unsigned accumulate, unsigned long long a_step, unsigned nks) {
  asm volatile(
      "{\n\t.reg .pred p, q, r1, r2, r3;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "setp.gt.u32 r1, %6, 1;\n\tsetp.gt.u32 r2, %6, 2;\n\tsetp.gt.u32 r3, %6, 3;\n\t"
      "add.u64 a1, %1, %5;\n\tadd.u64 a2, a1, %5;\n\tadd.u64 a3, a2, %5;\n\t"
      "add.u64 b1, %2, 2;\n\tadd.u64 b2, %2, 4;\n\tadd.u64 b3, %2, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
      "@r1 tcgen05.mma.cta_group::1.kind::tf32 [%0], a1, b1, %3, q;\n\t"
      "@r2 tcgen05.mma.cta_group::1.kind::tf32 [%0], a2, b2, %3, q;\n\t"
      "@r3 tcgen05.mma.cta_group::1.kind::tf32 [%0], a3, b3, %3, q;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "l"(a_step), "r"(nks)
      : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// ---- thread-block cluster helpers (K-split variant of the halo kernel) ----
__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of this CTA's shared-memory location `addr` inside CTA `rank`
__device__ __forceinline__ unsigned mapa_shared(unsigned addr, unsigned rank) {
  unsigned r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f4(unsigned cluster_addr, float a, float b, float c, float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Every thread of every CTA of the cluster (whole warps: .aligned).  An execution barrier only: what it orders here is
// "barriers initialised (and made visible by fence.mbarrier_init) before any remote arrival" and "no CTA exits before
// the others are done with its shared memory" -- data is handed over through part_full, with its own release / acquire.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
// mbar_wait whose acquire covers writes made by other CTAs of the cluster before their (release.cluster) arrivals
__device__ __forceinline__ bool mbar_wait_cluster(unsigned long long *bar, unsigned parity, volatile int *abort_flag, unsigned limit) {
  const unsigned addr = smem_u32(bar);
  for (unsigned it = 0; it < limit; ++it) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ float4 f4add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

__device__ __forceinline__ void tmem_ld16(unsigned taddr, float *v) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// One group of 16 accumulator columns of one pixel: optional residual add, incremental activation against the
// reservoir, store.  The activation is a template argument: with a run-time switch every one of the 32 calls below
// carried the code of all three functions, and the executed path hopped over ~50 KB of instructions -- after an L2
// flush each hop is an instruction-cache miss served from DRAM (measured: 4 us of a 5.4 us epilogue).
// ReLU and "none" are inlined; sigmoid and tanh go through one shared out-of-line copy (ACT = MIE_ACT_SIGMOID stands
// for both): inlining 32 copies of expf / tanhf cost 180 registers and with them the third resident block.
__device__ __noinline__ float tc_act_call(int op, float x) { return act_apply(op, x); }
template <int ACT>
__device__ __forceinline__ float tc_act(int op, float x) {
  if (ACT == MIE_ACT_RELU) return fmaxf(x, 0.0f);
  if (ACT == MIE_ACT_NONE) return x;
  return tc_act_call(op, x);
}

template <int ACT>
__device__ __forceinline__ bool tc_epilogue_group_t(const TcParams &p, const float *v, int64_t pix, int co, bool any_d) {
  bool flag = false;
  const int nq = min(4, (p.cout - co) >> 2);  // channel quads of this group that exist
  float4 d[4], x[4], base[4];
  // all loads of the group first, then the arithmetic, then the stores
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    d[h] = make_float4(v[h * 4], v[h * 4 + 1], v[h * 4 + 2], v[h * 4 + 3]);
    if (h < nq) {
      if (p.addend) d[h] = f4add(d[h], *reinterpret_cast<const float4 *>(p.addend + pix * p.addend_ps + co + h * 4));
      if (ACT != MIE_ACT_NONE && any_d) {
        x[h] = *reinterpret_cast<const float4 *>(p.res + pix * p.res_ps + co + h * 4);
        if (p.emitted) base[h] = *reinterpret_cast<const float4 *>(p.emitted + pix * p.emitted_ps + co + h * 4);
      }
    }
  }
  // The 16 channels of this call are one send-decision group of a thresholded layer (MIE_THR_GROUP): all four quads
  // are evaluated first, then written -- as computed when the group is sent (and added to the carry), as zeros when it
  // is withheld.  A lossless layer (thr == 0, no carry) sends every group.
  float4 o[4];
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    if (h >= nq) continue;
    o[h] = d[h];
    if (ACT != MIE_ACT_NONE) {
      if (any_d) {
        const float4 xn = f4add(x[h], d[h]);
        *reinterpret_cast<float4 *>(p.res + pix * p.res_ps + co + h * 4) = xn;
        if (!p.emitted)
          base[h] = make_float4(tc_act<ACT>(p.act, x[h].x), tc_act<ACT>(p.act, x[h].y), tc_act<ACT>(p.act, x[h].z), tc_act<ACT>(p.act, x[h].w));
        o[h] = make_float4(tc_act<ACT>(p.act, xn.x) - base[h].x, tc_act<ACT>(p.act, xn.y) - base[h].y,
                           tc_act<ACT>(p.act, xn.z) - base[h].z, tc_act<ACT>(p.act, xn.w) - base[h].w);
      } else {
        o[h] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    flag |= fabsf(o[h].x) > p.thr || fabsf(o[h].y) > p.thr || fabsf(o[h].z) > p.thr || fabsf(o[h].w) > p.thr;
  }
  const bool withheld = !flag && (p.thr > 0.0f || p.emitted != nullptr);
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    if (h >= nq) continue;
    *reinterpret_cast<float4 *>(p.out + pix * p.out_ps + co + h * 4) = withheld ? make_float4(0.f, 0.f, 0.f, 0.f) : o[h];
    if (ACT != MIE_ACT_NONE && p.emitted && flag)
      *reinterpret_cast<float4 *>(p.emitted + pix * p.emitted_ps + co + h * 4) = f4add(base[h], o[h]);
  }
  return flag;
}

__device__ __forceinline__ bool tc_epilogue_group(const TcParams &p, const float *v, int64_t pix, int co, bool any_d) {
  switch (p.act) {
    case MIE_ACT_RELU: return tc_epilogue_group_t<MIE_ACT_RELU>(p, v, pix, co, any_d);
    case MIE_ACT_SIGMOID:
    case MIE_ACT_TANH: return tc_epilogue_group_t<MIE_ACT_SIGMOID>(p, v, pix, co, any_d);
    default: return tc_epilogue_group_t<MIE_ACT_NONE>(p, v, pix, co, any_d);
  }
}

// Epilogue of one accumulator row (= one output pixel, all NB channels of the block).  Called by all 32 lanes of an
// epilogue warp (the tensor-memory loads are warp-collective); returns whether the pixel was sent.
__device__ __forceinline__ void tmem_ld16_sum(unsigned taddr, unsigned acc2, float *v) {
  tmem_ld16(taddr, v);
  if (acc2) {   // a second partial accumulator (two MMA issuers): the sum is the result
    float w[16];
    tmem_ld16(taddr + acc2, w);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] += w[i];
  }
}

// [c_lo, c_hi) is the column range this warp stores (two warps may share a pixel, each taking half the columns);
// the "did anything change" scan always covers all NB columns.
__device__ __forceinline__ bool tc_epilogue_pixel(const TcParams &p, int NB, unsigned taddr, bool valid, int64_t pix,
                                                  int co0, unsigned long long *acc_empty_bar, int lane, unsigned acc2 = 0,
                                                  int c_lo = 0, int c_hi = 1 << 30) {
      // does this pixel carry any change?  (pixels of an active tile outside the dilated support are all
      // zero: they skip the reservoir read-modify-write)
      bool any_d = true;
      if (p.act != MIE_ACT_NONE && !p.emitted) {
        any_d = false;
        for (int c = 0; c < NB; c += 16) {
          float v[16];
          tmem_ld16_sum(taddr + c, acc2, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) any_d |= (v[j] != 0.0f);
        }
        if (valid && p.addend && !any_d)
          for (int c = 0; c < NB && co0 + c < p.cout; ++c) any_d |= (p.addend[pix * p.addend_ps + co0 + c] != 0.0f);
      }
      c_hi = min(c_hi, NB);
      bool flag = false;    // some group of this thread's channel range was sent
      for (int c = c_lo; c < c_hi; c += 16) {
        float v[16];
        tmem_ld16_sum(taddr + c, acc2, v);  // every lane of the warp takes part (aligned), valid or not
        if (valid && co0 + c < p.cout) flag |= tc_epilogue_group(p, v, pix, co0 + c, any_d);
      }
      // the accumulator has been read: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar);
      return valid && flag;
}

// ---- coalesced epilogue (lossless layers: no threshold, no carry) ----------------------------------------------
// The accumulator arrives one pixel per lane, so a lane that stores its own pixel makes every warp-wide access touch
// 32 different 128-byte lines for 16 bytes each.  Here a group of 16 channels goes through a 2 KB staging buffer per
// warp instead ([32 pixels][4 x float4], the float4 slot XOR-swizzled by the pixel so that both the row-wise write
// and the transposed read are free of bank conflicts), and is then handled with four lanes per pixel: one warp
// access covers eight neighbouring pixels x 64 contiguous bytes, for the reservoir read-modify-write, the residual
// addend and the output alike.  A float4 whose change is exactly zero leaves the reservoir untouched (x + 0 = x and
// f(x) - f(x) = 0, so the result equals the full update).
// Returns a mask with bit l set when pixel l of the warp (lane l's accumulator row) emitted a non-zero value.
template <int ACT>
__device__ __forceinline__ unsigned tc_epilogue_rows_t(const TcParams &p, float4 *stage, const float *v, int lane, int64_t pix,
                                                       unsigned valid_mask, int co) {
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int j = 0; j < 4; ++j) stage[lane * 4 + (j ^ sw)] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  __syncwarp();
  unsigned sent = 0;
  const int j = lane & 3, cj = co + 4 * j;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int pl = it * 8 + (lane >> 2);
    float4 d = stage[pl * 4 + (j ^ ((pl >> 1) & 3))];
    const int64_t px = __shfl_sync(0xffffffffu, pix, pl);
    const bool ok = ((valid_mask >> pl) & 1u) && cj < p.cout;
    bool flag = false;
    if (ok) {
      if (p.addend) d = f4add(d, *reinterpret_cast<const float4 *>(p.addend + px * p.addend_ps + cj));
      float4 o = d;
      if (ACT != MIE_ACT_NONE) {
        if (d.x != 0.0f || d.y != 0.0f || d.z != 0.0f || d.w != 0.0f) {
          float4 *rp = reinterpret_cast<float4 *>(p.res + px * p.res_ps + cj);
          const float4 x = *rp;
          const float4 xn = f4add(x, d);
          *rp = xn;
          o = make_float4(tc_act<ACT>(p.act, xn.x) - tc_act<ACT>(p.act, x.x), tc_act<ACT>(p.act, xn.y) - tc_act<ACT>(p.act, x.y),
                          tc_act<ACT>(p.act, xn.z) - tc_act<ACT>(p.act, x.z), tc_act<ACT>(p.act, xn.w) - tc_act<ACT>(p.act, x.w));
        }
      }
      flag = fabsf(o.x) > 0.0f || fabsf(o.y) > 0.0f || fabsf(o.z) > 0.0f || fabsf(o.w) > 0.0f;
      *reinterpret_cast<float4 *>(p.out + px * p.out_ps + cj) = o;
    }
    unsigned bal = __ballot_sync(0xffffffffu, flag);
    bal |= bal >> 1;
    bal |= bal >> 2;   // bit 4k: any of the four lanes of pixel it * 8 + k
#pragma unroll
    for (int k = 0; k < 8; ++k) sent |= ((bal >> (4 * k)) & 1u) << (it * 8 + k);
  }
  __syncwarp();   // the next group overwrites the buffer
  return sent;
}

// One accumulator row per lane, columns [c_lo, c_hi) of the block's NB; same contract as tc_epilogue_pixel.
__device__ __forceinline__ bool tc_epilogue_pixel_coalesced(const TcParams &p, int NB, unsigned taddr, bool valid, int64_t pix,
                                                            int co0, unsigned long long *acc_empty_bar, int lane, float4 *stage,
                                                            unsigned acc2, int c_lo, int c_hi) {
  const unsigned valid_mask = __ballot_sync(0xffffffffu, valid);
  c_hi = min(c_hi, NB);
  unsigned sent = 0;
  bool released = false;
  for (int c = c_lo; c < c_hi; c += 16) {
    float v[16];
    tmem_ld16_sum(taddr + c, acc2, v);
    if (c + 16 >= c_hi) {   // last read of this warp: hand the accumulator back before the global traffic
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar);
      released = true;
    }
    if (co0 + c >= p.cout) continue;
    switch (p.act) {
      case MIE_ACT_RELU: sent |= tc_epilogue_rows_t<MIE_ACT_RELU>(p, stage, v, lane, pix, valid_mask, co0 + c); break;
      case MIE_ACT_SIGMOID:
      case MIE_ACT_TANH: sent |= tc_epilogue_rows_t<MIE_ACT_SIGMOID>(p, stage, v, lane, pix, valid_mask, co0 + c); break;
      default: sent |= tc_epilogue_rows_t<MIE_ACT_NONE>(p, stage, v, lane, pix, valid_mask, co0 + c); break;
    }
  }
  if (!released) {
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(acc_empty_bar);
  }
  return valid && ((sent >> lane) & 1u);
}

// Asks for the lines the epilogue of one pixel will read (reservoir, residual addend, carry) while the MMAs of the item
// are still running: the accumulator arrives to loads that hit the cache instead of starting a DRAM round trip each.
__device__ __forceinline__ void tc_epilogue_prefetch(const TcParams &p, int64_t pix, int co0, int c_lo, int c_hi) {
  c_hi = min(c_hi, p.cout - co0);
  for (int c = c_lo; c < c_hi; c += 32) {
    if (p.act != MIE_ACT_NONE) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p.res + pix * p.res_ps + co0 + c));
      if (p.emitted) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.emitted + pix * p.emitted_ps + co0 + c));
    }
    if (p.addend) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.addend + pix * p.addend_ps + co0 + c));
  }
}

struct TcMaps {
  CUtensorMap in[4];  // stride 1: [0] only; stride 2: [row parity * 2 + column parity]
  CUtensorMap w;
};

// Zeroes the stale tiles of the output field.  Run by the epilogue warps (`tid` = index within them, `nthreads` = how
// many they are) before their first accumulator arrives: the producer and the MMA issuer do not wait for it.
__device__ __forceinline__ void tc_zero_tile(const TcParams &p, int t, int THo, int TWo, int tid, int nthreads) {
  const int tx = t % TWo, ty = (t / TWo) % THo, n = t / (TWo * THo);
  for (int i = tid; i < 64 * p.cout; i += nthreads) {
    const int px = i / p.cout, c = i - px * p.cout;
    const int oy = ty * 8 + (px >> 3), ox = tx * 8 + (px & 7);
    if (oy < p.hout && ox < p.wout) p.out[((int64_t)(n * p.hout + oy) * p.wout + ox) * p.out_ps + c] = 0.0f;
  }
}
__device__ __forceinline__ void tc_zero_stale(const TcParams &p, int ntiles_total, int THo, int TWo, int tid, int nthreads) {
  const int n_stale = p.stale ? min(p.counts[1], p.max_tiles) : 0;
  for (int s = blockIdx.x; s < n_stale; s += gridDim.x) {
    const int t = p.stale[s];
    if (t < 0 || t >= ntiles_total) { if (tid == 0) atomicOr(&p.counts[3], MIE_ERR_BAD_TILE); continue; }
    tc_zero_tile(p, t, THo, TWo, tid, nthreads);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// "Own tiles" mode (mie_conv_args.own_tiles): the convolution needs no tile list from a launch before it.  The output
// tiles are dealt to the thread blocks in static pairs (2P, 2P+1), pair P to group P mod G, a group being the n_cblk
// blocks (or clusters) that finish the column blocks of the same pixels.  After the grid dependency wait every block
// tests the tiles of its group against the input words (dilate_flag: one round trip to L2, all loads in flight at once),
// compacts the active ones in ascending order into shared memory and pairs them up as work items; all blocks of a group
// arrive at the same list.  At full activity this spreads the work exactly as the global list does; at partial activity a
// block's share is what is active among its own tiles.  Stale tiles are zeroed by the one block of the group that also
// reads the previous word (column block 0, cluster rank 0).
// Tile words: a tile that a single block finishes is cleared by that block before its epilogue ORs the sent pixels in, as
// after a separate dilation.  A tile that several blocks finish cannot be cleared by one of them without racing the
// others' ORs; there the epilogue warps OR into a scratch word and draw a ticket, and the warp that draws the last ticket
// stores the finished word and leaves both scratch entries zero.
// ---------------------------------------------------------------------------------------------------------------
constexpr int OWN_MAX = 256;   // tiles one group can own; the host sends larger shares to the separate dilation launch

struct OwnShared {
  int list[OWN_MAX];           // active tiles from the front (ascending), stale tiles from the back
  int n_active, n_stale;
  uint8_t flags[OWN_MAX];
};
template <bool OWN> struct OwnSharedT : OwnShared {};
template <> struct OwnSharedT<false> { int list[1]; int n_active, n_stale; };

// Every thread of the block.  (Inlined: as a function of its own, called by all kernels, it made an E2Depth step 3 % slower.)
__device__ __forceinline__ void own_scan(const uint64_t *in_bits, int Hin, int Win, int Hout, int Wout, int k, int stride, int pad,
                                             const uint64_t *union_bits, uint64_t *out_bits /* null unless this block reads and
                                             clears the previous words */, OwnShared &sh, int g, int G, int ntiles_total, bool single) {
  const int SP = (ntiles_total + 1) >> 1;
  const int n_own = g < SP ? 2 * ((SP - g + G - 1) / G) : 0;
  for (int idx = threadIdx.x; idx < n_own; idx += blockDim.x) {
    const int t = 2 * (g + (idx >> 1) * G) + (idx & 1);
    sh.flags[idx] = t < ntiles_total ? dilate_flag(t, in_bits, Hin, Win, Hout, Wout, k, stride, pad, union_bits, out_bits, single)
                                     : (uint8_t)0;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    int na = 0, ns = 0;
    const unsigned below = (1u << threadIdx.x) - 1u;
    for (int base = 0; base < n_own; base += 32) {
      const int idx = base + (int)threadIdx.x;
      const int f = idx < n_own ? sh.flags[idx] : 0;
      const unsigned ba = __ballot_sync(0xffffffffu, f == 1), bs = __ballot_sync(0xffffffffu, f == 2);
      const int t = 2 * (g + (idx >> 1) * G) + (idx & 1);
      if (f == 1) sh.list[na + __popc(ba & below)] = t;
      if (f == 2) sh.list[OWN_MAX - 1 - (ns + __popc(bs & below))] = t;
      na += __popc(ba);
      ns += __popc(bs);
    }
    if (threadIdx.x == 0) { sh.n_active = na; sh.n_stale = ns; }
  }
  __syncthreads();
}

__device__ __forceinline__ void tc_zero_stale_own(const TcParams &p, const OwnShared &sh, int THo, int TWo, int tid, int nthreads) {
  for (int s = 0; s < sh.n_stale; ++s) tc_zero_tile(p, sh.list[OWN_MAX - 1 - s], THo, TWo, tid, nthreads);
}

// One lane per (epilogue warp, tile): `v` = this warp's sent pixels, already shifted into 32-bit half `half32` of the
// tile word; `total` = warps that contribute to a tile over all blocks.
__device__ __forceinline__ void own_contribute(const TcParams &p, int t, int half32, unsigned v, int total) {
  if (v) atomicOr(reinterpret_cast<unsigned *>(p.own_words + t) + half32, v);
  __threadfence();
  if (atomicAdd(p.own_tickets + t, 1) == total - 1) {
    __threadfence();
    reinterpret_cast<unsigned long long *>(p.out_bits32)[t] = atomicExch(p.own_words + t, 0ull);
    p.own_tickets[t] = 0;
  }
}

// ---------------------------------------------------------------------------------------------------------------
// K-split (cluster variants of both kernels): the CS thread blocks of a cluster work on the same item, each reducing
// 1/CS of the input-channel chunks, so each holds partial sums for all NB columns.  A block sends every other block
// the partial sums of that block's column slice (remote shared-memory stores, layout [source][16-column group]
// [channel quad][128 rows] float4: a warp stores 512 contiguous bytes per quad), receives the partial sums of its own
// slice, adds them in a fixed order and finishes only that slice with the usual fused epilogue.
// Called by whole epilogue warps after the accumulator is complete; lane = accumulator row m.  This warp takes the
// groups g0, g0 + gstep, ... of every slice.  part_full must have been initialised with (CS - 1) x (epilogue warps)
// arrivals.  Returns false when a wait ran out; *sent tells whether this row's pixel emitted anything.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ bool ksplit_finish(const TcParams &p, int NB, unsigned CS, unsigned crank, unsigned taddr, unsigned acc2,
                                              unsigned part_base, const unsigned char *part_ptr, unsigned long long *part_full,
                                              unsigned parity, int m, int lane, int g0, int gstep, bool valid, int64_t pix,
                                              int co0, volatile int *abort_flag, unsigned limit, bool *sent) {
  const int SW = NB / (int)CS, ng = SW >> 4;     // slice width, 16-column groups per slice
  const int slice0 = (int)crank * SW;
  for (unsigned j = 0; j < CS; ++j) {
    if (j == crank) continue;
    const unsigned src = crank < j ? crank : crank - 1u;   // this block's index among the sources of block j
    for (int gi = g0; gi < ng; gi += gstep) {
      float v[16];
      tmem_ld16_sum(taddr + (unsigned)((int)j * SW + gi * 16), acc2, v);
      const unsigned dst = mapa_shared(part_base + ((((src * (unsigned)ng + (unsigned)gi) * 4u) * 128u + (unsigned)m) << 4), j);
#pragma unroll
      for (int h = 0; h < 4; ++h) st_cluster_f4(dst + 2048u * h, v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
    }
  }
  // one fence for all the stores above, then lane j tells block j (its release is cumulative over the warp's stores)
  asm volatile("fence.acq_rel.cluster;" ::: "memory");
  __syncwarp();
  if ((unsigned)lane < CS && (unsigned)lane != crank) mbar_arrive_cluster(mapa_shared(smem_u32(part_full), (unsigned)lane));
  if (!mbar_wait_cluster(part_full, parity, abort_flag, limit)) return false;
  bool flag = false;
  for (int gi = g0; gi < ng; gi += gstep) {
    float v[16];
    tmem_ld16_sum(taddr + (unsigned)(slice0 + gi * 16), acc2, v);
    for (unsigned sidx = 0; sidx + 1u < CS; ++sidx) {
      const float4 *sp = reinterpret_cast<const float4 *>(part_ptr + (((((size_t)sidx * ng + gi) * 4u) * 128u + (unsigned)m) << 4));
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float4 w = sp[h * 128];
        v[4 * h] += w.x; v[4 * h + 1] += w.y; v[4 * h + 2] += w.z; v[4 * h + 3] += w.w;
      }
    }
    const int co = co0 + slice0 + gi * 16;
    if (valid && co < p.cout) {
      // a group whose change is exactly zero skips the reservoir (x + 0 = x and f(x) - f(x) = 0: same result)
      bool any_d = true;
      if (p.act != MIE_ACT_NONE && !p.emitted && !p.addend) {
        any_d = false;
#pragma unroll
        for (int i = 0; i < 16; ++i) any_d |= (v[i] != 0.0f);
      }
      flag |= tc_epilogue_group(p, v, pix, co, any_d);
    }
  }
  *sent = valid && flag;
  return true;
}

// ---------------------------------------------------------------------------------------------------------------
// Halo-resident variant for stride-1 layers with k >= 3.
//
// The per-tap kernel below fetches the shifted 8x8x32 input box of every filter tap again (9 or 25 times the same
// pixels), which makes the L2 -> shared-memory path its bound.  Here the (8+k-1)^2 halo of each of the two tiles
// is fetched ONCE per 32-channel chunk and kept in shared memory in the un-swizzled operand layout
//     [halo row y][tile 0|1][16-byte channel group c (8)][halo column x][4 channels],
// in which the 8 pixels x..x+7 of one channel group are one contiguous 128-byte core matrix for ANY x.  A filter
// tap (ky,kx) is then nothing but the descriptor start address  base + ky*2*ROW + kx*16  (ROW = 8*Wh*16 bytes),
// with leading offset Wh*16 (next channel group) and stride offset ROW (next 8-pixel group).  Consecutive groups
// alternate between the two tiles, so accumulator row m holds tile (m>>3)&1, pixel row m>>4, pixel column m&7.
// Only the filter slices (NB x 32 floats per tap and chunk) stream through the stage ring.
// Roles (384 threads): warp 0 = halo producer (one row per lane), warp 1 = filter producer, warps 2 and 3 = MMA
// issuers (warp 2 owns the tensor memory), warps 4..11 = epilogue: two warps per tensor-memory lane quarter, each
// taking half of the block's channels (the epilogue is a chain of dependent global loads per 16 channels; with
// four warps it, not the MMAs, set the pace of layers with many work items per block).  One thread issues a tcgen05.mma about every
// 45 ns whatever its shape, which for blocks of <= 128 channels is several times the tensor core's own time: two
// issuers take alternate pipeline stages and accumulate into separate accumulators that the epilogue adds.
constexpr int HALO_THREADS = 384;
constexpr int HALO_MAX_STAGES = 12;

// KSPLIT: the cluster variant is a separate instantiation, so that the plain one carries neither its code nor its registers.
// OWN: the own-tiles mode, again a separate instantiation: the list-mode kernels are compiled exactly as if it did not exist
// (with the mode as a run-time flag every layer ran 1.5 us longer in list mode, too).
template <bool KSPLIT, bool OWN>
__global__ void __launch_bounds__(HALO_THREADS, 1)
conv_tc_halo_kernel(const TcParams p, const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_w) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int NB = p.nb;
  const unsigned b_bytes = (unsigned)NB * 128u;                 // one filter slice: NB rows of 32 floats, 128-byte swizzle
  const unsigned st_bytes = b_bytes * (unsigned)p.tps;          // one stage: `tps` consecutive taps of one channel chunk
  const int Wh = 8 + p.k - 1, Hh = 8 + p.k - 1;
  const unsigned row_bytes = 8u * (unsigned)Wh * 16u;           // one halo row of one tile, all 8 channel groups
  const unsigned a_buf_bytes = (unsigned)Hh * 2u * row_bytes;   // both tiles
  // b_full[i][s]: slot s holds a stage for MMA issuer i.  One barrier per (issuer, slot): an issuer then observes every
  // phase of every barrier it waits on, whatever the ring depth.  (With one barrier per slot and an odd ring a slot
  // changes hands every lap; the issuer would wait for lap L without having seen lap L-1 complete, and a parity wait
  // cannot tell "lap L done" from "lap L-2 done".)
  __shared__ unsigned long long b_full[2][HALO_MAX_STAGES], b_empty[HALO_MAX_STAGES], a_full[2], a_empty[2], acc_full[2], acc_empty[2];
  __shared__ unsigned long long part_full;   // K-split: every other CTA of the cluster has delivered its partial sums
  __shared__ OwnSharedT<OWN> s_own;          // own-tiles mode: this block's tile list (a stub in the list-mode kernels)
  __shared__ unsigned s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // K-split: the CS CTAs of a cluster work on the same item, CTA `crank` reducing chunks [ch_lo, ch_hi); a cluster has
  // at most one item (the host sizes the grid so), hence `bid` / `nblk` below index clusters, not CTAs.
  const unsigned CS = KSPLIT ? (unsigned)p.ksplit : 1u;
  const unsigned crank = CS > 1u ? cluster_ctarank() : 0u;
  const int bid = (int)(blockIdx.x / CS), nblk = (int)(gridDim.x / CS);
  if (tid == 0) { TC_TRACE(0); TC_TRACE_G(14); }
  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(&map_in)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(&map_w)) : "memory");
  }
  const int THo = (p.hout + 7) >> 3, TWo = (p.wout + 7) >> 3;
  const int ntiles_total = p.n * THo * TWo;
  unsigned acc_cols = 32;
  while ((int)acc_cols < NB) acc_cols <<= 1;
  const unsigned NI = (unsigned)p.issuers;
  const unsigned tmem_cols = 2 * NI * acc_cols;   // per item buffer: one accumulator per issuer

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&b_full[0][s], 1); mbar_init(&b_full[1][s], 1); mbar_init(&b_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&a_full[b], 1); mbar_init(&a_empty[b], NI); mbar_init(&acc_full[b], NI); mbar_init(&acc_empty[b], 8); }
    mbar_init(&part_full, CS > 1u ? (CS - 1u) * 8u : 1u);   // one arrival per epilogue warp of every other CTA
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = s_tmem_base;
  if (CS > 1u) cluster_sync_all();   // no CTA may receive a remote arrival before its barriers exist

  // everything above touched no global memory: it may overlap the tail of the previous kernel in the stream
  if (tid == 0) TC_TRACE(1);
  grid_dependency_wait();
  grid_dependency_trigger();
  constexpr bool own = OWN;
  bool head_ok = true;
  if constexpr (!OWN) {
    head_ok = run_head_job(p.head, p.spin_limit);   // block 0 makes the tile lists, the others wait for them
    if (tid == (int)blockDim.x - 1) count_head_job_passed(p.head);   // a lane of the last epilogue warp: off the critical path
  }
  const int n_cblk = p.cout_pad / NB;
  // work items of this block: item0, item0 + item_step, ... < n_items; item -> (tile pair, column block); tiles from `lst`
  int item0 = bid, item_step = nblk, n_active;
  const int32_t *lst = p.list;
  const bool own_multi = own && n_cblk * (int)CS > 1;   // several blocks finish a tile: its word goes through the scratch
  int pre0 = -1, pre1 = -1;
  if constexpr (OWN) {
    // own-tiles mode: this block's group tests its share of the tiles itself and works through a list in shared memory
    const int G = nblk / n_cblk, g = bid / n_cblk;
    own_scan(p.head.in_bits, p.head.Hin, p.head.Win, p.head.Hout, p.head.Wout, p.head.k, p.head.stride, p.head.pad, p.head.union_bits,
             (bid % n_cblk == 0 && crank == 0u) ? p.head.out_bits : nullptr, s_own, g < G ? g : 0x3fffffff, G, ntiles_total, !own_multi);
    lst = s_own.list;
    n_active = s_own.n_active;
    item0 = bid % n_cblk;
    item_step = n_cblk;
    if (n_active > 0) pre0 = lst[0];
    if (n_active > 1) pre1 = lst[1];
  } else {
    // the producer asks for the tile-list entries of its first item together with the device-side count, before the
    // count is known: one round trip to memory instead of two on the path count -> list -> first operand load
    if (warp == 0) {
      const int e = 2 * (bid / n_cblk);
      if (e < p.max_tiles) pre0 = p.list[e];
      if (e + 1 < p.max_tiles) pre1 = p.list[e + 1];
    }
    n_active = head_ok ? min(p.counts[0], p.max_tiles) : 0;
  }
  if (tid == 0) TC_TRACE(2);

  if (tid == 0) TC_TRACE(3);

  const int n_pairs = (n_active + 1) >> 1;
  const int n_items = n_pairs * n_cblk;
  const int n_chunks = p.cin_pad >> 5;
  const int ch_lo = (int)crank * (n_chunks / (int)CS), ch_hi = ch_lo + n_chunks / (int)CS;
  const int taps = p.k * p.k;
  const unsigned b_base = smem_u32(smem);
  const unsigned a_base = b_base + (unsigned)p.stages * st_bytes;
  const unsigned part_base = a_base + 2u * a_buf_bytes;   // K-split: [source CTA][16-column group][4 channel quads][128 rows] float4

  if (warp == 0) {
    // =========================== halo producer: lane = 2 * halo row + tile ===========================
    const int hy = lane >> 1, slot = lane & 1;
    unsigned uses = 0;
    for (int item = item0; item < n_items && !p.withhold_loads; item += item_step) {
      const int pair = item / n_cblk;
      const bool first = item == item0;
      int t0 = first ? pre0 : lst[2 * pair];
      int t1 = (2 * pair + 1 < n_active) ? (first ? pre1 : lst[2 * pair + 1]) : -1;
      // An entry outside the field is reported and skipped: the epilogue ignores it too, its half of the operand is
      // filled from tile 0 (any in-range load) or left out, and the partner tile of the pair is computed as usual.
      const bool bad0 = t0 < 0 || t0 >= ntiles_total, bad1 = (2 * pair + 1 < n_active) && (t1 < 0 || t1 >= ntiles_total);
      if ((bad0 || bad1) && lane == 0) atomicOr(&p.counts[3], MIE_ERR_BAD_TILE);
      if (bad0) t0 = 0;
      if (bad1) t1 = -1;
      const int t = slot ? t1 : t0;
      const int x0 = (t >= 0) ? (t % TWo) * 8 - p.pad : 0, y0 = (t >= 0) ? ((t / TWo) % THo) * 8 - p.pad : 0, n0 = (t >= 0) ? t / (TWo * THo) : 0;
      const unsigned tx_bytes = (t1 >= 0 ? 2u : 1u) * (unsigned)Hh * row_bytes;
      bool ok = true;
      if (lane == 0 && item == item0) TC_TRACE_V(4, clock64() + (t0 & 0));
      for (int chunk = ch_lo; chunk < ch_hi; ++chunk, ++uses) {
        const unsigned buf = uses & 1u;
        if (lane == 0) {
          if (uses >= 2) ok = mbar_wait(&a_empty[buf], ((uses >> 1) - 1) & 1u, &s_abort, p.spin_limit);
          if (ok) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&a_full[buf])), "r"(tx_bytes) : "memory");
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (hy < Hh && t >= 0)
          tma_load_5d_raw(a_base + buf * a_buf_bytes + (unsigned)lane * row_bytes, &map_in, smem_u32(&a_full[buf]), 0, x0, chunk * 8, y0 + hy, n0);
        if (lane == 0 && uses == 0) TC_TRACE(5);
      }
      if (!ok || s_abort) break;
    }
  } else if (warp == 1) {
    // =========================== filter producer ===========================
    if (lane == 0) {
      unsigned s = 0, wait_parity = 0, stage_addr = b_base, gs = 0;   // gs: running stage number; issuer gs % NI takes it
      bool first_pass = true, ok = true;
      for (int item = item0; item < n_items && ok && !s_abort && !p.withhold_loads; item += item_step) {
        const int cbn = (item % n_cblk) * NB;
        for (int chunk = ch_lo; chunk < ch_hi && ok; ++chunk) {
          for (int tap = 0; tap < taps; tap += p.tps) {
            if (!first_pass && !mbar_wait(&b_empty[s], wait_parity, &s_abort, p.spin_limit)) { ok = false; break; }
            const unsigned bar = smem_u32(&b_full[NI == 2u ? (gs & 1u) : 0u][s]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(st_bytes) : "memory");
            tma_load_4d_raw(stage_addr, &map_w, bar, 0, cbn, chunk, tap);
            if (first_pass && s == 0) TC_TRACE(6);
            stage_addr += st_bytes;
            ++gs;
            if (++s == (unsigned)p.stages) { s = 0; stage_addr = b_base; if (!first_pass) wait_parity ^= 1u; first_pass = false; }
          }
        }
      }
    }
  } else if (warp == 2 || warp == 3) {
    // =========================== MMA issuers ===========================
    const unsigned me = (unsigned)warp - 2u;
    if (lane == 0 && me < NI) {
      const unsigned idesc = make_idesc_tf32(NB);
      const unsigned long long b_hi = make_smem_desc(0) & 0xFFFFFFFF00000000ull;
      const unsigned b_lo_flags = (unsigned)(make_smem_desc(0) & 0xFFFF0000ull);
      const unsigned long long a_tmpl = make_smem_desc_plain(0, (unsigned)Wh * 16u, row_bytes);
      const unsigned long long a_hi = a_tmpl & 0xFFFFFFFF00000000ull;
      const unsigned a_lo_flags = (unsigned)(a_tmpl & 0xFFFF0000ull);
      const unsigned long long a_step = 2ull * (unsigned)Wh;     // two channel groups (K = 8) in 16-byte units
      const unsigned spc = (unsigned)(taps / p.tps);              // stages per channel chunk
      const unsigned nst = (unsigned)p.stages;
      const unsigned period = (NI == 2u && (nst & 1u)) ? 2u * nst : nst;
      unsigned g = 0;                                             // running stage number (all items of this block)
      unsigned item_idx = 0, uses = 0;
      bool ok = true;
      for (int item = item0; item < n_items && ok && !s_abort; item += item_step, ++item_idx) {
        const unsigned buf = item_idx & 1u;
        if (item_idx >= 2 && !mbar_wait(&acc_empty[buf], ((item_idx >> 1) - 1) & 1u, &s_abort, p.spin_limit)) break;
        tc_fence_after();
        const unsigned tmem_d = tmem_base + (buf * NI + me) * acc_cols;
        unsigned accumulate = 0;
        for (int chunk = ch_lo; chunk < ch_hi && ok; ++chunk, ++uses, g += spc) {
          const unsigned abuf = uses & 1u;
          if (!mbar_wait(&a_full[abuf], (uses >> 1) & 1u, &s_abort, p.spin_limit)) { ok = false; break; }
          if (me == 0 && uses == 0) TC_TRACE(7);
          const unsigned halo = a_base + abuf * a_buf_bytes;
          const unsigned nks = (unsigned)min(4, (p.cin - chunk * 32 + 7) >> 3);   // K-slices holding real channels
          bool issued = false;
          for (unsigned st = (NI == 2u) ? ((me - g) & 1u) : 0u; st < spc; st += NI) {
            const unsigned gs = g + st, lap = gs / nst, slot = gs - lap * nst;
            // the u-th stage this issuer takes from this slot: the pair (issuer, slot) recurs every lcm(ring, issuers) stages
            const unsigned use = gs / period;
            if (!mbar_wait(&b_full[me][slot], use & 1u, &s_abort, p.spin_limit)) { ok = false; break; }
            if (me == 0 && gs == 0) TC_TRACE(8);
            tc_fence_after();
            const unsigned t0 = st * (unsigned)p.tps;
            unsigned ky = t0 / (unsigned)p.k, kx = t0 - ky * (unsigned)p.k;
            unsigned row_addr = halo + ky * 2u * row_bytes, tap_addr = row_addr + kx * 16u;
            unsigned b_addr = b_base + slot * st_bytes;
            for (int j = 0; j < p.tps; ++j, b_addr += b_bytes) {
              const unsigned a_lo = a_lo_flags | ((tap_addr & 0x3FFFFu) >> 4);
              const unsigned b_lo = b_lo_flags | ((b_addr & 0x3FFFFu) >> 4);
              umma_tf32_step(tmem_d, a_hi | a_lo, b_hi | b_lo, idesc, accumulate, a_step, nks);
              accumulate = 1u;
              tap_addr += 16u;
              if (++kx == (unsigned)p.k) { kx = 0; row_addr += 2u * row_bytes; tap_addr = row_addr; }
            }
            umma_commit(&b_empty[slot]);
            issued = true;
          }
          if (!ok) break;
          // the halo buffer is free once the MMAs of both issuers have read it
          if (issued) umma_commit(&a_empty[abuf]);
          else mbar_arrive(&a_empty[abuf]);
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);
        if (me == 0 && item_idx == 0) TC_TRACE(9);
      }
    }
  } else {
    // =========================== epilogue (warps 4..11) ===========================
    const int q = warp & 3;
    const int half = (warp - 4) >> 2;                  // which half of the block's channels this warp stores
    // the two warps of a pair split the block's channels in halves of at least one 16-channel group (the unit of the
    // epilogue and of a thresholded layer's send decision); narrower blocks leave the pixel to the first warp
    const bool whole = NB < 32;
    const int c_lo = whole ? (half ? NB : 0) : half * (NB >> 1);
    const int c_hi = whole ? NB : c_lo + (NB >> 1);
    const int m = q * 32 + lane;                       // accumulator row
    const int slot = (m >> 3) & 1, pxi = ((m >> 4) << 3) | (m & 7);
    if constexpr (OWN) { if (bid % n_cblk == 0 && crank == 0u) tc_zero_stale_own(p, s_own, THo, TWo, tid - 128, HALO_THREADS - 128); }
    else if (head_ok) tc_zero_stale(p, ntiles_total, THo, TWo, tid - 128, HALO_THREADS - 128);
    unsigned item_idx = 0;
    for (int item = item0; item < n_items; item += item_step, ++item_idx) {
      const int pair = item / n_cblk, cb = item - pair * n_cblk;
      const int li = 2 * pair + slot;
      int t = (li < n_active) ? lst[li] : -1;
      if (t < 0 || t >= ntiles_total) t = -1;
      const unsigned buf = item_idx & 1u;
      const int tx = (t >= 0) ? t % TWo : 0, ty = (t >= 0) ? (t / TWo) % THo : 0, n = (t >= 0) ? t / (TWo * THo) : 0;
      const int oy = ty * 8 + (pxi >> 3), ox = tx * 8 + (pxi & 7);
      const bool valid = (t >= 0) && oy < p.hout && ox < p.wout;
      const int64_t pix = (int64_t)(n * p.hout + oy) * p.wout + ox;
      const unsigned taddr = tmem_base + buf * NI * acc_cols + ((unsigned)(q * 32) << 16);
      const unsigned acc2 = NI == 2u ? acc_cols : 0u;
      bool sent;
      if (KSPLIT) {
        // ---- K-split: exchange partial sums with the other blocks of the cluster, finish this block's column slice
        if (valid) tc_epilogue_prefetch(p, pix, cb * NB + (int)crank * (NB / (int)CS), 0, NB / (int)CS);
        if (!mbar_wait(&acc_full[buf], (item_idx >> 1) & 1u, &s_abort, p.spin_limit)) break;
        if (tid == 128 && item_idx == 0) TC_TRACE(10);
        tc_fence_after();
        if (!ksplit_finish(p, NB, CS, crank, taddr, acc2, part_base, smem + (size_t)p.stages * st_bytes + 2u * a_buf_bytes,
                           &part_full, item_idx & 1u, m, lane, half, 2, valid, pix, cb * NB, &s_abort, p.spin_limit, &sent))
          break;
        if (tid == 128 && item_idx == 0) TC_TRACE(3);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      } else {
      if (valid) tc_epilogue_prefetch(p, pix, cb * NB, c_lo, c_hi);
      if (!mbar_wait(&acc_full[buf], (item_idx >> 1) & 1u, &s_abort, p.spin_limit)) break;
      if (tid == 128 && item_idx == 0) TC_TRACE(10);
      tc_fence_after();
      // (the coalesced epilogue of the per-tap kernel measured slower here: with eight epilogue warps and the MMAs of
      // the next item running, the staging round trip costs more than the scattered accesses)
      sent = tc_epilogue_pixel(p, NB, taddr, valid, pix, cb * NB, &acc_empty[buf], lane, acc2, c_lo, c_hi);
      }
      if (tid == 128 && item_idx == 0) TC_TRACE(11);
      // ballot bytes: [tile 0 row 2q][tile 1 row 2q][tile 0 row 2q+1][tile 1 row 2q+1]
      const unsigned bal = __ballot_sync(0xffffffffu, sent);
      if ((lane == 0 || lane == 8) && t >= 0) {
        const unsigned sh = lane;                      // 0 for tile 0, 8 for tile 1
        const unsigned rows = ((bal >> sh) & 0xFFu) | (((bal >> (16 + sh)) & 0xFFu) << 8);
        if (own_multi) own_contribute(p, t, q >> 1, rows << ((q & 1) * 16), n_cblk * (int)CS * 8);
        else if (rows) atomicOr(p.out_bits32 + 2 * (size_t)t + (q >> 1), rows << ((q & 1) * 16));
      }
    }
  }

  // ---- teardown ----
  // the single-lane roles leave 31 lanes of their warp idle: reconverge before the block-wide barrier, which
  // every warp must reach as a whole
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  // K-split: no CTA leaves while another one of its cluster may still store into its shared memory or arrive on its
  // barrier (every wait above is bounded, so every CTA gets here).  A cluster without an item exchanges nothing; all
  // of its CTAs see the same item count, so they skip the barrier together.
  if (CS > 1u && item0 < n_items) cluster_sync_all();
  if (s_abort) {
    if (tid == 0) atomicOr(&p.counts[3], MIE_ERR_WAIT_EXPIRED);
    if (warp == 0) { const long long t0 = clock64(); while (clock64() - t0 < 2000000) { } }
    __syncthreads();
  }
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
  if (tid == 0) { TC_TRACE(12); TC_TRACE_G(15); TC_TRACE_V(13, (long long)n_items); }
  run_tail_job(p.tail);
}

// COALESCED: the epilogue variant (and its 8 KB of staging buffers) is a compile-time choice, so that the wide-block
// instantiation carries neither the code nor the shared memory of the other.
// KSPLIT: cluster variant (see ksplit_finish), a separate instantiation of the direct-epilogue kernel.
template <bool COALESCED, bool KSPLIT, bool OWN>
__global__ void __launch_bounds__(TC_THREADS, COALESCED ? 3 : 2)
conv_tc_kernel(const TcParams p, const __grid_constant__ TcMaps maps) {
  static_assert(!(COALESCED && KSPLIT), "the cluster variant uses the direct epilogue");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // 1024-byte alignment of every stage is what the 128-byte swizzle of TMA and of the MMA descriptors assume
  unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int NB = p.nb;
  const int stage_bytes = A_STAGE_BYTES + NB * 128;
  __shared__ unsigned long long full_bar[8], empty_bar[8], acc_full[2], acc_empty[2];
  __shared__ unsigned long long part_full;   // K-split: every other block of the cluster has delivered its partial sums
  __shared__ OwnSharedT<OWN> s_own;          // own-tiles mode: this block's tile list (a stub in the list-mode kernels)
  __shared__ float4 s_epi[COALESCED ? 4 : 1][COALESCED ? 128 : 1];   // staging buffers of the coalesced epilogue, one per epilogue warp
  __shared__ unsigned s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // K-split: `bid` / `nblk` index clusters; a cluster has at most one item (the host sizes the grid so)
  const unsigned CS = KSPLIT ? (unsigned)p.ksplit : 1u;
  const unsigned crank = CS > 1u ? cluster_ctarank() : 0u;
  const int bid = (int)(blockIdx.x / CS), nblk = (int)(gridDim.x / CS);
  if (tid == 0) { TC_TRACE(0); TC_TRACE_G(14); }
  if (tid == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(&maps.in[0])) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<unsigned long long>(&maps.w)) : "memory");
  }
  const int THo = (p.hout + 7) >> 3, TWo = (p.wout + 7) >> 3;
  const int ntiles_total = p.n * THo * TWo;
  unsigned acc_cols = 32;            // columns of one accumulator (power of two >= NB)
  while ((int)acc_cols < NB) acc_cols <<= 1;
  const unsigned tmem_cols = 2 * acc_cols;  // two accumulators: the epilogue of one item overlaps the MMAs of the next

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
    mbar_init(&part_full, CS > 1u ? (CS - 1u) * 4u : 1u);   // one arrival per epilogue warp of every other block
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = s_tmem_base;
  if (CS > 1u) cluster_sync_all();   // no block may receive a remote arrival before its barriers exist

  // everything above touched no global memory: it may overlap the tail of the previous kernel in the stream
  if (tid == 0) TC_TRACE(1);
  grid_dependency_wait();
  grid_dependency_trigger();
  constexpr bool own = OWN;
  bool head_ok = true;
  if constexpr (!OWN) {
    head_ok = run_head_job(p.head, p.spin_limit);   // block 0 makes the tile lists, the others wait for them
    if (tid == (int)blockDim.x - 1) count_head_job_passed(p.head);   // a lane of the last epilogue warp: off the critical path
  }
  const int n_cblk = p.cout_pad / NB;
  // work items of this block: item0, item0 + item_step, ... < n_items; item -> (tile pair, column block); tiles from `lst`
  int item0 = bid, item_step = nblk, n_active;
  const int32_t *lst = p.list;
  const bool own_multi = own && n_cblk * (int)CS > 1;   // several blocks finish a tile: its word goes through the scratch
  int pre0 = -1, pre1 = -1;
  if constexpr (OWN) {
    // own-tiles mode: this block's group tests its share of the tiles itself and works through a list in shared memory
    const int G = nblk / n_cblk, g = bid / n_cblk;
    own_scan(p.head.in_bits, p.head.Hin, p.head.Win, p.head.Hout, p.head.Wout, p.head.k, p.head.stride, p.head.pad, p.head.union_bits,
             (bid % n_cblk == 0 && crank == 0u) ? p.head.out_bits : nullptr, s_own, g < G ? g : 0x3fffffff, G, ntiles_total, !own_multi);
    lst = s_own.list;
    n_active = s_own.n_active;
    item0 = bid % n_cblk;
    item_step = n_cblk;
    if (n_active > 0) pre0 = lst[0];
    if (n_active > 1) pre1 = lst[1];
  } else {
    // the producer asks for the tile-list entries of its first item together with the device-side count, before the
    // count is known: one round trip to memory instead of two on the path count -> list -> first operand load
    if (warp == 0) {
      const int e = 2 * (bid / n_cblk);
      if (e < p.max_tiles) pre0 = p.list[e];
      if (e + 1 < p.max_tiles) pre1 = p.list[e + 1];
    }
    n_active = head_ok ? min(p.counts[0], p.max_tiles) : 0;
  }
  if (tid == 0) TC_TRACE(2);

  if (tid == 0) TC_TRACE(3);

  const int n_pairs = (n_active + 1) >> 1;
  const int n_items = n_pairs * n_cblk;
  const int n_chunks = p.cin_pad >> 5;
  const int ch_lo = (int)crank * (n_chunks / (int)CS), ch_hi = ch_lo + n_chunks / (int)CS;   // this block's chunks
  const int taps = p.k * p.k;

  if (warp == 0) {
    // =========================== TMA producer ===========================
    // One thread issues every copy, so its scalar instructions are on the critical path: stage index, phase,
    // stage address and tap coordinates are running counters -- no division, no 64-bit multiply in the loop.
    if (lane == 0) {
      unsigned s = 0, wait_parity = 0;     // parity of the "stage is free" phase this pass around the ring waits for
      bool first_pass = true;
      const unsigned smem_base = smem_u32(smem);
      unsigned stage_addr = smem_base;
      const unsigned b_bytes = (unsigned)NB * 128u;
      for (int item = item0; item < n_items && !s_abort && !p.withhold_loads; item += item_step) {
        const int pair = item / n_cblk, cb = item - pair * n_cblk;
        const bool first = item == item0;
        int t0 = first ? pre0 : lst[2 * pair];
        int t1 = (2 * pair + 1 < n_active) ? (first ? pre1 : lst[2 * pair + 1]) : -1;
        // an entry outside the field is reported and skipped (see the halo kernel's producer)
        const bool bad0 = t0 < 0 || t0 >= ntiles_total, bad1 = (2 * pair + 1 < n_active) && (t1 < 0 || t1 >= ntiles_total);
        if (bad0 || bad1) atomicOr(&p.counts[3], MIE_ERR_BAD_TILE);
        if (bad0) t0 = 0;
        if (bad1) t1 = -1;
        const int x0 = (t0 % TWo) * 8, y0 = ((t0 / TWo) % THo) * 8, n0 = t0 / (TWo * THo);
        const int x1 = (t1 >= 0) ? (t1 % TWo) * 8 : 0, y1 = (t1 >= 0) ? ((t1 / TWo) % THo) * 8 : 0, n1 = (t1 >= 0) ? t1 / (TWo * THo) : 0;
        const unsigned tx_bytes = (t1 >= 0 ? A_STAGE_BYTES : A_STAGE_BYTES / 2) + b_bytes;
        const int cbn = cb * NB;
        if (item == item0) { TC_TRACE_V(4, clock64() + (t0 & 0)); }
        bool ok = true;
        for (int chunk = ch_lo; chunk < ch_hi && ok; ++chunk) {
          const int c0 = chunk * 32;
          int tap = 0;
          for (int ky = 0; ky < p.k && ok; ++ky) {
            int dy = ky - p.pad, pyb = 0;
            if (p.stride == 2) { pyb = (dy & 1) * 2; dy = (dy - (dy & 1)) >> 1; }
            for (int kx = 0; kx < p.k; ++kx, ++tap) {
              if (!first_pass && !mbar_wait(&empty_bar[s], wait_parity, &s_abort, p.spin_limit)) { ok = false; break; }
              int dx = kx - p.pad, mi = 0;
              if (p.stride == 2) { mi = pyb + (dx & 1); dx = (dx - (dx & 1)) >> 1; }
              const unsigned bar = smem_u32(&full_bar[s]);
              asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tx_bytes) : "memory");
              tma_load_4d_raw(stage_addr, &maps.in[mi], bar, c0, x0 + dx, y0 + dy, n0);
              if (t1 >= 0) tma_load_4d_raw(stage_addr + A_STAGE_BYTES / 2, &maps.in[mi], bar, c0, x1 + dx, y1 + dy, n1);
              tma_load_4d_raw(stage_addr + A_STAGE_BYTES, &maps.w, bar, 0, cbn, chunk, tap);
              stage_addr += (unsigned)stage_bytes;
              if (++s == (unsigned)p.stages) { s = 0; stage_addr = smem_base; if (!first_pass) wait_parity ^= 1u; if (first_pass) TC_TRACE(5); first_pass = false; }
            }
          }
        }
        if (item == item0) TC_TRACE(6);
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    // Same care as the producer: a lean loop issues an MMA every ~70 cycles, one that rebuilds descriptors and
    // divides by the stage count needs ~250.  Descriptors are pre-built; a stage only adds its address.
    if (lane == 0) {
      const unsigned idesc = make_idesc_tf32(NB);
      const unsigned smem_base = smem_u32(smem);
      const unsigned long long desc_hi = make_smem_desc(0) & 0xFFFFFFFF00000000ull;   // stride, version, swizzle
      const unsigned desc_lo_flags = (unsigned)(make_smem_desc(0) & 0xFFFF0000ull);     // leading-offset field
      unsigned s = 0, parity = 0, stage_addr = smem_base, item_idx = 0;
      const int k_iters = (ch_hi - ch_lo) * taps;
      for (int item = item0; item < n_items && !s_abort; item += item_step, ++item_idx) {
        // the epilogue must have drained this accumulator (used two items ago)
        const unsigned buf = item_idx & 1u;
        if (item_idx >= 2 && !mbar_wait(&acc_empty[buf], ((item_idx >> 1) - 1) & 1u, &s_abort, p.spin_limit)) break;
        tc_fence_after();
        const unsigned tmem_d = tmem_base + buf * acc_cols;
        bool ok = true;
        unsigned accumulate = 0;
        for (int ki = 0; ki < k_iters; ++ki) {
          if (!mbar_wait(&full_bar[s], parity, &s_abort, p.spin_limit)) { ok = false; break; }
          if (ki == 0 && item_idx == 0) TC_TRACE(7);
          tc_fence_after();
          const unsigned a_lo = desc_lo_flags | ((stage_addr & 0x3FFFFu) >> 4);
          const unsigned b_lo = desc_lo_flags | (((stage_addr + A_STAGE_BYTES) & 0x3FFFFu) >> 4);
          // 4 x (K = 8 tf32 = 32 bytes = 2 descriptor units) inside the 128-byte swizzled row
          umma_tf32_x4(tmem_d, desc_hi | a_lo, desc_hi | b_lo, idesc, accumulate);
          accumulate = 1u;
          umma_commit(&empty_bar[s]);  // arrives once the MMAs above have finished reading the stage
          stage_addr += (unsigned)stage_bytes;
          if (++s == (unsigned)p.stages) { s = 0; stage_addr = smem_base; parity ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&acc_full[buf]);
        if (item_idx == 0) TC_TRACE(8);
      }
    }
  } else {
    // =========================== epilogue (warps 2..5) ===========================
    // (a second set of four epilogue warps, as in the halo kernel, measured slower here: this kernel's small
    // layers gain more from a third resident block per SM than from a shorter epilogue)
    const int q = warp & 3;           // tensor-memory lane group this warp may read: lanes 32q .. 32q+31
    const int m = q * 32 + lane;      // accumulator row = pixel of the pair
    const int slot = m >> 6, pxi = m & 63;
    if constexpr (OWN) { if (bid % n_cblk == 0 && crank == 0u) tc_zero_stale_own(p, s_own, THo, TWo, tid - 64, TC_THREADS - 64); }
    else if (head_ok) tc_zero_stale(p, ntiles_total, THo, TWo, tid - 64, TC_THREADS - 64);
    unsigned item_idx = 0;
    for (int item = item0; item < n_items; item += item_step, ++item_idx) {
      const int pair = item / n_cblk, cb = item - pair * n_cblk;
      const int li = 2 * pair + slot;
      int t = (li < n_active) ? lst[li] : -1;
      if (t < 0 || t >= ntiles_total) t = -1;
      const unsigned buf = item_idx & 1u;
      const int tx = (t >= 0) ? t % TWo : 0, ty = (t >= 0) ? (t / TWo) % THo : 0, n = (t >= 0) ? t / (TWo * THo) : 0;
      const int oy = ty * 8 + (pxi >> 3), ox = tx * 8 + (pxi & 7);
      const bool valid = (t >= 0) && oy < p.hout && ox < p.wout;
      const int64_t pix = (int64_t)(n * p.hout + oy) * p.wout + ox;
      if (valid) {
        if (KSPLIT) tc_epilogue_prefetch(p, pix, cb * NB + (int)crank * (NB / (int)CS), 0, NB / (int)CS);
        else tc_epilogue_prefetch(p, pix, cb * NB, 0, NB);
      }
      if (tid == 64 && item_idx == 0) TC_TRACE_V(9, clock64() + (t & 0));
      if (!mbar_wait(&acc_full[buf], (item_idx >> 1) & 1u, &s_abort, p.spin_limit)) break;
      if (tid == 64 && item_idx == 0) TC_TRACE(10);
      tc_fence_after();
      const unsigned taddr = tmem_base + buf * acc_cols + ((unsigned)(q * 32) << 16);
      bool sent;
      if (KSPLIT) {
        if (!ksplit_finish(p, NB, CS, crank, taddr, 0u, smem_u32(smem) + (unsigned)(p.stages * stage_bytes),
                           smem + (size_t)p.stages * stage_bytes, &part_full, item_idx & 1u, m, lane, 0, 1, valid, pix, cb * NB,
                           &s_abort, p.spin_limit, &sent))
          break;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
      } else {
        sent = COALESCED ? tc_epilogue_pixel_coalesced(p, NB, taddr, valid, pix, cb * NB, &acc_empty[buf], lane, s_epi[COALESCED ? warp - 2 : 0], 0u, 0, NB)
                         : tc_epilogue_pixel(p, NB, taddr, valid, pix, cb * NB, &acc_empty[buf], lane);
      }
      if (tid == 64 && item_idx == 0) TC_TRACE(11);
      const unsigned sent_bits = __ballot_sync(0xffffffffu, sent);
      if (lane == 0 && t >= 0) {
        // two epilogue warps share a tile (32 pixels each)
        if (own_multi) own_contribute(p, t, q & 1, sent_bits, n_cblk * (int)CS * 2);
        else if (sent_bits) atomicOr(p.out_bits32 + 2 * (size_t)t + (q & 1), sent_bits);
      }
    }
  }

  // ---- teardown ------------------------------------------------------------------------------------
  __syncwarp();  // single-lane roles: the whole warp reaches the block-wide barrier together
  tc_fence_before();
  __syncthreads();
  if (CS > 1u && item0 < n_items) cluster_sync_all();   // K-split: no block leaves while another may still store into its shared memory
  if (s_abort) {
    if (tid == 0) atomicOr(&p.counts[3], MIE_ERR_WAIT_EXPIRED);
    // give copies that may still be in flight time to land before shared memory is released
    if (warp == 0) { const long long t0 = clock64(); while (clock64() - t0 < 2000000) { } }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
  if (tid == 0) { TC_TRACE(12); TC_TRACE_G(15); TC_TRACE_V(13, (long long)n_items); }
  run_tail_job(p.tail);
}



typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void *ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) {
    if (e != cudaSuccess) set_cuda_error(e);
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

// Tensor maps are a pure function of their arguments, and a layer asks for the same ones every step: the encoded
// descriptors are remembered (per host thread, direct-mapped, 256 entries), so only the first launch of a layer at a
// given geometry and buffer set pays the driver's encoding call.
struct MapKey {
  const void *base;
  int rank, swizzle;
  cuuint64_t dims[5], strides[4];
  cuuint32_t box[5];
};
struct MapSlot {
  bool used;
  MapKey key;
  CUtensorMap map;
};

bool encode(EncodeTiledFn fn, CUtensorMap *m, int rank, const void *base, const cuuint64_t *dims, const cuuint64_t *strides_bytes,
            const cuuint32_t *box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  static thread_local MapSlot cache[256];
  MapKey k;
  memset(&k, 0, sizeof(k));
  k.base = base; k.rank = rank; k.swizzle = (int)swizzle;
  for (int i = 0; i < rank; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) k.strides[i] = strides_bytes[i];
  unsigned long long h = 1469598103934665603ull;
  const unsigned char *kb = reinterpret_cast<const unsigned char *>(&k);
  for (size_t i = 0; i < sizeof(k); ++i) h = (h ^ kb[i]) * 1099511628211ull;
  MapSlot &slot = cache[(h ^ (h >> 32)) & 255u];
  if (slot.used && memcmp(&slot.key, &k, sizeof(k)) == 0) {
    *m = slot.map;
    return true;
  }
  cuuint32_t es[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void *>(base), dims, strides_bytes, box, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  slot.used = true;
  slot.key = k;
  slot.map = *m;
  return true;
}

// Process-wide options of the tensor-core path (mie_set_option / mie_get_option).
int g_opt_tc_thresholded = 1;               // MIE_OPT_TC_THRESHOLDED
unsigned g_opt_spin_limit = SPIN_LIMIT;     // MIE_OPT_TC_SPIN_LIMIT
int g_opt_withhold_loads = 0;               // MIE_OPT_TC_WITHHOLD_LOADS
int g_opt_ksplit = 1;                       // MIE_OPT_TC_KSPLIT
int g_opt_own_kernels = 7;                  // MIE_OPT_TC_OWN_KERNELS

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute of a kernel: the largest value set so far is
// remembered per device, so a process that drives several GPUs raises the limit on each of them.
constexpr int MAX_DEVICES = 64;
template <typename Kernel>
int ensure_dynamic_smem(Kernel kernel, int *set_per_device, size_t smem) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
  if (dev < 0 || dev >= MAX_DEVICES) return MIE_EUNSUPPORTED;
  if ((int)smem > set_per_device[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_cuda_error(e); return MIE_ECUDA; }
    set_per_device[dev] = (int)smem;
  }
  return MIE_OK;
}

// Shared memory the halo kernel's operands may take (KB) and the largest filter ring (slots); MIE_TC_RING_KB /
// MIE_TC_RING_CAP in the environment override them for A/B measurements.
int halo_ring_kb() {
  static const int v = []() { const char *e = getenv("MIE_TC_RING_KB"); const int x = e ? atoi(e) : 0; return (x >= 128 && x <= 224) ? x : 200; }();
  return v;
}
int halo_ring_cap() {
  static const int v = []() { const char *e = getenv("MIE_TC_RING_CAP"); const int x = e ? atoi(e) : 0; return (x >= 2 && x <= HALO_MAX_STAGES) ? x : 4; }();
  return v;
}

// MIE_TC_HALO=0 in the environment keeps every layer on the per-tap kernel (for A/B measurements).
bool halo_enabled() {
  static const bool on = []() { const char *e = getenv("MIE_TC_HALO"); return !(e && e[0] == '0'); }();
  return on;
}

}  // namespace

// Whether the tensor-core path can take this convolution (host-side rules only).
bool tc_eligible(const mie_conv_args *a) {
  if (a->in2 || a->accum) return false;   // the 1x1 head kernel's extras
  if (!a->wpacked_tc) return false;
  if (a->refresh || a->bias) return false;   // dense evaluation (full fp32, bias, reservoir set) is the FP32 kernel's
  if (!(a->stride == 1 || a->stride == 2)) return false;
  if (a->k != 1 && a->k != 3 && a->k != 5 && a->k != 7) return false;
  if (a->in_ps % 4 || !aligned16(a->in)) return false;                           // TMA: 16-byte strides and base
  const bool halo_shape = a->stride == 1 && a->k >= 3 && a->k <= 7;
  // a channel count that is no multiple of 4 is taken when the pixel stride covers the rounded-up count: the
  // padding channels are read and meet zero filter entries (the same contract as the FP32 path's vector loads)
  if (a->cin % 4 && !(halo_shape && a->in_ps >= (a->cin + 3) / 4 * 4)) return false;
  if (a->cout % 4 || a->out_ps % 4 || !aligned16(a->out)) return false;          // float4 epilogue
  if (a->res && (a->res_ps % 4 || !aligned16(a->res))) return false;
  if (a->emitted && (a->emitted_ps % 4 || !aligned16(a->emitted))) return false;
  if (a->addend && (a->addend_ps % 4 || !aligned16(a->addend))) return false;
  if (a->cout_pad % 16) return false;
  if (a->thr > 0.0f || a->emitted) {
    // Thresholded layers (groups of 16 channels of a pixel are sent or withheld, optionally with a carry buffer) run
    // on the FP32 kernel unless MIE_OPT_TC_THRESHOLDED is set.  The epilogue works in 16-channel groups, which are the
    // decision unit, so any block width takes part.
    if (!g_opt_tc_thresholded) return false;
  }
  // Too shallow to pay off.  (The 5x5 head of E2Depth, 5 -> 32 channels, would run 3x faster here than on the
  // FP32 path, but it sees the raw input delta: truncating O(1) values to TF32 every step random-walks in the
  // first reservoir and measured 1.1e-3 of the output range against 1.3e-5 with the head in FP32.)
  if ((int64_t)a->cin * a->k * a->k < 256) return false;
  if (a->stride == 2 && ((a->hin & 1) || (a->win & 1))) return false;            // parity views need even extents
  return true;
}

// Channels per block and cluster size of a tensor-core convolution (host-side rules only).
static void tc_block_shape(const mie_conv_args *a, int *nb_out, int *ksplit_out) {
  const int cin_pad32 = (a->cin + 31) / 32 * 32;
  // channels per block: as wide as fits 256 accumulator columns; narrowed (down to 32) only while the layer
  // could not keep about half of the SMs busy even at full activity -- the small-image layers of a UNet have
  // a few dozen tiles but thousands of reduction steps.  Measured on B200: a pipeline stage costs about
  // 0.6 us whatever its width, so narrowing pays only until the work items cover the machine once.
  // MIE_TC_NB_MAX in the environment caps the block width (A/B measurements)
  static const int nb_max = []() { const char *e = getenv("MIE_TC_NB_MAX"); const int x = e ? atoi(e) : 0; return (x == 32 || x == 64 || x == 128) ? x : 256; }();
  int nb = nb_max;
  while (nb > 16 && a->cout_pad % nb) nb >>= 1;
  const int64_t pairs = (a->max_tiles + 1) / 2;
  while (nb > 32 && a->cout_pad % (nb / 2) == 0 && pairs * (a->cout_pad / nb) < 64) nb >>= 1;
  // K-split: a layer with so few tile pairs that even 32-channel blocks leave each block a chain of hundreds of
  // dependent MMA stages takes wide blocks instead and spreads the input-channel chunks of every block over a cluster of
  // 2 or 4 thread blocks, which exchange their partial sums through distributed shared memory (ksplit_finish).
  // Conditions: every cluster gets at most one work item (grid = items x cluster size <= one wave), the chunks divide
  // evenly, and a block's slice of the columns is a whole number of 16-channel groups.
  int ksplit = 1;
  if (g_opt_ksplit && a->k >= 3 && a->k <= 7) {
    int nbw = 128;
    while (nbw > 32 && a->cout_pad % nbw) nbw >>= 1;
    const int n_chunks = cin_pad32 / 32;
    const int64_t items_w = pairs * (a->cout_pad / nbw);
    const bool halo = a->stride == 1 && (cin_pad32 > 32 || a->k >= 5) && halo_enabled();   // which kernel takes the layer
    const int Wh = 8 + a->k - 1;
    const int a_bytes = 2 * (Wh * 2 * 8 * Wh * 16);
    for (int cs = 4; cs >= 2 && ksplit == 1; cs >>= 1) {
      const int part_bytes = (cs - 1) * (nbw / cs) * 512;
      // the received partial sums take shared memory from the operand ring.  Halo kernel: split only while two ring
      // slots of a whole filter row each still fit (with single-tap stages the wide block measured no faster than the
      // narrow ones); per-tap kernel: three stages must fit.
      const bool fits = halo ? 2 * a->k * nbw * 128 <= 200 * 1024 - a_bytes - part_bytes
                             : 3 * (A_STAGE_BYTES + nbw * 128) + part_bytes <= 200 * 1024;
      // worth it from about 70 operand stages per item on (the per-tap kernel's stages are single taps: from 50)
      if (a->cout_pad % nbw == 0 && n_chunks % cs == 0 && n_chunks / cs >= 1 && items_w * cs <= MIE_SM_COUNT &&
          (nbw / cs) % 16 == 0 && n_chunks * a->k * a->k >= (halo ? 72 : 50) && fits)
        ksplit = cs;
    }
    if (ksplit > 1) nb = nbw;
  }
  *nb_out = nb;
  *ksplit_out = ksplit;
}

int launch_conv_tc(const mie_conv_args *a, cudaStream_t st) {
  EncodeTiledFn fn = get_encode();
  if (!fn) return MIE_ECUDA;
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.spin_limit = g_opt_spin_limit;
  p.withhold_loads = g_opt_withhold_loads;
  p.cin = a->cin; p.cout = a->cout; p.cout_pad = a->cout_pad;
  p.cin_pad = (a->cin + 31) / 32 * 32;
  p.n = a->n; p.hin = a->hin; p.win = a->win; p.hout = a->hout; p.wout = a->wout;
  p.k = a->k; p.stride = a->stride; p.pad = a->pad;
  p.list = a->list; p.stale = a->stale; p.counts = a->counts; p.max_tiles = a->max_tiles;
  p.out = a->out; p.out_ps = a->out_ps; p.out_bits32 = reinterpret_cast<unsigned int *>(a->out_bits);
  p.act = a->act; p.thr = a->thr; p.res = a->res; p.res_ps = a->res_ps;
  p.emitted = a->emitted; p.emitted_ps = a->emitted_ps; p.addend = a->addend; p.addend_ps = a->addend_ps;
  p.tail = tail_for_kernel(a->tail);
  p.head = tail_for_kernel(a->head);
  p.ksplit = 1;
  int nb, ksplit;
  tc_block_shape(a, &nb, &ksplit);
  // Own-tiles mode: the grid must consist of whole groups of n_cblk blocks (or clusters), and a group's share of the tiles
  // must fit the list in its shared memory.  own_grid() returns the grid to launch; when the mode was asked for and
  // cannot be had, it enqueues the separate dilation and the kernel reads the global lists as usual.
  int own_status = MIE_OK;
  const int own_mask = g_opt_own_kernels;   // kind: 1 per-tap, 2 per-tap as clusters, 4 halo, 8 halo as clusters
  auto own_grid = [&](int64_t grid, int kind) -> int64_t {
    if (!a->own_tiles) return grid;
    const int n_cblk = a->cout_pad / nb;
    const int64_t groups = grid / n_cblk, sp = ((int64_t)a->max_tiles + 1) / 2;
    const int64_t ntiles = (int64_t)a->n * divup(a->hout, 8) * divup(a->wout, 8);
    if ((own_mask & kind) && groups >= 1 && 2 * ((sp + groups - 1) / groups) <= OWN_MAX && a->max_tiles == ntiles) {
      p.own = 1;
      p.head = *a->head;
      p.own_words = static_cast<unsigned long long *>(a->own_scratch);
      p.own_tickets = reinterpret_cast<int *>(static_cast<char *>(a->own_scratch) + 8 * ntiles);
      return groups * n_cblk;
    }
    const mie_tail_job *h = a->head;
    own_status = mie_tiles_dilate(h->in_bits, h->N, h->Hin, h->Win, h->Hout, h->Wout, h->k, h->stride, h->pad, h->union_bits,
                                  h->out_bits, h->list, h->stale, h->counts, h->flags, st);
    p.head = mie_tail_job{};
    return grid;
  };
  p.nb = nb;
  int acc_cols = 32;
  while (acc_cols < nb) acc_cols <<= 1;
  const int64_t max_items = (int64_t)((a->max_tiles + 1) / 2) * (a->cout_pad / nb);

  // ---- halo-resident kernel: stride 1, k in {3,5,7} ----
  // Two shapes stay on the per-tap kernel: blocks of 256 channels with more work items than SMs (bound by the
  // tensor core itself, not by instruction issue: per-tap measured 15 % faster), and layers of a single channel
  // chunk with a 3x3 filter (the halo is used for 9 taps only once: per-tap measured 8 % faster on 32 -> 32 channels).
  if (a->stride == 1 && a->k >= 3 && a->k <= 7 && !(nb == 256 && max_items > MIE_SM_COUNT) && (p.cin_pad > 32 || a->k >= 5) && halo_enabled()) {
    const int Wh = 8 + a->k - 1;
    const int a_bytes = 2 * (Wh * 2 * 8 * Wh * 16);          // two buffers of [Hh][2 tiles][8 groups][Wh][16 B]
    // A stage holds `tps` consecutive taps of one channel chunk (one TMA): the issuing thread pays its wait /
    // fence / commit once per stage, so stages are made as fat as shared memory allows -- a whole filter (k*k
    // taps), else one filter row (k taps), else a single tap -- even if only two ring slots remain (measured:
    // 5-tap stages x 2 slots beat 1-tap stages x 4 slots by 25 % on a 5x5 256->128 layer).
    const int part_bytes = ksplit > 1 ? (ksplit - 1) * (nb / ksplit) * 512 : 0;   // partial sums received from the cluster
    const int budget = halo_ring_kb() * 1024 - a_bytes - part_bytes;
    int tps = 0, stages = 0;
    const int cand[3] = {a->k * a->k, a->k, 1};
    for (int i = 0; i < 3 && !tps; ++i)
      if (2 * cand[i] * nb * 128 <= budget) { tps = cand[i]; stages = budget / (cand[i] * nb * 128); if (stages > halo_ring_cap()) stages = halo_ring_cap(); }
    p.tps = tps ? tps : 1;
    const int b_bytes = p.tps * nb * 128;
    p.issuers = (2 * 2 * acc_cols <= 512 && (p.cin_pad / 32 / ksplit) * (a->k * a->k / p.tps) >= 2) ? 2 : 1;   // stages per CTA
    // (Two issuers take alternate stages; each waits on its own "full" barrier per slot, so the ring may be odd.)
    if (stages >= 2) {
      p.stages = stages;
      const size_t smem = (size_t)stages * b_bytes + a_bytes + part_bytes + 1024;
      int blocks_per_sm = (int)((220 * 1024) / (smem + 2048));
      const int by_tmem = 512 / (2 * p.issuers * acc_cols);
      if (blocks_per_sm > by_tmem) blocks_per_sm = by_tmem;
      if (blocks_per_sm > 1) blocks_per_sm = 1;   // registers: 384 threads x ~112
      if (blocks_per_sm < 1) blocks_per_sm = 1;
      CUtensorMap map_in, map_w;
      const cuuint64_t dims[5] = {4, (cuuint64_t)a->win, (cuuint64_t)((a->cin + 3) / 4), (cuuint64_t)a->hin, (cuuint64_t)a->n};
      const cuuint64_t str[4] = {(cuuint64_t)a->in_ps * 4, 16, (cuuint64_t)a->win * a->in_ps * 4, (cuuint64_t)a->hin * a->win * a->in_ps * 4};
      const cuuint32_t box[5] = {4, (cuuint32_t)Wh, 8, 1, 1};
      const cuuint64_t nch = (cuuint64_t)(p.cin_pad / 32);
      const cuuint64_t wdims[4] = {32, (cuuint64_t)a->cout_pad, nch, (cuuint64_t)(a->k * a->k)};
      const cuuint64_t wstr[3] = {128, (cuuint64_t)a->cout_pad * 128, nch * a->cout_pad * 128};
      const cuuint32_t box_w[4] = {32, (cuuint32_t)nb, 1, (cuuint32_t)p.tps};
      if (encode(fn, &map_in, 5, a->in, dims, str, box, CU_TENSOR_MAP_SWIZZLE_NONE) && encode(fn, &map_w, 4, a->wpacked_tc, wdims, wstr, box_w)) {
        const int64_t cap = (int64_t)MIE_SM_COUNT * blocks_per_sm;
        int grid = max_items < cap ? (int)max_items : (int)cap;
        if (grid < 1) grid = 1;
        grid = (int)own_grid(ksplit > 1 ? max_items : grid, ksplit > 1 ? 8 : 4);   // clusters: one per possible item, as below
        if (own_status != MIE_OK) return own_status;
        static int halo_smem_set[MAX_DEVICES] = {0};
        if (ksplit > 1) {
          static int halo_ks_smem_set[MAX_DEVICES] = {0};
          static int halo_ks_own_smem_set[MAX_DEVICES] = {0};
          p.ksplit = ksplit;
          if (p.own) {
            { const int s_ = ensure_dynamic_smem(conv_tc_halo_kernel<true, true>, halo_ks_own_smem_set, smem); if (s_ != MIE_OK) return s_; }
            launch_chained_cluster(conv_tc_halo_kernel<true, true>, dim3((unsigned)(max_items * ksplit)), dim3(HALO_THREADS), smem, st,
                                   (unsigned)ksplit, p, map_in, map_w);
            return check_launch();
          }
          { const int s_ = ensure_dynamic_smem(conv_tc_halo_kernel<true, false>, halo_ks_smem_set, smem); if (s_ != MIE_OK) return s_; }
          launch_chained_cluster(conv_tc_halo_kernel<true, false>, dim3((unsigned)(max_items * ksplit)), dim3(HALO_THREADS), smem, st,
                                 (unsigned)ksplit, p, map_in, map_w);
          return check_launch();
        }
        if (p.own) {
          static int halo_own_smem_set[MAX_DEVICES] = {0};
          { const int s_ = ensure_dynamic_smem(conv_tc_halo_kernel<false, true>, halo_own_smem_set, smem); if (s_ != MIE_OK) return s_; }
          launch_chained(conv_tc_halo_kernel<false, true>, dim3(grid), dim3(HALO_THREADS), smem, st, p, map_in, map_w);
          return check_launch();
        }
        { const int s_ = ensure_dynamic_smem(conv_tc_halo_kernel<false, false>, halo_smem_set, smem); if (s_ != MIE_OK) return s_; }
        launch_chained(conv_tc_halo_kernel<false, false>, dim3(grid), dim3(HALO_THREADS), smem, st, p, map_in, map_w);
        return check_launch();
      }
      // a tensor map the driver refuses (unusual strides): the per-tap kernel below takes the layer
    }
  }

  const int stage_bytes = A_STAGE_BYTES + nb * 128;
  // Narrow blocks (few MMAs per item: the epilogue is exposed) take the coalesced epilogue; wide blocks, whose epilogue
  // hides behind the next item's MMAs, measured faster on the direct one.
  const bool coalesced = nb <= 32 && a->thr == 0.0f && !a->emitted && (a->cout & 3) == 0 && ksplit == 1;
  const int epi_bytes = coalesced ? 8192 : 0;   // static staging buffers of the coalesced epilogue
  int stages = (200 * 1024) / stage_bytes;
  if (stages > 8) stages = 8;
  // Pipeline depth beyond 3 measured no gain (2 measured worse), while blocks of up to 128 channels are bound by the
  // latency of each work item (load -> MMA -> reservoir read-modify-write): keep them shallow so that 2-3 blocks
  // share an SM.
  // Narrow blocks may go deeper while three blocks still share an SM: a block that holds a single work item of few
  // stages (3x3, one channel chunk) then has all its loads in flight at once instead of waiting for freed slots.
  if (nb <= 128 && stages > 3) {
    const int deep = ((220 * 1024) / 3 - 3072 - epi_bytes) / stage_bytes;
    stages = deep > 3 ? (deep < stages ? deep : stages) : 3;
  }
  { // MIE_TC_TAP_STAGES in the environment forces the per-tap ring depth (A/B measurements)
    static const int forced = []() { const char *e = getenv("MIE_TC_TAP_STAGES"); const int x = e ? atoi(e) : 0; return (x >= 2 && x <= 8) ? x : 0; }();
    if (forced && forced * stage_bytes <= 200 * 1024) stages = forced;
  }
  const int part_bytes = ksplit > 1 ? (ksplit - 1) * (nb / ksplit) * 512 : 0;   // partial sums received from the cluster
  if (ksplit > 1) {
    stages = (200 * 1024 - part_bytes) / stage_bytes;
    if (stages > 4) stages = 4;
  }
  if (stages < 2) return MIE_EUNSUPPORTED;
  p.stages = stages;
  const size_t smem = (size_t)stages * stage_bytes + part_bytes + 1024;
  int blocks_per_sm = (int)((220 * 1024) / (smem + 2048 + epi_bytes));
  { const int by_tmem = 512 / (2 * acc_cols); if (blocks_per_sm > by_tmem) blocks_per_sm = by_tmem; }
  // registers: the coalesced instantiation (79) fits three blocks of 192 threads, the direct one (142) two
  if (blocks_per_sm > (coalesced ? 3 : 2)) blocks_per_sm = coalesced ? 3 : 2;
  if (blocks_per_sm < 1) blocks_per_sm = 1;

  TcMaps maps;
  memset(&maps, 0, sizeof(maps));
  const cuuint32_t box_in[4] = {32, 8, 8, 1};
  if (a->stride == 1) {
    const cuuint64_t dims[4] = {(cuuint64_t)a->cin, (cuuint64_t)a->win, (cuuint64_t)a->hin, (cuuint64_t)a->n};
    const cuuint64_t str[3] = {(cuuint64_t)a->in_ps * 4, (cuuint64_t)a->win * a->in_ps * 4, (cuuint64_t)a->hin * a->win * a->in_ps * 4};
    if (!encode(fn, &maps.in[0], 4, a->in, dims, str, box_in)) return MIE_EINVAL;
  } else {
    for (int py = 0; py < 2; ++py)
      for (int px = 0; px < 2; ++px) {
        const cuuint64_t dims[4] = {(cuuint64_t)a->cin, (cuuint64_t)((a->win - px + 1) / 2), (cuuint64_t)((a->hin - py + 1) / 2), (cuuint64_t)a->n};
        const cuuint64_t str[3] = {(cuuint64_t)a->in_ps * 8, (cuuint64_t)a->win * a->in_ps * 8, (cuuint64_t)a->hin * a->win * a->in_ps * 4};
        const float *base = a->in + ((int64_t)py * a->win + px) * a->in_ps;
        if (!encode(fn, &maps.in[py * 2 + px], 4, base, dims, str, box_in)) return MIE_EINVAL;
      }
  }
  {
    // filter stored [tap][32-channel chunk][cout_pad][32]: the box of one (tap, chunk, channel block) is contiguous
    const cuuint64_t nch = (cuuint64_t)(p.cin_pad / 32);
    const cuuint64_t dims[4] = {32, (cuuint64_t)a->cout_pad, nch, (cuuint64_t)(a->k * a->k)};
    const cuuint64_t str[3] = {128, (cuuint64_t)a->cout_pad * 128, nch * a->cout_pad * 128};
    const cuuint32_t box_w[4] = {32, (cuuint32_t)nb, 1, 1};
    if (!encode(fn, &maps.w, 4, a->wpacked_tc, dims, str, box_w)) return MIE_EINVAL;
  }
  const int64_t cap = (int64_t)MIE_SM_COUNT * blocks_per_sm;
  int grid = max_items < cap ? (int)max_items : (int)cap;
  if (grid < 1) grid = 1;
  grid = (int)own_grid(ksplit > 1 ? max_items : grid, ksplit > 1 ? 2 : 1);
  if (own_status != MIE_OK) return own_status;
  if (ksplit > 1) {
    static int ks_smem_set[MAX_DEVICES] = {0};
    static int ks_own_smem_set[MAX_DEVICES] = {0};
    p.ksplit = ksplit;
    if (p.own) {
      { const int s_ = ensure_dynamic_smem(conv_tc_kernel<false, true, true>, ks_own_smem_set, smem); if (s_ != MIE_OK) return s_; }
      launch_chained_cluster(conv_tc_kernel<false, true, true>, dim3((unsigned)(max_items * ksplit)), dim3(TC_THREADS), smem, st,
                             (unsigned)ksplit, p, maps);
      return check_launch();
    }
    { const int s_ = ensure_dynamic_smem(conv_tc_kernel<false, true, false>, ks_smem_set, smem); if (s_ != MIE_OK) return s_; }
    launch_chained_cluster(conv_tc_kernel<false, true, false>, dim3((unsigned)(max_items * ksplit)), dim3(TC_THREADS), smem, st,
                           (unsigned)ksplit, p, maps);
    return check_launch();
  }
  static int smem_set[4][MAX_DEVICES] = {{0}};
  {
    const int s_ = coalesced ? (p.own ? ensure_dynamic_smem(conv_tc_kernel<true, false, true>, smem_set[3], smem)
                                      : ensure_dynamic_smem(conv_tc_kernel<true, false, false>, smem_set[1], smem))
                             : (p.own ? ensure_dynamic_smem(conv_tc_kernel<false, false, true>, smem_set[2], smem)
                                      : ensure_dynamic_smem(conv_tc_kernel<false, false, false>, smem_set[0], smem));
    if (s_ != MIE_OK) return s_;
  }
  if (coalesced) {
    if (p.own) launch_chained(conv_tc_kernel<true, false, true>, dim3(grid), dim3(TC_THREADS), smem, st, p, maps);
    else launch_chained(conv_tc_kernel<true, false, false>, dim3(grid), dim3(TC_THREADS), smem, st, p, maps);
  } else {
    if (p.own) launch_chained(conv_tc_kernel<false, false, true>, dim3(grid), dim3(TC_THREADS), smem, st, p, maps);
    else launch_chained(conv_tc_kernel<false, false, false>, dim3(grid), dim3(TC_THREADS), smem, st, p, maps);
  }
  return check_launch();
}

}  // namespace mie

// [k*k][cin_pad/32][cout_pad][32] <- w[cout][cin][ky][kx], rounded to TF32 (round to nearest, ties away), zero padded
__global__ void pack_weights_tc_kernel(const float *__restrict__ w, int cout, int cin, int k, int cin_pad, int cout_pad,
                                       float *__restrict__ wp, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    // i = ((tap * n_chunks + chunk) * cout_pad + co) * 32 + ci_in_chunk
    const int cl = (int)(i % 32);
    int64_t rest = i / 32;
    const int co = (int)(rest % cout_pad);
    rest /= cout_pad;
    const int nch = cin_pad / 32;
    const int ci = (int)(rest % nch) * 32 + cl;
    const int tap = (int)(rest / nch);
    float v = 0.0f;
    if (co < cout && ci < cin) v = w[((int64_t)co * cin + ci) * k * k + tap];
    unsigned u = __float_as_uint(v);
    u = (u + 0x1000u) & 0xFFFFE000u;  // keep 10 mantissa bits
    wp[i] = __uint_as_float(u);
  }
}

#ifdef MIE_TC_TRACE
extern "C" int mie_debug_trace(long long *host, int n) {
  return cudaMemcpyFromSymbol(host, g_tc_trace, sizeof(long long) * (size_t)(n < 1024 * 16 ? n : 1024 * 16)) == cudaSuccess ? 0 : 1;
}
#endif

extern "C" int mie_conv_cluster_size(const mie_conv_args *a) {
  if (!a || !tc_eligible(a)) return 0;
  int nb, ksplit;
  tc_block_shape(a, &nb, &ksplit);
  return ksplit;
}

extern "C" int mie_set_option(int option, int value) {
  switch (option) {
    case MIE_OPT_TC_THRESHOLDED: g_opt_tc_thresholded = value ? 1 : 0; return MIE_OK;
    case MIE_OPT_TC_SPIN_LIMIT:
      if (value < 0) return MIE_EINVAL;
      g_opt_spin_limit = value == 0 ? SPIN_LIMIT : (unsigned)value;
      return MIE_OK;
    case MIE_OPT_TC_WITHHOLD_LOADS: g_opt_withhold_loads = value ? 1 : 0; return MIE_OK;
    case MIE_OPT_TC_KSPLIT: g_opt_ksplit = value ? 1 : 0; return MIE_OK;
    case MIE_OPT_TC_OWN_KERNELS:
      if (value < 0 || value > 15) return MIE_EINVAL;
      g_opt_own_kernels = value;
      return MIE_OK;
    case MIE_OPT_LAUNCH_COUNT: __atomic_store_n(&g_launch_count, (unsigned long long)(value < 0 ? 0 : value), __ATOMIC_RELAXED); return MIE_OK;
    default: return MIE_EINVAL;
  }
}

extern "C" int mie_get_option(int option, int *value) {
  if (!value) return MIE_EINVAL;
  switch (option) {
    case MIE_OPT_TC_THRESHOLDED: *value = g_opt_tc_thresholded; return MIE_OK;
    case MIE_OPT_TC_SPIN_LIMIT: *value = (int)g_opt_spin_limit; return MIE_OK;
    case MIE_OPT_TC_WITHHOLD_LOADS: *value = g_opt_withhold_loads; return MIE_OK;
    case MIE_OPT_TC_KSPLIT: *value = g_opt_ksplit; return MIE_OK;
    case MIE_OPT_TC_OWN_KERNELS: *value = g_opt_own_kernels; return MIE_OK;
    case MIE_OPT_LAUNCH_COUNT: *value = (int)(__atomic_load_n(&g_launch_count, __ATOMIC_RELAXED) & 0x7FFFFFFFull); return MIE_OK;
    default: return MIE_EINVAL;
  }
}

extern "C" int mie_conv_pack_dims_tc(int cin, int cout, int k, int *cin_pad, int *cout_pad, int64_t *n_floats) {
  if (cin <= 0 || cout <= 0 || k <= 0) return MIE_EINVAL;
  const int cp = divup(cin, 32) * 32, op = divup(cout, 32) * 32;
  if (cin_pad) *cin_pad = cp;
  if (cout_pad) *cout_pad = op;
  if (n_floats) *n_floats = (int64_t)k * k * cp * op;
  return MIE_OK;
}

extern "C" int mie_pack_conv_weights_tc(const float *w_oihw, int cout, int cin, int k, float *wpacked, void *stream) {
  if (!w_oihw || !wpacked) return MIE_EINVAL;
  int cp, op;
  int64_t total;
  int s = mie_conv_pack_dims_tc(cin, cout, k, &cp, &op, &total);
  if (s != MIE_OK) return s;
  int blocks = (int)((total + 255) / 256);
  if (blocks > MIE_SM_COUNT * 8) blocks = MIE_SM_COUNT * 8;
  pack_weights_tc_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(w_oihw, cout, cin, k, cp, op, wpacked, total);
  return check_launch();
}

