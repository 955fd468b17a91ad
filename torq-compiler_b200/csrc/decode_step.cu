// One persistent kernel for a whole decode step of the Gemma-3-style graph the op list
// describes (embed, then per layer: RMSNorm -> qkv projection -> q/k norm + RoPE + KV append
// -> attention -> o projection -> post norm + residual -> pre-FFN norm -> gate/up projection
// -> GeGLU -> down projection -> post norm + residual; final norm, LM head, arg max).
//
// Why one kernel: at decode batch sizes a layer streams 26.8 MB of int8 weights, 4 us of HBM
// time, through five dependent stages. As separate launches each stage pays a launch gap and
// a cold start of its weight stream; here one CTA per SM stays resident and
//   * a producer warp streams this CTA's share of every weight matrix of every layer through
//     a ring of shared-memory slots with bulk asynchronous copies. Weights do not depend on
//     activations, so the stream runs ahead across stage boundaries by the depth of the ring
//     (most of a layer) and HBM never idles while the CTAs synchronise;
//   * 16 consumer warps turn the int8 rows into fp16 fragments (exact) and feed mma.sync
//     m16n8k16 with the weights as the 16-row operand and up to 8 tokens as the 8-column
//     operand, fp32 accumulation. The activations are bf16 values held as fp16 (exact inside
//     fp16's normal range; a per-token power of two is taken out first when a token's largest
//     magnitude would not fit). A slot holds 16 weight rows x 1152 bytes of K; the
//     warps split its K range, a 17th warp adds their partial tiles in a fixed order and
//     applies the stage's epilogue (bf16 scale, GeGLU, logits + running arg max);
//   * stages hand their results over in one of two ways. A projection's output (a few KB) travels
//     as 32-bit words {epoch tag, bf16 value}: the reader spins on the words it needs until they
//     carry the stage's tag, so the data IS the signal: one L2 round trip, no fence, no counter.
//     The K-split projections of tensor parallelism travel the same way through peer memory, as 64-bit words
//     {tag, fp32 partial result}, one per GPU and element. Where a stage's result is large (attention partial
//     sums, the GeGLU vector) or needs every GPU's candidates (the arg max) a grid-wide barrier is used (one
//     counter in global memory, cooperative launch). Every wait is bounded. Each CTA keeps the residual
//     stream in shared memory and recomputes the small norms itself, so only the projections'
//     outputs cross between CTAs.
// The tensor work is HBM-bound (1.25 instructions per weight byte to build the fragments is
// the on-chip cost), which is why the operands go through mma.sync registers and not through
// a shared-memory staging pass for tcgen05.
//
// Rounding points are those of the per-op kernels in decoder.cu; only the order of fp32
// additions inside the norms and the K reduction differs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>

#include "kernels.h"
#include "status_word.cuh"

namespace tb200 {

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kReducerWarp = 16;
constexpr int kProducerWarp = 17;
constexpr int kThreads = 18 * 32;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kSegBytes = 1152;               // bytes of K of one weight row per slot
constexpr int kRowStride = 1216;              // = 64 mod 128: rows g, g+1 fall in different 64-byte halves
constexpr int kSlotBytes = 16 * kRowStride;   // 16 rows per slot
constexpr int kLongSeg = 2304;                // long rows: bytes of K per slot ...
constexpr int kLongStride = 2368;             // ... at this row distance (= 64 mod 128), 8 rows per slot
constexpr int kPartFloats = kConsumerWarps * 128;
constexpr int kD = 256;                       // head dim
// limit of every bounded wait of the kernel in ns, copied from the launch arguments by thread 0 before the
// first block-wide barrier
__shared__ unsigned long long s_wait_limit_ns;

// status codes written to the device status word when a bounded wait gives up
enum { kErrFull = 16, kErrEmpty = 17, kErrGrid = 18, kErrPartFull = 19, kErrPartEmpty = 20 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ float bf2f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
__device__ __forceinline__ uint16_t f2bf(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
__device__ __forceinline__ float rbf(float f) { return bf2f(f2bf(f)); }
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(2000u)  // the thread may sleep up to 2 us per try; it wakes when the phase completes
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait on a shared-memory barrier. Gives up (false) when the limit passes or when any
// CTA has already reported a failure in the status word; a thread that gave up keeps running
// its (statically bounded) loops without waiting again, so no barrier partner is left alone.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code, bool ok) {
  if (!ok) return false;
#pragma unroll 1
  for (int i = 0; i < 4096; i++)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (*(volatile int*)status != 0) return false;
    if (globaltimer_ns() - t0 > s_wait_limit_ns) {
      report_expired_wait(status, code);
      return false;
    }
  }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_gpu(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Tagged hand-over of a projection's output: element = (tag << 16) | bf16 bits, one 32-bit store.
// The tag is the low 16 bits of an epoch that grows by one per (launch, layer, projection); a buffer is
// rewritten every layer, so a stale word always carries an older tag than the one waited for.
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_v4(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Spins until the word carries `tag`; returns its bf16 payload as a float. Bounded like every wait.
__device__ __forceinline__ float wait_tagged(const uint32_t* p, uint32_t tag, int* status, bool& ok) {
  uint32_t w = ld_relaxed_u32(p);
  if ((w >> 16) == tag || !ok) return __uint_as_float(w << 16);
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++) {
      w = ld_relaxed_u32(p);
      if ((w >> 16) == tag) return __uint_as_float(w << 16);
    }
    if (*(volatile int*)status != 0 || globaltimer_ns() - t0 > s_wait_limit_ns) {
      report_expired_wait(status, (int)kErrGrid);
      ok = false;
      return 0.f;
    }
  }
}
// Across GPUs the hand-over word is 64 bits {tag, fp32 partial result}: one store through peer memory carries the
// value and its signal (no fence, no barrier; one NVLink crossing), and the reader polls its own GPU's memory.
__device__ __forceinline__ void st_tagged_sys(float* inbox_word, float value, uint32_t tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(value);
  asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(inbox_word), "l"(w) : "memory");
}
__device__ __forceinline__ float wait_tagged_sys(const float* inbox_word, uint32_t tag, int* status, bool& ok) {
  unsigned long long w;
  asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(inbox_word) : "memory");
  if ((uint32_t)(w >> 32) == tag || !ok) return __uint_as_float((uint32_t)w);
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++) {
      asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(w) : "l"(inbox_word) : "memory");
      if ((uint32_t)(w >> 32) == tag) return __uint_as_float((uint32_t)w);
    }
    if (*(volatile int*)status != 0 || globaltimer_ns() - t0 > s_wait_limit_ns) {
      report_expired_wait(status, (int)kErrGrid);
      ok = false;
      return 0.f;
    }
  }
}
// The same for four consecutive words (16-byte aligned).
__device__ __forceinline__ uint4 wait_tagged4(const uint32_t* p, uint32_t tag, int* status, bool& ok) {
  uint4 w = ld_relaxed_v4(p);
  auto good = [&](const uint4& v) { return (v.x >> 16) == tag && (v.y >> 16) == tag && (v.z >> 16) == tag && (v.w >> 16) == tag; };
  if (good(w) || !ok) return w;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++) {
      w = ld_relaxed_v4(p);
      if (good(w)) return w;
    }
    if (*(volatile int*)status != 0 || globaltimer_ns() - t0 > s_wait_limit_ns) {
      report_expired_wait(status, (int)kErrGrid);
      ok = false;
      return make_uint4(0, 0, 0, 0);
    }
  }
}

// Grid barriers. Counters only ever grow (64 bits): a launch starts from the bases its
// predecessor left behind. Barriers inside one GPU use the local counter, one count per CTA.
// A barrier that spans the tensor-parallel peers is hierarchical: every CTA adds to a gathering
// counter of its own GPU, and only the CTA whose count completes the GPU's G arrivals adds one to the
// barrier counter on every GPU through peer memory (tp - 1 NVLink atomics per GPU and barrier, not
// G * (tp - 1)); the waiters' target therefore grows by tp per barrier. Two (gathering, barrier)
// counter pairs alternate, so that a GPU that is one barrier ahead never adds to the counter its peers
// are still waiting on; which pair comes next is carried from launch to launch with the bases (a launch
// has one cross-GPU barrier, the arg max's).
// Counter block (byte offsets): local 0, barrier 8 and 16, their bases 24, 32, 40, exit count 48, epoch of
// the tagged hand-overs 56, next pair 60, gathering 64 and 72.
struct BarrierState {
  unsigned long long local, global[2];  // expected values
  int parity;
};
// Arrival side: everything this thread (and, through the preceding CTA-level synchronisation,
// its CTA) wrote is made visible before the count goes up.
// fence = false: the caller has already fenced (every lane of the reducer warp fences its own stores).
__device__ __forceinline__ void grid_arrive(const DecodeStepArgs& a, bool all_gpus, int parity, bool fence = true) {
  if (all_gpus && a.tp > 1) {
    if (fence) __threadfence_system();
    unsigned long long* gather = (unsigned long long*)(a.scratch + a.counter_off + 64 + 8 * parity);
    const unsigned long long old = atomicAdd(gather, 1ull);
    if ((old + 1ull) % (unsigned long long)a.grid == 0ull) {
      // every CTA of this GPU has arrived (each after its own system-scope fence): tell every GPU, this one first
      __threadfence_system();
      const unsigned long long off = a.counter_off + 8 + 8 * parity;
      atomicAdd_system((unsigned long long*)(a.scratch + off), 1ull);
      for (int r = 0; r < a.tp; r++)
        if (r != a.rank) atomicAdd_system((unsigned long long*)(a.peer_scratch[r] + off), 1ull);
    }
  } else {
    if (fence) __threadfence();
    atomicAdd((unsigned long long*)(a.scratch + a.counter_off), 1ull);
  }
}
// Waiting side (one thread per CTA). Bounded like mbar_wait.
__device__ __forceinline__ bool grid_wait(const DecodeStepArgs& a, bool all_gpus, int parity, unsigned long long target,
                                          int* status, bool ok) {
  if (!ok) return false;
  const bool sys = all_gpus && a.tp > 1;
  const unsigned long long* counter = (const unsigned long long*)(a.scratch + a.counter_off + (sys ? 8 + 8 * parity : 0));
#pragma unroll 1
  for (int i = 0; i < 4096; i++)
    if ((sys ? ld_acquire_sys(counter) : ld_acquire_gpu(counter)) >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; i++)
      if ((sys ? ld_acquire_sys(counter) : ld_acquire_gpu(counter)) >= target) return true;
    if (*(volatile int*)status != 0) return false;
    if (globaltimer_ns() - t0 > s_wait_limit_ns) {
      report_expired_wait(status, (int)kErrGrid);
      return false;
    }
  }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// four signed bytes -> two fp16x2 words (k, k+1) and (k+2, k+3); exact.
// 0x6400 | u is the fp16 number 1024 + u (u = byte + 128); subtracting 1152 leaves the byte's value.
__device__ __forceinline__ void s8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  const uint32_t p01 = __byte_perm(u, 0x64646464u, 0x5140), p23 = __byte_perm(u, 0x64646464u, 0x5342);
  asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(p01), "r"(0x64806480u));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(p23), "r"(0x64806480u));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.0f + tanhf(k0 * (x + k1 * x * x * x)));
}

// Position in a ring of n entries: index and how many times the ring has wrapped (parity used
// by the barriers). Advanced by all parties in the same order.
struct RingPos {
  uint32_t idx, wraps;
  __device__ __forceinline__ void advance(uint32_t n) {
    if (++idx == n) {
      idx = 0;
      wraps++;
    }
  }
};

// One projection as seen by one CTA: which weight rows it owns and how they are tiled.
enum PhaseKind { kRows = 0, kPairs = 1, kLogits = 2 };
struct Phase {
  const int8_t* W;
  const uint16_t* scale;
  int K, N;       // row length (bytes), total rows (pairs phase: rows of one half, i.e. I)
  int kind;
  int first, count;  // this CTA's first row (or gate/up pair) and how many
  int ntiles, nseg;
  int rpt;        // weight rows (or pairs) per tile
  int seg;        // bytes of K per slot
  int stride;     // byte distance of consecutive rows inside a slot
  int whole;      // the tile's rows are one contiguous run of global memory, copied at once
};
enum { kQkv = 0, kO = 1, kGateUp = 2, kDown = 3, kLmHead = 4 };

// Slot geometry. Rows no longer than kSegBytes: a tile is 16 whole rows, contiguous in global
// memory, fetched by one bulk copy (two for a gate/up tile: 8 gate rows and the 8 matching up
// rows). Longer rows (the down projection): 8 rows per tile, kLongSeg bytes of each per slot,
// one copy per row. Few large copies matter: the copy engine's cost is per request.
__device__ __forceinline__ Phase make_phase(const DecodeStepArgs& a, const DecodeLayerDesc* L, int which, const int* a_first,
                                            const int* a_count) {
  Phase p;
  p.kind = kRows;
  switch (which) {
    case kQkv: p.W = (const int8_t*)(a.consts + L->w_qkv); p.scale = (const uint16_t*)(a.consts + L->s_qkv);
      p.K = a.H; p.N = (a.n_q + 2) * kD; break;
    case kO: p.W = (const int8_t*)(a.consts + L->w_o); p.scale = (const uint16_t*)(a.consts + L->s_o);
      p.K = a.o_k; p.N = a.H; break;  // a.o_k < n_q * 256 when a head is shared by two tensor-parallel GPUs
    case kGateUp: p.W = (const int8_t*)(a.consts + L->w_gu); p.scale = (const uint16_t*)(a.consts + L->s_gu);
      p.K = a.H; p.N = a.I; p.kind = kPairs; break;
    case kDown: p.W = (const int8_t*)(a.consts + L->w_down); p.scale = (const uint16_t*)(a.consts + L->s_down);
      p.K = a.I; p.N = a.H; break;
    default: p.W = (const int8_t*)(a.consts + a.lm_w); p.scale = (const uint16_t*)(a.consts + a.lm_s);
      p.K = a.H; p.N = a.V; p.kind = kLogits; break;
  }
  p.first = a_first[which];
  p.count = a_count[which];
  if (p.K <= kSegBytes) {
    p.whole = 1;
    p.rpt = p.kind == kPairs ? 8 : 16;
    p.seg = p.K;
    p.stride = p.K;
  } else {
    p.whole = 0;
    p.rpt = 8;
    p.seg = kLongSeg;
    p.stride = kLongStride;
  }
  p.ntiles = (p.count + p.rpt - 1) / p.rpt;
  p.nseg = (p.K + p.seg - 1) / p.seg;
  return p;
}
// weight row held by slot row j of tile t, or -1
__device__ __forceinline__ int tile_row(const Phase& p, int t, int j) {
  if (p.kind == kPairs) {
    const int pi = 8 * t + (j & 7);
    if (pi >= p.count) return -1;
    return (j < 8 ? 0 : p.N) + p.first + pi;
  }
  if (j >= p.rpt) return -1;
  const int r = p.rpt * t + j;
  return r < p.count ? p.first + r : -1;
}

// Shared-memory map (byte offsets from the start of dynamic shared memory):
//   ring | xin (fp16 activations of the running projection; attention scratch in between)
//   | xs (bf16 residual stream) | part (2 partial-tile buffers) | red (reductions, softmax
//   coefficients, per-token activation scale, RoPE tables) | barriers
struct Smem {
  char* base;
  uint32_t ring, bars;  // shared-space byte addresses
  uint32_t xin_addr;
  uint32_t off_xin, off_xs, off_part, off_red, off_bars;
};
constexpr int kRedSums = 0;        // 256 floats: block reductions
constexpr int kRedCoef = 1024;     // 512 floats: softmax merge coefficients and totals
constexpr int kRedXscale = 3072;   // 8 floats: power-of-two scale taken out of each token's activations
constexpr int kRedRows = 3200;     // int [5] first row and int [5] row count of this CTA per projection
constexpr int kRedRope = 4096;     // 2 tables x 128 x (cos, sin)
constexpr int kRedBytes = 6144;
// barriers: full[nslots], empty[nslots], part_full[2], part_empty[2], then the give-up flag

// ------------------------------------------------------------------------------------------
// Consumer-side helpers (threads 0..511)
// ------------------------------------------------------------------------------------------

// v[b] <- reduction over the 512 consumer threads of v[b], b < BT, combined in warp order
template <int BT, bool MAX>
__device__ __forceinline__ void consumer_reduce(float (&v)[BT], float* red, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int b = 0; b < BT; b++) {
    float x = v[b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float y = __shfl_xor_sync(0xffffffffu, x, o);
      x = MAX ? fmaxf(x, y) : x + y;
    }
    if (lane == 0) red[warp * BT + b] = x;
  }
  bar_consumers();
#pragma unroll
  for (int b = 0; b < BT; b++) {
    float s = MAX ? 0.f : 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; w++) s = MAX ? fmaxf(s, red[w * BT + b]) : s + red[w * BT + b];
    v[b] = s;
  }
  bar_consumers();
}

// power of two that brings a token's largest magnitude under 2^15, so that the fp16 copy of
// its activations cannot overflow; returns the factor the products must be multiplied back by
__device__ __forceinline__ float fp16_guard(float amax, float& down) {
  int ex = 0;
  frexpf(amax, &ex);  // amax < 2^ex
  if (!(amax < 3.0e38f) || ex <= 15) {
    down = 1.0f;
    return 1.0f;
  }
  down = ldexpf(1.0f, 15 - ex);
  return ldexpf(1.0f, ex - 15);
}

constexpr int kNormElems = 4;  // elements of a hidden vector per consumer thread (H <= 2048)
struct NormWeights {
  float post[kNormElems], pre[kNormElems];  // 1 + w
};
// Fetched before the grid barrier that precedes the norm, so that the weights are in registers
// when the projection's output becomes visible.
__device__ __forceinline__ NormWeights load_norm_weights(const uint16_t* w_post, const uint16_t* w_pre, int H, int tid) {
  NormWeights nw;
#pragma unroll
  for (int e = 0; e < kNormElems; e++) {
    const int i = tid + e * kConsumerThreads;
    nw.post[e] = (w_post && i < H) ? 1.0f + bf2f(__ldg(w_post + i)) : 0.f;
    nw.pre[e] = i < H ? 1.0f + bf2f(__ldg(w_pre + i)) : 0.f;
  }
  return nw;
}

// The norm vectors of a layer (six short constants, read once per step, so always an HBM miss) are pulled
// into L2 a layer ahead: the loads in front of each norm then cost an L2 round trip, not a DRAM one.
__device__ __forceinline__ void prefetch_layer_constants(const DecodeStepArgs& a, const DecodeLayerDesc* L, int tid) {
  const int lines = (a.H * 2 + 127) / 128;
  if (tid < 4 * lines) {
    const int which = tid / lines, line = tid - which * lines;
    const unsigned long long off = which == 0 ? L->in_norm : which == 1 ? L->post_attn_norm : which == 2 ? L->pre_ffn_norm : L->post_ffn_norm;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(a.consts + off + (size_t)line * 128));
  } else if (tid < 4 * lines + 8) {
    const int j = tid - 4 * lines;
    asm volatile("prefetch.global.L2 [%0];" ::"l"(a.consts + (j < 4 ? L->q_norm : L->k_norm) + (size_t)(j & 3) * 128));
  }
}

// Residual update and the norm that feeds the next projection:
//   if src: xs <- bf16(xs + bf16(src * rsqrt(mean(src^2) + eps) * (1 + w_post)))
//   xin    <- fp16(bf16(xs * rsqrt(mean(xs^2) + eps) * (1 + w_pre)))   (exact: |value| <= sqrt(H) * |1 + w|)
// src is a [B, H] bf16 tensor in global memory written by other CTAs before the last barrier.
// With tensor parallelism the projection's output arrives as one fp32 partial result per GPU
// (inbox [tp][B][H] of tagged 64-bit words at byte offset `inbox` of the scratch area, written by the
// peers' reducer warps); each is awaited by its tag, they are added in rank order and rounded to bf16,
// the same on every GPU. An inbox word is rewritten only after every CTA of this GPU has read it: a peer's
// next partial result for it depends, through the projection in between, on rows that every CTA here
// produces after this read.
__device__ __forceinline__ float load_projection(const DecodeStepArgs& a, const uint32_t* src, uint32_t tag,
                                                 unsigned long long inbox, int b, int i, int* status, bool& ok) {
  if (a.tp <= 1) return wait_tagged(src + (size_t)b * a.H + i, tag, status, ok);
  const float* in = (const float*)(a.scratch + inbox);  // 64-bit words {tag, value}: two floats per element
  float s = 0.f;
  for (int r = 0; r < a.tp; r++) s += wait_tagged_sys(in + 2 * (((size_t)r * a.B + b) * a.H + i), tag, status, ok);
  return rbf(s);
}
template <int BT>
__device__ __forceinline__ void residual_norm(const DecodeStepArgs& a, const uint32_t* src, uint32_t tag,
                                              unsigned long long inbox, const NormWeights& nw, uint16_t* xs, char* xin,
                                              int xin_stride, float* red, int tid, int* status, bool& ok) {
  const int H = a.H;
  float ss[BT];
  if (src) {
    float sv[BT][kNormElems];
#pragma unroll
    for (int b = 0; b < BT; b++) {
      ss[b] = 0.f;
#pragma unroll
      for (int e = 0; e < kNormElems; e++) {
        const int i = tid + e * kConsumerThreads;
        sv[b][e] = (b < a.B && i < H) ? load_projection(a, src, tag, inbox, b, i, status, ok) : 0.f;
        ss[b] += sv[b][e] * sv[b][e];
      }
    }
    consumer_reduce<BT, false>(ss, red, tid);
#pragma unroll
    for (int b = 0; b < BT; b++) {
      const float inv = rsqrtf(ss[b] / (float)H + a.eps);
      ss[b] = 0.f;
#pragma unroll
      for (int e = 0; e < kNormElems; e++) {
        const int i = tid + e * kConsumerThreads;
        if (b < a.B && i < H) {
          const float n = rbf(sv[b][e] * inv * nw.post[e]);
          const uint16_t x = f2bf(bf2f(xs[b * H + i]) + n);
          xs[b * H + i] = x;
          ss[b] += bf2f(x) * bf2f(x);
        }
      }
    }
  } else {
#pragma unroll
    for (int b = 0; b < BT; b++) {
      ss[b] = 0.f;
#pragma unroll
      for (int e = 0; e < kNormElems; e++) {
        const int i = tid + e * kConsumerThreads;
        if (b < a.B && i < H) {
          const float v = bf2f(xs[b * H + i]);
          ss[b] += v * v;
        }
      }
    }
  }
  consumer_reduce<BT, false>(ss, red, tid);
#pragma unroll
  for (int b = 0; b < BT; b++) {
    const float inv = rsqrtf(ss[b] / (float)H + a.eps);
#pragma unroll
    for (int e = 0; e < kNormElems; e++) {
      const int i = tid + e * kConsumerThreads;
      if (b < a.B && i < H)
        *(__half*)(xin + (size_t)b * xin_stride + 2 * i) = __float2half_rn(rbf(bf2f(xs[b * H + i]) * inv * nw.pre[e]));
    }
  }
  if (tid < 8) ((float*)((char*)red + kRedXscale))[tid] = 1.0f;
  bar_consumers();
}

// The tensor part of one projection for one consumer warp: walks the CTA's slots of this
// phase in the producer's order, multiplies its share of each slot's K range, and hands one
// partial 16x8 tile per weight tile to the reducer warp.
__device__ __forceinline__ void consume_phase(const Phase& p, const Smem& sm, int nslots, int B, int xin_stride,
                                              RingPos& ring, RingPos& tile, int* status, bool& ok, int warp, int lane) {
  const int g = lane >> 2, tig = lane & 3;
  const uint32_t x_row = sm.xin_addr + (uint32_t)g * xin_stride + tig * 32;
  for (int t = 0; t < p.ntiles; t++) {
    // four independent accumulators: a dependent mma.sync chain costs ~130 cycles per link here
    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f},
          c3[4] = {0.f, 0.f, 0.f, 0.f};
    const bool upper = p.kind == kPairs || (p.rpt == 16 && (p.count - 16 * t) > 8);  // rows g+8 hold data
    for (int s = 0; s < p.nseg; s++) {
      const uint32_t slot = ring.idx;
      ok = mbar_wait(sm.bars + 8 * slot, ring.wraps & 1, status, kErrFull, ok);
      ring.advance(nslots);
      const int seg_bytes = min(p.seg, p.K - s * p.seg);
      const int kbs = seg_bytes >> 6;
      const uint32_t wbase = sm.ring + slot * kSlotBytes + g * p.stride + tig * 16;
      // the warp that takes the first K block rotates with the tile so that no scheduler
      // is always the one with an extra block
      for (int kb = (warp + 2 * t + 5 * s) & 15; kb < kbs; kb += 16) {
        const uint4 wa = lds128(wbase + kb * 64);
        uint4 wb = make_uint4(0, 0, 0, 0);
        if (upper) wb = lds128(wbase + 8 * p.stride + kb * 64);
        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
        if (g < B) {
          const uint32_t xa = x_row + (uint32_t)(s * p.seg + kb * 64) * 2;
          x0 = lds128(xa);
          x1 = lds128(xa + 16);
        }
        uint32_t a0, a1 = 0, a2, a3 = 0;
        s8x4_to_f16x4(wa.x, a0, a2);
        if (upper) s8x4_to_f16x4(wb.x, a1, a3);
        mma_f16(c0, a0, a1, a2, a3, x0.x, x0.y);
        s8x4_to_f16x4(wa.y, a0, a2);
        if (upper) s8x4_to_f16x4(wb.y, a1, a3);
        mma_f16(c1, a0, a1, a2, a3, x0.z, x0.w);
        s8x4_to_f16x4(wa.z, a0, a2);
        if (upper) s8x4_to_f16x4(wb.z, a1, a3);
        mma_f16(c2, a0, a1, a2, a3, x1.x, x1.y);
        s8x4_to_f16x4(wa.w, a0, a2);
        if (upper) s8x4_to_f16x4(wb.w, a1, a3);
        mma_f16(c3, a0, a1, a2, a3, x1.z, x1.w);
      }
      __syncwarp();
      // after a failed wait nothing is signalled any more: the partner's own bounded wait ends it
      if (lane == 0 && ok) mbar_arrive(sm.bars + 8 * (nslots + slot));  // slot drained by this warp
    }
    const uint32_t buf = tile.idx, round = tile.wraps;
    tile.advance(2);
    if (round > 0) ok = mbar_wait(sm.bars + 8 * (2 * nslots + 2 + buf), (round - 1) & 1, status, kErrPartEmpty, ok);
    float4* dst = (float4*)(sm.base + sm.off_part) + (buf * kPartFloats / 4 + warp * 32 + lane);
    *dst = make_float4((c0[0] + c1[0]) + (c2[0] + c3[0]), (c0[1] + c1[1]) + (c2[1] + c3[1]), (c0[2] + c1[2]) + (c2[2] + c3[2]),
                       (c0[3] + c1[3]) + (c2[3] + c3[3]));
    __syncwarp();
    if (lane == 0 && ok) mbar_arrive(sm.bars + 8 * (2 * nslots + buf));
  }
}

// Optional per-stage timestamps of CTA 0 (consumer thread 0), for profiling the stage chain.
__device__ __forceinline__ void trace_mark(const DecodeStepArgs& a, int blk, int tid, int& idx) {
  if (a.trace_off && blk == 0 && tid == 0) {
    unsigned long long* t = (unsigned long long*)(a.scratch + a.trace_off);
    if (idx < a.trace_len) t[idx] = globaltimer_ns();
  }
  idx++;
}

// Attention work split. Stage 1: every CTA takes one slice of the key window of every batch row
// (a handful of keys: the cache is read by all SMs at once); warp = (pair of query heads
// hp = warp & 1, token lane tl = warp >> 1): keys tl, tl + 8, ... of the slice; the single KV
// head is read by both head pairs (second read from L1). The CTA's running (max, sum, acc[256])
// per head goes to global memory. Stage 2, after a grid barrier: every CTA merges the slices for
// a few of the B * n_q * 256 output columns, one column per warp at a time, lanes over slices.
constexpr int kTokenLanes = 8;
struct KeyRange {
  int t_first, t_end, pos;
};
__device__ __forceinline__ KeyRange key_range(const DecodeStepArgs& a, const DecodeLayerDesc* L, int slice, int tl) {
  KeyRange r;
  int pos = __ldg(a.pos);
  pos = pos < 0 ? 0 : (pos >= a.T ? a.T - 1 : pos);
  const int t_lo = L->window > 0 ? max(0, pos - L->window + 1) : 0;
  const int span = pos + 1 - t_lo;
  const int per = (span + a.grid - 1) / a.grid;
  const int t0 = t_lo + slice * per;
  r.t_first = t0 + tl;
  r.t_end = min(pos + 1, t0 + per);
  r.pos = pos;
  return r;
}
// Long before the attention stage runs: pull this CTA's cache lines towards L2.
__device__ __forceinline__ void prefetch_keys(const DecodeStepArgs& a, const DecodeLayerDesc* L, int blk, int warp, int lane) {
  if ((warp & 1) || lane >= 8) return;
  const KeyRange r = key_range(a, L, blk, warp >> 1);
  for (int b = 0; b < a.B; b++) {
    const char* kc = a.arena + L->kcache + (size_t)b * a.T * kD * 2;
    const char* vc = a.arena + L->vcache + (size_t)b * a.T * kD * 2;
    for (int t = r.t_first; t < r.t_end; t += kTokenLanes)
      if (t != r.pos) {
        const char* p = (lane < 4 ? kc : vc) + (size_t)t * kD * 2 + (lane & 3) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
      }
  }
}

// Attention scratch inside the activation staging area (dead between the qkv and o projections)
constexpr int kAttnQs = 0;                       // float [4][256]: queries after norm, RoPE and scaling
constexpr int kAttnKs = 4 * kD * 4;              // bf16 [256]: the new key
constexpr int kAttnVs = kAttnKs + kD * 2;        // bf16 [256]: the new value
constexpr int kAttnAcc = kAttnVs + kD * 2;       // float [8 token lanes][4 heads][258]: (max, sum, acc[256])
constexpr int kAttnScratchBytes = kAttnAcc + kTokenLanes * 4 * (kD + 2) * 4;

// 1 + w of the q-norm (warps 0..n_q-1) or k-norm (warp n_q) elements a lane works on; fetched
// before the barrier that releases the attention stage
struct HeadNormWeights {
  float w[8];
};
__device__ __forceinline__ HeadNormWeights load_head_norm_weights(const DecodeStepArgs& a, const DecodeLayerDesc* L, int warp,
                                                                  int lane) {
  HeadNormWeights r;
#pragma unroll
  for (int j = 0; j < 8; j++) r.w[j] = 0.f;
  if (warp <= a.n_q) {
    const uint16_t* w = (const uint16_t*)(a.consts + (warp < a.n_q ? L->q_norm : L->k_norm));
#pragma unroll
    for (int j = 0; j < 4; j++) {
      r.w[j] = 1.0f + bf2f(__ldg(w + 4 * lane + j));
      r.w[4 + j] = 1.0f + bf2f(__ldg(w + 128 + 4 * lane + j));
    }
  }
  return r;
}

// Stage 1 for batch row b: q/k head norms, RoPE and the KV append (warps 0..n_q+1, one head each;
// CTA 0 writes the cache); the keys of the CTA's slice; the 8 token lanes merged per head; the
// CTA's partial per head published.
__device__ void attention_slice(const DecodeStepArgs& a, const DecodeLayerDesc* L, const Smem& sm, const HeadNormWeights& nw,
                                int b, int blk, int tid, uint32_t tag, int* status, bool& ok) {
  const int warp = tid >> 5, lane = tid & 31;
  const int G = a.grid;
  char* scratch = sm.base + sm.off_xin;
  float* qs = (float*)(scratch + kAttnQs);
  uint16_t* ks = (uint16_t*)(scratch + kAttnKs);
  uint16_t* vs = (uint16_t*)(scratch + kAttnVs);
  float* comb = (float*)(scratch + kAttnAcc);
  const float2* rope = (const float2*)(sm.base + sm.off_red + kRedRope) + L->rope_table * 128;
  const int hp = warp & 1, tl = warp >> 1;
  const KeyRange kr = key_range(a, L, blk, tl);
  const int pos = kr.pos;
  const uint32_t* qkv = (const uint32_t*)(a.scratch + a.qkv_off) + (size_t)b * (a.n_q + 2) * kD;
  uint16_t* kcache = (uint16_t*)(a.arena + L->kcache) + (size_t)b * a.T * kD;
  uint16_t* vcache = (uint16_t*)(a.arena + L->vcache) + (size_t)b * a.T * kD;
  // this warp's first keys and values: issued before anything else so that the cache latency
  // overlaps the head norms (the entry for the new position comes from shared memory)
  constexpr int kBatch = 2;
  uint4 kk[kBatch], vv[kBatch];
#pragma unroll
  for (int j = 0; j < kBatch; j++) {
    const int t = kr.t_first + kTokenLanes * j;
    kk[j] = vv[j] = make_uint4(0, 0, 0, 0);
    if (t < kr.t_end && t != pos) {
      kk[j] = __ldg((const uint4*)(kcache + (size_t)t * kD + lane * 8));
      vv[j] = __ldg((const uint4*)(vcache + (size_t)t * kD + lane * 8));
    }
  }
  if (warp < a.n_q + 2) {
    const int hh = warp;
    // this lane's elements: [4*lane, 4*lane+4) of each half of the head
    // tagged words written by the qkv projection's reducers: the wait for them is the stage's barrier
    const uint4 t_lo = wait_tagged4(qkv + hh * kD + 4 * lane, tag, status, ok);
    const uint4 t_hi = wait_tagged4(qkv + hh * kD + 128 + 4 * lane, tag, status, ok);
    const uint2 lo2 = make_uint2((t_lo.x & 0xffffu) | (t_lo.y << 16), (t_lo.z & 0xffffu) | (t_lo.w << 16));
    const uint2 hi2 = make_uint2((t_hi.x & 0xffffu) | (t_hi.y << 16), (t_hi.z & 0xffffu) | (t_hi.w << 16));
    const uint32_t raw[4] = {lo2.x, lo2.y, hi2.x, hi2.y};
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      v[2 * j] = __uint_as_float(raw[j] << 16);
      v[2 * j + 1] = __uint_as_float(raw[j] & 0xffff0000u);
    }
    if (hh == a.n_q + 1) {  // v head: copied as is
      *(uint2*)(vs + 4 * lane) = lo2;
      *(uint2*)(vs + 128 + 4 * lane) = hi2;
      if (blk == 0) {
        *(uint2*)(vcache + (size_t)pos * kD + 4 * lane) = lo2;
        *(uint2*)(vcache + (size_t)pos * kD + 128 + 4 * lane) = hi2;
      }
    } else {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 8; j++) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)kD + a.eps);
      float n[8];
#pragma unroll
      for (int j = 0; j < 8; j++) n[j] = rbf(v[j] * inv * nw.w[j]);
      uint16_t r1[4], r2[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 cs = rope[4 * lane + j];  // (cos, sin) of pos * theta^(-i/128)
        r1[j] = f2bf(n[j] * cs.x - n[4 + j] * cs.y);
        r2[j] = f2bf(n[4 + j] * cs.x + n[j] * cs.y);
      }
      if (hh < a.n_q) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          qs[hh * kD + 4 * lane + j] = bf2f(r1[j]) * a.attn_scale;
          qs[hh * kD + 128 + 4 * lane + j] = bf2f(r2[j]) * a.attn_scale;
        }
      } else {
        const uint2 p1 = make_uint2(r1[0] | ((uint32_t)r1[1] << 16), r1[2] | ((uint32_t)r1[3] << 16));
        const uint2 p2 = make_uint2(r2[0] | ((uint32_t)r2[1] << 16), r2[2] | ((uint32_t)r2[3] << 16));
        *(uint2*)(ks + 4 * lane) = p1;
        *(uint2*)(ks + 128 + 4 * lane) = p2;
        if (blk == 0) {
          *(uint2*)(kcache + (size_t)pos * kD + 4 * lane) = p1;
          *(uint2*)(kcache + (size_t)pos * kD + 128 + 4 * lane) = p2;
        }
      }
    }
  }
  bar_consumers();
  // ---- keys: two heads per warp ----
  float m[2], l[2], acc[2][8];
#pragma unroll
  for (int h = 0; h < 2; h++) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) acc[h][j] = 0.f;
  }
  if (kr.t_first < kr.t_end) {
    float qv[2][8];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const float4 q0 = *(const float4*)(qs + (2 * hp + h) * kD + lane * 8),
                   q1 = *(const float4*)(qs + (2 * hp + h) * kD + lane * 8 + 4);
      qv[h][0] = q0.x; qv[h][1] = q0.y; qv[h][2] = q0.z; qv[h][3] = q0.w;
      qv[h][4] = q1.x; qv[h][5] = q1.y; qv[h][6] = q1.z; qv[h][7] = q1.w;
    }
    for (int tb = kr.t_first; tb < kr.t_end; tb += kTokenLanes * kBatch) {
      if (tb != kr.t_first) {
#pragma unroll
        for (int j = 0; j < kBatch; j++) {
          const int t = tb + kTokenLanes * j;
          if (t < kr.t_end && t != pos) {
            kk[j] = __ldg((const uint4*)(kcache + (size_t)t * kD + lane * 8));
            vv[j] = __ldg((const uint4*)(vcache + (size_t)t * kD + lane * 8));
          }
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; j++) {
        const int t = tb + kTokenLanes * j;
        if (t < kr.t_end) {
          uint4 k4 = kk[j], v4 = vv[j];
          if (t == pos) {  // the new key/value come from shared memory, not from the cache line just written
            k4 = *(const uint4*)(ks + lane * 8);
            v4 = *(const uint4*)(vs + lane * 8);
          }
          const uint32_t kw[4] = {k4.x, k4.y, k4.z, k4.w}, vw[4] = {v4.x, v4.y, v4.z, v4.w};
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int q = 0; q < 4; q++) {
            const float ke = __uint_as_float(kw[q] << 16), ko = __uint_as_float(kw[q] & 0xffff0000u);
            s0 = fmaf(qv[0][2 * q], ke, s0); s0 = fmaf(qv[0][2 * q + 1], ko, s0);
            s1 = fmaf(qv[1][2 * q], ke, s1); s1 = fmaf(qv[1][2 * q + 1], ko, s1);
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            s0 += __shfl_xor_sync(0xffffffffu, s0, o);
            s1 += __shfl_xor_sync(0xffffffffu, s1, o);
          }
          const float sc[2] = {s0, s1};
#pragma unroll
          for (int h = 0; h < 2; h++) {
            const float m_new = fmaxf(m[h], sc[h]);
            const float corr = expf(m[h] - m_new), pr = expf(sc[h] - m_new);
            l[h] = l[h] * corr + pr;
#pragma unroll
            for (int q = 0; q < 4; q++) {
              acc[h][2 * q] = acc[h][2 * q] * corr + pr * __uint_as_float(vw[q] << 16);
              acc[h][2 * q + 1] = acc[h][2 * q + 1] * corr + pr * __uint_as_float(vw[q] & 0xffff0000u);
            }
            m[h] = m_new;
          }
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; h++) {
    float* dst = comb + (tl * 4 + 2 * hp + h) * (kD + 2);
    if (lane == 0) {
      dst[0] = m[h];
      dst[1] = l[h];
    }
    float2* d2 = (float2*)(dst + 2 + lane * 8);
    d2[0] = make_float2(acc[h][0], acc[h][1]);
    d2[1] = make_float2(acc[h][2], acc[h][3]);
    d2[2] = make_float2(acc[h][4], acc[h][5]);
    d2[3] = make_float2(acc[h][6], acc[h][7]);
  }
  bar_consumers();
  // ---- merge the 8 token lanes: thread = (head, pair of dims) ----
  {
    float2* part_ml = (float2*)(a.scratch + a.attn_ml_off);
    float* part_acc = (float*)(a.scratch + a.attn_part_off);
    const int h = tid >> 7, d2 = tid & 127;
    if (h < a.n_q) {
      float mm = -INFINITY;
#pragma unroll
      for (int q = 0; q < kTokenLanes; q++) mm = fmaxf(mm, comb[(q * 4 + h) * (kD + 2)]);
      float ll = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int q = 0; q < kTokenLanes; q++) {
        const float* cq = comb + (q * 4 + h) * (kD + 2);
        if (cq[1] > 0.f) {
          const float e = expf(cq[0] - mm);
          const float2 av = *(const float2*)(cq + 2 + 2 * d2);
          ll += cq[1] * e;
          o0 += av.x * e;
          o1 += av.y * e;
        }
      }
      const size_t row = ((size_t)b * a.n_q + h) * G + blk;
      if (d2 == 0) part_ml[row] = make_float2(mm, ll);
      *(float2*)(part_acc + row * kD + 2 * d2) = make_float2(o0, o1);
    }
  }
}

// Stage 2: columns [C * blk / G, C * (blk + 1) / G) of the B * n_q * 256 attention outputs. A warp
// merges one column at a time: lanes take slices s = lane, lane + 32, ...; fixed order everywhere.
__device__ void attention_merge(const DecodeStepArgs& a, int blk, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  const int G = a.grid;
  const int C = a.B * a.n_q * kD;
  const int c_first = (int)((long long)C * blk / G), c_end = (int)((long long)C * (blk + 1) / G);
  const float2* part_ml = (const float2*)(a.scratch + a.attn_ml_off);
  const float* part_acc = (const float*)(a.scratch + a.attn_part_off);
  uint16_t* out = (uint16_t*)(a.scratch + a.attn_out_off);
  constexpr int kPerLane = 8;  // up to 256 slices (CTAs)
  for (int c = c_first + warp; c < c_end; c += kConsumerWarps) {
    const int bh = c / kD, d = c % kD;
    float2 ml[kPerLane];
    float av[kPerLane];
#pragma unroll
    for (int j = 0; j < kPerLane; j++) {
      const int s = lane + 32 * j;
      ml[j] = make_float2(-INFINITY, 0.f);
      av[j] = 0.f;
      if (s < G) {
        ml[j] = __ldcg(part_ml + (size_t)bh * G + s);
        av[j] = __ldcg(part_acc + ((size_t)bh * G + s) * kD + d);
      }
    }
    float mm = -INFINITY;
#pragma unroll
    for (int j = 0; j < kPerLane; j++) mm = fmaxf(mm, ml[j].x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int j = 0; j < kPerLane; j++)
      if (ml[j].y > 0.f) {
        const float e = expf(ml[j].x - mm);
        ll += ml[j].y * e;
        oo += av[j] * e;
      }
    ll = warp_sum(ll);
    oo = warp_sum(oo);
    if (lane == 0) out[c] = f2bf(oo / ll);
  }
}

// Input of the o projection: the attention output (bf16, global), staged as guarded fp16.
template <int BT>
__device__ __forceinline__ void stage_attention(const DecodeStepArgs& a, const Smem& sm, int xin_stride, int tid) {
  const uint16_t* src = (const uint16_t*)(a.scratch + a.attn_out_off);
  char* xin = sm.base + sm.off_xin;
  float* red = (float*)(sm.base + sm.off_red);
  float* xscale = (float*)(sm.base + sm.off_red + kRedXscale);
  // this GPU's K slice of the o projection: columns [o_k_offset, o_k_offset + o_k) of the local attention output
  const int width = a.n_q * kD, vec = a.o_k / 8;  // <= 128 vectors of 8 values per batch row
  uint4 v[BT];
  float amax[BT];
#pragma unroll
  for (int b = 0; b < BT; b++) {
    amax[b] = 0.f;
    v[b] = make_uint4(0, 0, 0, 0);
    if (b < a.B && tid < vec) {
      v[b] = __ldcg((const uint4*)(src + (size_t)b * width + a.o_k_offset) + tid);
      const uint32_t w[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
#pragma unroll
      for (int j = 0; j < 4; j++)
        amax[b] = fmaxf(amax[b], fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xffff0000u))));
    }
  }
  consumer_reduce<BT, true>(amax, red, tid);
#pragma unroll
  for (int b = 0; b < BT; b++) {
    float down;
    const float up = fp16_guard(amax[b], down);
    if (tid == 0 && b < a.B) xscale[b] = up;
    if (b < a.B && tid < vec) {
      const uint32_t w[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const __half2 h2 = __floats2half2_rn(__uint_as_float(w[j] << 16) * down, __uint_as_float(w[j] & 0xffff0000u) * down);
        o[j] = *(const uint32_t*)&h2;
      }
      *(uint4*)(xin + (size_t)b * xin_stride + 16 * tid) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  bar_consumers();
}

// Input of the down projection: the GeGLU output written by all CTAs, staged as guarded fp16.
template <int BT>
__device__ __forceinline__ void stage_activations(const DecodeStepArgs& a, const Smem& sm, int xin_stride, int tid) {
  const uint16_t* act = (const uint16_t*)(a.scratch + a.act_off);
  char* xin = sm.base + sm.off_xin;
  float* red = (float*)(sm.base + sm.off_red);
  float* xscale = (float*)(sm.base + sm.off_red + kRedXscale);
  const int vec = a.I / 8;
  float amax[BT];
#pragma unroll
  for (int b = 0; b < BT; b++) amax[b] = 0.f;
  for (int c = tid; c < vec; c += kConsumerThreads)
#pragma unroll
    for (int b = 0; b < BT; b++)
      if (b < a.B) {
        const uint4 v = __ldcg((const uint4*)(act + (size_t)b * a.I) + c);
        *(uint4*)(xin + (size_t)b * xin_stride + 16 * c) = v;  // raw bf16 for now
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++)
          amax[b] = fmaxf(amax[b], fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xffff0000u))));
      }
  consumer_reduce<BT, true>(amax, red, tid);
  float down[BT];
#pragma unroll
  for (int b = 0; b < BT; b++) {
    const float up = fp16_guard(amax[b], down[b]);
    if (tid == 0 && b < a.B) xscale[b] = up;
  }
  for (int c = tid; c < vec; c += kConsumerThreads)
#pragma unroll
    for (int b = 0; b < BT; b++)
      if (b < a.B) {
        uint4* p = (uint4*)(xin + (size_t)b * xin_stride + 16 * c);
        const uint4 v = *p;
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const __half2 h2 = __floats2half2_rn(__uint_as_float(w[j] << 16) * down[b],
                                               __uint_as_float(w[j] & 0xffff0000u) * down[b]);
          o[j] = *(const uint32_t*)&h2;
        }
        *p = make_uint4(o[0], o[1], o[2], o[3]);
      }
  bar_consumers();
}

// ------------------------------------------------------------------------------------------
// Reducer warp: adds the 16 partial tiles in warp order and applies the stage's epilogue
// ------------------------------------------------------------------------------------------
struct ArgBest {
  float v[2];
  int i[2];
};
struct TileScales {
  float lo, hi;
};
__device__ __forceinline__ TileScales load_tile_scales(const Phase& p, int t, int g) {
  TileScales s;
  s.lo = s.hi = 0.f;
  if (t < p.ntiles) {
    const int r_lo = tile_row(p, t, g), r_hi = tile_row(p, t, g + 8);
    if (r_lo >= 0) s.lo = bf2f(__ldg(p.scale + r_lo));
    if (r_hi >= 0) s.hi = bf2f(__ldg(p.scale + r_hi));
  }
  return s;
}
__device__ __forceinline__ void reduce_phase(const DecodeStepArgs& a, const Phase& p, const Smem& sm, int nslots,
                                             RingPos& tile, int* status, bool& ok, int lane, void* out, unsigned long long inbox,
                                             uint32_t tag, ArgBest* best) {
  const int g = lane >> 2, tig = lane & 3;
  const float* xscale = (const float*)(sm.base + sm.off_red + kRedXscale);
  // the scales of the next tiles are requested ahead: their latency must not sit between two tiles
  TileScales q0 = load_tile_scales(p, 0, g), q1 = load_tile_scales(p, 1, g), q2 = load_tile_scales(p, 2, g),
             q3 = load_tile_scales(p, 3, g);
  for (int t = 0; t < p.ntiles; t++) {
    const int r_lo = tile_row(p, t, g), r_hi = tile_row(p, t, g + 8);
    const TileScales cur = q0;
    q0 = q1; q1 = q2; q2 = q3;
    q3 = load_tile_scales(p, t + 4, g);
    const uint32_t buf = tile.idx, round = tile.wraps;
    tile.advance(2);
    ok = mbar_wait(sm.bars + 8 * (2 * nslots + buf), round & 1, status, kErrPartFull, ok);
    const float4* src = (const float4*)(sm.base + sm.off_part) + (buf * kPartFloats / 4 + lane);
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < kConsumerWarps; w++) {
      const float4 v = src[w * 32];
      c[0] += v.x; c[1] += v.y; c[2] += v.z; c[3] += v.w;
    }
    const int b0 = 2 * tig, b1 = 2 * tig + 1;
    const float xs0 = xscale[b0], xs1 = xscale[b1];  // written by the consumers before this tile's products
    __syncwarp();
    if (lane == 0 && ok) mbar_arrive(sm.bars + 8 * (2 * nslots + 2 + buf));
    c[0] *= xs0; c[1] *= xs1; c[2] *= xs0; c[3] *= xs1;  // exact: powers of two
    const float s_lo = cur.lo, s_hi = cur.hi;
    if (p.kind == kRows && inbox) {
      // tensor parallel, K split over the GPUs: fp32 partial result, tagged, to every GPU's inbox [rank][B][N]
      for (int r = 0; r < a.tp; r++) {
        float* y = (float*)(a.peer_scratch[r] + inbox) + 2 * (size_t)a.rank * a.B * p.N;
        if (r_lo >= 0) {
          if (b0 < a.B) st_tagged_sys(y + 2 * ((size_t)b0 * p.N + r_lo), c[0] * s_lo, tag);
          if (b1 < a.B) st_tagged_sys(y + 2 * ((size_t)b1 * p.N + r_lo), c[1] * s_lo, tag);
        }
        if (r_hi >= 0) {
          if (b0 < a.B) st_tagged_sys(y + 2 * ((size_t)b0 * p.N + r_hi), c[2] * s_hi, tag);
          if (b1 < a.B) st_tagged_sys(y + 2 * ((size_t)b1 * p.N + r_hi), c[3] * s_hi, tag);
        }
      }
    } else if (p.kind == kRows) {
      uint32_t* y = (uint32_t*)out;  // tagged words: the store is the signal
      const uint32_t th = tag << 16;
      if (r_lo >= 0) {
        if (b0 < a.B) y[(size_t)b0 * p.N + r_lo] = th | f2bf(c[0] * s_lo);
        if (b1 < a.B) y[(size_t)b1 * p.N + r_lo] = th | f2bf(c[1] * s_lo);
      }
      if (r_hi >= 0) {
        if (b0 < a.B) y[(size_t)b0 * p.N + r_hi] = th | f2bf(c[2] * s_hi);
        if (b1 < a.B) y[(size_t)b1 * p.N + r_hi] = th | f2bf(c[3] * s_hi);
      }
    } else if (p.kind == kPairs) {
      // rows g hold gate, rows g+8 the matching up row: act = bf16(bf16(gelu(gate)) * up). This vector is
      // 6 times longer than the others: plain bf16 and a grid barrier (tagged words would double what every
      // CTA has to read through its load/store unit).
      uint16_t* y = (uint16_t*)out;
      if (r_lo >= 0) {
        const int col = r_lo;  // index inside the intermediate vector
        if (b0 < a.B) y[(size_t)b0 * p.N + col] = f2bf(rbf(gelu_tanh(rbf(c[0] * s_lo))) * rbf(c[2] * s_hi));
        if (b1 < a.B) y[(size_t)b1 * p.N + col] = f2bf(rbf(gelu_tanh(rbf(c[1] * s_lo))) * rbf(c[3] * s_hi));
      }
    } else {
      const float v[4] = {c[0] * s_lo, c[1] * s_lo, c[2] * s_hi, c[3] * s_hi};
      const int rr[4] = {r_lo, r_lo, r_hi, r_hi};
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int bb = (q & 1) ? b1 : b0;
        if (rr[q] >= 0 && bb < a.B) {
          if (a.logits) a.logits[(size_t)bb * p.N + rr[q]] = v[q];
          if (v[q] > best->v[q & 1]) {  // rows are visited in rising order: ties keep the lower index
            best->v[q & 1] = v[q];
            best->i[q & 1] = rr[q] + a.vocab_offset;
          }
        }
      }
    }
  }
}

template <int BT>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const DecodeStepArgs a) {
  extern __shared__ __align__(128) char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blk = blockIdx.x, G = gridDim.x;
  const int nslots = a.nslots;
  Smem sm;
  sm.base = smem_raw;
  sm.ring = smem_u32(smem_raw);
  sm.off_xin = (uint32_t)nslots * kSlotBytes;
  sm.off_xs = sm.off_xin + a.xin_bytes;
  sm.off_part = sm.off_xs + (((uint32_t)a.B * a.H * 2 + 127) & ~127u);
  sm.off_red = sm.off_part + 2 * kPartFloats * 4;
  sm.off_bars = sm.off_red + kRedBytes;
  sm.xin_addr = sm.ring + sm.off_xin;
  sm.bars = sm.ring + sm.off_bars;
  const int xin_stride = a.xin_stride;
  const DecodeLayerDesc* layers = (const DecodeLayerDesc*)(a.consts + a.layers_off);
  const unsigned long long* bases = (const unsigned long long*)(a.scratch + a.counter_off + 24);
  // epoch of the tagged hand-overs: one per (launch, layer, projection); the tag is its low 16 bits
  const uint32_t epoch_base = *(const uint32_t*)(a.scratch + a.counter_off + 56);
  auto tag_of = [&](int layer, int which) { return (epoch_base + 4u * (uint32_t)layer + (uint32_t)which + 1u) & 0xffffu; };
  int* status = a.status;
  volatile int* gave_up = (volatile int*)(smem_raw + sm.off_bars + 8 * (2 * nslots + 4));

  if (tid == 0) {
    for (int s = 0; s < nslots; s++) {
      mbar_init(sm.bars + 8 * s, 1);                          // full: the producer's expect_tx arrival
      mbar_init(sm.bars + 8 * (nslots + s), kConsumerWarps);  // empty: one arrival per consumer warp
    }
    for (int i = 0; i < 2; i++) {
      mbar_init(sm.bars + 8 * (2 * nslots + i), kConsumerWarps);  // partial tile written
      mbar_init(sm.bars + 8 * (2 * nslots + 2 + i), 1);           // partial tile read
    }
    *gave_up = 0;
    s_wait_limit_ns = a.wait_ns;
    // rows of each projection owned by this CTA (the same in every layer)
    int* rf = (int*)(smem_raw + sm.off_red + kRedRows);
    const int rows_of[5] = {(a.n_q + 2) * kD, a.H, a.I, a.H, a.V};
    for (int w = 0; w < 5; w++) {
      rf[w] = (int)((long long)rows_of[w] * blk / G);
      rf[5 + w] = (int)((long long)rows_of[w] * (blk + 1) / G) - rf[w];
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  const int* row_first = (const int*)(smem_raw + sm.off_red + kRedRows);
  const int* row_count = row_first + 5;
  bool ok = true;
  BarrierState bs;  // followed by the consumer threads; thread 0 stores it for the next launch
  bs.local = bases[0];
  bs.global[0] = bases[1];
  bs.global[1] = bases[2];
  bs.parity = *(const int*)(a.scratch + a.counter_off + 60);
  if (warp == kProducerWarp) {
    // ---------------- producer: stream this CTA's weight rows, in consumption order ----------------
    RingPos pc{0, 0};
    uint32_t issued = 0;
    for (int l = 0; l <= a.n_layers; l++) {
      const int first_phase = l < a.n_layers ? kQkv : kLmHead, last_phase = l < a.n_layers ? kDown : kLmHead;
      for (int which = first_phase; which <= last_phase; which++) {
        const Phase p = make_phase(a, layers + (l < a.n_layers ? l : 0), which, row_first, row_count);
        for (int t = 0; t < p.ntiles; t++) {
          const int row = lane < 16 ? tile_row(p, t, lane) : -1;
          const int nvalid = __popc(__ballot_sync(0xffffffffu, row >= 0));
          for (int s = 0; s < p.nseg; s++) {
            const uint32_t slot = pc.idx, use = pc.wraps;
            pc.advance(nslots);
            issued++;
            if (use > 0) ok = mbar_wait(sm.bars + 8 * (nslots + slot), (use - 1) & 1, status, kErrEmpty, ok);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) continue;  // nothing more is issued after a failed wait
            const int seg_bytes = min(p.seg, p.K - s * p.seg);
            const uint32_t full = sm.bars + 8 * slot, dst = sm.ring + slot * kSlotBytes;
            if (lane == 0) mbar_expect_tx(full, (uint32_t)(nvalid * seg_bytes));
            __syncwarp();
            if (p.whole) {
              // rows 0..n-1 (and, for gate/up, rows 8..8+n-1) of the slot are runs of consecutive rows
              const int runs = p.kind == kPairs ? 2 : 1, n = nvalid / runs;
              if (lane < runs)
                bulk_g2s(dst + lane * 8 * p.stride, p.W + (size_t)tile_row(p, t, lane * 8) * p.K, (uint32_t)(n * p.K), full);
            } else if (row >= 0) {
              bulk_g2s(dst + lane * p.stride, p.W + (size_t)row * p.K + (size_t)s * p.seg, (uint32_t)seg_bytes, full);
            }
          }
        }
      }
    }
    // On the failure path the consumers may have stopped waiting: make sure every copy that was
    // issued has landed before the CTA can exit.
    if (!ok && lane == 0) {
      for (uint32_t q = issued > (uint32_t)nslots ? issued - nslots : 0; q < issued; q++) {
        const unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(sm.bars + 8 * (q % nslots), (q / nslots) & 1) && globaltimer_ns() - t0 < 100000000ull) {
        }
      }
    }
  } else if (warp == kReducerWarp) {
    // ---------------- reducer ----------------
    RingPos tiles{0, 0};
    int gpar = bs.parity;  // which of the two cross-GPU counter pairs the next cross-GPU barrier uses
    ArgBest best;
    best.v[0] = best.v[1] = -INFINITY;
    best.i[0] = best.i[1] = 0x7fffffff;
    for (int l = 0; l < a.n_layers; l++) {
      const DecodeLayerDesc* L = layers + l;
      for (int which = kQkv; which <= kDown; which++) {
        const Phase p = make_phase(a, L, which, row_first, row_count);
        void* out = a.scratch + (which == kQkv ? a.qkv_off : which == kO ? a.o_off : which == kGateUp ? a.act_off : a.d_off);
        // o and down are split along K over the tensor-parallel GPUs: partial results to every inbox
        const bool split_k = a.tp > 1 && (which == kO || which == kDown);
        reduce_phase(a, p, sm, nslots, tiles, status, ok, lane, out,
                     split_k ? (which == kO ? a.inbox_o_off : a.inbox_d_off) : 0ull, tag_of(l, which), &best);
        if (which == kGateUp) {  // the long activation vector: grid barrier
          __threadfence();
          __syncwarp();
          if (lane == 0) grid_arrive(a, false, 0, false);
        }  // otherwise the tagged words are the signal
      }
    }
    {
      const Phase p = make_phase(a, layers, kLmHead, row_first, row_count);
      reduce_phase(a, p, sm, nslots, tiles, status, ok, lane, nullptr, 0ull, 0u, &best);
      // lanes with the same token pair differ in bits 2..4
#pragma unroll
      for (int q = 0; q < 2; q++) {
        float v = best.v[q];
        int i = best.i[q];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, o);
          const int oi = __shfl_xor_sync(0xffffffffu, i, o);
          if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
          }
        }
        const int bb = 2 * (lane & 3) + q;
        if ((lane >> 2) == 0 && bb < a.B) {
          // every GPU collects every GPU's candidates: [rank][CTA][8] values, then the same of indices
          for (int r = 0; r < a.tp; r++) {
            float* pv = (float*)(a.peer_scratch[r] + a.amax_off);
            int* pi = (int*)(pv + (size_t)a.tp * G * 8);
            pv[((size_t)a.rank * G + blk) * 8 + bb] = v;
            pi[((size_t)a.rank * G + blk) * 8 + bb] = i;
          }
        }
      }
      if (a.tp > 1) __threadfence_system();
      else __threadfence();
      __syncwarp();
      if (lane == 0) grid_arrive(a, true, gpar, false);
    }
  } else {
    // ---------------- consumers ----------------
    uint16_t* xs = (uint16_t*)(smem_raw + sm.off_xs);
    char* xin = smem_raw + sm.off_xin;
    float* red = (float*)(smem_raw + sm.off_red);
    RingPos slots{0, 0}, tiles{0, 0};
    // all_gpus: the barrier follows a stage whose results cross the tensor-parallel GPUs
    auto wait_grid = [&](bool all_gpus, bool poll = true) {
      const bool sys = all_gpus && a.tp > 1;
      unsigned long long target;
      const int parity = bs.parity;
      if (sys) {
        target = (bs.global[parity] += (unsigned long long)a.tp);
        bs.parity ^= 1;
      } else {
        target = (bs.local += (unsigned long long)G);
      }
      if (!poll) return;  // only the count is advanced
      if (tid == 0) {
        const bool r = grid_wait(a, sys, parity, target, status, ok);
        if (!r) *gave_up = 1;
      }
      bar_consumers();
      if (*gave_up) ok = false;
    };
    // RoPE tables for this position: (cos, sin)(pos * theta^(-i/128)) for the (at most two) bases
    if (tid < 256) {
      int pos = __ldg(a.pos);
      pos = pos < 0 ? 0 : (pos >= a.T ? a.T - 1 : pos);
      const int i = tid & 127;
      const float inv_freq = powf(a.theta[tid >> 7], -(float)i / 128.0f);
      float sn, cs;
      sincosf((float)pos * inv_freq, &sn, &cs);
      ((float2*)(smem_raw + sm.off_red + kRedRope))[tid] = make_float2(cs, sn);
    }
    // embedding: xs[b, i] = bf16(bf16(E[tok, i] * scale[tok]) * mult)
    for (int b = 0; b < a.B; b++) {
      int tk = __ldg(a.tokens + b);
      tk = tk < 0 ? 0 : (tk >= a.V_embed ? a.V_embed - 1 : tk);
      const float s = bf2f(__ldg((const uint16_t*)(a.consts + a.embed_s) + tk));
      const int8_t* row = (const int8_t*)(a.consts + a.embed_w) + (size_t)tk * a.H;
      for (int i = tid; i < a.H; i += kConsumerThreads) xs[b * a.H + i] = f2bf(rbf((float)row[i] * s) * a.embed_mult);
    }
    prefetch_layer_constants(a, layers, tid);
    bar_consumers();
    int mark = 0;
    trace_mark(a, blk, tid, mark);
    for (int l = 0; l < a.n_layers; l++) {
      const DecodeLayerDesc* L = layers + l;
      prefetch_keys(a, L, blk, warp, lane);  // well ahead of the attention stage
      if (l + 1 < a.n_layers) prefetch_layer_constants(a, layers + l + 1, tid);
      // ---- qkv projection (input: norm of the residual stream, updated with the previous layer's MLP output) ----
      {
        const NormWeights nw = load_norm_weights(l > 0 ? (const uint16_t*)(a.consts + layers[l - 1].post_ffn_norm) : nullptr,
                                                 (const uint16_t*)(a.consts + L->in_norm), a.H, tid);
        trace_mark(a, blk, tid, mark);
        residual_norm<BT>(a, l > 0 ? (const uint32_t*)(a.scratch + a.d_off) : nullptr, tag_of(l - 1, kDown), a.inbox_d_off, nw, xs,
                          xin, xin_stride, red, tid, status, ok);
      }
      trace_mark(a, blk, tid, mark);
      consume_phase(make_phase(a, L, kQkv, row_first, row_count), sm, nslots, a.B, xin_stride, slots, tiles, status, ok, warp, lane);
      trace_mark(a, blk, tid, mark);
      // ---- attention over the cache: slices, barrier, merge ----
      {
        const HeadNormWeights hw = load_head_norm_weights(a, L, warp, lane);
        bar_consumers();  // every warp is done with the staged activations: their space becomes attention scratch
        trace_mark(a, blk, tid, mark);
        for (int b = 0; b < a.B; b++) {
          attention_slice(a, L, sm, hw, b, blk, tid, tag_of(l, kQkv), status, ok);
          bar_consumers();
        }
      }
      if (tid == 0) grid_arrive(a, false, 0);
      trace_mark(a, blk, tid, mark);
      wait_grid(false);
      trace_mark(a, blk, tid, mark);
      attention_merge(a, blk, tid);
      bar_consumers();
      if (tid == 0) grid_arrive(a, false, 0);
      trace_mark(a, blk, tid, mark);
      // ---- o projection ----
      wait_grid(false);
      trace_mark(a, blk, tid, mark);
      stage_attention<BT>(a, sm, xin_stride, tid);
      trace_mark(a, blk, tid, mark);
      consume_phase(make_phase(a, L, kO, row_first, row_count), sm, nslots, a.B, xin_stride, slots, tiles, status, ok, warp, lane);
      trace_mark(a, blk, tid, mark);
      // ---- gate/up projection + GeGLU ----
      {
        const NormWeights nw = load_norm_weights((const uint16_t*)(a.consts + L->post_attn_norm),
                                                 (const uint16_t*)(a.consts + L->pre_ffn_norm), a.H, tid);
        trace_mark(a, blk, tid, mark);
        residual_norm<BT>(a, (const uint32_t*)(a.scratch + a.o_off), tag_of(l, kO), a.inbox_o_off, nw, xs, xin, xin_stride, red, tid,
                          status, ok);
      }
      trace_mark(a, blk, tid, mark);
      consume_phase(make_phase(a, L, kGateUp, row_first, row_count), sm, nslots, a.B, xin_stride, slots, tiles, status, ok, warp, lane);
      trace_mark(a, blk, tid, mark);
      // ---- down projection ----
      wait_grid(false);
      trace_mark(a, blk, tid, mark);
      stage_activations<BT>(a, sm, xin_stride, tid);
      trace_mark(a, blk, tid, mark);
      consume_phase(make_phase(a, L, kDown, row_first, row_count), sm, nslots, a.B, xin_stride, slots, tiles, status, ok, warp, lane);
      trace_mark(a, blk, tid, mark);
    }
    {
      const NormWeights nw = load_norm_weights((const uint16_t*)(a.consts + layers[a.n_layers - 1].post_ffn_norm),
                                               (const uint16_t*)(a.consts + a.final_norm), a.H, tid);
      trace_mark(a, blk, tid, mark);
      residual_norm<BT>(a, (const uint32_t*)(a.scratch + a.d_off), tag_of(a.n_layers - 1, kDown), a.inbox_d_off, nw, xs, xin,
                        xin_stride, red, tid, status, ok);
    }
    trace_mark(a, blk, tid, mark);
    consume_phase(make_phase(a, layers, kLmHead, row_first, row_count), sm, nslots, a.B, xin_stride, slots, tiles, status, ok, warp, lane);
    trace_mark(a, blk, tid, mark);
    wait_grid(true, blk == 0);  // only CTA 0 needs the other CTAs' candidates
    if (blk == 0) {
      trace_mark(a, blk, tid, mark);
      // greedy ids: best (value, lowest index) over the candidates of every CTA of every GPU
      const int cand = a.tp * G;
      const float* pv = (const float*)(a.scratch + a.amax_off);
      const int* pi = (const int*)(pv + (size_t)cand * 8);
      if (warp < a.B) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c = lane; c < cand; c += 32) {
          const float ov = __ldcg(pv + c * 8 + warp);
          const int oi = __ldcg(pi + c * 8 + warp);
          if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, o);
          const int oi = __shfl_xor_sync(0xffffffffu, i, o);
          if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
          }
        }
        if (lane == 0) a.out_ids[warp] = ok ? i : -1;
      }
    }
  }
  __syncthreads();
  // the last CTA to leave stores where the counters will stand once this launch's counts are all
  // in: the bases of the next launch
  if (tid == 0) {
    unsigned int* exit_count = (unsigned int*)(a.scratch + a.counter_off + 48);
    const unsigned int old = atomicAdd(exit_count, 1u);
    if (old == (unsigned int)G - 1) {
      unsigned long long* next = (unsigned long long*)(a.scratch + a.counter_off + 24);
      next[0] = bs.local;
      next[1] = bs.global[0];
      next[2] = bs.global[1];
      *(int*)(a.scratch + a.counter_off + 60) = bs.parity;
      *(uint32_t*)(a.scratch + a.counter_off + 56) = epoch_base + 4u * (uint32_t)a.n_layers;
      *exit_count = 0;
      __threadfence();
    }
  }
}

}  // namespace

// Shared-memory plan for batch B: activation staging (bf16 rows of the longest projection
// input, padded so that consecutive tokens start 16 bytes apart modulo 128), residual stream,
// two partial-tile buffers, reduction scratch, barriers; the rest becomes ring slots.
bool decode_step_supported(int B, int H, int n_q, int n_kv, int D, int I, int V) {
  return B >= 1 && B <= 8 && n_kv == 1 && D == kD && n_q >= 1 && n_q <= 4 && H % 64 == 0 && I % 64 == 0 &&
         (n_q * D) % 64 == 0 && V >= 16 && H <= kSegBytes && I <= 32768;
}

namespace {
struct SmemPlan {
  int nslots, xin_stride, xin_bytes, total;
};
SmemPlan plan_smem(int B, int H, int n_q, int I, int max_bytes) {
  SmemPlan s;
  int kmax = H > I ? H : I;
  if (n_q * kD > kmax) kmax = n_q * kD;
  s.xin_stride = ((kmax * 2 + 127) / 128) * 128 + 16;
  s.xin_bytes = B * s.xin_stride;
  const int attn_scratch = kAttnScratchBytes;
  if (s.xin_bytes < attn_scratch) s.xin_bytes = attn_scratch;
  s.xin_bytes = (s.xin_bytes + 127) & ~127;
  const int fixed = s.xin_bytes + ((B * H * 2 + 127) & ~127) + 2 * kPartFloats * 4 + kRedBytes + 8 * (2 * 16 + 4 + 1) + 128;
  s.nslots = (max_bytes - fixed) / kSlotBytes;
  if (s.nslots > 16) s.nslots = 16;
  s.total = fixed + s.nslots * kSlotBytes;
  return s;
}
}  // namespace

size_t decode_step_scratch_bytes(int B, int H, int n_q, int I, int n_layers, int sm_count, int tp, DecodeStepArgs* offsets) {
  // qkv | o | act | d (bf16), attention partials, arg-max partials, barrier counters
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += (bytes + 255) & ~(size_t)255;
    return at;
  };
  // Regions that other GPUs write come first: their offsets depend only on B, H, the group size and the
  // SM count, which are the same on every member (a shard's MLP width may differ from its peers').
  offsets->counter_off = take(256);
  offsets->amax_off = take((size_t)tp * sm_count * 8 * 8);
  offsets->inbox_o_off = tp > 1 ? take((size_t)tp * B * H * 8) : 0;  // tagged 64-bit words
  offsets->inbox_d_off = tp > 1 ? take((size_t)tp * B * H * 8) : 0;
  // projection outputs as tagged 32-bit words
  offsets->qkv_off = take((size_t)B * (n_q + 2) * kD * 4);
  offsets->o_off = take((size_t)B * H * 4);
  offsets->act_off = take((size_t)B * I * 2);  // plain bf16
  offsets->d_off = take((size_t)B * H * 4);
  offsets->attn_slices = sm_count;
  offsets->attn_out_off = take((size_t)B * n_q * kD * 2);
  offsets->attn_ml_off = take((size_t)B * n_q * sm_count * 8);
  offsets->attn_part_off = take((size_t)B * n_q * sm_count * kD * 4);
  offsets->trace_len = 16 * n_layers + 8;
  offsets->trace_off = take((size_t)offsets->trace_len * 8);
  return off;
}

cudaError_t launch_decode_step(DecodeStepArgs a, cudaStream_t stream) {
  int dev = 0, sms = 0, max_smem = 0, coop = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (!coop) return cudaErrorNotSupported;
  const SmemPlan sp = plan_smem(a.B, a.H, a.n_q, a.I, max_smem);
  if (sp.nslots < 2) return cudaErrorInvalidConfiguration;
  a.nslots = sp.nslots;
  a.xin_stride = sp.xin_stride;
  a.xin_bytes = sp.xin_bytes;
  a.wait_ns = wait_limit_ns();
  void (*kernel)(const DecodeStepArgs) = a.B <= 1 ? decode_step_kernel<1>
                                         : a.B <= 2 ? decode_step_kernel<2>
                                         : a.B <= 4 ? decode_step_kernel<4>
                                                    : decode_step_kernel<8>;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.total);
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, sp.total);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorInvalidConfiguration;
  if (a.grid != sms) return cudaErrorInvalidValue;  // the scratch layout was sized for this many CTAs
  void* params[] = {&a};
  return cudaLaunchCooperativeKernel((const void*)kernel, dim3(sms), dim3(kThreads), params, (size_t)sp.total, stream);
}

}  // namespace tb200
