// int8 GEMM on the 5th-generation tensor cores (tcgen05.mma kind::i8) with the
// requantising epilogue fused: the kernel behind 1x1 convolutions and
// fully_connected (a 1x1 conv on NHWC is the row-major GEMM
// [N*H*W, IC] x [OC, IC]^T, compiler/torq/Conversions/LinalgToTorqHL/Conv2DMatmulPattern.cpp:47-57).
//
//   out[m, n] = clamp( apply_scale_32( sum_k A[m,k] * W[n,k] + bias'[n], M[n], S[n] ) + ozp )
//
// bias' already holds bias - izp * sum_k W[n,k] (1x1 convs have no padding, so the
// input zero point folds into a per-channel constant).
//
// These GEMMs are skinny (K = 16..1280 bytes per row, M in the millions) and bound by
// HBM and by the integer epilogue, not by the tensor pipe. The structure follows from that:
//   * one persistent CTA per SM, 576 threads;
//   * warp 0 = TMA producer. The swizzle width follows K (32 / 64 / 128-byte rows), so a
//     stage of A is 128 rows x 32..128 B and the ring holds up to 16 stages: many small
//     loads in flight instead of a few padded ones;
//   * when the whole weight matrix fits (<= 96 KB) it is loaded into shared memory once
//     and stays; otherwise its tile travels with each A stage;
//   * warp 1 = MMA issuer, one elected lane, accumulators in TMEM, 4 stages of <= 128 columns;
//   * warps 2..17 = epilogue, the part that bounds the kernel (about a dozen integer
//     instructions per output): 4 groups of 4 warps, group g drains accumulator stage g,
//     so 16 warps keep the schedulers busy. tcgen05.ld 32 columns, int64 rescale on CUDA
//     cores from 16-byte per-channel constants in shared memory, packed clamp; the int8
//     tile is staged in shared memory and leaves with one TMA store, so global memory sees
//     full lines instead of 16-byte pieces at a row stride;
//   * single-thread roles carry no divisions: tile coordinates and ring indices advance
//     incrementally.
// The same kernel runs KH x KW convolutions as implicit GEMM (CONV = true): an M tile is a
// TH x TW patch of output pixels of one image (TH * TW = 128); for every tap (kh, kw) and block
// of input channels the producer loads the patch's input pixels with ONE 4-D TMA box
// {channels, TW pixels at the conv stride, TH rows at the conv stride, 1 image} whose start is
// shifted by the tap, and the issuer accumulates all taps into the same TMEM tile (K runs over
// (kh, kw, ic), the order of OHWI weights). Padding costs nothing: out-of-range pixels are
// zero-filled by the copy engine. Zero fill means "x = 0", while the op pads with the input zero
// point, so border pixels get a per-class correction izp * sum of the padded taps' weights,
// added in the epilogue from a small table (classes = which rows x which columns of the window
// fall outside). The output tile leaves through a 4-D TMA store, which clips ragged edges.
// Every mbarrier wait is bounded: on expiry the kernel records a code in the device
// status word and every role drains to the common exit, where TMEM is freed.
#include <cuda.h>
#include <type_traits>
#include <cuda_runtime.h>

#include <cstdlib>
#include <mutex>

#include "kernels.h"
#include "tcgen05_ptx.cuh"
#include "dependent_launch.cuh"

namespace tb200 {

namespace {

constexpr int kBM = 128;
constexpr int kMaxStages = 16;
constexpr int kEpiGroups = 4;                    // each group = 4 warps = the 128 TMEM lanes of one accumulator
constexpr int kEpiWarps = 4 * kEpiGroups;
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kSmemBudget = 216 * 1024;          // dynamic shared memory the kernel may use (227 KB less the static part)
constexpr int kResidentWeightBytes = 64 * 1024;  // weights up to this size stay in shared memory

// Debugging aid (TB200_GEMM_TRACE=1): CTA 0 records %globaltimer stamps of its roles, 512 slots per role
// (0 producer, 1 MMA issuer, 2.. epilogue groups); tb200_debug_read_gemm_trace copies them out.
constexpr int kTraceSlots = 512;
__device__ unsigned long long g_gemm_trace[6 * kTraceSlots];
__device__ __forceinline__ void trace_stamp(int on, int role, int& idx, unsigned tag) {
  if (on && blockIdx.x == 0 && idx < kTraceSlots) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_gemm_trace[role * kTraceSlots + idx++] = (t << 8) | tag;
  }
}

struct GemmTcParams {
  int trace;
  const ChanParams* chan;
  int8_t* out;
  long long ldc;
  int M, N, BN, n_tiles, m_tiles, k_blocks, k_last_steps;
  int row_bytes;        // 32, 64 or 128: bytes of K per shared-memory row (= swizzle width)
  int stages;           // A (or A+W) ring depth
  int w_resident;       // weights loaded once
  int out_zp, clamp_min, clamp_max;
  const int4* q4;       // compact per-channel records of the EPI 1 / 2 kernels
  int acc_stride, acc_stages, tmem_cols;
  int gpt, BNh;         // epilogue groups per accumulator (1 or 2) and the columns each of them drains (BN / gpt)
  // implicit-GEMM convolution (CONV kernels): tile = TH x TW output pixels, TW a power of two
  int tw_log2, TH, tiles_w, tiles_per_img, OH, OW, cstride, pad_t, pad_l, KW, icb_per_tap;
  // khs > 1 (stride-1 convolutions, TW >= 8): one load per (kw, channel block) brings the TH + khs - 1 input rows all
  // khs kernel rows of that column need; the operand of kernel row kh starts kh * TW rows into the stage, a whole
  // number of 8-row swizzle atoms, so the descriptors stay the plain K-major ones. k_loads = stage loads per tile.
  int khs, k_loads, patch_rows;
  // halo (stride 1, resident weights): the tile's patch is 16 pixels wide and TH + KH - 1 rows high, loaded once per
  // channel block; tap (kh, kw) reads it kh * 16 + kw rows in, so the last KW - 1 pixels of every 16 (whose operand
  // rows run into the next patch row) are computed and dropped: tw_valid = 16 - (KW - 1) output columns per tile.
  // kcols = kernel columns the issuer walks inside one stage (KW with halo, else 1).
  int halo, tw_valid, kcols;
  // s2 (3x3 at stride 2, IC 16 / 32 / 64, even width, resident weights): the input is read as pixel PAIRS - rows of
  // 2 * IC bytes, two horizontally adjacent pixels - one patch of 33 input rows x 9 pairs per tile of 16 x 8 outputs.
  // Output column ox of tap kw reads pixel 2 * ox + kw - pad_l: pair ox + a, half b, so the tap's operand starts
  // (kh * 9 + a) rows and b * IC bytes into the patch; the eight outputs of a tile row are eight consecutive pairs
  // (one 8-row group) and the next tile row is two input rows = 18 pairs further (the descriptor's group stride).
  int s2, a_row_bytes, s2_stage_bytes, s2_pair0;  // pair width, bytes of a stage, pair offset of the patch origin (-1 or 0)
  const int32_t* corr;  // [row classes * col classes][n_tiles * BN] border corrections, or null
  const uint8_t* rcls;  // [OH] row class
  const uint8_t* ccls;  // [OW] column class
  const uint8_t* cls_nonzero;  // [classes] 1 when the class has a non-zero correction
  int ncc;              // column classes
  const int8_t* lut;    // 256-entry table applied to the int8 result (a fused tosa.table), or null
  // ADD kernels: out = clamp(q4(t_self[result] + t_other[res])), the operand tables built in the prologue by the
  // same apply_scale_32 as binary_kernel; res is laid out like out
  const int8_t* res;
  int self_zp, self_mult, self_shift, self_lshift, other_zp, other_mult, other_shift, other_lshift, add_dr, add_sign;
  int add_clamp_min, add_clamp_max;
  int4 add_q4;
  int tma_store;        // stage the output tile in shared memory and write it with one TMA store
  uint32_t staging_off; // byte offset of the staging buffers inside dynamic shared memory
  int* status;
  unsigned long long wait_ns;  // limit of every mbarrier wait
};


// EPI: 0 = the general rescale from the 32-byte ChanParams (any shift, 64-bit arithmetic); 1 / 2 = the compact
// Q4 records (common.cuh: one 16-byte shared-memory load, one 32-bit multiply-high per output) with / without
// the sign term of DOUBLE_ROUND; 3 = as 1 with the clamp being the whole int8 range (two saturating packs).
// LUT: a 256-entry table is applied to the result. Integer instructions issue at half rate on this machine,
// so whatever the epilogue does per output is a template choice, not a branch.
template <int EPI, bool CONV, bool LUT, bool ADD = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, GemmTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages], bar_empty[kMaxStages], bar_acc_full[4], bar_acc_empty[4],
      bar_w;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) int4 cp_s[kEpiGroups][128];  // per epilogue group: the Q4 records of its current n tile
  __shared__ __align__(16) uint8_t lut_s[256];           // fused table, indexed by value + 128
  __shared__ int add_t[ADD ? 512 : 1];                   // fused add: operand tables by raw byte, [0..255] own result, [256..511] other

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const bool shared_rows = CONV && p.khs > 1;
  const uint32_t a_stage_bytes = CONV && p.s2 ? (uint32_t)p.s2_stage_bytes : (uint32_t)(shared_rows ? p.patch_rows : kBM) * p.row_bytes;
  const uint32_t w_tile_bytes = (uint32_t)p.BN * p.row_bytes;  // one (n tile, k block) of the weights
  const uint32_t stage_bytes = a_stage_bytes + (p.w_resident ? 0u : w_tile_bytes * (shared_rows ? (uint32_t)p.khs : 1u));
  const uint32_t smem_w = smem_base;  // resident weights: [n_tiles][k_blocks] tiles
  const uint32_t smem_ring = smem_base + (p.w_resident ? (uint32_t)p.n_tiles * p.k_blocks * w_tile_bytes : 0u);
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 4; s++) {
      mbar_init(smem_u32(&bar_acc_full[s]), 1);
      mbar_init(smem_u32(&bar_acc_empty[s]), 4 * p.gpt);  // one arrival per epilogue warp that drains the stage
    }
    mbar_init(smem_u32(&bar_w), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (LUT && threadIdx.x >= 64 && threadIdx.x < 64 + 256) lut_s[threadIdx.x - 64] = (uint8_t)p.lut[threadIdx.x - 64];
  if (ADD && threadIdx.x >= 64 && threadIdx.x < 64 + 256) {
    const int v = (int)(int8_t)(threadIdx.x - 64);
    add_t[threadIdx.x - 64] = apply_scale_32((v - p.self_zp) * (1 << p.self_lshift), p.self_mult, p.self_shift, p.add_dr != 0);
    add_t[256 + threadIdx.x - 64] = apply_scale_32((v - p.other_zp) * (1 << p.other_lshift), p.other_mult, p.other_shift, p.add_dr != 0);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // everything above touched only shared memory, TMEM and constants; the next kernel may be scheduled from here on,
  // and what follows waits for the kernel before this one (the producer first sends for the resident weights)
  if (threadIdx.x == 0) grid_dependency_release();
  if (threadIdx.x != 0) grid_dependency_wait();

  // tile t -> (n, m) with n the slow index: a CTA keeps one n tile (its constants) for a long run
  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      if (p.w_resident) {
        const uint32_t bw = smem_u32(&bar_w);
        mbar_expect_tx(bw, (uint32_t)p.n_tiles * p.k_blocks * w_tile_bytes);
        for (int n = 0; n < p.n_tiles; n++)
          for (int kb = 0; kb < p.k_blocks; kb++)
            tma_load_2d(smem_w + (uint32_t)(n * p.k_blocks + kb) * w_tile_bytes, &tmB, kb * p.row_bytes, n * p.BN, bw);
      }
      grid_dependency_wait();
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int tr = 0;
      int n = blockIdx.x / p.m_tiles, m = blockIdx.x - n * p.m_tiles;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        // convolution: where the tile's patch starts in the input, and the tap / channel block of kb
        int img = 0, ih0 = 0, iw0 = 0, kh = 0, kw = 0, icb = 0;
        if (CONV) {
          img = m / p.tiles_per_img;
          const int r = m - img * p.tiles_per_img;
          const int ty = r / p.tiles_w, tx = r - ty * p.tiles_w;
          ih0 = ty * p.TH * p.cstride - p.pad_t;
          iw0 = tx * p.tw_valid * p.cstride - p.pad_l;
        }
        for (int kb = 0; kb < p.k_loads; kb++) {
          if (!(ok = mbar_wait(smem_u32(&bar_empty[s]), phase ^ 1, p.status, 1, p.wait_ns))) break;
          trace_stamp(p.trace, 0, tr, 1);
          const uint32_t full = smem_u32(&bar_full[s]);
          const uint32_t dst = smem_ring + (uint32_t)s * stage_bytes;
          mbar_expect_tx(full, CONV && p.s2 ? (uint32_t)(33 * 9 * p.a_row_bytes) : stage_bytes);  // s2: the stage is padded to 1 KB
          if (CONV && p.s2) {
            // one patch of pixel pairs per tile: 9 pairs from pair (first output column + s2_pair0), 33 input rows
            tma_load_4d(dst, &tmA, 0, (iw0 + p.pad_l) / 2 + p.s2_pair0, ih0, img, full);
          } else if (shared_rows) {
            // one patch of TH + khs - 1 rows for this kernel column and channel block; the weights of its khs taps
            tma_load_4d(dst, &tmA, icb * p.row_bytes, iw0 + kw, ih0, img, full);
            if (!p.w_resident)
              for (int r = 0; r < p.khs; r++)
                tma_load_2d(dst + a_stage_bytes + (uint32_t)r * w_tile_bytes, &tmB,
                            ((r * p.KW + kw) * p.icb_per_tap + icb) * p.row_bytes, n * p.BN, full);
            if (++icb == p.icb_per_tap) {
              icb = 0;
              kw++;
            }
          } else {
            if (CONV) {
              // zero fill outside the frame; the channel coordinate is a multiple of 32 bytes
              tma_load_4d(dst, &tmA, icb * p.row_bytes, iw0 + kw, ih0 + kh, img, full);
              if (++icb == p.icb_per_tap) {
                icb = 0;
                if (++kw == p.KW) {
                  kw = 0;
                  kh++;
                }
              }
            } else
              tma_load_2d(dst, &tmA, kb * p.row_bytes, m * kBM, full);
            if (!p.w_resident) tma_load_2d(dst + a_stage_bytes, &tmB, kb * p.row_bytes, n * p.BN, full);
          }
          if (++s == p.stages) {
            s = 0;
            phase ^= 1;
          }
        }
        m += gridDim.x;
        while (m >= p.m_tiles) {
          m -= p.m_tiles;
          n++;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    // At N <= 128 an instruction takes the tensor pipe only 27-36 ns (about 50-70 cycles): the work between two
    // issues must stay below that or the pipe idles. So the whole warp walks the loop with warp-uniform values (one
    // elected lane issues), the descriptors are kept as 32-bit low words (the shared-memory address field cannot
    // carry out of its 14 bits) stepped by additions, and the K steps of a row are unrolled at compile time.
    {
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      const int steps_full = p.row_bytes / 32;
      bool ok = true;
      if (p.w_resident) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_w), 0, p.status, 5, p.wait_ns));
      const uint64_t desc0_ring = make_smem_desc(smem_ring, p.row_bytes);
      const uint64_t desc0_w = make_smem_desc(p.w_resident ? smem_w : smem_ring + a_stage_bytes, p.row_bytes);
      const uint32_t desc_hi = (uint32_t)(desc0_ring >> 32);
      const uint32_t ring_lo = (uint32_t)desc0_ring, w_lo = (uint32_t)desc0_w;
      const uint32_t stage_units = stage_bytes >> 4, w_tile_units = w_tile_bytes >> 4;
      const uint32_t tap_units = CONV ? (uint32_t)((p.row_bytes << p.tw_log2) >> 4) : 0u;  // TW rows
      // weights of kernel row r + 1 relative to row r: KW * icb_per_tap k blocks on (resident), or the next tile of the stage
      const uint32_t w_row_units = p.w_resident ? (uint32_t)(p.KW * p.icb_per_tap) * w_tile_units : w_tile_units;
      const uint32_t w_col_units = (uint32_t)p.icb_per_tap * w_tile_units;  // halo: the next kernel column's weights
      const uint32_t row_units = (uint32_t)p.row_bytes >> 4;                // halo: the patch one pixel further
      const bool halo33 = p.halo && p.khs == 3 && p.kcols == 3;
      // s2: the A descriptor has its own width (pairs) and a group stride of two input rows (18 pairs); column kw of a
      // tap starts a pairs and b pixels into the patch row: kw - pad_l + 2 = 2 * (a + 1) + b
      uint32_t s2_a_hi = 0, s2_col0 = 0, s2_col1 = 0, s2_col2 = 0, s2_row_units = 0;
      if (CONV && p.s2) {
        uint64_t d = make_smem_desc(0, p.a_row_bytes);
        d &= ~((uint64_t)0x3FFF << 32);
        d |= (uint64_t)((18 * p.a_row_bytes) >> 4) << 32;
        s2_a_hi = (uint32_t)(d >> 32);
        const uint32_t pair_units = (uint32_t)p.a_row_bytes >> 4, pix_units = pair_units >> 1;
        auto col = [&](int kw) {
          const int v = kw - p.pad_l - 2 * p.s2_pair0;  // pixels from the patch origin
          return (uint32_t)(v >> 1) * pair_units + (uint32_t)(v & 1) * pix_units;
        };
        s2_col0 = col(0); s2_col1 = col(1); s2_col2 = col(2);
        s2_row_units = 9 * pair_units;
      }
      const bool rows3 = shared_rows && !p.halo && p.khs == 3;
      // The waits of the hot loop are short polls; a poll that fails leaves the loop, the bounded wait runs out here
      // and the loop is entered again where it stopped. (With the bounded wait's loop inside, the same issue sequence
      // ran at 86 ns per instruction instead of 49: measured with resident operands.)
      auto run = [&](auto steps_c) {
        constexpr int STEPS = decltype(steps_c)::value;
        int s = 0;
        uint32_t phase = 0;
        int n = blockIdx.x / p.m_tiles, m = blockIdx.x - n * p.m_tiles;
        int as = 0;
        uint32_t acc_phase = 0;
        int tr = 0;
        uint32_t a_lo = ring_lo;                   // descriptor of stage s
        uint32_t bar = smem_u32(&bar_full[0]);     // full barrier of stage s
        const uint32_t bar_empty_off = smem_u32(&bar_empty[0]) - smem_u32(&bar_full[0]);
        int t = blockIdx.x, kb = 0;
        bool tile_open = false;
        uint32_t tmem_d = 0, accum = 0, b_kb = 0;
        for (;;) {
          int failed = 0;  // 1: the accumulator stage is not drained yet, 2: the operand stage has not landed yet
          while (t < total_tiles) {
            if (!tile_open) {
              if (!__all_sync(0xffffffffu, mbar_poll(smem_u32(&bar_acc_empty[as]), acc_phase ^ 1, 8))) {
                failed = 1;
                break;
              }
              trace_stamp(p.trace, 1, tr, 1);
              tile_open = true;
              tmem_d = tmem_base + (uint32_t)(as * p.acc_stride);
              accum = 0;
              b_kb = w_lo + (uint32_t)(n * p.k_blocks) * w_tile_units;  // resident weights: k block 0 of this n tile
            }
            if (!__all_sync(0xffffffffu, mbar_poll(bar, phase, 8))) {
              failed = 2;
              break;
            }
            tc_fence_after();
            uint32_t b_lo = p.w_resident ? b_kb : w_lo + (a_lo - ring_lo);
            if (CONV && p.s2) {
              uint32_t ar = a_lo, bc = b_lo;
#pragma unroll
              for (int r = 0; r < 3; r++) {
#pragma unroll
                for (int c = 0; c < 3; c++) {
                  const uint32_t ac = ar + (c == 0 ? s2_col0 : c == 1 ? s2_col1 : s2_col2);
#pragma unroll
                  for (int k = 0; k < STEPS; k++) {
                    mma_i8_ab_elect(tmem_d, ac + 2 * k, s2_a_hi, bc + 2 * k, desc_hi, idesc, accum);
                    accum = 1;
                  }
                  bc += w_col_units;
                }
                ar += s2_row_units;
              }
            } else if (CONV && halo33) {
              // 3x3 over a halo patch, the common case, fully unrolled: the operand of tap (r, c) starts r * 16 + c
              // rows into the patch, a compile-time distance once the row width (32 * STEPS bytes) is one
              uint32_t bc = b_lo;
#pragma unroll
              for (int r = 0; r < 3; r++)
#pragma unroll
                for (int c = 0; c < 3; c++) {
#pragma unroll
                  for (int k = 0; k < STEPS; k++) {
                    mma_i8_lo_elect(tmem_d, a_lo + (uint32_t)((r * 16 + c) * 2 * STEPS + 2 * k), bc + 2 * k, desc_hi, idesc, accum);
                    accum = 1;
                  }
                  bc += w_col_units;
                }
            } else if (CONV && rows3) {
              // three kernel rows sharing one load per kernel column, unrolled
#pragma unroll
              for (int r = 0; r < 3; r++) {
#pragma unroll
                for (int k = 0; k < STEPS; k++) {
                  mma_i8_lo_elect(tmem_d, a_lo + (uint32_t)r * tap_units + 2 * k, b_lo + 2 * k, desc_hi, idesc, accum);
                  accum = 1;
                }
                b_lo += w_row_units;
              }
            } else if (shared_rows) {
              uint32_t ar = a_lo;
              for (int r = 0; r < p.khs; r++) {
                uint32_t ac = ar, bc = b_lo;
                for (int c = 0; c < p.kcols; c++) {
#pragma unroll
                  for (int k = 0; k < STEPS; k++) {
                    mma_i8_lo_elect(tmem_d, ac + 2 * k, bc + 2 * k, desc_hi, idesc, accum);
                    accum = 1;
                  }
                  ac += row_units;
                  bc += w_col_units;
                }
                ar += tap_units;
                b_lo += w_row_units;
              }
            } else if (kb == p.k_blocks - 1 && p.k_last_steps != STEPS) {
              for (int k = 0; k < p.k_last_steps; k++) {
                mma_i8_lo_elect(tmem_d, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc, accum);
                accum = 1;
              }
            } else {
#pragma unroll
              for (int k = 0; k < STEPS; k++) {
                mma_i8_lo_elect(tmem_d, a_lo + 2 * k, b_lo + 2 * k, desc_hi, idesc, accum);
                accum = 1;
              }
            }
            mma_commit_elect(bar + bar_empty_off);  // frees the stage once the MMAs have read it
            b_kb += w_tile_units;
            a_lo += stage_units;
            bar += 8;
            if (++s == p.stages) {
              s = 0;
              phase ^= 1;
              a_lo = ring_lo;
              bar = smem_u32(&bar_full[0]);
            }
            if (++kb == p.k_loads) {
              mma_commit_elect(smem_u32(&bar_acc_full[as]));
              trace_stamp(p.trace, 1, tr, 3);
              kb = 0;
              tile_open = false;
              if (++as == p.acc_stages) {
                as = 0;
                acc_phase ^= 1;
              }
              t += gridDim.x;
              m += gridDim.x;
              while (m >= p.m_tiles) {
                m -= p.m_tiles;
                n++;
              }
            }
          }
          if (!failed) break;
          trace_stamp(p.trace, 1, tr, 4 + failed);  // 5: waited for an accumulator, 6: waited for operands
          ok = __all_sync(0xffffffffu, failed == 1 ? mbar_wait(smem_u32(&bar_acc_empty[as]), acc_phase ^ 1, p.status, 2, p.wait_ns)
                                                   : mbar_wait(bar, phase, p.status, 3, p.wait_ns));
          if (!ok) break;
          trace_stamp(p.trace, 1, tr, 7);
        }
      };
      if (ok) {
        if (steps_full == 4) run(std::integral_constant<int, 4>{});
        else if (steps_full == 2) run(std::integral_constant<int, 2>{});
        else run(std::integral_constant<int, 1>{});
      }
    }
  } else {
    // ------------------------------------------------ epilogue: 4 groups of 4 warps; group g owns accumulator
    // stage g and takes this CTA's tiles g, g + 4, g + 8, ...
    const int q = warp & 3;                // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;
    // gpt == 1: group g drains accumulator stage g alone. gpt == 2 (tiles wider than 128 columns, two
    // stages): groups 2s and 2s + 1 drain stage s together, each its half of the columns.
    const int astage = p.gpt == 2 ? group >> 1 : group;
    const int col_half = p.gpt == 2 ? (group & 1) * p.BNh : 0;
    const int e = (threadIdx.x - 64) & 127;
    int4* cps = cp_s[group];
    const uint32_t lo2 = (uint32_t)(p.clamp_min & 0xffff) * 0x10001u;
    const uint32_t hi2 = (uint32_t)(p.clamp_max & 0xffff) * 0x10001u;
    const bool vec_ok = (p.ldc & 15) == 0;
    const int nfull = p.BNh >> 5;
    const uint32_t tile_bytes = (uint32_t)kBM * p.BNh;
    // one staging tile per group for the TMA store of the output
    uint8_t* const stage_tile = smem_raw + (smem_base - smem_u32(smem_raw)) + p.staging_off + (size_t)group * tile_bytes;
    const int row_in_tile = q * 32 + lane;
    // convolution: the pixel of this accumulator row inside the tile; with a halo patch only tw_valid of its 16
    // columns are outputs, and the staged tile holds just those
    const int px_x = CONV ? (row_in_tile & ((1 << p.tw_log2) - 1)) : 0, px_y = CONV ? (row_in_tile >> p.tw_log2) : 0;
    const bool px_valid = !CONV || px_x < p.tw_valid;
    uint8_t* const srow = stage_tile + (size_t)(CONV ? px_y * p.tw_valid + px_x : row_in_tile) * p.BNh;
    const int bar_id = 1 + group;
    auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory"); };
    int loaded_n = -1;
    uint32_t acc_phase = 0;
    bool ok = true;
    int tr = 0;
    const int tr_on = p.trace && e == 0;
    const int t_first = blockIdx.x + astage * gridDim.x;
    int n = t_first / p.m_tiles, m = t_first - n * p.m_tiles;
    for (int t = t_first; t < total_tiles; t += p.acc_stages * gridDim.x) {
      const ChanParams* chan_n = p.chan + (size_t)n * p.BN + col_half;
      if (EPI != 0 && n != loaded_n) {
        group_sync();
        if (e < p.BNh) cps[e] = p.q4[(size_t)n * p.BN + col_half + e];
        group_sync();
        loaded_n = n;
      }
      trace_stamp(tr_on, 2 + group, tr, 1);
      if (ok) ok = mbar_wait(smem_u32(&bar_acc_full[astage]), acc_phase, p.status, 4, p.wait_ns);
      trace_stamp(tr_on, 2 + group, tr, 2);
      if (ok) {
        tc_fence_after();
        const int row = m * kBM + row_in_tile;
        // convolution: this thread's output pixel and its border class
        int img = 0, oh0 = 0, ow0 = 0;
        const int32_t* corr_row = nullptr;
        if (CONV) {
          img = m / p.tiles_per_img;
          const int r = m - img * p.tiles_per_img;
          const int ty = r / p.tiles_w, tx = r - ty * p.tiles_w;
          oh0 = ty * p.TH;
          ow0 = tx * p.tw_valid;
          const int oh = oh0 + px_y, ow = ow0 + px_x;
          if (p.corr && px_valid && oh < p.OH && ow < p.OW) {
            const int cls = p.rcls[oh] * p.ncc + p.ccls[ow];
            if (p.cls_nonzero[cls]) corr_row = p.corr + (size_t)cls * p.n_tiles * p.BN + (size_t)n * p.BN + col_half;
          }
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(astage * p.acc_stride + col_half);
        int8_t* orow = p.out + (long long)row * p.ldc + (long long)n * p.BN + col_half;
        const int8_t* rrow = ADD ? p.res + (long long)row * p.ldc + (long long)n * p.BN + col_half : nullptr;
        const int ncol0 = n * p.BN + col_half;
        if (p.tma_store) {
          // this group's previous store must have read the staging tile before it is overwritten
          if (e == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          group_sync();
        }
        trace_stamp(tr_on, 2 + group, tr, 3);

        // requantise 16 accumulators starting at tile column c0 and store them
        auto emit16 = [&](const uint32_t* v, int c0) {
          uint32_t w4[4];
#pragma unroll
          for (int g = 0; g < 4; g++) {
            int r[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              int acc = (int)v[g * 4 + j];
              if (CONV && corr_row) acc += corr_row[c0 + g * 4 + j];
              if (EPI == 1 || EPI == 3) {
                r[j] = scale_q4_sign(acc, cps[c0 + g * 4 + j]);
              } else if (EPI == 2) {
                r[j] = scale_q4(acc, cps[c0 + g * 4 + j]);
              } else {
                const ChanParams c = chan_n[c0 + g * 4 + j];
                r[j] = scale_cp<false>(acc + c.bias, c) + p.out_zp;
              }
            }
            w4[g] = EPI == 3 ? sat_pack4(r[0], r[1], r[2], r[3]) : clamp_pack4(r[0], r[1], r[2], r[3], lo2, hi2);
            if (ADD) {
              // the other operand's four bytes (same row and columns of a tensor laid out like the result)
              uint32_t xo = 0;
              if (row < p.M) {
                if (vec_ok && ncol0 + c0 + g * 4 + 4 <= p.N) {
                  xo = *reinterpret_cast<const uint32_t*>(rrow + c0 + g * 4);
                } else {
#pragma unroll
                  for (int j = 0; j < 4; j++)
                    if (ncol0 + c0 + g * 4 + j < p.N) xo |= (uint32_t)(uint8_t)rrow[c0 + g * 4 + j] << (8 * j);
                }
              }
              int s4[4];
#pragma unroll
              for (int j = 0; j < 4; j++) {
                const int v = add_t[(w4[g] >> (8 * j)) & 0xff] + add_t[256 + ((xo >> (8 * j)) & 0xff)];
                const int v4 = v * 4 + p.add_q4.x;
                const int neg = p.add_sign ? (v4 >> 31) : 0;
                const int r1 = (__mulhi(v4, p.add_q4.y) + p.add_q4.z + neg + neg) >> p.add_q4.w;
                s4[j] = max(p.add_clamp_min, min(p.add_clamp_max, r1));
              }
              w4[g] = (uint32_t)(s4[0] & 0xff) | ((uint32_t)(s4[1] & 0xff) << 8) | ((uint32_t)(s4[2] & 0xff) << 16) | ((uint32_t)s4[3] << 24);
            }
            if (LUT) {  // out = table[value + 128], byte by byte
              const uint32_t x = w4[g] ^ 0x80808080u;
              w4[g] = (uint32_t)lut_s[x & 0xff] | ((uint32_t)lut_s[(x >> 8) & 0xff] << 8) |
                      ((uint32_t)lut_s[(x >> 16) & 0xff] << 16) | ((uint32_t)lut_s[x >> 24] << 24);
            }
          }
          if (p.tma_store) {
            if (px_valid) *reinterpret_cast<uint4*>(srow + c0) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          } else if (row < p.M) {
            if (vec_ok && ncol0 + c0 + 16 <= p.N) {
              *reinterpret_cast<uint4*>(orow + c0) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; j++)
                if (ncol0 + c0 + j < p.N) orow[c0 + j] = (int8_t)(w4[j >> 2] >> (8 * (j & 3)));
            }
          }
        };

        for (int c = 0; c < nfull; c++) {
          uint32_t v[32];
          tmem_ld32_issue(taddr + c * 32, v);
          tmem_ld_wait32(v);
          emit16(v, c * 32);
          emit16(v + 16, c * 32 + 16);
        }
        if (p.BNh & 16) {
          uint32_t vt[16];
          tmem_ld16(taddr + nfull * 32, vt);
          emit16(vt, nfull * 32);
        }
        tc_fence_before();
        __syncwarp();
        trace_stamp(tr_on, 2 + group, tr, 4);
        if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[astage]));  // this warp's share of the TMEM stage is drained
        if (p.tma_store) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // staged bytes -> visible to the TMA engine
          group_sync();
          if (e == 0) {
            if (CONV) tma_store_4d(&tmC, ncol0, ow0, oh0, img, smem_u32(stage_tile));
            else tma_store_2d(&tmC, ncol0, m * kBM, smem_u32(stage_tile));
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          trace_stamp(tr_on, 2 + group, tr, 5);
        }
      }
      acc_phase ^= 1;
      m += p.acc_stages * gridDim.x;
      while (m >= p.m_tiles) {
        m -= p.m_tiles;
        n++;
      }
    }
    if (p.tma_store && e == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // ------------------------------------------------ common exit: free TMEM
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    if (*(volatile int*)p.status != 0) __nanosleep(1000000);  // let copies in flight land after a failed wait
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// Output tensor [rows, cols] with a row pitch; box = [box_rows, box_cols], dense rows in shared memory.
bool encode_2d_plain(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch,
                     uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 2-D byte tensor [rows, cols] with a row pitch; box = [box_rows, row_bytes], swizzle width = row_bytes.
bool encode_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch, uint32_t box_rows,
               int row_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {(cuuint32_t)row_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_32B;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Input of a convolution as a 4-D tensor {C, W, H, N}: box = {row_bytes channels, TW pixels at the
// conv stride, TH rows at the conv stride, 1 image}, which lands in shared memory as 128 rows of
// row_bytes, the same K-major layout the 2-D loads produce. Out-of-range elements read as zero.
bool encode_conv_input(CUtensorMap* map, const void* base, int N, int H, int W, int C, int row_bytes, int TW, int TH,
                       int stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)C, (cuuint64_t)W * C, (cuuint64_t)H * W * C};
  cuuint32_t box[4] = {(cuuint32_t)row_bytes, (cuuint32_t)(TW * stride), (cuuint32_t)(TH * stride), 1};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  const CUtensorMapSwizzle sw = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                  : CU_TENSOR_MAP_SWIZZLE_32B;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Input of a stride-2 convolution as pixel pairs {2C, W / 2, H, N} (W even): box = {2C bytes, 9 pairs, 33 rows, 1 image}.
bool encode_conv_input_pairs(CUtensorMap* map, const void* base, int N, int H, int W, int C) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const int rb = 2 * C;
  cuuint64_t dims[4] = {(cuuint64_t)rb, (cuuint64_t)(W / 2), (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)rb, (cuuint64_t)W * C, (cuuint64_t)H * W * C};
  cuuint32_t box[4] = {(cuuint32_t)rb, 9, 33, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapSwizzle sw = rb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : rb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Output {OC, OW, OH, N}: box = {BN, TW, TH, 1}, dense in shared memory; the store clips ragged edges.
bool encode_conv_output(CUtensorMap* map, const void* base, int N, int OH, int OW, int OC, int BN, int TW, int TH) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)OC, (cuuint64_t)OW, (cuuint64_t)OH, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)OC, (cuuint64_t)OW * OC, (cuuint64_t)OH * OW * OC};
  cuuint32_t box[4] = {(cuuint32_t)BN, (cuuint32_t)TW, (cuuint32_t)TH, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace


namespace {
int gemm_trace_on() {
  const char* e = getenv("TB200_GEMM_TRACE");
  return e && *e && *e != '0';
}
}  // namespace

// Copies the role timestamps of the last traced launch's CTA 0 (6 roles x 512 slots, (ns << 8) | tag, 0 = unused).
int read_gemm_trace(unsigned long long* out, int n) {
  if (n > 6 * kTraceSlots) n = 6 * kTraceSlots;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(out, g_gemm_trace, (size_t)n * sizeof(unsigned long long)) != cudaSuccess) return -1;
  static unsigned long long zeros[6 * kTraceSlots];
  cudaMemcpyToSymbol(g_gemm_trace, zeros, sizeof(zeros));
  return n;
}

namespace {
typedef void (*GemmKernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, GemmTcParams);
// [EPI][LUT] for the plain GEMM and for the implicit-GEMM convolution
GemmKernelFn gemm_kernel_for(bool conv, int epi, bool lut, bool add = false) {
  // the fused residual add exists for the plain GEMM without a table
  static const GemmKernelFn addk[4] = {gemm_i8_tc_kernel<0, false, false, true>, gemm_i8_tc_kernel<1, false, false, true>,
                                       gemm_i8_tc_kernel<2, false, false, true>, gemm_i8_tc_kernel<3, false, false, true>};
  if (add) return addk[epi];
  static const GemmKernelFn plain[4][2] = {
      {gemm_i8_tc_kernel<0, false, false>, gemm_i8_tc_kernel<0, false, true>},
      {gemm_i8_tc_kernel<1, false, false>, gemm_i8_tc_kernel<1, false, true>},
      {gemm_i8_tc_kernel<2, false, false>, gemm_i8_tc_kernel<2, false, true>},
      {gemm_i8_tc_kernel<3, false, false>, gemm_i8_tc_kernel<3, false, true>},
  };
  static const GemmKernelFn convk[4][2] = {
      {gemm_i8_tc_kernel<0, true, false>, gemm_i8_tc_kernel<0, true, true>},
      {gemm_i8_tc_kernel<1, true, false>, gemm_i8_tc_kernel<1, true, true>},
      {gemm_i8_tc_kernel<2, true, false>, gemm_i8_tc_kernel<2, true, true>},
      {gemm_i8_tc_kernel<3, true, false>, gemm_i8_tc_kernel<3, true, true>},
  };
  return conv ? convk[epi][lut ? 1 : 0] : plain[epi][lut ? 1 : 0];
}
// Every kernel needs its dynamic shared-memory limit raised once per device.
cudaError_t gemm_kernels_set_smem(bool conv) {
  for (int e = 0; e < 4; e++)
    for (int l = 0; l < 2; l++) {
      const cudaError_t err = cudaFuncSetAttribute(gemm_kernel_for(conv, e, l != 0), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
      if (err != cudaSuccess) return err;
    }
  for (int e = 0; e < 4 && !conv; e++) {
    const cudaError_t err = cudaFuncSetAttribute(gemm_kernel_for(false, e, false, true), cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (err != cudaSuccess) return err;
  }
  return cudaSuccess;
}
// EPI 1 with a clamp that is the whole int8 range packs with two saturating conversions (EPI 3)
int gemm_epi_variant(int epi, int clamp_min, int clamp_max) { return epi == 1 && clamp_min <= -128 && clamp_max >= 127 ? 3 : epi; }
}  // namespace

GemmTcGeometry gemm_tc_geometry(int N, int K, long long M) {
  GemmTcGeometry g{};
  g.row_bytes = K <= 32 ? 32 : K <= 64 ? 64 : 128;
  g.k_blocks = (K + g.row_bytes - 1) / g.row_bytes;
  g.Kpad = g.k_blocks * g.row_bytes;
  const int npad = (N + 15) / 16 * 16;
  // narrow tiles: at most 128 columns, four accumulator stages, one epilogue group per tile; least padding wins
  int best_tiles = 0, best_bn = 0, best_total = 1 << 30;
  const int t0 = (npad + 127) / 128;
  for (int tiles = t0; tiles <= t0 + 2; tiles++) {
    const int bn = ((npad + tiles - 1) / tiles + 15) / 16 * 16;
    if (bn * tiles < best_total) {
      best_total = bn * tiles;
      best_tiles = tiles;
      best_bn = bn;
    }
  }
  g.BN = best_bn;
  g.n_tiles = best_tiles;
  g.gpt = 1;
  // few rows and a small weight matrix (a classifier's FC): narrower column tiles until every SM has one. The A tile
  // is then re-read by more CTAs out of L2, 128 / BN times the weight bytes in all, so this pays only while the
  // whole product is latency-bound (measured: 1000 x 1280 at 256 rows 27 -> 19 us; 8192 x 8192 at one row 45 -> 70 us)
  {
    const long long m_tiles = (M + kBM - 1) / kBM;
    if (m_tiles * g.n_tiles < 148 && (long long)npad * g.Kpad <= (2ll << 20)) {
      int bn = g.BN;
      while (bn > 32 && m_tiles * ((npad + bn - 1) / bn) < 148) bn -= 16;
      if (bn != g.BN) {
        g.n_tiles = (npad + bn - 1) / bn;
        g.BN = ((npad + g.n_tiles - 1) / g.n_tiles + 15) / 16 * 16;
      }
    }
  }
  // wide tiles: 160..256 columns (a multiple of 32), two accumulator stages, two epilogue groups per tile.
  // Each A tile then meets twice as many weight columns per load and the MMA reads less shared memory per
  // multiply-accumulate. Taken when it pads no more than 1/16 beyond the narrow choice.
  static int max_bn = -1;  // TB200_GEMM_MAX_BN=128 keeps the narrow tiles (A/B aid)
  if (max_bn < 0) { const char* e = getenv("TB200_GEMM_MAX_BN"); max_bn = e && atoi(e) >= 16 ? atoi(e) : 256; }
  if (npad > 128 && max_bn > 128) {
    int wt = 0, wbn = 0, wtotal = 1 << 30;
    const int w0 = (npad + 255) / 256;
    for (int tiles = w0; tiles <= w0 + 2; tiles++) {
      const int bn = ((npad + tiles - 1) / tiles + 31) / 32 * 32;
      if (bn <= 128 || bn > 256) continue;
      if (bn * tiles < wtotal) {
        wtotal = bn * tiles;
        wt = tiles;
        wbn = bn;
      }
    }
    // wide tiles only when they still give every SM a tile: few rows want many small tiles
    const long long m_tiles = (M + kBM - 1) / kBM;
    if (wt > 0 && wtotal <= best_total + best_total / 16 && m_tiles * wt >= 148) {
      g.BN = wbn;
      g.n_tiles = wt;
      g.gpt = 2;
    }
  }
  return g;
}

bool gemm_tc_supported(long long M, int N, int K, long long lda) {
  return M >= 1 && M < (1ll << 31) && N >= 1 && K >= 16 && (K % 16) == 0 && (lda % 16) == 0 && lda >= K;
}

struct GemmTcState {
  const void* a = nullptr;
  const void* w = nullptr;
  const void* c = nullptr;
  CUtensorMap tmA, tmB, tmC;
};

GemmTcState* gemm_tc_state_new() { return new GemmTcState(); }
void gemm_tc_state_free(GemmTcState* s) { delete s; }

cudaError_t launch_gemm_i8_tc(const GemmTcArgs& a, GemmTcState* st, cudaStream_t stream) {
  const GemmTcGeometry g = gemm_tc_geometry(a.N, a.K, a.M);
  if (st->a != a.a) {
    if (!encode_2d(&st->tmA, a.a, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)a.lda, kBM, g.row_bytes))
      return cudaErrorInvalidValue;
    st->a = a.a;
  }
  if (st->w != a.w) {
    if (!encode_2d(&st->tmB, a.w, (uint64_t)g.n_tiles * g.BN, (uint64_t)g.Kpad, (uint64_t)g.Kpad, (uint32_t)g.BN,
                   g.row_bytes))
      return cudaErrorInvalidValue;
    st->w = a.w;
  }
  // Long K with wide tiles: the epilogue is a small share of the tile's time and the ring needs the shared memory
  // more than the output staging does, so the result leaves with 16-byte stores from registers.
  const bool tma_store = (a.ldc % 16) == 0 && ((uintptr_t)a.out % 16) == 0 && !(g.gpt == 2 && g.k_blocks >= 16);
  if (tma_store && st->c != a.out) {
    if (!encode_2d_plain(&st->tmC, a.out, (uint64_t)a.M, (uint64_t)a.N, (uint64_t)a.ldc, kBM, (uint32_t)(g.BN / g.gpt)))
      return cudaErrorInvalidValue;
    st->c = a.out;
  }
  GemmTcParams p{};
  p.tma_store = tma_store;
  p.chan = a.chan;
  p.out = a.out;
  p.ldc = a.ldc;
  p.M = (int)a.M;
  p.N = a.N;
  p.BN = g.BN;
  p.n_tiles = g.n_tiles;
  p.m_tiles = (int)((a.M + kBM - 1) / kBM);
  p.k_blocks = g.k_blocks;
  p.k_loads = g.k_blocks;
  p.khs = 1;
  p.kcols = 1;
  p.k_last_steps = ((a.K - (g.k_blocks - 1) * g.row_bytes) + 31) / 32;
  p.row_bytes = g.row_bytes;
  const size_t w_bytes = (size_t)g.n_tiles * g.BN * g.Kpad;
  p.w_resident = w_bytes <= (size_t)kResidentWeightBytes;
  const size_t stage_bytes = (size_t)kBM * g.row_bytes + (p.w_resident ? 0 : (size_t)g.BN * g.row_bytes);
  const size_t staging_bytes = tma_store ? (size_t)kEpiGroups * kBM * (g.BN / g.gpt) : 0;  // one (half) tile per group
  const size_t ring_budget = (size_t)kSmemBudget - 1024 - (p.w_resident ? w_bytes : 0) - staging_bytes;
  int stages = (int)(ring_budget / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return cudaErrorInvalidConfiguration;
  p.stages = stages;
  p.out_zp = a.out_zp;
  p.clamp_min = a.clamp_min;
  p.clamp_max = a.clamp_max;
  p.q4 = a.q4;
  int stride = 32;
  while (stride < g.BN) stride <<= 1;
  p.acc_stride = stride;
  p.gpt = g.gpt;
  p.BNh = g.BN / g.gpt;
  p.acc_stages = kEpiGroups / g.gpt;  // 4 stages of <= 128 columns or 2 of <= 256 fill the 512 TMEM columns
  p.tmem_cols = p.acc_stages * stride;
  p.status = a.status;
  p.wait_ns = wait_limit_ns();
  p.trace = gemm_trace_on();
  p.lut = a.lut;
  p.staging_off = (uint32_t)((p.w_resident ? w_bytes : 0) + (size_t)stages * stage_bytes);
  const size_t smem = 1024 + p.staging_off + staging_bytes;
  static std::atomic<unsigned long long> attr_set{0};
  if (first_use_on_device(attr_set)) {
    const cudaError_t e = gemm_kernels_set_smem(false);
    if (e != cudaSuccess) return e;
    mark_used_on_device(attr_set);
  }
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = tiles < current_sm_count() ? tiles : current_sm_count();
  const bool fused_add = a.res != nullptr;
  if (fused_add) {
    if (a.lut || a.add.kind != 0 || a.add.epi == 0) return cudaErrorInvalidValue;
    const BinaryArgs& d = a.add;
    p.res = a.res;
    const bool sa = a.add_self_is_a != 0;
    p.self_zp = sa ? d.a_zp : d.b_zp; p.self_mult = sa ? d.a_mult : d.b_mult; p.self_shift = sa ? d.a_shift : d.b_shift;
    p.self_lshift = sa ? d.a_lshift : d.b_lshift;
    p.other_zp = sa ? d.b_zp : d.a_zp; p.other_mult = sa ? d.b_mult : d.a_mult; p.other_shift = sa ? d.b_shift : d.a_shift;
    p.other_lshift = sa ? d.b_lshift : d.a_lshift;
    p.add_dr = d.double_round;
    p.add_sign = d.epi == 1;
    p.add_clamp_min = d.clamp_min; p.add_clamp_max = d.clamp_max;
    p.add_q4 = d.q4;
  }
  return launch_dependent_if(tiles >= kDependentMinBlocks / 2, gemm_kernel_for(false, gemm_epi_variant(a.epi, a.clamp_min, a.clamp_max), a.lut != nullptr, fused_add), dim3(grid), dim3(kThreads), smem, stream, st->tmA, st->tmB, st->tmC, p);
}

// ---- convolution as implicit GEMM ----
ConvTcGeometry conv_tc_geometry(int N, int OH, int OW, int IC, int OC, int KH, int KW, int stride) {
  ConvTcGeometry g{};
  // channel block = swizzle width: the widest of 128 / 64 / 32 bytes with the least padding of IC. A last
  // block that reaches beyond IC is fine: the copy engine fills the missing channels with zeros and the
  // packed weights hold zeros there.
  int best_pad = 1 << 30;
  for (int rb = 128; rb >= 32; rb >>= 1) {
    const int padded = (IC + rb - 1) / rb * rb;
    if (padded < best_pad) {
      best_pad = padded;
      g.row_bytes = rb;
    }
  }
  g.icb_per_tap = (IC + g.row_bytes - 1) / g.row_bytes;
  g.k_blocks = KH * KW * g.icb_per_tap;
  g.Kpad = g.k_blocks * g.row_bytes;
  // Patch shape TW * TH = 128. Stride-1 convolutions with more than one kernel row share one load of TH + KH - 1
  // input rows among the KH taps of a kernel column (TW >= 8 so that a kernel row's operand starts on a whole
  // 8-row swizzle atom): the shape with the fewest rows through the copy engine. Otherwise the least padded area
  // (ties: the wider patch, longer contiguous runs). Measured on 3x3 convolutions of 32..128 channels at 48..112
  // pixels: once the loads are shared, 8-, 16- and 32-pixel-wide patches take the same time (the kernel is then
  // bound per tile, not by rows or runs of the copy engine), so the rule stays the simple one.
  g.khs = (stride == 1 && KH > 1) ? KH : 1;
  long long best = -1;
  for (int tw = 128; tw >= (g.khs > 1 ? 8 : 4); tw >>= 1) {
    const int th = 128 / tw;
    const long long tiles = (long long)((OW + tw - 1) / tw) * ((OH + th - 1) / th);
    const long long cost = g.khs > 1 ? tiles * (th + KH - 1) * tw : tiles * tw * th;
    if (best < 0 || cost < best) {
      best = cost;
      g.TW = tw;
      g.TH = th;
    }
  }
  g.TWv = g.TW;
  g.tiles_w = (OW + g.TW - 1) / g.TW;
  g.tiles_h = (OH + g.TH - 1) / g.TH;
  GemmTcGeometry n = gemm_tc_geometry(OC, g.Kpad, (long long)N * g.tiles_w * g.tiles_h * kBM);
  // Halo patches: the copy engine works row by row (a pixel's channel block is a row), and a load per kernel
  // column moves every input pixel KW times. With the weights resident in shared memory one 16-pixel-wide patch
  // per tile and channel block serves all KH * KW taps: tap (kh, kw) is the same patch read kh * 16 + kw rows in.
  // Taken when it moves fewer rows than the per-column loads.
  static int no_halo = -1;  // TB200_CONV_NO_HALO=1: A/B aid
  if (no_halo < 0) { const char* e = getenv("TB200_CONV_NO_HALO"); no_halo = e && *e && *e != '0'; }
  if (!no_halo && stride == 1 && KH > 1 && KW > 1 && KW <= 5) {
    const int twv = 16 - (KW - 1), th = 8;
    const int tiles_w = (OW + twv - 1) / twv, tiles_h = (OH + th - 1) / th;
    const GemmTcGeometry nh = gemm_tc_geometry(OC, g.Kpad, (long long)N * tiles_w * tiles_h * kBM);
    const long long rows_halo = (long long)tiles_w * tiles_h * (th + KH - 1) * 16;
    const long long rows_cols = (long long)g.tiles_w * g.tiles_h * (g.TH + KH - 1) * g.TW * KW;
    // the weights must stay in shared memory beside the output staging tiles and at least three patches
    const size_t need = (size_t)nh.n_tiles * nh.BN * g.Kpad + (size_t)kEpiGroups * kBM * (nh.BN / nh.gpt) +
                        3 * (size_t)(th + KH - 1) * 16 * g.row_bytes + 1024;
    if (need <= (size_t)kSmemBudget && rows_halo < rows_cols) {
      g.halo = 1;
      g.TW = 16;
      g.TWv = twv;
      g.TH = th;
      g.tiles_w = tiles_w;
      g.tiles_h = tiles_h;
      n = nh;
    }
  }
  g.BN = n.BN;
  g.n_tiles = n.n_tiles;
  g.gpt = n.gpt;
  return g;
}

// Stride-2 3x3 over pixel pairs (see GemmTcParams::s2): what the launch needs beyond the geometry.
static bool conv_s2_eligible(int W, int IC, int KH, int KW, int stride, int pad_l) {
  static int off = -1;  // TB200_CONV_NO_S2=1: A/B aid
  if (off < 0) { const char* e = getenv("TB200_CONV_NO_S2"); off = e && *e && *e != '0'; }
  return !off && stride == 2 && KH == 3 && KW == 3 && (W % 2) == 0 && (IC == 16 || IC == 32 || IC == 64) && (pad_l == 0 || pad_l == 1);
}

ConvTcGeometry conv_tc_geometry_padded(int N, int OH, int OW, int W, int IC, int OC, int KH, int KW, int stride, int pad_l) {
  ConvTcGeometry g = conv_tc_geometry(N, OH, OW, IC, OC, KH, KW, stride);
  if (!conv_s2_eligible(W, IC, KH, KW, stride, pad_l)) return g;
  const int tiles_w = (OW + 7) / 8, tiles_h = (OH + 15) / 16;
  const GemmTcGeometry n = gemm_tc_geometry(OC, g.Kpad, (long long)N * tiles_w * tiles_h * kBM);
  const size_t stage = ((size_t)33 * 9 * 2 * IC + 1023) / 1024 * 1024;
  const size_t need = (size_t)n.n_tiles * n.BN * g.Kpad + (size_t)kEpiGroups * kBM * (n.BN / n.gpt) + 3 * stage + 1024;
  if (need > (size_t)kSmemBudget) return g;
  g.s2 = 1;
  g.halo = 0;
  g.khs = 1;
  g.TW = 8; g.TWv = 8; g.TH = 16;
  g.tiles_w = tiles_w; g.tiles_h = tiles_h;
  g.BN = n.BN; g.n_tiles = n.n_tiles; g.gpt = n.gpt;
  return g;
}

bool conv_tc_supported(int N, int H, int W, int IC, int OC, int KH, int KW, int stride_h, int stride_w, int dil_h, int dil_w,
                       int OH, int OW) {
  if (IC % 16 != 0 || OC % 16 != 0 || stride_h != stride_w || stride_h < 1 || stride_h > 2 || dil_h != 1 || dil_w != 1 ||
      KH < 1 || KW < 1 || KH * KW > 49 || KH * KW == 1)
    return false;
  const ConvTcGeometry g = conv_tc_geometry(N, OH, OW, IC, OC, KH, KW, stride_h);
  if (g.TW * stride_w > 256 || g.TH * stride_h > 256) return false;  // TMA box extents
  if ((long long)N * g.tiles_w * g.tiles_h >= (1ll << 30)) return false;
  return H >= 1 && W >= 1;
}

cudaError_t launch_conv_i8_tc(const ConvTcArgs& a, GemmTcState* st, cudaStream_t stream) {
  const ConvTcGeometry g = conv_tc_geometry_padded(a.N, a.OH, a.OW, a.W, a.IC, a.OC, a.KH, a.KW, a.stride, a.pad_l);
  const int patch_h = g.khs > 1 ? g.TH + a.KH - 1 : g.TH;  // rows of one load
  if (st->a != a.x) {
    if (g.s2 ? !encode_conv_input_pairs(&st->tmA, a.x, a.N, a.H, a.W, a.IC)
             : !encode_conv_input(&st->tmA, a.x, a.N, a.H, a.W, a.IC, g.row_bytes, g.TW, patch_h, a.stride))
      return cudaErrorInvalidValue;
    st->a = a.x;
  }
  if (st->w != a.w) {
    if (!encode_2d(&st->tmB, a.w, (uint64_t)g.n_tiles * g.BN, (uint64_t)g.Kpad, (uint64_t)g.Kpad, (uint32_t)g.BN, g.row_bytes))
      return cudaErrorInvalidValue;
    st->w = a.w;
  }
  if (((uintptr_t)a.out % 16) != 0) return cudaErrorInvalidValue;
  if (st->c != a.out) {
    if (!encode_conv_output(&st->tmC, a.out, a.N, a.OH, a.OW, a.OC, g.BN / g.gpt, g.TWv, g.TH)) return cudaErrorInvalidValue;
    st->c = a.out;
  }
  GemmTcParams p{};
  p.tma_store = 1;
  p.chan = a.chan;
  p.out = a.out;
  p.ldc = a.OC;
  p.N = a.OC;
  p.BN = g.BN;
  p.n_tiles = g.n_tiles;
  p.tiles_w = g.tiles_w;
  p.tiles_per_img = g.tiles_w * g.tiles_h;
  p.m_tiles = a.N * p.tiles_per_img;
  p.M = p.m_tiles * kBM;
  p.k_blocks = g.k_blocks;
  p.k_last_steps = g.row_bytes / 32;
  p.row_bytes = g.row_bytes;
  p.TH = g.TH;
  p.tw_log2 = 0;
  while ((1 << p.tw_log2) < g.TW) p.tw_log2++;
  p.OH = a.OH; p.OW = a.OW; p.cstride = a.stride; p.pad_t = a.pad_t; p.pad_l = a.pad_l; p.KW = a.KW;
  p.icb_per_tap = g.icb_per_tap;
  p.khs = g.khs;
  p.halo = g.halo;
  p.tw_valid = g.TWv;
  p.kcols = g.halo ? a.KW : 1;
  p.k_loads = g.s2 ? 1 : g.halo ? g.icb_per_tap : g.khs > 1 ? a.KW * g.icb_per_tap : g.k_blocks;
  p.patch_rows = patch_h * g.TW;
  p.s2 = g.s2;
  p.a_row_bytes = 2 * a.IC;
  p.s2_stage_bytes = (int)(((size_t)33 * 9 * 2 * a.IC + 1023) / 1024 * 1024);
  p.s2_pair0 = a.pad_l == 1 ? -1 : 0;
  p.corr = a.corr; p.rcls = a.rcls; p.ccls = a.ccls; p.cls_nonzero = a.cls_nonzero; p.ncc = a.ncc;
  const size_t w_bytes = (size_t)g.n_tiles * g.BN * g.Kpad;
  p.w_resident = g.halo || g.s2 || w_bytes <= (size_t)kResidentWeightBytes;
  const size_t stage_bytes = g.s2 ? (size_t)p.s2_stage_bytes
                                  : (size_t)(g.khs > 1 ? p.patch_rows : kBM) * g.row_bytes +
                                        (p.w_resident ? 0 : (size_t)g.BN * g.row_bytes * g.khs);
  const size_t staging_bytes = (size_t)kEpiGroups * kBM * (g.BN / g.gpt);
  const size_t ring_budget = (size_t)kSmemBudget - 1024 - (p.w_resident ? w_bytes : 0) - staging_bytes;
  int stages = (int)(ring_budget / stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return cudaErrorInvalidConfiguration;
  {  // A/B aid: TB200_CONV_STAGES=<n> caps the ring depth (the convolution always stores through the TMA: the
     // register store path indexes rows as a plain GEMM does and is not valid for patch tiles)
    const char* e = getenv("TB200_CONV_STAGES");
    if (e && atoi(e) >= 2 && atoi(e) < stages) stages = atoi(e);
  }
  p.stages = stages;
  p.out_zp = a.out_zp; p.clamp_min = a.clamp_min; p.clamp_max = a.clamp_max; p.q4 = a.q4;
  int stride = 32;
  while (stride < g.BN) stride <<= 1;
  p.acc_stride = stride;
  p.gpt = g.gpt;
  p.BNh = g.BN / g.gpt;
  p.acc_stages = kEpiGroups / g.gpt;
  p.tmem_cols = p.acc_stages * stride;
  p.status = a.status;
  p.wait_ns = wait_limit_ns();
  p.trace = gemm_trace_on();
  p.lut = a.lut;
  p.staging_off = (uint32_t)((p.w_resident ? w_bytes : 0) + (size_t)stages * stage_bytes);
  const size_t smem = 1024 + p.staging_off + staging_bytes;
  static std::atomic<unsigned long long> attr_set{0};
  if (first_use_on_device(attr_set)) {
    const cudaError_t e = gemm_kernels_set_smem(true);
    if (e != cudaSuccess) return e;
    mark_used_on_device(attr_set);
  }
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = tiles < current_sm_count() ? tiles : current_sm_count();
  return launch_dependent_if(tiles >= kDependentMinBlocks / 2, gemm_kernel_for(true, gemm_epi_variant(a.epi, a.clamp_min, a.clamp_max), a.lut != nullptr), dim3(grid), dim3(kThreads), smem, stream, st->tmA, st->tmB, st->tmC, p);
}

}  // namespace tb200
