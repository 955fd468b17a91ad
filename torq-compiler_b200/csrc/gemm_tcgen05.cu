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
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0      : TMA producer  - A tile 128 x 128 B and W tile BN x 128 B per K block,
//                 128-byte swizzled, 4-stage ring guarded by full/empty mbarriers
//   warp 1      : MMA issuer    - one elected lane issues tcgen05.mma (M=128, N=BN, K=32),
//                 accumulators in TMEM, double buffered (2 x BN columns)
//   warps 2..9  : epilogue      - two groups of 4 warps, group g drains accumulator stage g
//                 (alternating tiles): tcgen05.ld 32 columns at a time with the next load in
//                 flight, int64 requant on CUDA cores, 16-byte stores; overlaps the MMAs
// Every mbarrier wait is bounded: on expiry the kernel records a code in the device
// status word and every role drains to the common exit, where TMEM is freed.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "kernels.h"

namespace tb200 {

namespace {

constexpr int kStages = 4;
constexpr int kBM = 128;
constexpr int kBK = 128;  // bytes of K per stage = one 128-byte swizzle row
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

struct GemmTcParams {
  const ChanParams* chan;
  int8_t* out;
  long long ldc;
  int M, N, BN, n_tiles, m_tiles, k_blocks, k_last_steps;
  int out_zp, clamp_min, clamp_max;
  int acc_stride, tmem_cols;
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

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
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false (and a code in the status word) if the phase does not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++)
      if (mbar_try_wait(bar, parity)) return true;
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      if (*(volatile int*)status == 0) *(volatile int*)status = code;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  // K-major operand, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused for this layout)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // descriptor version of sm_100
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

// Issue a 32-column load without waiting; tmem_ld_wait32 completes it. The wait names the
// destination registers as operands so that no use of them can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
      "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait32(uint32_t (&v)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                 "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
                 "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]),
                 "+r"(v[23]), "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]),
                 "+r"(v[30]), "+r"(v[31])
               :
               : "memory");
}

template <bool HI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages], bar_empty[kStages], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) ChanParams cp_s[2][256];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t b_stage_bytes = (uint32_t)p.BN * kBK;
  const uint32_t smem_a = smem_base;
  const uint32_t smem_b = smem_base + kStages * kBM * kBK;
  const int total_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(smem_u32(&bar_acc_full[s]), 1);
      mbar_init(smem_u32(&bar_acc_empty[s]), kEpiWarps / 2);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int m = t / p.n_tiles, n = t - m * p.n_tiles;
        for (int kb = 0; kb < p.k_blocks; kb++) {
          if (!(ok = mbar_wait(smem_u32(&bar_empty[s]), phase ^ 1, p.status, 1))) break;
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_expect_tx(full, kBM * kBK + b_stage_bytes);
          tma_load_2d(smem_a + s * (kBM * kBK), &tmA, kb * kBK, m * kBM, full);
          tma_load_2d(smem_b + s * b_stage_bytes, &tmB, kb * kBK, n * p.BN, full);
          if (++s == kStages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      int s = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, it++) {
        const int as = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!(ok = mbar_wait(smem_u32(&bar_acc_empty[as]), acc_phase ^ 1, p.status, 2))) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(as * p.acc_stride);
        for (int kb = 0; kb < p.k_blocks; kb++) {
          if (!(ok = mbar_wait(smem_u32(&bar_full[s]), phase, p.status, 3))) break;
          tc_fence_after();
          const int steps = (kb == p.k_blocks - 1) ? p.k_last_steps : (kBK / 32);
          const uint64_t da = make_smem_desc(smem_a + s * (kBM * kBK));
          const uint64_t db = make_smem_desc(smem_b + s * b_stage_bytes);
          for (int k = 0; k < steps; k++) mma_i8(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          mma_commit(smem_u32(&bar_empty[s]));  // frees the smem stage once the MMAs have read it
          if (++s == kStages) {
            s = 0;
            phase ^= 1;
          }
        }
        if (ok) mma_commit(smem_u32(&bar_acc_full[as]));
      }
    }
  } else {
    // ------------------------------------------------ epilogue: two groups of 4 warps, alternating tiles
    const int q = warp & 3;                // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;     // group g drains accumulator stage g
    const int e = (threadIdx.x - 64) & 127;
    ChanParams* cps = cp_s[group];
    const uint32_t lo2 = (uint32_t)(p.clamp_min & 0xffff) * 0x10001u;
    const uint32_t hi2 = (uint32_t)(p.clamp_max & 0xffff) * 0x10001u;
    const bool vec_ok = (p.ldc & 15) == 0;
    const int nfull = p.BN >> 5;
    int loaded_n = -1;
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x, it++) {
      if ((it & 1) != group) continue;
      const int m = t / p.n_tiles, n = t - m * p.n_tiles;
      if (n != loaded_n) {
        if (group == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
        for (int i = e; i < p.BN; i += 128) cps[i] = p.chan[n * p.BN + i];
        if (group == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
        loaded_n = n;
      }
      const uint32_t acc_phase = (it >> 1) & 1;
      if (ok) ok = mbar_wait(smem_u32(&bar_acc_full[group]), acc_phase, p.status, 4);
      if (!ok) continue;  // keep taking part in the named barriers above
      tc_fence_after();
      const int row = m * kBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(group * p.acc_stride);
      int8_t* orow = p.out + (long long)row * p.ldc + (long long)n * p.BN;
      const int ncol0 = n * p.BN;

      // requantise 16 accumulators starting at tile column c0 and store them
      auto emit16 = [&](const uint32_t* v, int c0) {
        uint32_t w4[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
          int r[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const ChanParams cp = cps[c0 + g * 4 + j];
            r[j] = scale_cp<HI>((int)v[g * 4 + j] + cp.bias, cp) + p.out_zp;
          }
          w4[g] = clamp_pack4(r[0], r[1], r[2], r[3], lo2, hi2);
        }
        if (row < p.M) {
          if (vec_ok && ncol0 + c0 + 16 <= p.N) {
            *reinterpret_cast<uint4*>(orow + c0) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
              if (ncol0 + c0 + j < p.N) orow[c0 + j] = (int8_t)(w4[j >> 2] >> (8 * (j & 3)));
          }
        }
      };

      uint32_t va[32], vb[32];
      if (nfull > 0) tmem_ld32_issue(taddr, va);
      tmem_ld_wait32(va);
      for (int c = 0; c < nfull; c += 2) {
        if (c + 1 < nfull) tmem_ld32_issue(taddr + (c + 1) * 32, vb);
        emit16(va, c * 32);
        emit16(va + 16, c * 32 + 16);
        tmem_ld_wait32(vb);
        if (c + 1 < nfull) {
          if (c + 2 < nfull) tmem_ld32_issue(taddr + (c + 2) * 32, va);
          emit16(vb, (c + 1) * 32);
          emit16(vb + 16, (c + 1) * 32 + 16);
          tmem_ld_wait32(va);
        }
      }
      if (p.BN & 16) {
        uint32_t vt[16];
        tmem_ld16(taddr + nfull * 32, vt);
        emit16(vt, nfull * 32);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[group]));
    }
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

// 2-D byte tensor [rows, cols] with a row pitch; box = [box_rows, 128 bytes], 128-byte swizzle.
bool encode_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

void gemm_tc_tiling(int N, int& BN, int& n_tiles) {
  const int npad = (N + 15) / 16 * 16;
  n_tiles = (npad + 255) / 256;
  BN = ((npad + n_tiles - 1) / n_tiles + 15) / 16 * 16;
}

bool gemm_tc_supported(long long M, int N, int K, long long lda) {
  return M >= 1 && N >= 1 && K >= 16 && (K % 16) == 0 && (lda % 16) == 0 && lda >= K;
}

struct GemmTcState {
  const void* a = nullptr;
  const void* w = nullptr;
  CUtensorMap tmA, tmB;
};

GemmTcState* gemm_tc_state_new() { return new GemmTcState(); }
void gemm_tc_state_free(GemmTcState* s) { delete s; }

cudaError_t launch_gemm_i8_tc(const GemmTcArgs& a, GemmTcState* st, cudaStream_t stream) {
  const int k_blocks = (a.K + kBK - 1) / kBK;
  if (st->a != a.a) {
    if (!encode_2d(&st->tmA, a.a, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)a.lda, kBM)) return cudaErrorInvalidValue;
    st->a = a.a;
  }
  if (st->w != a.w) {
    if (!encode_2d(&st->tmB, a.w, (uint64_t)a.n_tiles * a.BN, (uint64_t)a.Kpad, (uint64_t)a.Kpad, (uint32_t)a.BN))
      return cudaErrorInvalidValue;
    st->w = a.w;
  }
  GemmTcParams p{};
  p.chan = a.chan;
  p.out = a.out;
  p.ldc = a.ldc;
  p.M = (int)a.M;
  p.N = a.N;
  p.BN = a.BN;
  p.n_tiles = a.n_tiles;
  p.m_tiles = (int)((a.M + kBM - 1) / kBM);
  p.k_blocks = k_blocks;
  p.k_last_steps = ((a.K - (k_blocks - 1) * kBK) + 31) / 32;
  p.out_zp = a.out_zp;
  p.clamp_min = a.clamp_min;
  p.clamp_max = a.clamp_max;
  int stride = 32;
  while (stride < a.BN) stride <<= 1;
  p.acc_stride = stride;
  p.tmem_cols = 2 * stride;
  p.status = a.status;
  const size_t smem = 1024 + (size_t)kStages * (kBM * kBK + (size_t)a.BN * kBK);
  static size_t smem_set = 0;
  if (smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(197 * 1024));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_i8_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(197 * 1024));
    if (e != cudaSuccess) return e;
    smem_set = 197 * 1024;
  }
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (a.hi_shift) gemm_i8_tc_kernel<true><<<grid, kThreads, smem, stream>>>(st->tmA, st->tmB, p);
  else gemm_i8_tc_kernel<false><<<grid, kThreads, smem, stream>>>(st->tmA, st->tmB, p);
  return cudaGetLastError();
}

}  // namespace tb200
