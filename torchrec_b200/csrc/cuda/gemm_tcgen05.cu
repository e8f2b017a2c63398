// bf16 GEMMs of the dense towers on the 5th-generation tensor cores (tcgen05 / TMEM / TMA), sm_100a.
//
// One persistent kernel, one CTA per SM, specialised warps:
//   warp 0      TMA producer: cp.async.bulk.tensor (128-byte swizzle) into a 4-stage shared-memory ring,
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BLOCK_N, K=16) with the
//               accumulator in tensor memory; tcgen05.commit releases ring slots and publishes tiles,
//   warps 2..5  epilogue: tcgen05.ld the 128 x BLOCK_N fp32 accumulator (double-buffered in TMEM so the
//               next tile's MMAs overlap this tile's epilogue), fuse bias / activation / the DCN-v2
//               "x0 * (acc + b) + x" update / a residual add, and store bf16 (or fp32, optionally with
//               red.add for split-K).
// Operand layouts: NT  C[M,N] = A[M,K] B[N,K]^T (both K-major, forward and input-gradient GEMMs) and
//                  TN  C[N,K] = A[M,N]^T B[M,K] (both MN-major, weight-gradient GEMMs, split over M).
// No load uses cluster multicast.  Every wait on an mbarrier has a time limit; on expiry the CTA raises a
// flag, drains its outstanding copies, frees its tensor memory and returns, and the host reports an error.
//
// The reference runs these products as library GEMMs (torchrec/modules/mlp.py:61-80,
// torchrec/modules/crossnet.py:178-181).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cuda.h>

#include "common.cuh"

namespace trb {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;  // 64 bf16 = 128 bytes = one swizzle span
constexpr int kThreads = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr long long kWaitCycles = 2000000000LL;  // about one second

enum GemmErr : int { ERR_NONE = 0, ERR_FULL_WAIT = 1, ERR_EMPTY_WAIT = 2, ERR_TMEM_FULL_WAIT = 3, ERR_TMEM_EMPTY_WAIT = 4, ERR_EPI_LOAD_WAIT = 5 };

struct GemmParams {
  int M, N, K;        // output rows, output cols, contraction length
  void* out;          // [M, ldc]
  int out_fp32;       // 1: fp32 output, 0: bf16
  int atomic_out;     // 1: red.add into fp32 output (split-K)
  int64_t ldc;
  const float* bias;  // [N] or null
  int act;            // 0 none, 1 relu, 2 sigmoid
  const __nv_bfloat16* mul;  // cross epilogue: y = mul * (acc + bias) + add
  const __nv_bfloat16* add;  // residual add (also the "+ x" of the cross epilogue)
  __nv_bfloat16* u_out;      // cross epilogue: also store u = acc + bias
  int k_splits;
  int kb_per_split;  // k-blocks per split; every split is non-empty
  int* err;
};

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait: false when the limit expired or another role aborted
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      atomicCAS(err, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(tmap), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the shared-memory sources of all committed stores have been read (the buffers may be overwritten)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all committed stores are complete
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make generic-proxy writes to shared memory visible to the async proxy (TMA)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32 columns of fp32: thread `lane` receives row `lane`, columns [c, c+32).  The load is asynchronous;
// tmem_ld_wait names the destination registers as in/out operands so that no use of them can be scheduled above the wait.
__device__ __forceinline__ void tmem_ld_32x32_issue(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                 "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
                 "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3FFFF) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= uint64_t(1) << 46;  // version
  d |= uint64_t(2) << 61;  // SWIZZLE_128B
  return d;
}

__host__ __device__ constexpr uint32_t make_idesc(int n, bool a_mn, bool b_mn) {
  // c_format F32 (1<<4), a/b format BF16 (1<<7, 1<<10), majors, N>>3 at bit 17, M>>4 at bit 24
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(a_mn) << 15) | (uint32_t(b_mn) << 16) |
         (uint32_t(n >> 3) << 17) | (uint32_t(kBlockM >> 4) << 24);
}

enum Epi : int { EPI_PLAIN = 0, EPI_BIAS = 1, EPI_BIAS_RELU = 2, EPI_BIAS_SIGMOID = 3, EPI_CROSS = 4, EPI_ADD = 5, EPI_F32 = 6, EPI_F32_ATOMIC = 7 };

constexpr int kEpiWarps = 8;
constexpr int kEpiBufBytes = 32 * 128;  // 32 rows x 64 bf16 columns, one TMA box

// bf16 epilogues stage their tiles in shared memory and move them with TMA; the fp32 ones write registers directly
__host__ __device__ constexpr bool epi_uses_tma(int epi) { return epi != EPI_F32 && epi != EPI_F32_ATOMIC; }

// Work item -> (output tile, contraction split).  The split is the slow index: the CTAs that run at the same time
// then work on the same slice of the contraction for different output tiles, so every operand slice is fetched
// from DRAM once and re-read from L2 by the other tiles of its row or column.
__device__ __forceinline__ int work_tile(int w, int k_splits, int tiles) { return k_splits == 1 ? w : w % tiles; }
__device__ __forceinline__ int work_split(int w, int k_splits, int tiles) { return k_splits == 1 ? 0 : w / tiles; }

template <int BLOCK_N, int EPI>
struct SmemLayout {
  static constexpr int kABytes = kBlockM * kBlockK * 2;   // 16 KB
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;   // 16 / 32 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  // the cross epilogue needs two staging buffers per warp (x0 -> u, x -> y); it gives up one pipeline stage for them
  static constexpr int kEpiBufs = !epi_uses_tma(EPI) ? 0 : (EPI == EPI_CROSS ? 2 : 1);
  static constexpr int kStages = (EPI == EPI_CROSS && BLOCK_N == 256) ? 3 : 4;
  static constexpr int kEpiBytes = kEpiWarps * kEpiBufs * kEpiBufBytes;
  static constexpr int kTotal = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == 1) return fmaxf(v, 0.f);
  if (act == 2) return 1.f / (1.f + __expf(-v));
  return v;
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
  uint4 pk;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  return pk;
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& pk, float (&v)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}

// One 32-row x 32-column piece of the accumulator: thread `lane` owns row `lane`, r[] are its 32 columns.
// All global loads of the piece are issued before any arithmetic so that their latencies overlap.
template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t (&r)[32], int64_t row_off, int col0) {
  constexpr bool kBias = EPI == EPI_BIAS || EPI == EPI_BIAS_RELU || EPI == EPI_BIAS_SIGMOID || EPI == EPI_CROSS;
  constexpr bool kMul = EPI == EPI_CROSS;
  constexpr bool kAdd = EPI == EPI_CROSS || EPI == EPI_ADD;
  float4 bias[8];
  uint4 mulv[4], addv[4];
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int col = col0 + g * 8;
    if (col < p.N) {
      if constexpr (kBias) {
        bias[2 * g] = __ldg(reinterpret_cast<const float4*>(p.bias + col));
        bias[2 * g + 1] = __ldg(reinterpret_cast<const float4*>(p.bias + col + 4));
      }
      if constexpr (kMul) mulv[g] = *reinterpret_cast<const uint4*>(p.mul + row_off + col);
      if constexpr (kAdd) addv[g] = *reinterpret_cast<const uint4*>(p.add + row_off + col);
    }
  }
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    const int col = col0 + g * 8;
    if (col >= p.N) continue;  // N % 8 == 0: a group of 8 columns is fully inside or outside
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
    if constexpr (kBias) {
      v[0] += bias[2 * g].x; v[1] += bias[2 * g].y; v[2] += bias[2 * g].z; v[3] += bias[2 * g].w;
      v[4] += bias[2 * g + 1].x; v[5] += bias[2 * g + 1].y; v[6] += bias[2 * g + 1].z; v[7] += bias[2 * g + 1].w;
    }
    if constexpr (EPI == EPI_BIAS_RELU) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
    }
    if constexpr (EPI == EPI_BIAS_SIGMOID) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 1.f / (1.f + __expf(-v[j]));
    }
    if constexpr (EPI == EPI_CROSS) {
      // u = acc + bias is stored in bf16 and y is computed from the rounded u, so that y == x0 * u + x exactly as saved
      const uint4 upk = pack_bf16x8(v);
      *reinterpret_cast<uint4*>(p.u_out + row_off + col) = upk;
      unpack_bf16x8(upk, v);
      float m[8];
      unpack_bf16x8(mulv[g], m);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= m[j];
    }
    if constexpr (kAdd) {
      float a[8];
      unpack_bf16x8(addv[g], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += a[j];
    }
    if constexpr (EPI == EPI_F32 || EPI == EPI_F32_ATOMIC) {
      float* o = reinterpret_cast<float*>(p.out) + row_off + col;
      if constexpr (EPI == EPI_F32_ATOMIC) {
        red_add_f32x4(o, make_float4(v[0], v[1], v[2], v[3]));
        red_add_f32x4(o + 4, make_float4(v[4], v[5], v[6], v[7]));
      } else {
        *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
      }
    } else {
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + row_off + col) = pack_bf16x8(v);
    }
  }
}

// MN_MAJOR = false: A[M,K], B[N,K] row-major (K contiguous).  tmapA box {64 k, 128 rows}, tmapB box {64 k, BLOCK_N rows}.
// MN_MAJOR = true : A[Kc,M], B[Kc,N] row-major (output dims contiguous, contraction along rows).
//                   tmap boxes are {64 cols, 64 rows}; a stage holds M/64 (resp. N/64) such boxes.
template <int BLOCK_N, bool MN_MAJOR, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                 const __grid_constant__ CUtensorMap tmapOut, const __grid_constant__ CUtensorMap tmapU,
                 const __grid_constant__ CUtensorMap tmapMul, const __grid_constant__ CUtensorMap tmapAdd, GemmParams p) {
  using L = SmemLayout<BLOCK_N, EPI>;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + kStages * L::kStageBytes;  // 1024-byte aligned: stage sizes are multiples of 1024
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + L::kEpiBytes);
  uint64_t* full = bars;                       // [kStages]
  uint64_t* empty = bars + kStages;            // [kStages]
  uint64_t* tmem_full = bars + 2 * kStages;    // [2]
  uint64_t* tmem_empty = bars + 2 * kStages + 2;  // [2]
  uint64_t* in_bars = bars + 2 * kStages + 4;  // [kEpiWarps] epilogue operand tiles have landed
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4 + kEpiWarps);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + kBlockM - 1) / kBlockM;
  const int n_tiles = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int kb_total = (p.K + kBlockK - 1) / kBlockK;
  const int kb_per_split = p.kb_per_split;
  const int tiles_total = m_tiles * n_tiles;
  const int num_work = tiles_total * p.k_splits;
  constexpr uint32_t kTmemCols = 2 * BLOCK_N;  // two accumulators

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], kEpiWarps);  // one arrival per epilogue warp
    }
    for (int w = 0; w < kEpiWarps; ++w) mbar_init(&in_bars[w], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const int tile = work_tile(w, p.k_splits, tiles_total), ks = work_split(w, p.k_splits, tiles_total);
        const int m_blk = tile / n_tiles, n_blk = tile - m_blk * n_tiles;
        const int kb0 = ks * kb_per_split, kb1 = min(kb_total, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.err, ERR_EMPTY_WAIT)) { ok = false; break; }
          uint8_t* sa = smem + s * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full[s], L::kStageBytes);
          if (!MN_MAJOR) {
            tma_load_2d(sa, &tmapA, &full[s], kb * kBlockK, m_blk * kBlockM);
            tma_load_2d(sb, &tmapB, &full[s], kb * kBlockK, n_blk * BLOCK_N);
          } else {
#pragma unroll
            for (int c = 0; c < kBlockM / 64; ++c)
              tma_load_2d(sa + c * 8192, &tmapA, &full[s], m_blk * kBlockM + c * 64, kb * kBlockK);
#pragma unroll
            for (int c = 0; c < BLOCK_N / 64; ++c)
              tma_load_2d(sb + c * 8192, &tmapB, &full[s], n_blk * BLOCK_N + c * 64, kb * kBlockK);
          }
        }
      }
      if (!ok) {
        // drain: wait (bounded) until the copies already issued have landed before the CTA may exit
        const long long t0 = clock64();
        for (uint32_t j = (it > kStages ? it - kStages : 0); j < it; ++j) {
          const int s = j % kStages;
          const uint32_t ph = (j / kStages) & 1;
          while (!mbar_try_wait(&full[s], ph) && clock64() - t0 < kWaitCycles) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BLOCK_N, MN_MAJOR, MN_MAJOR);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++tile_it) {
        const int ks = work_split(w, p.k_splits, tiles_total);
        const int kb0 = ks * kb_per_split, kb1 = min(kb_total, kb0 + kb_per_split);
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1, abort_flag, p.err, ERR_TMEM_EMPTY_WAIT)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BLOCK_N;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, p.err, ERR_FULL_WAIT)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            uint64_t da, db;
            if (!MN_MAJOR) {
              da = make_smem_desc(sa + k * 32, 16, 1024);
              db = make_smem_desc(sb + k * 32, 16, 1024);
            } else {
              da = make_smem_desc(sa + k * 2048, 8192, 1024);
              db = make_smem_desc(sb + k * 2048, 8192, 1024);
            }
            umma_bf16(tmem_d, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tcgen05_commit(&empty[s]);  // slot reusable once these MMAs have read it
        }
        if (ok) tcgen05_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    // Two warps share each TMEM lane quarter (warp % 4) and split the tile's columns in halves.  The TMEM load of
    // the next 32-column piece is in flight while the current one is processed.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    constexpr int kPieces = BLOCK_N / 64;  // 32-column pieces per warp
    uint32_t tile_it = 0;
    bool ok = true;
    if constexpr (epi_uses_tma(EPI)) {
      // bf16 output through shared memory and TMA.  A warp owns 32 rows x 64 columns at a time ("box": two TMEM
      // pieces).  Operand tiles of the fused epilogue (x0 and x of the cross layer, the residual) arrive by TMA load
      // into the same buffers the results leave from: lane `l` reads the 16-byte chunks of its row, computes, and
      // writes the result over them; one lane then issues the TMA store.  Chunk c of row l sits at c ^ (l & 7),
      // the 128-byte swizzle of the tensor maps, which also keeps the 16-byte accesses free of bank conflicts.
      constexpr bool kBias = EPI == EPI_BIAS || EPI == EPI_BIAS_RELU || EPI == EPI_BIAS_SIGMOID || EPI == EPI_CROSS;
      constexpr bool kMul = EPI == EPI_CROSS;
      constexpr bool kAdd = EPI == EPI_CROSS || EPI == EPI_ADD;
      constexpr bool kIn = kMul || kAdd;
      constexpr int kBoxes = BLOCK_N / 128;  // boxes per warp per tile
      const int ew = warp - 2;
      uint8_t* bufA = epi_smem + ew * L::kEpiBufs * kEpiBufBytes;  // cross: x0 -> u.  otherwise: (residual ->) out
      uint8_t* bufB = bufA + (L::kEpiBufs > 1 ? kEpiBufBytes : 0);  // cross: x -> y
      uint8_t* bufOut = EPI == EPI_CROSS ? bufB : bufA;
      uint64_t* in_bar = &in_bars[ew];
      uint32_t in_uses = 0;
      bool in_flight = false;
      const uint32_t sw = uint32_t(lane & 7);
      auto load_operands = [&](int row0, int col0) {
        // previous stores must have read the buffers before new data may land in them
        if (lane == 0) {
          tma_store_wait_read();
          mbar_expect_tx(in_bar, (int(kMul) + int(kAdd)) * kEpiBufBytes);
          if constexpr (kMul) tma_load_2d(bufA, &tmapMul, in_bar, col0, row0);
          if constexpr (kAdd) tma_load_2d(bufOut, &tmapAdd, in_bar, col0, row0);
        }
        in_flight = true;
      };
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++tile_it) {
        const int tile = work_tile(w, p.k_splits, tiles_total);
        const int m_blk = tile / n_tiles, n_blk = tile - m_blk * n_tiles;
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        const int row0 = m_blk * kBlockM + q * 32;
        const int colbase = n_blk * BLOCK_N + half * (BLOCK_N / 2);
        const bool rows_ok = row0 < p.M;
        if constexpr (kIn) {
          // operands of the first box travel while the MMAs of this tile may still be running
          if (rows_ok && colbase < p.N) load_operands(row0, colbase);
          if constexpr (kBoxes > 1) {
            if (lane == 0 && rows_ok && colbase + 64 < p.N) {
              if constexpr (kMul) tma_prefetch_2d(&tmapMul, colbase + 64, row0);
              if constexpr (kAdd) tma_prefetch_2d(&tmapAdd, colbase + 64, row0);
            }
          }
        }
        if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.err, ERR_TMEM_FULL_WAIT)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tbase = tmem_base + (uint32_t(q * 32) << 16) + acc * BLOCK_N + half * (BLOCK_N / 2);
        uint32_t r[2][32];
        tmem_ld_32x32_issue(tbase, r[0]);
#pragma unroll
        for (int c = 0; c < kPieces; ++c) {
          const int box = c >> 1, h = c & 1;
          const int col0 = colbase + box * 64;
          const bool active = rows_ok && col0 < p.N;
          tmem_ld_wait(r[c & 1]);
          if (c + 1 < kPieces) {
            tmem_ld_32x32_issue(tbase + (c + 1) * 32, r[(c + 1) & 1]);
          } else {
            // every TMEM read of this tile has completed: hand the accumulator back to the MMA warp
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          }
          if (h == 0) {
            if constexpr (kIn) {
              if (active && box > 0) load_operands(row0, col0);
              if (in_flight) {
                const bool landed = mbar_wait(in_bar, in_uses & 1, abort_flag, p.err, ERR_EPI_LOAD_WAIT);
                if (__all_sync(0xffffffffu, landed)) {
                  ++in_uses;
                  in_flight = false;
                } else {
                  ok = false;
                }
              }
            } else {
              if (active && lane == 0) tma_store_wait_read();
              __syncwarp();
            }
          }
          if (!ok) {
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            break;
          }
          if (active) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int chunk = h * 4 + g;
              const int col = col0 + chunk * 8;
              const uint32_t off = uint32_t(lane) * 128u + ((uint32_t(chunk) ^ sw) << 4);
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[c & 1][g * 8 + j]);
              if constexpr (kBias) {
                if (col < p.N) {
                  const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + col));
                  const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + col + 4));
                  v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                  v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                }
              }
              if constexpr (EPI == EPI_BIAS_RELU) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
              }
              if constexpr (EPI == EPI_BIAS_SIGMOID) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = 1.f / (1.f + __expf(-v[j]));
              }
              if constexpr (EPI == EPI_CROSS) {
                // u = acc + bias is stored in bf16 and y is computed from the rounded u, so that y == x0 * u + x as saved
                uint4* pa = reinterpret_cast<uint4*>(bufA + off);
                const uint4 upk = pack_bf16x8(v);
                float m[8];
                unpack_bf16x8(*pa, m);
                *pa = upk;
                unpack_bf16x8(upk, v);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] *= m[j];
              }
              uint4* po = reinterpret_cast<uint4*>(bufOut + off);
              if constexpr (kAdd) {
                float a[8];
                unpack_bf16x8(*po, a);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += a[j];
              }
              *po = pack_bf16x8(v);
            }
            if (h == 1) {
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                if constexpr (EPI == EPI_CROSS) tma_store_2d(&tmapU, bufA, col0, row0);
                tma_store_2d(&tmapOut, bufOut, col0, row0);
                tma_store_commit();
              }
            }
          }
        }
      }
      if (lane == 0) {
        if (!ok && in_flight) {
          // operand tiles may still be on their way into shared memory: give them a bounded time to land
          const long long t0 = clock64();
          while (!mbar_try_wait(in_bar, in_uses & 1) && clock64() - t0 < kWaitCycles) {
          }
        }
        tma_store_wait_all();
      }
    } else {
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x, ++tile_it) {
        const int tile = work_tile(w, p.k_splits, tiles_total);
        const int m_blk = tile / n_tiles, n_blk = tile - m_blk * n_tiles;
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!mbar_wait(&tmem_full[acc], acc_ph, abort_flag, p.err, ERR_TMEM_FULL_WAIT)) { ok = false; break; }
        tcgen05_fence_after();
        const int row = m_blk * kBlockM + q * 32 + lane;
        const bool row_ok = row < p.M;
        const int64_t row_off = int64_t(row) * p.ldc;
        const int colbase = n_blk * BLOCK_N + half * (BLOCK_N / 2);
        const uint32_t tbase = tmem_base + (uint32_t(q * 32) << 16) + acc * BLOCK_N + half * (BLOCK_N / 2);
        uint32_t r[2][32];
        tmem_ld_32x32_issue(tbase, r[0]);
#pragma unroll
        for (int c = 0; c < kPieces; ++c) {
          tmem_ld_wait(r[c & 1]);
          if (c + 1 < kPieces) tmem_ld_32x32_issue(tbase + (c + 1) * 32, r[(c + 1) & 1]);
          const int col0 = colbase + c * 32;
          if (row_ok && col0 < p.N) epilogue_chunk<EPI>(p, r[c & 1], row_off, col0);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// ---- host ------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
  static EncodeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q);
    TORCH_CHECK(e == cudaSuccess && f != nullptr, "cuTensorMapEncodeTiled is not available");
    return reinterpret_cast<EncodeFn>(f);
  }();
  return fn;
}

// 2-D bf16 row-major tensor [rows, cols]; box = {box_cols (inner), box_rows}; 128-byte swizzle, zero fill
static CUtensorMap make_tmap(const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows) {
  CUtensorMap m;
  cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(ld) * 2};
  cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  TORCH_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * 2) % 16 == 0, "TMA operand must be 16-byte aligned");
  CUresult r = get_encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", int(r));
  return m;
}

static int num_sms() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

static at::Tensor& err_flag(const at::Device& dev) {
  static std::vector<at::Tensor> flags(64);
  auto& f = flags[dev.index() < 0 ? 0 : dev.index()];
  if (!f.defined()) f = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return f;
}

template <bool MN_MAJOR>
static void launch_gemm(const at::Tensor& a, const at::Tensor& b, GemmParams p) {
  auto stream = at::cuda::getCurrentCUDAStream();
  p.err = err_flag(a.device()).data_ptr<int>();
  {
    const int kb_total = (p.K + kBlockK - 1) / kBlockK;
    p.k_splits = std::max(1, std::min(p.k_splits, kb_total));
    p.kb_per_split = (kb_total + p.k_splits - 1) / p.k_splits;
    p.k_splits = (kb_total + p.kb_per_split - 1) / p.kb_per_split;  // drop splits that would be empty
  }
  const bool wide = p.N > 128;
  CUtensorMap ta, tb;
  if (!MN_MAJOR) {
    ta = make_tmap(a.data_ptr(), a.size(0), a.size(1), a.stride(0), kBlockK, kBlockM);
    tb = make_tmap(b.data_ptr(), b.size(0), b.size(1), b.stride(0), kBlockK, wide ? 256 : 128);
  } else {
    ta = make_tmap(a.data_ptr(), a.size(0), a.size(1), a.stride(0), 64, kBlockK);
    tb = make_tmap(b.data_ptr(), b.size(0), b.size(1), b.stride(0), 64, kBlockK);
  }
  const int BN = wide ? 256 : 128;
  const int m_tiles = (p.M + kBlockM - 1) / kBlockM, n_tiles = (p.N + BN - 1) / BN;
  const int work = m_tiles * n_tiles * p.k_splits;
  const int grid = std::min(work, num_sms());
  int epi;
  if (p.out_fp32) epi = p.atomic_out ? EPI_F32_ATOMIC : EPI_F32;
  else if (p.u_out) epi = EPI_CROSS;
  else if (p.add) epi = EPI_ADD;
  else if (p.bias) epi = p.act == 1 ? EPI_BIAS_RELU : (p.act == 2 ? EPI_BIAS_SIGMOID : EPI_BIAS);
  else epi = EPI_PLAIN;
  TORCH_CHECK(!(p.out_fp32 && (p.bias || p.act || p.add || p.mul)), "fp32 output supports the plain product only");
  TORCH_CHECK(p.bias || p.act == 0, "an activation needs a bias operand (pass zeros)");
  // bf16 epilogues move 32-row x 64-column boxes of the output (and of the fused operands) by TMA
  CUtensorMap t_out = ta, t_u = ta, t_mul = ta, t_add = ta;
  if (epi_uses_tma(epi)) {
    t_out = make_tmap(p.out, p.M, p.N, p.ldc, 64, 32);
    t_u = p.u_out ? make_tmap(p.u_out, p.M, p.N, p.ldc, 64, 32) : t_out;
    t_mul = p.mul ? make_tmap(p.mul, p.M, p.N, p.ldc, 64, 32) : t_out;
    t_add = p.add ? make_tmap(p.add, p.M, p.N, p.ldc, 64, 32) : t_out;
  }
  auto launch = [&](auto kernel, int smem) {
    // the attribute is per kernel instantiation; setting it is cheap and idempotent
    TRB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    kernel<<<grid, kThreads, smem, stream>>>(ta, tb, t_out, t_u, t_mul, t_add, p);
  };
#define TRB_GEMM_CASE(E)                                                                              \
  case E:                                                                                             \
    if (wide) launch(gemm_bf16_kernel<256, MN_MAJOR, E>, SmemLayout<256, E>::kTotal);                 \
    else launch(gemm_bf16_kernel<128, MN_MAJOR, E>, SmemLayout<128, E>::kTotal);                      \
    break;
  if constexpr (MN_MAJOR) {
    switch (epi) {
      TRB_GEMM_CASE(EPI_F32)
      TRB_GEMM_CASE(EPI_F32_ATOMIC)
      default: TORCH_CHECK(false, "unsupported epilogue for the TN product");
    }
  } else {
    switch (epi) {
      TRB_GEMM_CASE(EPI_PLAIN)
      TRB_GEMM_CASE(EPI_BIAS)
      TRB_GEMM_CASE(EPI_BIAS_RELU)
      TRB_GEMM_CASE(EPI_BIAS_SIGMOID)
      TRB_GEMM_CASE(EPI_CROSS)
      TRB_GEMM_CASE(EPI_ADD)
      TRB_GEMM_CASE(EPI_F32)
      default: TORCH_CHECK(false, "unsupported epilogue for the NT product");
    }
  }
#undef TRB_GEMM_CASE
  TRB_CUDA_CHECK(cudaGetLastError());
}

static void check_nt(const at::Tensor& a, const at::Tensor& b) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "gemm_nt: a [M,K], b [N,K]");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && a.size(1) % 8 == 0 && b.size(0) % 8 == 0);
}

// act(a @ b^T + bias) -> bf16 (or fp32)
at::Tensor gemm_nt_bf16(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& bias, int64_t act,
                        bool out_fp32) {
  check_nt(a, b);
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  at::Tensor out = at::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  if (M == 0) return out;
  GemmParams p{};
  p.M = int(M); p.N = int(N); p.K = int(K);
  p.out = out.data_ptr(); p.out_fp32 = out_fp32 ? 1 : 0; p.ldc = N;
  at::Tensor bias_c;
  if (bias.has_value() && bias->defined()) {
    bias_c = bias->to(at::kFloat).contiguous();
    TORCH_CHECK(bias_c.numel() == N);
    p.bias = bias_c.data_ptr<float>();
  }
  p.act = int(act);
  p.k_splits = 1;
  launch_gemm<false>(a, b, p);
  return out;
}

// u = a @ b^T + bias ; y = x0 * u + xl
std::tuple<at::Tensor, at::Tensor> gemm_nt_bf16_cross(const at::Tensor& a, const at::Tensor& b, const at::Tensor& bias,
                                                      const at::Tensor& x0, const at::Tensor& xl) {
  check_nt(a, b);
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  TORCH_CHECK(x0.is_contiguous() && xl.is_contiguous() && x0.size(0) == M && x0.size(1) == N && xl.sizes() == x0.sizes());
  TORCH_CHECK(x0.scalar_type() == at::kBFloat16 && xl.scalar_type() == at::kBFloat16);
  at::Tensor u = at::empty({M, N}, a.options()), y = at::empty({M, N}, a.options());
  if (M == 0) return {u, y};
  at::Tensor bias_c = bias.to(at::kFloat).contiguous();
  GemmParams p{};
  p.M = int(M); p.N = int(N); p.K = int(K);
  p.out = y.data_ptr(); p.ldc = N;
  p.bias = bias_c.data_ptr<float>();
  p.mul = reinterpret_cast<const __nv_bfloat16*>(x0.data_ptr());
  p.add = reinterpret_cast<const __nv_bfloat16*>(xl.data_ptr());
  p.u_out = reinterpret_cast<__nv_bfloat16*>(u.data_ptr());
  p.k_splits = 1;
  launch_gemm<false>(a, b, p);
  return {u, y};
}

// a @ b^T + add
at::Tensor gemm_nt_bf16_add(const at::Tensor& a, const at::Tensor& b, const at::Tensor& add) {
  check_nt(a, b);
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  TORCH_CHECK(add.is_contiguous() && add.size(0) == M && add.size(1) == N && add.scalar_type() == at::kBFloat16);
  at::Tensor out = at::empty({M, N}, a.options());
  if (M == 0) return out;
  GemmParams p{};
  p.M = int(M); p.N = int(N); p.K = int(K);
  p.out = out.data_ptr(); p.ldc = N;
  p.add = reinterpret_cast<const __nv_bfloat16*>(add.data_ptr());
  p.k_splits = 1;
  launch_gemm<false>(a, b, p);
  return out;
}

// a^T @ b : a [Mc, N], b [Mc, K] -> [N, K] fp32 (weight gradient), split over the contraction.  With `acc` the product is
// ADDED into that tensor (every work item reduces into it with red.add), which lets a weight gradient land directly in a
// pre-zeroed flat gradient buffer: no output allocation, no zero fill, no accumulation pass afterwards.
static at::Tensor gemm_tn_impl(const at::Tensor& a, const at::Tensor& b, c10::optional<at::Tensor> acc) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(0) == b.size(0) && a.stride(1) == 1 && b.stride(1) == 1);
  TORCH_CHECK(a.size(1) % 8 == 0 && b.size(1) % 8 == 0);
  c10::cuda::CUDAGuard guard(a.device());
  const int64_t Mc = a.size(0), N = a.size(1), K = b.size(1);
  GemmParams p{};
  p.M = int(N); p.N = int(K); p.K = int(Mc);
  const int BN = p.N > 128 ? 256 : 128;
  const int tiles = ((p.M + kBlockM - 1) / kBlockM) * ((p.N + BN - 1) / BN);
  const int kb_total = int((Mc + kBlockK - 1) / kBlockK);
  // split the contraction so that the work items fill whole waves of the persistent grid: estimate
  // rounds x (k-blocks per item + epilogue) for every candidate and keep the cheapest
  int splits = 1;
  {
    const int sms = num_sms();
    const int max_splits = std::max(1, std::min(kb_total / 4, 64));
    double best = 1e30;
    for (int s = 1; s <= max_splits; ++s) {
      const int kbps = (kb_total + s - 1) / s;
      const int s_eff = (kb_total + kbps - 1) / kbps;
      const int rounds = (tiles * s_eff + sms - 1) / sms;
      const double cost = double(rounds) * (kbps + 4.0) + 0.25 * s_eff;  // mild penalty on atomic traffic
      if (cost < best) { best = cost; splits = s_eff; }
    }
  }
  const bool into = acc.has_value() && acc->defined();
  at::Tensor out;
  if (into) {
    out = *acc;
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.dim() == 2 && out.size(0) == N && out.size(1) == K && out.is_contiguous(),
                "accumulator must be a contiguous fp32 [N, K] tensor");
    if (Mc == 0) return out;
  } else {
    out = splits > 1 ? at::zeros({N, K}, a.options().dtype(at::kFloat)) : at::empty({N, K}, a.options().dtype(at::kFloat));
    if (Mc == 0) return out.zero_();
  }
  p.out = out.data_ptr(); p.out_fp32 = 1; p.atomic_out = (splits > 1 || into) ? 1 : 0; p.ldc = K;
  p.k_splits = splits;
  launch_gemm<true>(a, b, p);
  return out;
}

at::Tensor gemm_tn_bf16(const at::Tensor& a, const at::Tensor& b) { return gemm_tn_impl(a, b, c10::nullopt); }

void gemm_tn_bf16_acc(const at::Tensor& a, const at::Tensor& b, at::Tensor acc) { gemm_tn_impl(a, b, acc); }

// nonzero after a kernel gave up waiting (one device-to-host read; resets the flag)
int64_t gemm_error_status() {
  int dev = 0;
  cudaGetDevice(&dev);
  at::Tensor& f = err_flag(at::Device(at::kCUDA, dev));
  const int v = f.item<int>();
  if (v != 0) f.zero_();
  return v;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("gemm_nt_bf16(Tensor a, Tensor b, Tensor? bias, int act, bool out_fp32) -> Tensor");
  m.def("gemm_nt_bf16_cross(Tensor a, Tensor b, Tensor bias, Tensor x0, Tensor xl) -> (Tensor, Tensor)");
  m.def("gemm_nt_bf16_add(Tensor a, Tensor b, Tensor add) -> Tensor");
  m.def("gemm_tn_bf16(Tensor a, Tensor b) -> Tensor");
  m.def("gemm_tn_bf16_acc(Tensor a, Tensor b, Tensor(a!) acc) -> ()");
  m.def("gemm_error_status() -> int");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("gemm_nt_bf16", &trb::gemm_nt_bf16);
  m.impl("gemm_nt_bf16_cross", &trb::gemm_nt_bf16_cross);
  m.impl("gemm_nt_bf16_add", &trb::gemm_nt_bf16_add);
  m.impl("gemm_tn_bf16", &trb::gemm_tn_bf16);
  m.impl("gemm_tn_bf16_acc", &trb::gemm_tn_bf16_acc);
}

TORCH_LIBRARY_IMPL(trb200, CompositeExplicitAutograd, m) { m.impl("gemm_error_status", &trb::gemm_error_status); }
