// Dot interaction on the tensor cores (bf16): Z = X X^T per sample, X = [dense; sparse] of shape [n <= 32, D].
//
// One warp owns one sample.  X is staged once in shared memory as bf16 rows with a 16-byte pad (conflict-free fragment loads),
// rows n..31 zero.  Forward: Z[32, 32] = X X^T as 2 x 4 tiles of mma.m16n8k16 over D / 16 k-steps (the two tiles below the
// diagonal are skipped); both operands are read from the same rows, so eight 32-bit shared loads per lane and k-step feed all
// fragments.  Backward: dX[32, D] = S X with S the symmetric [32, 32] matrix of pair gradients (zero diagonal), built in shared
// memory from the incoming gradient; 2 x D/8 tiles over two k-steps.
//
// The op is memory-bound (one read of X, one small write) once the 27 x 27 x 128 multiply-adds per sample leave the CUDA
// cores; per-sample tiles are far below the 64-row minimum of tcgen05.mma, so the warp-level mma is the fitting instruction
// here.  The reference gets the op from torch (triu_indices + bmm, torchrec/models/dlrm.py:222-254).
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

namespace trb {

constexpr int kDotRows = 32;        // padded number of vectors per sample
constexpr int kDotWarps = 4;        // samples per CTA

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// stage X of sample b into `xs` ([32][pitch] bf16, pitch = D + 8); D % 8 == 0
__device__ __forceinline__ void dot_stage_x(const __nv_bfloat16* __restrict__ dense, const __nv_bfloat16* __restrict__ sparse, int64_t b, int F,
                                            int D, __nv_bfloat16* xs, int pitch, int lane) {
  const int vec_per_row = D / 8;
  const int n = F + 1;
  for (int i = lane; i < kDotRows * vec_per_row; i += 32) {
    const int r = i / vec_per_row, v = i - r * vec_per_row;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r == 0) val = *reinterpret_cast<const uint4*>(dense + b * D + v * 8);
    else if (r < n) val = *reinterpret_cast<const uint4*>(sparse + (b * F + (r - 1)) * D + v * 8);
    *reinterpret_cast<uint4*>(xs + r * pitch + v * 8) = val;
  }
}

__global__ void __launch_bounds__(32 * kDotWarps) dot_fwd_mma_kernel(const __nv_bfloat16* __restrict__ dense, const __nv_bfloat16* __restrict__ sparse,
                                                                    __nv_bfloat16* __restrict__ out, int64_t B, int F, int D, int out_dim) {
  extern __shared__ __align__(16) unsigned char dot_smem[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t b = int64_t(blockIdx.x) * kDotWarps + wib;
  if (b >= B) return;
  const int pitch = D + 8;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(dot_smem) + size_t(wib) * kDotRows * pitch;
  dot_stage_x(dense, sparse, b, F, D, xs, pitch, lane);
  __syncwarp();
  const int g = lane >> 2, t4 = lane & 3;
  float c[2][4][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int t = 0; t < 4; ++t)
#pragma unroll
      for (int k = 0; k < 4; ++k) c[m][t][k] = 0.f;
  for (int k0 = 0; k0 < D; k0 += 16) {
    // x[q][h]: row g + 8 q, columns k0 + 8 h + 2 t4 .. + 1
    uint32_t x[4][2];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
      for (int h = 0; h < 2; ++h) x[q][h] = *reinterpret_cast<const uint32_t*>(xs + (g + 8 * q) * pitch + k0 + 8 * h + 2 * t4);
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const uint32_t a[4] = {x[2 * m][0], x[2 * m + 1][0], x[2 * m][1], x[2 * m + 1][1]};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        if (m == 1 && t < 2) continue;  // rows 16..31 x columns 0..15 lie below the diagonal
        mma_bf16_16816(c[m][t], a, x[t][0], x[t][1]);
      }
    }
  }
  __nv_bfloat16* o = out + b * int64_t(out_dim);
  // the dense vector is passed through in front of the pair terms (rows of `out` have an odd length: 2-byte stores only)
  for (int d = lane; d < D; d += 32) o[d] = xs[d];
  const int n = F + 1;
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (m == 1 && t < 2) continue;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = 16 * m + g + 8 * (k >> 1), j = 8 * t + 2 * t4 + (k & 1);
        if (i < j && j < n) o[D + i * n - i * (i + 1) / 2 + (j - i - 1)] = __float2bfloat16(c[m][t][k]);
      }
    }
}

__global__ void __launch_bounds__(32 * kDotWarps) dot_bwd_mma_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ dense,
                                                                    const __nv_bfloat16* __restrict__ sparse, __nv_bfloat16* __restrict__ ddense,
                                                                    __nv_bfloat16* __restrict__ dsparse, int64_t B, int F, int D, int out_dim) {
  extern __shared__ __align__(16) unsigned char dot_smem[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t b = int64_t(blockIdx.x) * kDotWarps + wib;
  if (b >= B) return;
  const int pitch = D + 8, spitch = kDotRows + 8;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(dot_smem) + size_t(wib) * (kDotRows * pitch + kDotRows * spitch);
  __nv_bfloat16* ss = xs + kDotRows * pitch;  // S [32][spitch]
  dot_stage_x(dense, sparse, b, F, D, xs, pitch, lane);
  for (int i = lane; i < kDotRows * spitch / 2; i += 32) reinterpret_cast<uint32_t*>(ss)[i] = 0u;
  __syncwarp();
  const int n = F + 1;
  const __nv_bfloat16* go = dout + b * int64_t(out_dim);
  {
    // pair p of row i sits at D + i n - i (i + 1) / 2 + (j - i - 1): walk the rows, lanes over j
    for (int i = 0; i < n - 1; ++i) {
      const int base = D + i * n - i * (i + 1) / 2;
      for (int j = i + 1 + lane; j < n; j += 32) {
        const __nv_bfloat16 v = go[base + (j - i - 1)];
        ss[i * spitch + j] = v;
        ss[j * spitch + i] = v;
      }
    }
  }
  __syncwarp();
  const int g = lane >> 2, t4 = lane & 3;
  // A fragments of S for both row tiles and both k-steps (K = 32)
  uint32_t a[2][2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      const __nv_bfloat16* p = ss + (16 * m + g) * spitch + 16 * ks + 2 * t4;
      a[m][ks][0] = *reinterpret_cast<const uint32_t*>(p);
      a[m][ks][1] = *reinterpret_cast<const uint32_t*>(p + 8 * spitch);
      a[m][ks][2] = *reinterpret_cast<const uint32_t*>(p + 8);
      a[m][ks][3] = *reinterpret_cast<const uint32_t*>(p + 8 * spitch + 8);
    }
  const unsigned short* xu = reinterpret_cast<const unsigned short*>(xs);
  for (int n0 = 0; n0 < D; n0 += 8) {
    float c[2][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int k = 0; k < 4; ++k) c[m][k] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      // B[k][col] = X[16 ks + k][n0 + col]: two consecutive k of one column are two rows of X
      const int r0 = 16 * ks + 2 * t4, col = n0 + g;
      const uint32_t b0 = uint32_t(xu[r0 * pitch + col]) | (uint32_t(xu[(r0 + 1) * pitch + col]) << 16);
      const uint32_t b1 = uint32_t(xu[(r0 + 8) * pitch + col]) | (uint32_t(xu[(r0 + 9) * pitch + col]) << 16);
#pragma unroll
      for (int m = 0; m < 2; ++m) mma_bf16_16816(c[m], a[m][ks], b0, b1);
    }
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int i = 16 * m + g + 8 * hh, d = n0 + 2 * t4;
        if (i >= n) continue;
        float v0 = c[m][2 * hh], v1 = c[m][2 * hh + 1];
        if (i == 0) {  // the dense vector also receives the pass-through gradient
          v0 += __bfloat162float(go[d]);
          v1 += __bfloat162float(go[d + 1]);
          *reinterpret_cast<__nv_bfloat162*>(ddense + b * D + d) = __floats2bfloat162_rn(v0, v1);
        } else {
          *reinterpret_cast<__nv_bfloat162*>(dsparse + (b * F + (i - 1)) * D + d) = __floats2bfloat162_rn(v0, v1);
        }
      }
  }
}

inline bool dot_mma_ok(int F, int D) { return F + 1 <= kDotRows && D % 16 == 0 && D >= 16 && D <= 512; }
inline size_t dot_fwd_mma_smem(int D) { return size_t(kDotWarps) * kDotRows * (D + 8) * sizeof(__nv_bfloat16); }
inline size_t dot_bwd_mma_smem(int D) { return size_t(kDotWarps) * (kDotRows * (D + 8) + kDotRows * (kDotRows + 8)) * sizeof(__nv_bfloat16); }

}  // namespace trb
