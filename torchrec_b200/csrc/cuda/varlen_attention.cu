// Self-attention over PACKED sequences (no padding): tokens of all sequences lie back to back in qkv [T, 3 * D]
// (q | k | v along the columns, D = heads * 64) with `offsets [B + 1]` giving the bounds; the cost is sum(len^2), not B * max_len^2.
//
// One CTA owns one (sequence, head).  K and V of the sequence (at most `n_cap` tokens, a few hundred) sit in shared memory for the
// whole CTA; every warp takes 16-query tiles and walks the keys 32 at a time with an online softmax, so registers do not grow with
// the length.  Matrix products run on the tensor cores through the warp-level mma.m16n8k16 (bf16 in, fp32 accumulate): a
// (sequence, head) problem is [len x 64] x [64 x len] with len around 100, far below what a 128-row tcgen05 tile with TMEM
// accumulators needs to pay off, and the softmax wants the scores in registers.  Probabilities go from the accumulator
// registers straight into the A operand of the second product; operands that must be read transposed come through ldmatrix.trans.
//
// Backward, same CTA shape, two phases over Q, K, V, dO in shared memory and no atomics: (A) a warp owns 16 keys and walks all
// queries: dV = Pd^T dO, dK = dS^T Q; (B) a warp owns 16 queries and walks all keys: dQ = dS K.  The scores are recomputed in
// both (7 small products instead of 5) from the saved log-sum-exp.
//
// Dropout on the probabilities is a hash of (seed, query token, head, key position) recomputed in the backward; no mask is stored.
// The reference model pads every sequence to max_len and calls the library's attention
// (examples/bert4rec/models/bert4rec.py of the reference, nn.TransformerEncoderLayer).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/library.h>

#include <cmath>

#include "common.cuh"

namespace trb {

constexpr int kAttnPad = 8;  // bf16 elements of padding per shared row: 16-byte aligned rows, conflict-free fragment loads

struct AttnDrop {
  uint32_t seed_lo, seed_hi;
  uint32_t keep_below;  // an element is kept iff its 32 hash bits are below this
  float scale;          // 2^32 / keep_below
  int on;
};

__device__ __forceinline__ uint32_t attn_hash32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}
__device__ __forceinline__ uint32_t attn_row_key(const AttnDrop& d, int64_t tok, int h, int H) {
  return attn_hash32(uint32_t(tok * H + h) ^ d.seed_lo) + d.seed_hi;
}
__device__ __forceinline__ float attn_keep(const AttnDrop& d, uint32_t row_key, int key) {
  if (!d.on) return 1.f;
  return attn_hash32(row_key ^ (uint32_t(key) * 0x9E3779B9u)) < d.keep_below ? d.scale : 0.f;
}

__device__ __forceinline__ void attn_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t attn_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t attn_ld32(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }

// A fragments (16 rows x DH) of rows r0 + g and r0 + g + 8 of a shared row-major array
template <int DH>
__device__ __forceinline__ void attn_a_frags(const __nv_bfloat16* base, int pitch, int r0, int g, int t4, uint32_t (&a)[DH / 16][4]) {
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
    const __nv_bfloat16* p = base + (r0 + g) * pitch + ks * 16 + 2 * t4;
    a[ks][0] = attn_ld32(p);
    a[ks][1] = attn_ld32(p + 8 * pitch);
    a[ks][2] = attn_ld32(p + 8);
    a[ks][3] = attn_ld32(p + 8 * pitch + 8);
  }
}

// c[t] (t = 0..3: 8-column tiles n0 + 8 t) += A[16 x DH] * Y[n0 .. n0 + 32)[DH]^T with Y row-major in shared memory
template <int DH>
__device__ __forceinline__ void attn_nt(float (&c)[4][4], const uint32_t (&a)[DH / 16][4], const __nv_bfloat16* y, int pitch, int n0, int g, int t4) {
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks)
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const __nv_bfloat16* p = y + (n0 + t * 8 + g) * pitch + ks * 16 + 2 * t4;
      attn_mma(c[t], a[ks], attn_ld32(p), attn_ld32(p + 8));
    }
}

// acc[16 x DH] += P[16 x 32] * Y[k0 .. k0 + 32)[DH]; P is given as accumulator-layout values p[t][k] (t: 8-column tiles)
template <int DH>
__device__ __forceinline__ void attn_nn(float (&acc)[DH / 8][4], const float (&p)[4][4], const __nv_bfloat16* y, int pitch, int k0, int lane) {
#pragma unroll
  for (int kk = 0; kk < 2; ++kk) {
    const uint32_t a[4] = {attn_pack(p[2 * kk][0], p[2 * kk][1]), attn_pack(p[2 * kk][2], p[2 * kk][3]), attn_pack(p[2 * kk + 1][0], p[2 * kk + 1][1]),
                           attn_pack(p[2 * kk + 1][2], p[2 * kk + 1][3])};
    const int row = k0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int d2 = 0; d2 < DH / 16; ++d2) {
      uint32_t b00, b01, b10, b11;
      const uint32_t addr = uint32_t(__cvta_generic_to_shared(y + row * pitch + d2 * 16 + (lane >> 4) * 8));
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(b00), "=r"(b01), "=r"(b10), "=r"(b11) : "r"(addr));
      attn_mma(acc[2 * d2], a, b00, b01);
      attn_mma(acc[2 * d2 + 1], a, b10, b11);
    }
  }
}

// rows [0, np) of one head's q, k or v (or of dout) into shared memory, zero beyond n
template <int DH>
__device__ __forceinline__ void attn_stage(const __nv_bfloat16* src, int64_t ld, int n, int np, __nv_bfloat16* dst, int tid, int nthreads) {
  constexpr int P = DH + kAttnPad;
  for (int i = tid; i < np * (DH / 8); i += nthreads) {
    const int r = i / (DH / 8), v = i - r * (DH / 8);
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < n) val = *reinterpret_cast<const uint4*>(src + r * ld + v * 8);
    *reinterpret_cast<uint4*>(dst + r * P + v * 8) = val;
  }
}

template <int DH, int WARPS>
__global__ void __launch_bounds__(32 * WARPS) varlen_attn_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const int64_t* __restrict__ offsets,
                                                                    __nv_bfloat16* __restrict__ out, float* __restrict__ lse2, int H, int n_cap, int np_cap,
                                                                    float scale_log2, AttnDrop drop, int* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  constexpr int P = DH + kAttnPad;
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int64_t tok0 = offsets[b];
  int n = int(offsets[b + 1] - tok0);
  if (n <= 0) return;
  const int D = H * DH;
  const int64_t ld = 3 * int64_t(D);
  if (n > n_cap) {  // longer than the launch was sized for: the tail gets zeros and the error word says so
    if (threadIdx.x == 0) atomicExch(err, 1);
    for (int i = threadIdx.x; i < (n - n_cap) * DH; i += blockDim.x) {
      const int r = n_cap + i / DH, d = i % DH;
      out[(tok0 + r) * D + h * DH + d] = __float2bfloat16(0.f);
      if (d == 0) lse2[(tok0 + r) * H + h] = 0.f;
    }
    n = n_cap;
  }
  const int np = (n + 31) & ~31;
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(attn_smem);
  __nv_bfloat16* Vs = Ks + np_cap * P;
  const __nv_bfloat16* head = qkv + tok0 * ld + h * DH;
  attn_stage<DH>(head + D, ld, n, np, Ks, threadIdx.x, blockDim.x);
  attn_stage<DH>(head + 2 * D, ld, n, np, Vs, threadIdx.x, blockDim.x);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  for (int q0 = warp * 16; q0 < n; q0 += WARPS * 16) {
    const int r0 = q0 + g, r1 = q0 + g + 8;
    uint32_t qa[DH / 16][4];
#pragma unroll
    for (int ks = 0; ks < DH / 16; ++ks) {
      const __nv_bfloat16* p0 = head + r0 * ld + ks * 16 + 2 * t4;
      const __nv_bfloat16* p1 = head + r1 * ld + ks * 16 + 2 * t4;
      qa[ks][0] = r0 < n ? attn_ld32(p0) : 0u;
      qa[ks][1] = r1 < n ? attn_ld32(p1) : 0u;
      qa[ks][2] = r0 < n ? attn_ld32(p0 + 8) : 0u;
      qa[ks][3] = r1 < n ? attn_ld32(p1 + 8) : 0u;
    }
    const uint32_t rk0 = attn_row_key(drop, tok0 + r0, h, H), rk1 = attn_row_key(drop, tok0 + r1, h, H);
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[DH / 8][4];
#pragma unroll
    for (int t = 0; t < DH / 8; ++t)
#pragma unroll
      for (int k = 0; k < 4; ++k) o[t][k] = 0.f;
    for (int kc = 0; kc < np; kc += 32) {
      float s[4][4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) s[t][k] = 0.f;
      attn_nt<DH>(s, qa, Ks, P, kc, g, t4);
      float c0 = -INFINITY, c1 = -INFINITY;
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int key = kc + t * 8 + 2 * t4 + (k & 1);
          const float v = key < n ? s[t][k] * scale_log2 : -INFINITY;
          s[t][k] = v;
          if (k < 2) c0 = fmaxf(c0, v); else c1 = fmaxf(c1, v);
        }
      c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, 1));
      c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, 2));
      c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, 1));
      c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, 2));
      const float mn0 = fmaxf(m0, c0), mn1 = fmaxf(m1, c1);  // finite: every chunk starts below n
      const float al0 = exp2f(m0 - mn0), al1 = exp2f(m1 - mn1);
      m0 = mn0;
      m1 = mn1;
      l0 *= al0;
      l1 *= al1;
#pragma unroll
      for (int t = 0; t < DH / 8; ++t) {
        o[t][0] *= al0;
        o[t][1] *= al0;
        o[t][2] *= al1;
        o[t][3] *= al1;
      }
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int key = kc + t * 8 + 2 * t4 + (k & 1);
          const float e = exp2f(s[t][k] - (k < 2 ? mn0 : mn1));
          if (k < 2) l0 += e; else l1 += e;
          s[t][k] = e * attn_keep(drop, k < 2 ? rk0 : rk1, key);
        }
      attn_nn<DH>(o, s, Vs, P, kc, lane);
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = 1.f / l0, i1 = 1.f / l1;
#pragma unroll
    for (int t = 0; t < DH / 8; ++t) {
      if (r0 < n) *reinterpret_cast<__nv_bfloat162*>(out + (tok0 + r0) * D + h * DH + t * 8 + 2 * t4) = __floats2bfloat162_rn(o[t][0] * i0, o[t][1] * i0);
      if (r1 < n) *reinterpret_cast<__nv_bfloat162*>(out + (tok0 + r1) * D + h * DH + t * 8 + 2 * t4) = __floats2bfloat162_rn(o[t][2] * i1, o[t][3] * i1);
    }
    if (t4 == 0) {
      if (r0 < n) lse2[(tok0 + r0) * H + h] = m0 + log2f(l0);
      if (r1 < n) lse2[(tok0 + r1) * H + h] = m1 + log2f(l1);
    }
  }
}

template <int DH, int WARPS>
__global__ void __launch_bounds__(32 * WARPS) varlen_attn_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ out,
                                                                    const __nv_bfloat16* __restrict__ dout, const float* __restrict__ lse2,
                                                                    const int64_t* __restrict__ offsets, __nv_bfloat16* __restrict__ dqkv, int H, int n_cap,
                                                                    int np_cap, float scale, float scale_log2, AttnDrop drop, int* __restrict__ err) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  constexpr int P = DH + kAttnPad;
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int64_t tok0 = offsets[b];
  int n = int(offsets[b + 1] - tok0);
  if (n <= 0) return;
  const int D = H * DH;
  const int64_t ld = 3 * int64_t(D);
  if (n > n_cap) {
    if (threadIdx.x == 0) atomicExch(err, 1);
    for (int i = threadIdx.x; i < (n - n_cap) * 3 * DH; i += blockDim.x) {
      const int r = n_cap + i / (3 * DH), c = i % (3 * DH);
      dqkv[(tok0 + r) * ld + (c / DH) * D + h * DH + (c % DH)] = __float2bfloat16(0.f);
    }
    n = n_cap;
  }
  const int np = (n + 31) & ~31;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(attn_smem);
  __nv_bfloat16* Ks = Qs + np_cap * P;
  __nv_bfloat16* Vs = Ks + np_cap * P;
  __nv_bfloat16* Gs = Vs + np_cap * P;  // dO
  float* lse_s = reinterpret_cast<float*>(Gs + np_cap * P);
  float* del_s = lse_s + np_cap;
  uint32_t* rk_s = reinterpret_cast<uint32_t*>(del_s + np_cap);
  const __nv_bfloat16* head = qkv + tok0 * ld + h * DH;
  attn_stage<DH>(head, ld, n, np, Qs, threadIdx.x, blockDim.x);
  attn_stage<DH>(head + D, ld, n, np, Ks, threadIdx.x, blockDim.x);
  attn_stage<DH>(head + 2 * D, ld, n, np, Vs, threadIdx.x, blockDim.x);
  attn_stage<DH>(dout + tok0 * D + h * DH, D, n, np, Gs, threadIdx.x, blockDim.x);
  for (int r = threadIdx.x; r < np; r += blockDim.x) {
    float del = 0.f, l = INFINITY;  // padded queries: exp2(s - inf) = 0, nothing flows
    if (r < n) {
      const __nv_bfloat16* orow = out + (tok0 + r) * D + h * DH;
      const __nv_bfloat16* grow = dout + (tok0 + r) * D + h * DH;
#pragma unroll
      for (int v = 0; v < DH / 8; ++v) {
        const uint4 a = *reinterpret_cast<const uint4*>(orow + v * 8), c = *reinterpret_cast<const uint4*>(grow + v * 8);
        const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* ch = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = __bfloat1622float2(ah[k]), y = __bfloat1622float2(ch[k]);
          del += x.x * y.x + x.y * y.y;
        }
      }
      l = lse2[(tok0 + r) * H + h];
    }
    del_s[r] = del;
    lse_s[r] = l;
    rk_s[r] = attn_row_key(drop, tok0 + r, h, H);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;

  // phase A: a warp owns 16 keys, walks the queries 32 at a time; everything is held transposed ([key][query])
  for (int j0 = warp * 16; j0 < n; j0 += WARPS * 16) {
    uint32_t ka[DH / 16][4], va[DH / 16][4];
    attn_a_frags<DH>(Ks, P, j0, g, t4, ka);
    attn_a_frags<DH>(Vs, P, j0, g, t4, va);
    float dk[DH / 8][4], dv[DH / 8][4];
#pragma unroll
    for (int t = 0; t < DH / 8; ++t)
#pragma unroll
      for (int k = 0; k < 4; ++k) dk[t][k] = dv[t][k] = 0.f;
    for (int qc = 0; qc < np; qc += 32) {
      float st[4][4], dp[4][4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) st[t][k] = dp[t][k] = 0.f;
      attn_nt<DH>(st, ka, Qs, P, qc, g, t4);
      attn_nt<DH>(dp, va, Gs, P, qc, g, t4);
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int q = qc + t * 8 + 2 * t4 + (k & 1);
          const int key = j0 + g + 8 * (k >> 1);
          const float a = exp2f(st[t][k] * scale_log2 - lse_s[q]);
          const float f = attn_keep(drop, rk_s[q], key);
          st[t][k] = a * f;
          dp[t][k] = a * (f * dp[t][k] - del_s[q]);
        }
      attn_nn<DH>(dv, st, Gs, P, qc, lane);
      attn_nn<DH>(dk, dp, Qs, P, qc, lane);
    }
    const int k0 = j0 + g, k1 = j0 + g + 8;
#pragma unroll
    for (int t = 0; t < DH / 8; ++t) {
      const int col = h * DH + t * 8 + 2 * t4;
      if (k0 < n) {
        *reinterpret_cast<__nv_bfloat162*>(dqkv + (tok0 + k0) * ld + D + col) = __floats2bfloat162_rn(dk[t][0] * scale, dk[t][1] * scale);
        *reinterpret_cast<__nv_bfloat162*>(dqkv + (tok0 + k0) * ld + 2 * D + col) = __floats2bfloat162_rn(dv[t][0], dv[t][1]);
      }
      if (k1 < n) {
        *reinterpret_cast<__nv_bfloat162*>(dqkv + (tok0 + k1) * ld + D + col) = __floats2bfloat162_rn(dk[t][2] * scale, dk[t][3] * scale);
        *reinterpret_cast<__nv_bfloat162*>(dqkv + (tok0 + k1) * ld + 2 * D + col) = __floats2bfloat162_rn(dv[t][2], dv[t][3]);
      }
    }
  }

  // phase B: a warp owns 16 queries, walks the keys 32 at a time
  for (int q0 = warp * 16; q0 < n; q0 += WARPS * 16) {
    uint32_t qa[DH / 16][4], ga[DH / 16][4];
    attn_a_frags<DH>(Qs, P, q0, g, t4, qa);
    attn_a_frags<DH>(Gs, P, q0, g, t4, ga);
    const int r0 = q0 + g, r1 = q0 + g + 8;
    const float ls0 = lse_s[r0], ls1 = lse_s[r1], de0 = del_s[r0], de1 = del_s[r1];
    const uint32_t rk0 = rk_s[r0], rk1 = rk_s[r1];
    float dq[DH / 8][4];
#pragma unroll
    for (int t = 0; t < DH / 8; ++t)
#pragma unroll
      for (int k = 0; k < 4; ++k) dq[t][k] = 0.f;
    for (int kc = 0; kc < np; kc += 32) {
      float s[4][4], dp[4][4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) s[t][k] = dp[t][k] = 0.f;
      attn_nt<DH>(s, qa, Ks, P, kc, g, t4);
      attn_nt<DH>(dp, ga, Vs, P, kc, g, t4);
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int key = kc + t * 8 + 2 * t4 + (k & 1);
          const float a = key < n ? exp2f(s[t][k] * scale_log2 - (k < 2 ? ls0 : ls1)) : 0.f;
          const float f = attn_keep(drop, k < 2 ? rk0 : rk1, key);
          dp[t][k] = a * (f * dp[t][k] - (k < 2 ? de0 : de1));
        }
      attn_nn<DH>(dq, dp, Ks, P, kc, lane);
    }
#pragma unroll
    for (int t = 0; t < DH / 8; ++t) {
      const int col = h * DH + t * 8 + 2 * t4;
      if (r0 < n) *reinterpret_cast<__nv_bfloat162*>(dqkv + (tok0 + r0) * ld + col) = __floats2bfloat162_rn(dq[t][0] * scale, dq[t][1] * scale);
      if (r1 < n) *reinterpret_cast<__nv_bfloat162*>(dqkv + (tok0 + r1) * ld + col) = __floats2bfloat162_rn(dq[t][2] * scale, dq[t][3] * scale);
    }
  }
}

static AttnDrop make_attn_drop(double p, int64_t seed) {
  AttnDrop d;
  d.on = p > 0.0 ? 1 : 0;
  d.seed_lo = uint32_t(uint64_t(seed));
  d.seed_hi = uint32_t(uint64_t(seed) >> 32);
  const double keep = std::min(4294967295.0, std::max(1.0, std::floor((1.0 - p) * 4294967296.0)));
  d.keep_below = uint32_t(keep);
  d.scale = d.on ? float(4294967296.0 / keep) : 1.f;
  return d;
}

constexpr int kAttnDH = 64;
constexpr int kAttnFwdWarps = 4;
constexpr int kAttnBwdWarps = 8;

static void attn_check(const at::Tensor& qkv, const at::Tensor& offsets, int64_t H, int64_t max_len) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.is_contiguous(), "qkv must be a contiguous bf16 CUDA matrix");
  TORCH_CHECK(offsets.is_cuda() && offsets.scalar_type() == at::kLong && offsets.dim() == 1 && offsets.is_contiguous() && offsets.numel() >= 1);
  TORCH_CHECK(H >= 1 && qkv.size(1) == 3 * H * kAttnDH, "varlen attention: head dimension must be 64");
  TORCH_CHECK(max_len >= 1 && max_len <= 384, "varlen attention: max_len must be in [1, 384]");
}

std::tuple<at::Tensor, at::Tensor> varlen_attn_fwd(const at::Tensor& qkv, const at::Tensor& offsets, int64_t H, int64_t max_len, double p, int64_t seed,
                                                   at::Tensor err) {
  attn_check(qkv, offsets, H, max_len);
  TORCH_CHECK(err.is_cuda() && err.scalar_type() == at::kInt && err.numel() >= 1);
  c10::cuda::CUDAGuard guard(qkv.device());
  const int64_t T = qkv.size(0), B = offsets.numel() - 1;
  const int D = int(H) * kAttnDH;
  at::Tensor out = at::empty({T, D}, qkv.options());
  at::Tensor lse = at::empty({T, H}, qkv.options().dtype(at::kFloat));
  if (T == 0 || B == 0) return {out, lse};
  const int np_cap = (int(max_len) + 31) & ~31;
  const size_t smem = size_t(2) * np_cap * (kAttnDH + kAttnPad) * sizeof(__nv_bfloat16);
  auto kern = varlen_attn_fwd_kernel<kAttnDH, kAttnFwdWarps>;
  TRB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  const float scale_log2 = float(1.4426950408889634 / std::sqrt(double(kAttnDH)));
  kern<<<unsigned(B * H), 32 * kAttnFwdWarps, smem, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(qkv.data_ptr()), offsets.data_ptr<int64_t>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()),
      lse.data_ptr<float>(), int(H), int(max_len), np_cap, scale_log2, make_attn_drop(p, seed), err.data_ptr<int>());
  TRB_CUDA_CHECK(cudaGetLastError());
  return {out, lse};
}

at::Tensor varlen_attn_bwd(const at::Tensor& dout, const at::Tensor& qkv, const at::Tensor& out, const at::Tensor& lse, const at::Tensor& offsets, int64_t H,
                           int64_t max_len, double p, int64_t seed, at::Tensor err) {
  attn_check(qkv, offsets, H, max_len);
  const int64_t T = qkv.size(0), B = offsets.numel() - 1;
  const int D = int(H) * kAttnDH;
  TORCH_CHECK(dout.is_cuda() && dout.scalar_type() == at::kBFloat16 && dout.is_contiguous() && dout.dim() == 2 && dout.size(0) == T && dout.size(1) == D);
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.sizes() == dout.sizes());
  TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == T * H);
  TORCH_CHECK(err.is_cuda() && err.scalar_type() == at::kInt && err.numel() >= 1);
  c10::cuda::CUDAGuard guard(qkv.device());
  at::Tensor dqkv = at::empty_like(qkv);
  if (T == 0 || B == 0) return dqkv;
  const int np_cap = (int(max_len) + 31) & ~31;
  const size_t smem = size_t(4) * np_cap * (kAttnDH + kAttnPad) * sizeof(__nv_bfloat16) + size_t(3) * np_cap * sizeof(float);
  TORCH_CHECK(smem <= 227 * 1024, "varlen attention backward: max_len ", max_len, " does not fit in shared memory");
  auto kern = varlen_attn_bwd_kernel<kAttnDH, kAttnBwdWarps>;
  TRB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  const float scale = float(1.0 / std::sqrt(double(kAttnDH)));
  kern<<<unsigned(B * H), 32 * kAttnBwdWarps, smem, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(qkv.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()),
      reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), lse.data_ptr<float>(), offsets.data_ptr<int64_t>(),
      reinterpret_cast<__nv_bfloat16*>(dqkv.data_ptr()), int(H), int(max_len), np_cap, scale, scale * 1.4426950408889634f, make_attn_drop(p, seed),
      err.data_ptr<int>());
  TRB_CUDA_CHECK(cudaGetLastError());
  return dqkv;
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def("varlen_attn_fwd(Tensor qkv, Tensor offsets, int heads, int max_len, float p, int seed, Tensor(a!) err) -> (Tensor, Tensor)");
  m.def("varlen_attn_bwd(Tensor dout, Tensor qkv, Tensor out, Tensor lse, Tensor offsets, int heads, int max_len, float p, int seed, Tensor(a!) err) -> Tensor");
}

TORCH_LIBRARY_IMPL(trb200, CUDA, m) {
  m.impl("varlen_attn_fwd", &trb::varlen_attn_fwd);
  m.impl("varlen_attn_bwd", &trb::varlen_attn_bwd);
}
