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
// Backward: two kernels of the same CTA shape and no atomics.  `varlen_attn_bwd_kv_kernel` keeps Q and dO of the sequence in shared
// memory, a warp owns 16 keys and walks all queries: dV = Pd^T dO, dK = dS^T Q (everything held transposed, [key][query]).
// `varlen_attn_bwd_q_kernel` keeps K and V in shared memory, a warp owns 16 queries and walks all keys: dQ = dS K.  The scores
// are recomputed in both (7 small products instead of 5) from the saved log-sum-exp; two arrays per kernel instead of four in
// one kernel lets three CTAs share an SM.
//
// Dropout on the probabilities: 8 bits per element from a hash of (seed, sequence, head, query pair, key pair) - one hash serves a
// 2 x 2 block, so both the query-major and the key-major kernels hash once per two elements; the keep probability is rounded
// to a multiple of 1/256 and the rescale factor matches the rounded value.  The backward recomputes the hash; no mask is stored.
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
  uint32_t keep_below;  // an element is kept iff its 8 hash bits are below this (1..256)
  float scale;          // 256 / keep_below
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
// per (sequence, head)
__device__ __forceinline__ uint32_t attn_drop_base(const AttnDrop& d, int64_t tok0, int h, int H) {
  return attn_hash32(uint32_t(tok0 * H + h) ^ d.seed_lo) + d.seed_hi;
}
// 32 bits for the 2 x 2 block (queries 2 qp, 2 qp + 1) x (keys 2 kp, 2 kp + 1); element (q, k) owns byte 2 (q & 1) + (k & 1)
__device__ __forceinline__ uint32_t attn_block_bits(uint32_t base, int qp, int kp) { return attn_hash32(base ^ ((uint32_t(qp) << 16) | uint32_t(kp))); }
__device__ __forceinline__ float attn_keep(const AttnDrop& d, uint32_t bits, int q_odd, int k_odd) {
  return ((bits >> (8 * (2 * q_odd + k_odd))) & 0xffu) < d.keep_below ? d.scale : 0.f;
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

// c[t] (t = 0..3: 8-column tiles n0 + 8 t) += A[16 x DH] * Y[n0 .. n0 + 32)[DH]^T with Y row-major in shared memory.
// One ldmatrix.x4 fetches the B fragments of a tile for two k-steps (four 8 x 8 blocks of 16 bytes per row).
template <int DH>
__device__ __forceinline__ void attn_nt(float (&c)[4][4], const uint32_t (&a)[DH / 16][4], const __nv_bfloat16* y, int pitch, int n0, int lane) {
  static_assert(DH % 32 == 0, "two k-steps per ldmatrix");
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const __nv_bfloat16* row = y + (n0 + t * 8 + (lane & 7)) * pitch + (lane >> 3) * 8;
#pragma unroll
    for (int k2 = 0; k2 < DH / 32; ++k2) {
      uint32_t b00, b01, b10, b11;
      const uint32_t addr = uint32_t(__cvta_generic_to_shared(row + k2 * 32));
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(b00), "=r"(b01), "=r"(b10), "=r"(b11) : "r"(addr));
      attn_mma(c[t], a[2 * k2], b00, b01);
      attn_mma(c[t], a[2 * k2 + 1], b10, b11);
    }
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
__global__ void __launch_bounds__(32 * WARPS, 3) varlen_attn_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const int64_t* __restrict__ offsets,
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
  const uint32_t dbase = attn_drop_base(drop, tok0, h, H);
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
      attn_nt<DH>(s, qa, Ks, P, kc, lane);
      if (kc + 32 > n) {  // only the last chunk has keys beyond the sequence
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (kc + t * 8 + 2 * t4 + (k & 1) >= n) s[t][k] = -INFINITY;
      }
      // running maxima on the raw scores (the softmax scale is positive, so it commutes with max and is folded into the exponent)
      float c0 = -INFINITY, c1 = -INFINITY;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        c0 = fmaxf(c0, fmaxf(s[t][0], s[t][1]));
        c1 = fmaxf(c1, fmaxf(s[t][2], s[t][3]));
      }
      c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, 1));
      c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, 2));
      c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, 1));
      c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, 2));
      const float mn0 = fmaxf(m0, c0), mn1 = fmaxf(m1, c1);  // finite: every chunk starts below n
      if (__any_sync(0xffffffffu, mn0 != m0 || mn1 != m1)) {  // a maximum moved: bring the running sums to the new reference
        const float al0 = exp2f((m0 - mn0) * scale_log2), al1 = exp2f((m1 - mn1) * scale_log2);
        l0 *= al0;
        l1 *= al1;
#pragma unroll
        for (int t = 0; t < DH / 8; ++t) {
          o[t][0] *= al0;
          o[t][1] *= al0;
          o[t][2] *= al1;
          o[t][3] *= al1;
        }
        m0 = mn0;
        m1 = mn1;
      }
      const float ms0 = m0 * scale_log2, ms1 = m1 * scale_log2;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float e = exp2f(fmaf(s[t][k], scale_log2, -(k < 2 ? ms0 : ms1)));
          if (k < 2) l0 += e; else l1 += e;
          s[t][k] = e;
        }
        if (drop.on) {  // rows r0 and r1 have the parity of g; the two keys of a tile are an aligned pair
          const int kp = ((kc + t * 8) >> 1) + t4;
          const uint32_t b0 = attn_block_bits(dbase, r0 >> 1, kp), b1 = attn_block_bits(dbase, r1 >> 1, kp);
          s[t][0] *= attn_keep(drop, b0, g & 1, 0);
          s[t][1] *= attn_keep(drop, b0, g & 1, 1);
          s[t][2] *= attn_keep(drop, b1, g & 1, 0);
          s[t][3] *= attn_keep(drop, b1, g & 1, 1);
        }
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
      if (r0 < n) lse2[(tok0 + r0) * H + h] = m0 * scale_log2 + log2f(l0);
      if (r1 < n) lse2[(tok0 + r1) * H + h] = m1 * scale_log2 + log2f(l1);
    }
  }
}

// A fragments of rows r0 + g, r0 + g + 8 of a global row-major array (row pitch ld), zero beyond n
template <int DH>
__device__ __forceinline__ void attn_a_frags_global(const __nv_bfloat16* base, int64_t ld, int r0, int n, int g, int t4, uint32_t (&a)[DH / 16][4]) {
  const int ra = r0 + g, rb = r0 + g + 8;
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
    const __nv_bfloat16* pa = base + ra * ld + ks * 16 + 2 * t4;
    const __nv_bfloat16* pb = base + rb * ld + ks * 16 + 2 * t4;
    a[ks][0] = ra < n ? attn_ld32(pa) : 0u;
    a[ks][1] = rb < n ? attn_ld32(pb) : 0u;
    a[ks][2] = ra < n ? attn_ld32(pa + 8) : 0u;
    a[ks][3] = rb < n ? attn_ld32(pb + 8) : 0u;
  }
}

// dK and dV: Q and dO of the sequence in shared memory; a warp owns 16 keys and walks the queries 32 at a time ([key][query] tiles)
template <int DH, int WARPS>
__global__ void __launch_bounds__(32 * WARPS, 3) varlen_attn_bwd_kv_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ out,
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
  if (n > n_cap) {  // the tail of a sequence that is longer than the launch was sized for gets zero gradients (k and v here)
    if (threadIdx.x == 0) atomicExch(err, 1);
    for (int i = threadIdx.x; i < (n - n_cap) * 2 * DH; i += blockDim.x) {
      const int r = n_cap + i / (2 * DH), c = i % (2 * DH);
      dqkv[(tok0 + r) * ld + (1 + c / DH) * D + h * DH + (c % DH)] = __float2bfloat16(0.f);
    }
    n = n_cap;
  }
  const int np = (n + 31) & ~31;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(attn_smem);
  __nv_bfloat16* Gs = Qs + np_cap * P;  // dO
  float* lse_s = reinterpret_cast<float*>(Gs + np_cap * P);
  float* del_s = lse_s + np_cap;
  const __nv_bfloat16* head = qkv + tok0 * ld + h * DH;
  attn_stage<DH>(head, ld, n, np, Qs, threadIdx.x, blockDim.x);
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
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const uint32_t dbase = attn_drop_base(drop, tok0, h, H);
  for (int j0 = warp * 16; j0 < n; j0 += WARPS * 16) {
    uint32_t ka[DH / 16][4], va[DH / 16][4];
    attn_a_frags_global<DH>(head + D, ld, j0, n, g, t4, ka);
    attn_a_frags_global<DH>(head + 2 * D, ld, j0, n, g, t4, va);
    float dk[DH / 8][4], dv[DH / 8][4];
#pragma unroll
    for (int t = 0; t < DH / 8; ++t)
#pragma unroll
      for (int k = 0; k < 4; ++k) dk[t][k] = dv[t][k] = 0.f;
    const int k0 = j0 + g, k1 = j0 + g + 8;  // both have the parity of g
    for (int qc = 0; qc < np; qc += 32) {
      float st[4][4], dp[4][4];
#pragma unroll
      for (int t = 0; t < 4; ++t)
#pragma unroll
        for (int k = 0; k < 4; ++k) st[t][k] = dp[t][k] = 0.f;
      attn_nt<DH>(st, ka, Qs, P, qc, lane);
      attn_nt<DH>(dp, va, Gs, P, qc, lane);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int q = qc + t * 8 + 2 * t4;  // queries q, q + 1: an aligned pair
        float f[4] = {1.f, 1.f, 1.f, 1.f};
        if (drop.on) {
          const uint32_t b0 = attn_block_bits(dbase, q >> 1, k0 >> 1), b1 = attn_block_bits(dbase, q >> 1, k1 >> 1);
          f[0] = attn_keep(drop, b0, 0, g & 1);
          f[1] = attn_keep(drop, b0, 1, g & 1);
          f[2] = attn_keep(drop, b1, 0, g & 1);
          f[3] = attn_keep(drop, b1, 1, g & 1);
        }
        const float2 ls = *reinterpret_cast<const float2*>(lse_s + q), de = *reinterpret_cast<const float2*>(del_s + q);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float a = exp2f(st[t][k] * scale_log2 - ((k & 1) ? ls.y : ls.x));
          st[t][k] = a * f[k];
          dp[t][k] = a * (f[k] * dp[t][k] - ((k & 1) ? de.y : de.x));
        }
      }
      attn_nn<DH>(dv, st, Gs, P, qc, lane);
      attn_nn<DH>(dk, dp, Qs, P, qc, lane);
    }
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
}

// dQ: K and V of the sequence in shared memory; a warp owns 16 queries and walks the keys 32 at a time
template <int DH, int WARPS>
__global__ void __launch_bounds__(32 * WARPS) varlen_attn_bwd_q_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ out,
                                                                      const __nv_bfloat16* __restrict__ dout, const float* __restrict__ lse2,
                                                                      const int64_t* __restrict__ offsets, __nv_bfloat16* __restrict__ dqkv, int H, int n_cap,
                                                                      int np_cap, float scale, float scale_log2, AttnDrop drop) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  constexpr int P = DH + kAttnPad;
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int64_t tok0 = offsets[b];
  int n = int(offsets[b + 1] - tok0);
  if (n <= 0) return;
  const int D = H * DH;
  const int64_t ld = 3 * int64_t(D);
  if (n > n_cap) {
    for (int i = threadIdx.x; i < (n - n_cap) * DH; i += blockDim.x) dqkv[(tok0 + n_cap + i / DH) * ld + h * DH + (i % DH)] = __float2bfloat16(0.f);
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
  const uint32_t dbase = attn_drop_base(drop, tok0, h, H);
  for (int q0 = warp * 16; q0 < n; q0 += WARPS * 16) {
    uint32_t qa[DH / 16][4], ga[DH / 16][4], oa[DH / 16][4];
    attn_a_frags_global<DH>(head, ld, q0, n, g, t4, qa);
    attn_a_frags_global<DH>(dout + tok0 * D + h * DH, D, q0, n, g, t4, ga);
    attn_a_frags_global<DH>(out + tok0 * D + h * DH, D, q0, n, g, t4, oa);
    const int r0 = q0 + g, r1 = q0 + g + 8;
    // delta = rowsum(dO * O): this lane's 16 columns of each row, then the four lanes of the row
    float de0 = 0.f, de1 = 0.f;
#pragma unroll
    for (int ks = 0; ks < DH / 16; ++ks)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ga[ks][j]));
        const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&oa[ks][j]));
        if (j & 1) de1 += x.x * y.x + x.y * y.y; else de0 += x.x * y.x + x.y * y.y;
      }
    de0 += __shfl_xor_sync(0xffffffffu, de0, 1);
    de0 += __shfl_xor_sync(0xffffffffu, de0, 2);
    de1 += __shfl_xor_sync(0xffffffffu, de1, 1);
    de1 += __shfl_xor_sync(0xffffffffu, de1, 2);
    const float ls0 = r0 < n ? lse2[(tok0 + r0) * H + h] : INFINITY, ls1 = r1 < n ? lse2[(tok0 + r1) * H + h] : INFINITY;
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
      attn_nt<DH>(s, qa, Ks, P, kc, lane);
      attn_nt<DH>(dp, ga, Vs, P, kc, lane);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        float f[4] = {1.f, 1.f, 1.f, 1.f};
        if (drop.on) {
          const int kp = ((kc + t * 8) >> 1) + t4;
          const uint32_t b0 = attn_block_bits(dbase, r0 >> 1, kp), b1 = attn_block_bits(dbase, r1 >> 1, kp);
          f[0] = attn_keep(drop, b0, g & 1, 0);
          f[1] = attn_keep(drop, b0, g & 1, 1);
          f[2] = attn_keep(drop, b1, g & 1, 0);
          f[3] = attn_keep(drop, b1, g & 1, 1);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int key = kc + t * 8 + 2 * t4 + (k & 1);
          const float a = key < n ? exp2f(s[t][k] * scale_log2 - (k < 2 ? ls0 : ls1)) : 0.f;
          dp[t][k] = a * (f[k] * dp[t][k] - (k < 2 ? de0 : de1));
        }
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
  const double keep = std::min(256.0, std::max(1.0, std::floor((1.0 - p) * 256.0 + 0.5)));
  d.keep_below = uint32_t(keep);
  d.scale = d.on ? float(256.0 / keep) : 1.f;
  return d;
}

constexpr int kAttnDH = 64;
constexpr int kAttnFwdWarps = 8;
constexpr int kAttnBwdWarps = 4;  // dK / dV kernel
constexpr int kAttnBwdQWarps = 4;

static void attn_check(const at::Tensor& qkv, const at::Tensor& offsets, int64_t H, int64_t max_len) {
  TORCH_CHECK(qkv.is_cuda() && qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.is_contiguous(), "qkv must be a contiguous bf16 CUDA matrix");
  TORCH_CHECK(offsets.is_cuda() && offsets.scalar_type() == at::kLong && offsets.dim() == 1 && offsets.is_contiguous() && offsets.numel() >= 1);
  TORCH_CHECK(H >= 1 && qkv.size(1) == 3 * H * kAttnDH, "varlen attention: head dimension must be 64");
  TORCH_CHECK(max_len >= 1 && max_len <= 768, "varlen attention: max_len must be in [1, 768]");
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
  const size_t rows_bytes = size_t(2) * np_cap * (kAttnDH + kAttnPad) * sizeof(__nv_bfloat16);
  const size_t smem_kv = rows_bytes + size_t(2) * np_cap * sizeof(float);
  auto kern_kv = varlen_attn_bwd_kv_kernel<kAttnDH, kAttnBwdWarps>;
  auto kern_q = varlen_attn_bwd_q_kernel<kAttnDH, kAttnBwdQWarps>;
  TRB_CUDA_CHECK(cudaFuncSetAttribute(kern_kv, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_kv)));
  TRB_CUDA_CHECK(cudaFuncSetAttribute(kern_q, cudaFuncAttributeMaxDynamicSharedMemorySize, int(rows_bytes)));
  const float scale = float(1.0 / std::sqrt(double(kAttnDH)));
  const AttnDrop drop = make_attn_drop(p, seed);
  auto stream = at::cuda::getCurrentCUDAStream();
  const auto* qp = reinterpret_cast<const __nv_bfloat16*>(qkv.data_ptr());
  const auto* op = reinterpret_cast<const __nv_bfloat16*>(out.data_ptr());
  const auto* gp = reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr());
  auto* dp = reinterpret_cast<__nv_bfloat16*>(dqkv.data_ptr());
  kern_kv<<<unsigned(B * H), 32 * kAttnBwdWarps, smem_kv, stream>>>(qp, op, gp, lse.data_ptr<float>(), offsets.data_ptr<int64_t>(), dp, int(H), int(max_len), np_cap,
                                                                   scale, scale * 1.4426950408889634f, drop, err.data_ptr<int>());
  TRB_CUDA_CHECK(cudaGetLastError());
  kern_q<<<unsigned(B * H), 32 * kAttnBwdQWarps, rows_bytes, stream>>>(qp, op, gp, lse.data_ptr<float>(), offsets.data_ptr<int64_t>(), dp, int(H), int(max_len), np_cap,
                                                                     scale, scale * 1.4426950408889634f, drop);
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
