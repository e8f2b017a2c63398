// Fused sparse-input distribution and pooled-output hand-over over peer-mapped memory (NVLink / NVSwitch), sm_100a.
//
// What a sharded embedding module needs per step, with W ranks of one node:
//
//   input side   every rank holds a KeyedJaggedTensor of its B_local samples (lengths [F, B_local], ids).  Rank d
//                must receive, for every table shard it owns, the ids of that table's features from ALL ranks.  A
//                (feature, shard) pair is a "job".  A job whose shard holds all rows of the table takes the feature's
//                ids as they are (table-wise / column-wise shards); jobs whose shards split the rows (row-wise,
//                table-row-wise, grid shards) take only the ids inside their row range, re-based to the shard.
//   kjt_dist_count    counts, per bag, how many ids fall into every row range of the row-split features, sums the
//                     per-(job) totals and stores them into every peer's table of sizes (plain peer stores), then
//                     raises the "sizes" flag.  No host round trip: sizes never leave the devices.
//   kjt_dist_scatter  waits for all peers' sizes (bounded), derives where each of its segments starts in every
//                     destination's receive buffer (jobs major, then source rank, then sample: the order the lookup
//                     kernel wants, so no re-concatenation pass follows), and writes lengths, ids and optional
//                     per-sample weights straight into the destinations' buffers.  Raises the "data" flag.
//   kjt_dist_recv_offsets  on the receiver: waits for the data flag of every source, then scans the received
//                     lengths into offsets.
//   output side  pooled_finalize turns the staging rows that the lookup kernels of all ranks stored into this rank's
//                buffer into the module's output: copies whole-shard columns, sums the W partial rows of row-split
//                tables in a fixed order (a deterministic reduce-scatter), applies the mean divisor and casts.
//                grad_publish is its mirror for the backward: it casts / scales the output gradient and pushes every column
//                block to the rank(s) that own the table, so the owners' backward kernels read local memory only.
//
// Receive buffers have a fixed capacity (ids per rank).  A step whose ids do not fit is detected from the sizes before
// anything is written: writers skip that destination and the destination records error 300, which the host raises.
//
// Only plain peer loads / stores are used (no bulk-tensor copies, no multicast).  Every wait is bounded.
//
// The reference performs the same redistribution with a size all-to-all, a host read of the sizes, one all-to-all
// per tensor and a permute (torchrec/distributed/dist_data.py:220-442), after bucketizing row-wise ids with a library
// op (torchrec/distributed/embedding_sharding.py:219-287); its outputs travel through pooled all-to-all /
// reduce-scatter collectives (torchrec/distributed/comm_ops.py:574-1073, :2038-2131).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cub/cub.cuh>

#include "common.cuh"
#include "peer_sync.cuh"

namespace trb {

constexpr int kChunk = 256;     // bags per work item
constexpr int kMaxShards = 16;  // row ranges per row-split feature (= kMaxPeers)
enum DistSlot : int { SLOT_SIZES = 0, SLOT_DATA = 1 };
enum JobCol : int { J_DEST = 0, J_LOCAL = 1, J_FEAT = 2, J_KIND = 3, J_SHARD = 4, kJobCols = 5 };  // J_SHARD: index into grp_jobs

struct DistParams {
  int W, rank, G, Q, B, nchunks, F_in, n_whole;
  const int32_t* jobs;            // [G, kJobCols]
  const int64_t* row_lo;          // [G] first table row of the job's shard
  const int64_t* row_hi;          // [G] one past its last row
  const int32_t* dest_job_start;  // [W + 1]; jobs are sorted by (destination, position at the destination)
  const int32_t* grp;             // [Q, 3] row-split feature: feature slot, first entry in grp_jobs, number of shards
  const int32_t* grp_jobs;        // job of every (row-split feature, shard), shards by ascending row range
  const int32_t* whole_jobs;      // [n_whole] jobs that take a feature's ids unchanged
  const int32_t* feat_pos;        // feature slot -> position of the feature in the incoming KJT
  const void* values;
  const void* offsets;            // [F_in * B + 1] of the incoming KJT
  const float* weights;           // per-id weights or null
  int off64;
  int32_t* send_len;   // [n_shards_total, B]      local scratch: per-bag counts of every row range
  int32_t* chunk_sum;  // [n_shards_total, nchunks]
  int32_t* counters;   // [2] tickets of the two kernels ("last block done")
  int32_t* epochs;     // [nslots]
  int* err;
  PeerPtrs flags;      // int32 [nslots, W]
  PeerPtrs sizes;      // int32 [2, W, G + 2] (double-buffered by epoch parity)
  PeerPtrs recv_len;   // int32 [J_max, W, B]
  PeerPtrs recv_val;   // ids [cap]
  PeerPtrs recv_w;     // float [cap] or null
  PeerPtrs recv_ret;   // int64 [cap] or null: (source rank << 32 | position of the id in the source's KJT), for unpooled lookups
  int has_ret;
  int64_t cap;
  long long wait_cycles;
};

__device__ __forceinline__ int64_t load_off(const void* p, int64_t i, int is64) {
  return is64 ? reinterpret_cast<const int64_t*>(p)[i] : int64_t(reinterpret_cast<const int32_t*>(p)[i]);
}

// shard (row range) of `id` among `ns` ascending ranges starting at s_lo[k]; -1 when outside all of them
__device__ __forceinline__ int shard_of(int64_t id, const int64_t* s_lo, int64_t hi_last, int ns) {
  if (id < s_lo[0] || id >= hi_last) return -1;
  int k = 0;
#pragma unroll 4
  for (int i = 1; i < ns; ++i) k += (id >= s_lo[i]) ? 1 : 0;
  return k;
}

// ---- count -------------------------------------------------------------------------------------------------------
template <typename idx_t>
__global__ void __launch_bounds__(256) kjt_dist_count_kernel(DistParams p) {
  __shared__ int64_t s_lo[kMaxShards];
  __shared__ int64_t s_hi_last;
  __shared__ int s_cnt[8][kMaxShards];
  __shared__ int s_last, s_epoch;
  const int tid = threadIdx.x, lane = tid & 31, wib = tid >> 5;
  const int nwork = p.nchunks * p.Q;
  const idx_t* values = reinterpret_cast<const idx_t*>(p.values);
  if (int(blockIdx.x) < nwork) {
    const int q = blockIdx.x / p.nchunks, c = blockIdx.x - q * p.nchunks;
    const int f = p.feat_pos[p.grp[q * 3]], first = p.grp[q * 3 + 1], ns = p.grp[q * 3 + 2];
    if (tid < ns) s_lo[tid] = p.row_lo[p.grp_jobs[first + tid]];
    if (tid == 0) s_hi_last = p.row_hi[p.grp_jobs[first + ns - 1]];
    __syncthreads();
    int my_total = 0;
    for (int i = 0; i < 32; ++i) {
      const int b = c * kChunk + wib * 32 + i;
      if (b >= p.B) break;
      const int64_t start = load_off(p.offsets, int64_t(f) * p.B + b, p.off64);
      const int64_t end = load_off(p.offsets, int64_t(f) * p.B + b + 1, p.off64);
      int cnt = 0;
      for (int64_t i0 = start; i0 < end; i0 += 32) {
        int sk = -1;
        if (i0 + lane < end) {
          sk = shard_of(int64_t(values[i0 + lane]), s_lo, s_hi_last, ns);
          if (sk < 0) atomicCAS(p.err, 0, 1);  // id outside the table
        }
        for (int k = 0; k < ns; ++k) {
          const unsigned m = __ballot_sync(0xffffffffu, sk == k);
          if (lane == k) cnt += __popc(m);
        }
      }
      if (lane < ns) p.send_len[int64_t(first + lane) * p.B + b] = cnt;
      my_total += cnt;
    }
    if (lane < kMaxShards) s_cnt[wib][lane] = my_total;
    __syncthreads();
    if (tid < ns) {
      int t = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += s_cnt[w][tid];
      p.chunk_sum[int64_t(first + tid) * p.nchunks + c] = t;
    }
  }
  // the block that finishes last publishes this rank's sizes to every peer
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int t = atomicAdd(&p.counters[0], 1);
    s_last = (t == int(gridDim.x) - 1);
    s_epoch = p.epochs[SLOT_SIZES] + 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const int epoch = s_epoch, parity = epoch & 1, stride = p.G + 2;
  for (int g = tid; g < stride; g += blockDim.x) {
    int64_t val;
    if (g == p.G) {
      val = p.B;
    } else if (g == p.G + 1) {
      val = load_off(p.offsets, int64_t(p.F_in) * p.B, p.off64);
    } else if (p.jobs[g * kJobCols + J_KIND] == 0) {
      const int f = p.feat_pos[p.jobs[g * kJobCols + J_FEAT]];
      val = load_off(p.offsets, int64_t(f + 1) * p.B, p.off64) - load_off(p.offsets, int64_t(f) * p.B, p.off64);
    } else {
      const int qs = p.jobs[g * kJobCols + J_SHARD];
      int t = 0;
      for (int c = 0; c < p.nchunks; ++c) t += p.chunk_sum[int64_t(qs) * p.nchunks + c];
      val = t;
    }
    for (int pr = 0; pr < p.W; ++pr)
      reinterpret_cast<int32_t*>(p.sizes.p[pr])[(int64_t(parity) * p.W + p.rank) * stride + g] = int32_t(val);
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.W) peer_signal_one(p.flags, tid, p.rank, p.W, SLOT_SIZES, epoch);
  if (tid == 0) {
    p.epochs[SLOT_SIZES] = epoch;
    p.counters[0] = 0;
  }
}

// ---- scatter -----------------------------------------------------------------------------------------------------
// Block-wide: where the segment (job g, source = this rank) starts in the destination's id buffer, and how many ids
// that destination receives in total.  `extra` values (one per thread) are added to the start (prefix of earlier chunks).
__device__ __forceinline__ void segment_base(const DistParams& p, const int32_t* S, int g, int64_t extra, int64_t* out_base,
                                             int64_t* out_total, int64_t* s_red) {
  const int tid = threadIdx.x, lane = tid & 31, wib = tid >> 5;
  const int d = p.jobs[g * kJobCols + J_DEST];
  const int g0 = p.dest_job_start[d], g1 = p.dest_job_start[d + 1], stride = p.G + 2;
  int64_t base = extra, total = 0;
  const int n = (g1 - g0) * p.W;
  for (int i = tid; i < n; i += blockDim.x) {
    const int gg = g0 + i / p.W, s = i - (i / p.W) * p.W;
    const int64_t v = S[int64_t(s) * stride + gg];
    total += v;
    if (gg < g || (gg == g && s < p.rank)) base += v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    base += __shfl_xor_sync(0xffffffffu, base, o);
    total += __shfl_xor_sync(0xffffffffu, total, o);
  }
  __syncthreads();
  if (lane == 0) {
    s_red[wib] = base;
    s_red[8 + wib] = total;
  }
  __syncthreads();
  if (tid == 0) {
    int64_t b = 0, t = 0;
    for (int w = 0; w < 8; ++w) {
      b += s_red[w];
      t += s_red[8 + w];
    }
    *out_base = b;
    *out_total = t;
  }
  __syncthreads();
}

template <typename idx_t>
__global__ void __launch_bounds__(256) kjt_dist_scatter_kernel(DistParams p) {
  __shared__ int64_t s_red[16];
  __shared__ int64_t s_base[kMaxShards], s_total;
  __shared__ int64_t s_lo[kMaxShards];
  __shared__ int64_t s_hi_last;
  __shared__ int s_dest[kMaxShards], s_jloc[kMaxShards];
  __shared__ int s_off[kMaxShards][kChunk];
  __shared__ int s_ok, s_last, s_epoch;
  const int tid = threadIdx.x, lane = tid & 31, wib = tid >> 5;
  const int c = blockIdx.x, y = blockIdx.y;
  const idx_t* values = reinterpret_cast<const idx_t*>(p.values);
  if (tid == 0) {
    s_ok = 1;
    s_epoch = p.epochs[SLOT_SIZES];
  }
  __syncthreads();
  const int epoch = s_epoch;
  if (tid < p.W && !peer_wait_one(p.flags, tid, p.rank, p.W, SLOT_SIZES, epoch, p.wait_cycles, p.err, 200)) s_ok = 0;
  __syncthreads();
  const int stride = p.G + 2;
  const int32_t* S = reinterpret_cast<const int32_t*>(p.sizes.p[p.rank]) + int64_t(epoch & 1) * p.W * stride;
  if (tid < p.W && s_ok && S[int64_t(tid) * stride + p.G] != p.B) {
    atomicCAS(p.err, 0, 250 + tid);  // ranks disagree on the per-rank batch size
    s_ok = 0;
  }
  __syncthreads();
  const int b0 = c * kChunk, b1 = min(b0 + kChunk, p.B);
  if (s_ok && b0 < p.B) {
    if (y < p.n_whole) {
      // a feature whose ids go unchanged to one destination: contiguous copies
      const int g = p.whole_jobs[y];
      const int d = p.jobs[g * kJobCols + J_DEST], j = p.jobs[g * kJobCols + J_LOCAL];
      const int f = p.feat_pos[p.jobs[g * kJobCols + J_FEAT]];
      segment_base(p, S, g, 0, &s_base[0], &s_total, s_red);
      if (s_total > p.cap) {
        if (d == p.rank && tid == 0) atomicCAS(p.err, 0, 300);
      } else {
        const int64_t fstart = load_off(p.offsets, int64_t(f) * p.B, p.off64);
        const int64_t src0 = load_off(p.offsets, int64_t(f) * p.B + b0, p.off64);
        const int64_t src1 = load_off(p.offsets, int64_t(f) * p.B + b1, p.off64);
        const int64_t dst = s_base[0] + (src0 - fstart);
        idx_t* out = reinterpret_cast<idx_t*>(p.recv_val.p[d]) + dst;
        for (int64_t i = tid; i < src1 - src0; i += blockDim.x) out[i] = values[src0 + i];
        if (p.weights) {
          float* wout = reinterpret_cast<float*>(p.recv_w.p[d]) + dst;
          for (int64_t i = tid; i < src1 - src0; i += blockDim.x) wout[i] = p.weights[src0 + i];
        }
        if (p.has_ret) {
          int64_t* rout = reinterpret_cast<int64_t*>(p.recv_ret.p[d]) + dst;
          for (int64_t i = tid; i < src1 - src0; i += blockDim.x) rout[i] = (int64_t(p.rank) << 32) | (src0 + i);
        }
        int32_t* lout = reinterpret_cast<int32_t*>(p.recv_len.p[d]) + (int64_t(j) * p.W + p.rank) * p.B;
        for (int b = b0 + tid; b < b1; b += blockDim.x)
          lout[b] = int32_t(load_off(p.offsets, int64_t(f) * p.B + b + 1, p.off64) - load_off(p.offsets, int64_t(f) * p.B + b, p.off64));
      }
    } else {
      // a row-split feature: every id goes to the shard whose row range holds it
      const int q = y - p.n_whole;
      const int f = p.feat_pos[p.grp[q * 3]], first = p.grp[q * 3 + 1], ns = p.grp[q * 3 + 2];
      if (tid < ns) {
        const int g = p.grp_jobs[first + tid];
        s_lo[tid] = p.row_lo[g];
        s_dest[tid] = p.jobs[g * kJobCols + J_DEST];
        s_jloc[tid] = p.jobs[g * kJobCols + J_LOCAL];
      }
      if (tid == 0) s_hi_last = p.row_hi[p.grp_jobs[first + ns - 1]];
      for (int k = 0; k < ns; ++k) {
        const int g = p.grp_jobs[first + k];
        int64_t extra = 0;
        for (int cc = tid; cc < c; cc += blockDim.x) extra += p.chunk_sum[int64_t(first + k) * p.nchunks + cc];
        segment_base(p, S, g, extra, &s_base[k], &s_total, s_red);
        if (tid == 0 && s_total > p.cap) {
          if (p.jobs[g * kJobCols + J_DEST] == p.rank) atomicCAS(p.err, 0, 300);
          s_base[k] = -1;
        }
        __syncthreads();
      }
      // per-bag start of every shard's ids inside this chunk; the counts themselves are the lengths the shard receives
      for (int k = wib; k < ns; k += 8) {
        int v[8], run = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int b = b0 + lane * 8 + i;
          v[i] = b < b1 ? p.send_len[int64_t(first + k) * p.B + b] : 0;
          run += v[i];
        }
        int incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += t;
        }
        int excl = incl - run;
        int32_t* lout = reinterpret_cast<int32_t*>(p.recv_len.p[s_dest[k]]) + (int64_t(s_jloc[k]) * p.W + p.rank) * p.B;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int bi = lane * 8 + i;
          s_off[k][bi] = excl;
          excl += v[i];
          if (b0 + bi < b1 && s_base[k] >= 0) lout[b0 + bi] = v[i];
        }
      }
      __syncthreads();
      for (int bi = wib; bi < b1 - b0; bi += 8) {
        const int b = b0 + bi;
        const int64_t start = load_off(p.offsets, int64_t(f) * p.B + b, p.off64);
        const int64_t end = load_off(p.offsets, int64_t(f) * p.B + b + 1, p.off64);
        int run = 0;  // lane k: ids of this bag already placed in shard k
        for (int64_t i0 = start; i0 < end; i0 += 32) {
          int sk = -1;
          int64_t id = 0;
          if (i0 + lane < end) {
            id = int64_t(values[i0 + lane]);
            sk = shard_of(id, s_lo, s_hi_last, ns);
          }
          int pos = 0;
          for (int k = 0; k < ns; ++k) {
            const unsigned m = __ballot_sync(0xffffffffu, sk == k);
            const int r = __shfl_sync(0xffffffffu, run, k);
            if (sk == k) pos = r + __popc(m & ((1u << lane) - 1u));
            if (lane == k) run += __popc(m);
          }
          if (sk >= 0 && s_base[sk] >= 0) {
            const int64_t dst = s_base[sk] + s_off[sk][bi] + pos;
            reinterpret_cast<idx_t*>(p.recv_val.p[s_dest[sk]])[dst] = idx_t(id - s_lo[sk]);
            if (p.weights) reinterpret_cast<float*>(p.recv_w.p[s_dest[sk]])[dst] = p.weights[i0 + lane];
            if (p.has_ret) reinterpret_cast<int64_t*>(p.recv_ret.p[s_dest[sk]])[dst] = (int64_t(p.rank) << 32) | (i0 + lane);
          }
        }
      }
    }
  }
  // the block that finishes last tells every destination that this rank's data has landed
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const int t = atomicAdd(&p.counters[1], 1);
    s_last = (t == int(gridDim.x * gridDim.y) - 1);
    s_epoch = p.epochs[SLOT_DATA] + 1;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence_system();
  if (tid < p.W) peer_signal_one(p.flags, tid, p.rank, p.W, SLOT_DATA, s_epoch);
  if (tid == 0) {
    p.epochs[SLOT_DATA] = s_epoch;
    p.counters[1] = 0;
  }
}

// ---- receiver: wait for every source, then lengths -> offsets ---------------------------------------------------
__global__ void kjt_dist_wait_kernel(PeerPtrs flags, int rank, int world, const int* epochs, long long wait_cycles, int* err) {
  const int p = threadIdx.x;
  if (p < world) peer_wait_one(flags, p, rank, world, SLOT_DATA, epochs[SLOT_DATA], wait_cycles, err, 220);
}

template <typename T>
__global__ void set_first_zero_kernel(T* out) { out[0] = T(0); }

// ---- finalize / grad publish ---------------------------------------------------------------------------------------
// segment descriptor rows of the int32 [n_seg, kSegCols] table
enum SegCol : int { SEG_OUT = 0, SEG_WIDTH = 1, SEG_SRC = 2, SEG_PARTS = 3, SEG_PSTRIDE = 4, SEG_MEAN_FEAT = 5, kSegCols = 6 };

__global__ void __launch_bounds__(256) pooled_finalize_kernel(const void* __restrict__ staging, int st_dtype, int64_t st_stride,
                                                              void* __restrict__ out, int out_dtype, int64_t out_stride,
                                                              const int32_t* __restrict__ seg, int n_seg, int B,
                                                              const void* __restrict__ kjt_offsets, int off64,
                                                              const int32_t* __restrict__ feat_pos, const int* __restrict__ err) {
  const int lane = threadIdx.x & 31;
  const int64_t wid = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= int64_t(B) * n_seg) return;
  const int b = int(wid / n_seg), s = int(wid - int64_t(b) * n_seg);
  const int32_t* d = seg + s * kSegCols;
  const int width = d[SEG_WIDTH], parts = d[SEG_PARTS], pstride = d[SEG_PSTRIDE];
  float scale = 1.f;
  if (d[SEG_MEAN_FEAT] >= 0) {
    const int f = feat_pos[d[SEG_MEAN_FEAT]];
    const int64_t len = load_off(kjt_offsets, int64_t(f) * B + b + 1, off64) - load_off(kjt_offsets, int64_t(f) * B + b, off64);
    scale = len > 0 ? 1.f / float(len) : 1.f;
  }
  const bool poisoned = *err != 0;  // a wait ran out somewhere in this step: never hand stale rows on as results
  for (int e = lane * 4; e < width; e += 128) {
    float4 acc = f4zero();
    for (int pp = 0; pp < parts; ++pp) {
      const float4 v = load4_dyn(staging, int64_t(b) * st_stride + d[SEG_SRC] + int64_t(pp) * pstride + e, st_dtype);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    if (poisoned) acc.x = acc.y = acc.z = acc.w = __int_as_float(0x7fc00000);
    store4_dyn(out, int64_t(b) * out_stride + d[SEG_OUT] + e, acc, out_dtype);
  }
}

// Gradient hand-over, the mirror of the forward: the rank that owns the samples pushes every column block of its output
// gradient to the rank(s) whose tables produced it, into row `rank * B + b` of the owner's local gradient slab
// [W * B, slab_stride].  The owners' backward kernels then read local memory only.  Row-split tables have several
// owners: the block goes to each of them (an all-gather by stores).
enum GSegCol : int { GS_SRC = 0, GS_WIDTH = 1, GS_DEST = 2, GS_DCOL = 3, GS_MEAN_FEAT = 4, kGSegCols = 5 };

__global__ void __launch_bounds__(256) grad_publish_kernel(const void* __restrict__ grad, int g_dtype, int64_t g_stride, PeerPtrs slabs,
                                                           int out_dtype, int64_t slab_stride, const int32_t* __restrict__ gseg, int n_seg,
                                                           int B, int rank, const void* __restrict__ kjt_offsets, int off64,
                                                           const int32_t* __restrict__ feat_pos, float scale_all) {
  const int lane = threadIdx.x & 31;
  const int64_t wid = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= int64_t(B) * n_seg) return;
  const int b = int(wid / n_seg), s = int(wid - int64_t(b) * n_seg);
  const int32_t* d = gseg + s * kGSegCols;
  const int width = d[GS_WIDTH];
  float scale = scale_all;
  if (d[GS_MEAN_FEAT] >= 0) {
    const int f = feat_pos[d[GS_MEAN_FEAT]];
    const int64_t len = load_off(kjt_offsets, int64_t(f) * B + b + 1, off64) - load_off(kjt_offsets, int64_t(f) * B + b, off64);
    if (len > 0) scale /= float(len);
  }
  void* out = slabs.p[d[GS_DEST]];
  const int64_t orow = (int64_t(rank) * B + b) * slab_stride + d[GS_DCOL];
  for (int e = lane * 4; e < width; e += 128) {
    float4 v = load4_dyn(grad, int64_t(b) * g_stride + d[GS_SRC] + e, g_dtype);
    v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
    store4_dyn(out, orow + e, v, out_dtype);
  }
}

// Sequence (unpooled) output: rows [0, n) of the peer-written buffer become a fresh tensor of the module's output dtype.  The
// copy frees the shared buffer for the next step and, like the pooled finalize, turns the result into NaN when a wait ran
// out in this step.
__global__ void __launch_bounds__(256) seq_finalize_kernel(const void* __restrict__ staging, int st_dtype, int64_t st_stride,
                                                           void* __restrict__ out, int out_dtype, int64_t n, int cols,
                                                           const int* __restrict__ err) {
  const int per_row = (cols + 3) / 4;
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n * per_row) return;
  const int64_t r = i / per_row;
  const int e = int(i - r * per_row) * 4;
  float4 v = load4_dyn(staging, r * st_stride + e, st_dtype);
  if (*err != 0) v.x = v.y = v.z = v.w = __int_as_float(0x7fc00000);
  store4_dyn(out, r * cols + e, v, out_dtype);
}

// ---- host side -----------------------------------------------------------------------------------------------------
static void fill_peers(PeerPtrs& dst, const std::vector<int64_t>& ptrs, int world) {
  TORCH_CHECK(int(ptrs.size()) == world, "one pointer per rank expected");
  for (int i = 0; i < kMaxPeers; ++i) dst.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
}

static int dtype_code(at::ScalarType t) {
  if (t == at::kFloat) return OUT_F32;
  if (t == at::kHalf) return OUT_F16;
  if (t == at::kBFloat16) return OUT_BF16;
  TORCH_CHECK(false, "unsupported dtype ", t);
}

// `topo`: int32 device tensors {jobs [G,5], dest_job_start [W+1], grp [Q,3], grp_jobs, whole_jobs, feat_pos};
// `rows`: int64 device tensors {row_lo [G], row_hi [G]}; `scratch`: int32 device tensors {send_len, chunk_sum, counters, epochs}.
static DistParams make_params(int64_t rank, int64_t B, const std::vector<at::Tensor>& topo, const std::vector<at::Tensor>& rows,
                              const std::vector<at::Tensor>& scratch, const at::Tensor& values, const at::Tensor& offsets,
                              const c10::optional<at::Tensor>& weights, const std::vector<int64_t>& flag_ptrs,
                              const std::vector<int64_t>& size_ptrs, const std::vector<int64_t>& len_ptrs,
                              const std::vector<int64_t>& val_ptrs, const std::vector<int64_t>& w_ptrs,
                              const std::vector<int64_t>& ret_ptrs, int64_t cap, int64_t wait_cycles, at::Tensor& err) {
  TORCH_CHECK(topo.size() == 6 && rows.size() == 2 && scratch.size() == 4);
  for (const auto& t : topo) TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous());
  for (const auto& t : rows) TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kLong && t.is_contiguous());
  for (const auto& t : scratch) TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous());
  TORCH_CHECK(values.is_cuda() && values.is_contiguous() && (values.scalar_type() == at::kInt || values.scalar_type() == at::kLong));
  TORCH_CHECK(offsets.is_cuda() && offsets.is_contiguous() && (offsets.scalar_type() == at::kInt || offsets.scalar_type() == at::kLong));
  DistParams p;
  p.W = int(flag_ptrs.size());
  TORCH_CHECK(p.W >= 1 && p.W <= kMaxPeers);
  p.rank = int(rank);
  p.G = int(topo[0].size(0));
  p.Q = int(topo[2].size(0));
  p.B = int(B);
  p.nchunks = int((B + kChunk - 1) / kChunk);
  p.n_whole = int(topo[4].numel());
  p.F_in = int((offsets.numel() - 1) / std::max<int64_t>(B, 1));
  TORCH_CHECK(offsets.numel() == int64_t(p.F_in) * B + 1, "offsets must have F*B+1 entries");
  p.jobs = topo[0].data_ptr<int32_t>();
  p.dest_job_start = topo[1].data_ptr<int32_t>();
  p.grp = topo[2].data_ptr<int32_t>();
  p.grp_jobs = topo[3].data_ptr<int32_t>();
  p.whole_jobs = topo[4].data_ptr<int32_t>();
  p.feat_pos = topo[5].data_ptr<int32_t>();
  p.row_lo = rows[0].data_ptr<int64_t>();
  p.row_hi = rows[1].data_ptr<int64_t>();
  p.values = values.data_ptr();
  p.offsets = offsets.data_ptr();
  p.off64 = offsets.scalar_type() == at::kLong ? 1 : 0;
  const bool weighted = weights.has_value() && weights->defined();
  if (weighted) TORCH_CHECK(weights->is_cuda() && weights->scalar_type() == at::kFloat && weights->is_contiguous() && !w_ptrs.empty());
  p.weights = weighted ? weights->data_ptr<float>() : nullptr;
  TORCH_CHECK(scratch[0].numel() >= topo[3].numel() * B && scratch[1].numel() >= topo[3].numel() * p.nchunks, "scratch too small");
  p.send_len = scratch[0].data_ptr<int32_t>();
  p.chunk_sum = scratch[1].data_ptr<int32_t>();
  p.counters = scratch[2].data_ptr<int32_t>();
  p.epochs = scratch[3].data_ptr<int32_t>();
  p.err = err.data_ptr<int>();
  fill_peers(p.flags, flag_ptrs, p.W);
  fill_peers(p.sizes, size_ptrs, p.W);
  fill_peers(p.recv_len, len_ptrs, p.W);
  fill_peers(p.recv_val, val_ptrs, p.W);
  if (weighted) fill_peers(p.recv_w, w_ptrs, p.W);
  else for (int i = 0; i < kMaxPeers; ++i) p.recv_w.p[i] = nullptr;
  p.has_ret = ret_ptrs.empty() ? 0 : 1;
  if (p.has_ret) fill_peers(p.recv_ret, ret_ptrs, p.W);
  else for (int i = 0; i < kMaxPeers; ++i) p.recv_ret.p[i] = nullptr;
  p.cap = cap;
  p.wait_cycles = (long long)wait_cycles;
  return p;
}

// phase: 0 = count + publish sizes, 1 = scatter.  They are separate ops so that a single-GPU emulation of several ranks
// can run every rank's count before any rank's scatter; a real rank calls them back to back.
void kjt_dist_send(int64_t phase, int64_t rank, int64_t B, std::vector<at::Tensor> topo, std::vector<at::Tensor> rows,
                   std::vector<at::Tensor> scratch, const at::Tensor& values, const at::Tensor& offsets,
                   const c10::optional<at::Tensor>& weights, std::vector<int64_t> flag_ptrs, std::vector<int64_t> size_ptrs,
                   std::vector<int64_t> len_ptrs, std::vector<int64_t> val_ptrs, std::vector<int64_t> w_ptrs,
                   std::vector<int64_t> ret_ptrs, int64_t cap, int64_t wait_cycles, at::Tensor err) {
  c10::cuda::CUDAGuard guard(values.device());
  DistParams p = make_params(rank, B, topo, rows, scratch, values, offsets, weights, flag_ptrs, size_ptrs, len_ptrs, val_ptrs,
                             w_ptrs, ret_ptrs, cap, wait_cycles, err);
  auto stream = at::cuda::getCurrentCUDAStream();
  const bool i64 = values.scalar_type() == at::kLong;
  if (phase == 0) {
    const int blocks = std::max(p.nchunks * p.Q, 1);
    if (i64) kjt_dist_count_kernel<int64_t><<<blocks, 256, 0, stream>>>(p);
    else kjt_dist_count_kernel<int32_t><<<blocks, 256, 0, stream>>>(p);
  } else {
    const int rows_y = p.n_whole + p.Q;
    TORCH_CHECK(rows_y >= 1 && rows_y <= 65535, "between 1 and 65535 (feature, shard group) pairs supported");
    dim3 grid(std::max(p.nchunks, 1), rows_y);
    if (i64) kjt_dist_scatter_kernel<int64_t><<<grid, 256, 0, stream>>>(p);
    else kjt_dist_scatter_kernel<int32_t><<<grid, 256, 0, stream>>>(p);
  }
  TRB_CUDA_CHECK(cudaGetLastError());
}

// Receiver: wait for all sources' data flags, then offsets[0] = 0, offsets[i+1] = sum(recv_len[0..i]) in `like`'s dtype.
at::Tensor kjt_dist_recv_offsets(const at::Tensor& recv_len, int64_t n, bool out64, std::vector<int64_t> flag_ptrs, int64_t rank,
                                 at::Tensor epochs, int64_t wait_cycles, at::Tensor err) {
  TORCH_CHECK(recv_len.is_cuda() && recv_len.scalar_type() == at::kInt && recv_len.numel() >= n);
  c10::cuda::CUDAGuard guard(recv_len.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int world = int(flag_ptrs.size());
  PeerPtrs f;
  fill_peers(f, flag_ptrs, world);
  kjt_dist_wait_kernel<<<1, 32, 0, stream>>>(f, int(rank), world, epochs.data_ptr<int>(), (long long)wait_cycles, err.data_ptr<int>());
  at::Tensor out = at::empty({n + 1}, recv_len.options().dtype(out64 ? at::kLong : at::kInt));
  auto run = [&](auto tag) {
    using T = decltype(tag);
    set_first_zero_kernel<T><<<1, 1, 0, stream>>>(out.data_ptr<T>());
    if (n == 0) return;
    size_t bytes = 0;
    cub::DeviceScan::InclusiveSum(nullptr, bytes, recv_len.data_ptr<int32_t>(), out.data_ptr<T>() + 1, n, stream);
    at::Tensor tmp = at::empty({int64_t(bytes)}, recv_len.options().dtype(at::kByte));
    cub::DeviceScan::InclusiveSum(tmp.data_ptr(), bytes, recv_len.data_ptr<int32_t>(), out.data_ptr<T>() + 1, n, stream);
  };
  if (out64) run(int64_t(0));
  else run(int32_t(0));
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

at::Tensor pooled_finalize(const at::Tensor& staging, int64_t st_stride, const at::Tensor& seg, int64_t B, int64_t out_cols,
                           at::ScalarType out_dtype, const at::Tensor& kjt_offsets, const at::Tensor& feat_pos, const at::Tensor& err) {
  TORCH_CHECK(staging.is_cuda() && seg.is_cuda() && seg.scalar_type() == at::kInt && seg.dim() == 2 && seg.size(1) == kSegCols);
  c10::cuda::CUDAGuard guard(staging.device());
  at::Tensor out = at::empty({B, out_cols}, staging.options().dtype(out_dtype));
  const int n_seg = int(seg.size(0));
  if (B == 0 || n_seg == 0) return out;
  const int64_t warps = B * n_seg;
  const int64_t blocks = (warps * 32 + 255) / 256;
  pooled_finalize_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      staging.data_ptr(), dtype_code(staging.scalar_type()), st_stride, out.data_ptr(), dtype_code(out_dtype), out_cols,
      seg.data_ptr<int32_t>(), n_seg, int(B), kjt_offsets.data_ptr(), kjt_offsets.scalar_type() == at::kLong ? 1 : 0,
      feat_pos.data_ptr<int32_t>(), err.data_ptr<int>());
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

at::Tensor seq_finalize(const at::Tensor& staging, int64_t n, at::ScalarType out_dtype, const at::Tensor& err) {
  TORCH_CHECK(staging.is_cuda() && staging.dim() == 2 && staging.is_contiguous() && n <= staging.size(0) && staging.size(1) % 4 == 0);
  c10::cuda::CUDAGuard guard(staging.device());
  const int cols = int(staging.size(1));
  at::Tensor out = at::empty({n, cols}, staging.options().dtype(out_dtype));
  if (n == 0) return out;
  const int64_t work = n * ((cols + 3) / 4);
  seq_finalize_kernel<<<(work + 255) / 256, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      staging.data_ptr(), dtype_code(staging.scalar_type()), cols, out.data_ptr(), dtype_code(out_dtype), n, cols, err.data_ptr<int>());
  TRB_CUDA_CHECK(cudaGetLastError());
  return out;
}

void grad_publish(const at::Tensor& grad, std::vector<int64_t> slab_ptrs, at::ScalarType slab_dtype, int64_t slab_stride, int64_t rank,
                  const at::Tensor& gseg, const at::Tensor& kjt_offsets, const at::Tensor& feat_pos, double scale) {
  TORCH_CHECK(grad.is_cuda() && grad.dim() == 2 && grad.stride(1) == 1);
  TORCH_CHECK((grad.stride(0) * grad.element_size()) % 8 == 0 && reinterpret_cast<uintptr_t>(grad.data_ptr()) % 16 == 0,
              "gradient rows must be 16-byte aligned");
  TORCH_CHECK(gseg.is_cuda() && gseg.scalar_type() == at::kInt && gseg.dim() == 2 && gseg.size(1) == kGSegCols && gseg.is_contiguous());
  c10::cuda::CUDAGuard guard(grad.device());
  const int64_t B = grad.size(0);
  const int n_seg = int(gseg.size(0));
  if (B == 0 || n_seg == 0) return;
  PeerPtrs slabs;
  fill_peers(slabs, slab_ptrs, int(slab_ptrs.size()));
  const int64_t blocks = (B * n_seg * 32 + 255) / 256;
  grad_publish_kernel<<<blocks, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      grad.data_ptr(), dtype_code(grad.scalar_type()), grad.stride(0), slabs, dtype_code(slab_dtype), slab_stride, gseg.data_ptr<int32_t>(),
      n_seg, int(B), int(rank), kjt_offsets.data_ptr(), kjt_offsets.scalar_type() == at::kLong ? 1 : 0, feat_pos.data_ptr<int32_t>(),
      float(scale));
  TRB_CUDA_CHECK(cudaGetLastError());
}

}  // namespace trb

TORCH_LIBRARY_FRAGMENT(trb200, m) {
  m.def(
      "kjt_dist_send(int phase, int rank, int B, Tensor[] topo, Tensor[] rows, Tensor[] scratch, Tensor values, Tensor offsets, "
      "Tensor? weights, int[] flag_ptrs, int[] size_ptrs, int[] len_ptrs, int[] val_ptrs, int[] w_ptrs, int[] ret_ptrs, int cap, int wait_cycles, "
      "Tensor(a!) err) -> ()");
  m.def(
      "kjt_dist_recv_offsets(Tensor recv_len, int n, bool out64, int[] flag_ptrs, int rank, Tensor epochs, int wait_cycles, "
      "Tensor(a!) err) -> Tensor");
  m.def(
      "pooled_finalize(Tensor staging, int st_stride, Tensor seg, int B, int out_cols, ScalarType out_dtype, Tensor kjt_offsets, "
      "Tensor feat_pos, Tensor err) -> Tensor");
  m.def("seq_finalize(Tensor staging, int n, ScalarType out_dtype, Tensor err) -> Tensor");
  m.def(
      "grad_publish(Tensor grad, int[] slab_ptrs, ScalarType slab_dtype, int slab_stride, int rank, Tensor gseg, Tensor kjt_offsets, "
      "Tensor feat_pos, float scale) -> ()");
}

TORCH_LIBRARY_IMPL(trb200, CompositeExplicitAutograd, m) {
  m.impl("kjt_dist_send", &trb::kjt_dist_send);
  m.impl("kjt_dist_recv_offsets", &trb::kjt_dist_recv_offsets);
  m.impl("pooled_finalize", &trb::pooled_finalize);
  m.impl("grad_publish", &trb::grad_publish);
  m.impl("seq_finalize", &trb::seq_finalize);
}
