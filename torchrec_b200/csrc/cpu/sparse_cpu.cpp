// Host implementations of the sparse-input operators (``torch.ops.trb200_cpu.*``): the data-loading and CPU-training path,
// and the sequential oracle of the device kernels.  Loops are parallelised with at::parallel_for where iterations are
// independent; the hash insert is sequential by construction.
//
// The reference takes the CPU forms of these operators from an external wheel (torchrec/sparse/jagged_tensor.py:32-48).
#include <ATen/ATen.h>
#include <ATen/Parallel.h>
#include <torch/library.h>

#include <algorithm>
#include <climits>
#include <vector>

#include "../cuda/zch_hash.h"

namespace trb_cpu {

template <typename F>
void dispatch_index(const at::Tensor& t, F&& f) {
  if (t.scalar_type() == at::kLong) f(int64_t(0));
  else if (t.scalar_type() == at::kInt) f(int32_t(0));
  else TORCH_CHECK(false, "expected an int32 or int64 tensor, got ", t.scalar_type());
}

// ---- complete cumsum ----------------------------------------------------------------------------
at::Tensor complete_cumsum(const at::Tensor& x) {
  TORCH_CHECK(x.dim() == 1);
  at::Tensor xc = x.contiguous();
  at::Tensor out = at::empty({x.numel() + 1}, x.options());
  auto run = [&](auto tag) {
    using T = decltype(tag);
    const T* in = xc.data_ptr<T>();
    T* o = out.data_ptr<T>();
    T acc = 0;
    o[0] = 0;
    for (int64_t i = 0; i < xc.numel(); ++i) { acc += in[i]; o[i + 1] = acc; }
  };
  if (x.scalar_type() == at::kLong) run(int64_t(0));
  else if (x.scalar_type() == at::kInt) run(int32_t(0));
  else if (x.scalar_type() == at::kFloat) run(float(0));
  else if (x.scalar_type() == at::kDouble) run(double(0));
  else TORCH_CHECK(false, "complete_cumsum: unsupported dtype ", x.scalar_type());
  return out;
}

// ---- permute_2d_sparse_data: lengths [T, B], permute [T'] ----------------------------------------
std::tuple<at::Tensor, at::Tensor, c10::optional<at::Tensor>> permute_2d_sparse_data(const at::Tensor& permute, const at::Tensor& lengths, const at::Tensor& values,
                                                                                     const c10::optional<at::Tensor>& weights) {
  TORCH_CHECK(lengths.dim() == 2 && values.dim() >= 1);
  const int64_t T = lengths.size(0), B = lengths.size(1), Tp = permute.numel();
  at::Tensor len_c = lengths.contiguous(), perm = permute.to(at::kLong).contiguous(), val_c = values.contiguous();
  at::Tensor out_len = at::empty({Tp, B}, lengths.options());
  std::vector<int64_t> in_off(T + 1, 0), out_off(Tp + 1, 0);
  const int64_t* pp = perm.data_ptr<int64_t>();
  dispatch_index(lengths, [&](auto tag) {
    using L = decltype(tag);
    const L* l = len_c.data_ptr<L>();
    L* ol = out_len.data_ptr<L>();
    for (int64_t t = 0; t < T; ++t) {
      int64_t s = 0;
      for (int64_t b = 0; b < B; ++b) s += l[t * B + b];
      in_off[t + 1] = in_off[t] + s;
    }
    for (int64_t t = 0; t < Tp; ++t) {
      TORCH_CHECK(pp[t] >= 0 && pp[t] < T, "permute_2d_sparse_data: permute entry out of range");
      std::copy(l + pp[t] * B, l + (pp[t] + 1) * B, ol + t * B);
      out_off[t + 1] = out_off[t] + (in_off[pp[t] + 1] - in_off[pp[t]]);
    }
  });
  std::vector<int64_t> shape = values.sizes().vec();
  shape[0] = out_off[Tp];
  at::Tensor out_val = at::empty(shape, values.options());
  const int64_t row_bytes = values.numel() ? int64_t(values.element_size()) * (values.numel() / std::max<int64_t>(values.size(0), 1)) : int64_t(values.element_size());
  const char* vs = static_cast<const char*>(val_c.data_ptr());
  char* vd = static_cast<char*>(out_val.data_ptr());
  c10::optional<at::Tensor> out_w;
  at::Tensor w_c;
  int64_t w_row = 0;
  if (weights.has_value() && weights->defined()) {
    w_c = weights->contiguous();
    std::vector<int64_t> ws = w_c.sizes().vec();
    ws[0] = out_off[Tp];
    out_w = at::empty(ws, w_c.options());
    w_row = int64_t(w_c.element_size()) * (w_c.numel() / std::max<int64_t>(w_c.size(0), 1));
  }
  at::parallel_for(0, Tp, 1, [&](int64_t b, int64_t e) {
    for (int64_t t = b; t < e; ++t) {
      const int64_t n = out_off[t + 1] - out_off[t];
      if (n == 0) continue;
      std::memcpy(vd + out_off[t] * row_bytes, vs + in_off[pp[t]] * row_bytes, size_t(n * row_bytes));
      if (out_w.has_value())
        std::memcpy(static_cast<char*>(out_w->data_ptr()) + out_off[t] * w_row, static_cast<const char*>(w_c.data_ptr()) + in_off[pp[t]] * w_row, size_t(n * w_row));
    }
  });
  return {out_len, out_val, out_w};
}

// ---- block bucketize: lengths [F*B], bucket = id / block_size[f] (ids past the last block wrap) ------
std::tuple<at::Tensor, at::Tensor, c10::optional<at::Tensor>, c10::optional<at::Tensor>, c10::optional<at::Tensor>> block_bucketize(
    const at::Tensor& lengths, const at::Tensor& indices, bool bucketize_pos, bool sequence, const at::Tensor& block_sizes, int64_t my_size,
    const c10::optional<at::Tensor>& weights, bool keep_orig_idx) {
  const int64_t n_bags = lengths.numel(), F = block_sizes.numel(), N = indices.numel();
  TORCH_CHECK(F > 0 && n_bags % F == 0 && my_size > 0);
  const int64_t B = n_bags / F;
  at::Tensor len_c = lengths.contiguous().view({-1}), idx_c = indices.contiguous(), blk = block_sizes.to(at::kLong).contiguous();
  at::Tensor new_len = at::zeros({my_size * n_bags}, lengths.options());
  at::Tensor new_idx = at::empty({N}, indices.options());
  c10::optional<at::Tensor> new_w, new_pos, unbucketize;
  at::Tensor w_c;
  if (weights.has_value() && weights->defined()) { w_c = weights->contiguous(); new_w = at::empty_like(w_c); TORCH_CHECK(w_c.scalar_type() == at::kFloat && w_c.numel() == N); }
  if (bucketize_pos) new_pos = at::empty({N}, indices.options());
  if (sequence) unbucketize = at::empty({N}, indices.options());
  const int64_t* bs = blk.data_ptr<int64_t>();
  dispatch_index(lengths, [&](auto ltag) {
    using L = decltype(ltag);
    dispatch_index(indices, [&](auto itag) {
      using I = decltype(itag);
      const L* l = len_c.data_ptr<L>();
      const I* idx = idx_c.data_ptr<I>();
      L* nl = new_len.data_ptr<L>();
      I* ni = new_idx.data_ptr<I>();
      std::vector<int64_t> off(n_bags + 1, 0);
      for (int64_t i = 0; i < n_bags; ++i) off[i + 1] = off[i] + l[i];
      TORCH_CHECK(off[n_bags] == N, "block_bucketize: lengths do not add up to the number of indices");
      auto bucket_of = [&](int64_t id, int64_t f, int64_t& local) {
        const int64_t b = bs[f];
        if (b > 0 && id < b * my_size) { const int64_t k = id / b; local = id - k * b; return k; }
        local = id / my_size;
        return id % my_size;
      };
      // pass 1: counts
      at::parallel_for(0, n_bags, 64, [&](int64_t b0, int64_t b1) {
        for (int64_t bag = b0; bag < b1; ++bag) {
          const int64_t f = bag / B;
          for (int64_t j = off[bag]; j < off[bag + 1]; ++j) { int64_t local; nl[bucket_of(int64_t(idx[j]), f, local) * n_bags + bag] += 1; }
        }
      });
      // output offsets, bucket-major
      std::vector<int64_t> noff(my_size * n_bags + 1, 0);
      for (int64_t i = 0; i < my_size * n_bags; ++i) noff[i + 1] = noff[i] + nl[i];
      // pass 2: scatter, keeping the order inside a bag
      at::parallel_for(0, n_bags, 64, [&](int64_t b0, int64_t b1) {
        std::vector<int64_t> cursor(my_size);
        for (int64_t bag = b0; bag < b1; ++bag) {
          const int64_t f = bag / B;
          for (int64_t k = 0; k < my_size; ++k) cursor[k] = noff[k * n_bags + bag];
          for (int64_t j = off[bag]; j < off[bag + 1]; ++j) {
            int64_t local;
            const int64_t k = bucket_of(int64_t(idx[j]), f, local);
            const int64_t dst = cursor[k]++;
            ni[dst] = keep_orig_idx ? idx[j] : I(local);
            if (new_w.has_value()) new_w->data_ptr<float>()[dst] = w_c.data_ptr<float>()[j];
            if (new_pos.has_value()) new_pos->data_ptr<I>()[dst] = I(j - off[bag]);
            if (unbucketize.has_value()) unbucketize->data_ptr<I>()[j] = I(dst);
          }
        }
      });
    });
  });
  return {new_len, new_idx, new_w, new_pos, unbucketize};
}

// ---- jagged [N, D] -> padded [B, L, D] ------------------------------------------------------------
at::Tensor jagged_to_padded_dense(const at::Tensor& values, const at::Tensor& offsets, int64_t max_length, double padding_value) {
  TORCH_CHECK(values.dim() == 2 && offsets.dim() == 1 && offsets.numel() >= 1);
  const int64_t B = offsets.numel() - 1, D = values.size(1);
  at::Tensor v = values.contiguous(), off = offsets.to(at::kLong).contiguous();
  at::Tensor out = at::full({B, max_length, D}, padding_value, values.options());
  const int64_t* o = off.data_ptr<int64_t>();
  const int64_t row = D * int64_t(values.element_size());
  const char* src = static_cast<const char*>(v.data_ptr());
  char* dst = static_cast<char*>(out.data_ptr());
  at::parallel_for(0, B, 16, [&](int64_t b0, int64_t b1) {
    for (int64_t b = b0; b < b1; ++b) {
      const int64_t n = std::min<int64_t>(o[b + 1] - o[b], max_length);
      if (n > 0) std::memcpy(dst + b * max_length * row, src + o[b] * row, size_t(n * row));
    }
  });
  return out;
}

// ---- multi-probe zero-collision hash, sequential (the device kernels document the algorithm) -------
std::tuple<at::Tensor, at::Tensor> zch_probe(const at::Tensor& ids, at::Tensor identities, c10::optional<at::Tensor> metadata, const at::Tensor& segments,
                                             int64_t input_hash_size, int64_t out_offset, int64_t max_probe, bool readonly, bool disable_fallback,
                                             const c10::optional<at::Tensor>& input_metadata, int64_t eviction_threshold, int64_t eviction_policy,
                                             int64_t reserved_slots) {
  TORCH_CHECK(ids.scalar_type() == at::kLong && identities.scalar_type() == at::kLong && identities.is_contiguous() && segments.scalar_type() == at::kLong);
  at::Tensor ids_c = ids.contiguous(), seg_c = segments.contiguous();
  const int64_t N = ids_c.numel(), S = identities.numel(), nb = seg_c.numel() - 1;
  at::Tensor slots = at::full({N}, -1, ids.options()), evicted = at::full({N}, -1, ids.options());
  int64_t* ident = identities.data_ptr<int64_t>();
  int32_t* meta = nullptr;
  const int32_t* in_meta = nullptr;
  at::Tensor in_meta_c;
  if (metadata.has_value() && metadata->defined()) { TORCH_CHECK(metadata->scalar_type() == at::kInt && metadata->numel() == S && metadata->is_contiguous()); meta = metadata->data_ptr<int32_t>(); }
  if (input_metadata.has_value() && input_metadata->defined()) { in_meta_c = input_metadata->contiguous(); TORCH_CHECK(in_meta_c.scalar_type() == at::kInt && in_meta_c.numel() == N); in_meta = in_meta_c.data_ptr<int32_t>(); }
  const int64_t* seg = seg_c.data_ptr<int64_t>();
  const int64_t* id = ids_c.data_ptr<int64_t>();
  int64_t* so = slots.data_ptr<int64_t>();
  int64_t* eo = evicted.data_ptr<int64_t>();
  auto range = [&](int64_t v, int64_t& lo, int64_t& size, int64_t& start) {
    const int64_t b = trb::zch_bucket(v, input_hash_size, nb);
    lo = seg[b] - out_offset;
    const int64_t hi = seg[b + 1] - out_offset;
    if (lo < 0 || hi > S || hi <= lo) return false;
    size = hi - lo;
    if (reserved_slots > 0 && reserved_slots < size) size -= reserved_slots;  // the reserved block at the end of the bucket is never probed
    start = int64_t(trb::zch_mix(uint64_t(v)) % uint64_t(size));
    return true;
  };
  // phase 1: hits refresh their score before anything is inserted or evicted
  for (int64_t i = 0; i < N; ++i) {
    int64_t lo, size, start;
    if (!range(id[i], lo, size, start)) continue;
    const int64_t probes = std::min<int64_t>(std::max<int64_t>(max_probe, 1), size);
    for (int64_t p = 0; p < probes; ++p) {
      const int64_t s = lo + (start + p) % size;
      if (ident[s] == id[i]) { so[i] = s; if (meta && in_meta) meta[s] = std::max(meta[s], in_meta[i]); break; }
      if (ident[s] == -1) break;
    }
  }
  for (int64_t i = 0; i < N && !readonly; ++i) {
    if (so[i] >= 0) continue;
    int64_t lo, size, start;
    if (!range(id[i], lo, size, start)) continue;
    const int32_t fresh = in_meta ? in_meta[i] : 0;
    const int64_t probes = std::min<int64_t>(std::max<int64_t>(max_probe, 1), size);
    int64_t lru_slot = -1;
    int32_t lru_meta = INT_MAX;
    for (int64_t p = 0; p < probes && so[i] < 0; ++p) {
      const int64_t s = lo + (start + p) % size;
      if (ident[s] == -1) { ident[s] = id[i]; if (meta) meta[s] = fresh; so[i] = s; break; }
      if (ident[s] == id[i]) { so[i] = s; if (meta && in_meta) meta[s] = std::max(meta[s], fresh); break; }
      if (!meta || eviction_policy == trb::ZCH_NO_EVICT) continue;
      if (eviction_policy == trb::ZCH_TTL) {
        if (meta[s] < int32_t(eviction_threshold)) { ident[s] = id[i]; meta[s] = fresh; so[i] = s; eo[i] = s; }
      } else if (meta[s] < lru_meta) { lru_meta = meta[s]; lru_slot = s; }
    }
    if (so[i] < 0 && eviction_policy == trb::ZCH_LRU && lru_slot >= 0 && lru_meta < fresh) { ident[lru_slot] = id[i]; meta[lru_slot] = fresh; so[i] = lru_slot; eo[i] = lru_slot; }
  }
  if (!disable_fallback)
    for (int64_t i = 0; i < N; ++i) {
      int64_t lo, size, start;
      if (so[i] >= 0 || !range(id[i], lo, size, start)) continue;
      const int64_t bucket = seg[trb::zch_bucket(id[i], input_hash_size, nb) + 1] - out_offset - lo;
      so[i] = (reserved_slots > 0 && reserved_slots < bucket) ? lo + size + int64_t(trb::zch_mix(uint64_t(id[i])) % uint64_t(reserved_slots)) : lo + start;
    }
  return {slots, evicted};
}

// ---- pruning remap (see the device kernel) ------------------------------------------------------------
at::Tensor itep_remap(const at::Tensor& values, const at::Tensor& feature_offsets, const at::Tensor& feature_buffer, const at::Tensor& address_lookup, at::Tensor row_util,
                      const at::Tensor& buffer_offsets, bool update_util) {
  TORCH_CHECK(values.scalar_type() == at::kLong && feature_offsets.scalar_type() == at::kLong && feature_buffer.scalar_type() == at::kInt);
  TORCH_CHECK(address_lookup.scalar_type() == at::kLong && row_util.scalar_type() == at::kFloat && row_util.is_contiguous() && buffer_offsets.scalar_type() == at::kLong);
  at::Tensor v = values.contiguous(), fo = feature_offsets.contiguous(), fb = feature_buffer.contiguous(), al = address_lookup.contiguous(), bo = buffer_offsets.contiguous();
  at::Tensor out = at::empty_like(v);
  const int64_t F = fb.numel();
  for (int64_t f = 0; f < F; ++f) {
    const int64_t b = fo.data_ptr<int64_t>()[f], e = fo.data_ptr<int64_t>()[f + 1];
    const int buf = fb.data_ptr<int32_t>()[f];
    for (int64_t i = b; i < e; ++i) {
      const int64_t x = v.data_ptr<int64_t>()[i];
      if (buf < 0) { out.data_ptr<int64_t>()[i] = x; continue; }
      const int64_t base = bo.data_ptr<int64_t>()[buf], size = bo.data_ptr<int64_t>()[buf + 1] - base;
      if (x < 0 || x >= size) { out.data_ptr<int64_t>()[i] = x; continue; }
      const int64_t en = al.data_ptr<int64_t>()[base + x];
      out.data_ptr<int64_t>()[i] = en >= 0 ? en : -(en + 1);
      if (update_util) row_util.data_ptr<float>()[base + x] += 1.f;
    }
  }
  return out;
}

}  // namespace trb_cpu

TORCH_LIBRARY(trb200_cpu, m) {
  m.def("complete_cumsum(Tensor x) -> Tensor", &trb_cpu::complete_cumsum);
  m.def("permute_2d_sparse_data(Tensor permute, Tensor lengths, Tensor values, Tensor? weights) -> (Tensor, Tensor, Tensor?)", &trb_cpu::permute_2d_sparse_data);
  m.def("block_bucketize(Tensor lengths, Tensor indices, bool bucketize_pos, bool sequence, Tensor block_sizes, int my_size, Tensor? weights, bool keep_orig_idx) -> (Tensor, Tensor, Tensor?, Tensor?, Tensor?)", &trb_cpu::block_bucketize);
  m.def("jagged_to_padded_dense(Tensor values, Tensor offsets, int max_length, float padding_value) -> Tensor", &trb_cpu::jagged_to_padded_dense);
  m.def("zch_probe(Tensor ids, Tensor(a!) identities, Tensor(b!)? metadata, Tensor segments, int input_hash_size, int out_offset, int max_probe, bool readonly, "
        "bool disable_fallback, Tensor? input_metadata, int eviction_threshold, int eviction_policy, int reserved_slots=0) -> (Tensor, Tensor)", &trb_cpu::zch_probe);
  m.def("itep_remap(Tensor values, Tensor feature_offsets, Tensor feature_buffer, Tensor address_lookup, Tensor(a!) row_util, Tensor buffer_offsets, bool update_util) -> Tensor", &trb_cpu::itep_remap);
}
