// Sequence packing for RL train batches: first-fit-decreasing bin assignment, one-pass row fill,
// and padded (left-pad prompt / right-pad completion) batch assembly. Host-only, plain C ABI over
// CSR-style inputs (one concatenated value array + offsets per field), so Python releases the GIL for
// the whole call (ctypes does that by itself) and output rows can live in pinned host memory.
//
// Behaviour matches the reference's packing extension (tunix/rl/_packing_ext.cc:496-569 FFD core,
// :195-336 row fill, :899-1173 padded assembly, :1177-1232 router-replay census):
//   * items are stable-sorted by descending length; each goes to the FIRST bin with room;
//   * after a placement the bin's next start is aligned up to `boundary`; a bin closes at
//     `max_segments` segments; what fits nowhere is returned as leftover (ascending original index);
//   * rows number segments 1..S (0 = padding), positions restart at 0 per segment, gaps and tails
//     are padded (ids = pad_id, masks / advantages / per-token = 0, routed experts = -1).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

#define TB_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

inline int64_t align_up(int64_t x, int64_t b) { return b <= 1 ? x : (x + b - 1) / b * b; }

struct Bin {
  int64_t rem;
  int64_t next_start;
  int segs;
};

// One chunk of FFD over `order` (descending length). Items that do not fit go to next_order.
void ffd_one_chunk(const int32_t* lengths, const std::vector<int32_t>& order, int pack_size, int64_t budget,
                   int max_segments, int64_t boundary, int32_t* bin_of, int32_t* start_of,
                   std::vector<int32_t>& next_order) {
  std::vector<Bin> bins(pack_size > 0 ? pack_size : 0, Bin{budget, 0, 0});
  int64_t max_rem = pack_size > 0 ? budget : -1;
  size_t pos = 0;
  for (; pos < order.size(); ++pos) {
    const int32_t it = order[pos];
    const int64_t n = lengths[it];
    bool placed = false;
    if (n <= max_rem) {
      for (int b = 0; b < pack_size; ++b) {
        Bin& bin = bins[b];
        if (bin.rem >= n) {
          bin_of[it] = b;
          start_of[it] = (int32_t)bin.next_start;
          const int64_t end = bin.next_start + n;
          bin.segs++;
          if (bin.segs >= max_segments) {
            bin.rem = -1;
          } else {
            bin.next_start = align_up(end, boundary);
            bin.rem = budget - bin.next_start;
          }
          placed = true;
          break;
        }
      }
    }
    if (!placed) {
      next_order.push_back(it);
      max_rem = -1;
      for (const Bin& b : bins) max_rem = std::max(max_rem, b.rem);
      if (max_rem < 0) {  // every bin is closed: the rest cannot be placed in this chunk
        ++pos;
        break;
      }
    } else {
      max_rem = -1;
      for (const Bin& b : bins) max_rem = std::max(max_rem, b.rem);
    }
  }
  for (; pos < order.size(); ++pos) next_order.push_back(order[pos]);
}

template <typename T>
inline void fill(T* p, int64_t n, T v) {
  for (int64_t i = 0; i < n; ++i) p[i] = v;
}

}  // namespace

// lengths[n] = prompt + completion tokens of each item.
// Outputs: bin_of[n] (-1 = leftover), start_of[n] (token offset inside its bin).
// Returns the number of placed items, or -1 for an invalid argument.
TB_HOST_API int tb_pack_ffd(const int32_t* lengths, int n, int pack_size, int64_t budget, int max_segments,
                            int64_t boundary, int32_t* bin_of, int32_t* start_of) {
  if (boundary <= 0 || n < 0) return -1;
  for (int i = 0; i < n; ++i) {
    bin_of[i] = -1;
    start_of[i] = 0;
  }
  if (n == 0 || pack_size <= 0 || max_segments <= 0) return 0;
  std::vector<int32_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return lengths[a] > lengths[b]; });
  std::vector<int32_t> next;
  ffd_one_chunk(lengths, order, pack_size, budget, max_segments, boundary, bin_of, start_of, next);
  return n - (int)next.size();
}

// Multi-chunk FFD under one call: chunk_of[n] (-1 leftover), bin_of[n], start_of[n].
// Stops early when min_buffered_tokens > 0 and fewer tokens than that remain. Returns the number of
// chunks, -1 for an invalid argument, -2 when an item can never be placed (longer than the budget).
TB_HOST_API int tb_pack_ffd_chunks(const int32_t* lengths, int n, int pack_size, int64_t budget,
                                   int max_segments, int64_t boundary, int64_t min_buffered_tokens,
                                   int32_t* chunk_of, int32_t* bin_of, int32_t* start_of) {
  if (boundary <= 0 || n < 0) return -1;
  for (int i = 0; i < n; ++i) {
    chunk_of[i] = -1;
    bin_of[i] = -1;
    start_of[i] = 0;
  }
  if (n == 0 || pack_size <= 0 || max_segments <= 0) return 0;
  std::vector<int32_t> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return lengths[a] > lengths[b]; });
  int chunk = 0;
  while (!order.empty()) {
    int64_t remaining = 0;
    for (int32_t it : order) remaining += lengths[it];
    if (min_buffered_tokens > 0 && remaining < min_buffered_tokens) break;
    std::vector<int32_t> next;
    std::vector<int32_t> tmp_bin(n, -1), tmp_start(n, 0);
    ffd_one_chunk(lengths, order, pack_size, budget, max_segments, boundary, tmp_bin.data(), tmp_start.data(), next);
    if (next.size() == order.size()) return -2;
    for (int32_t it : order)
      if (tmp_bin[it] >= 0) {
        chunk_of[it] = chunk;
        bin_of[it] = tmp_bin[it];
        start_of[it] = tmp_start[it];
      }
    order.swap(next);
    ++chunk;
  }
  return chunk;
}

// Fill one chunk of n_bins rows of `budget` tokens. Items are given in CSR form:
//   prompt_ids[prompt_off[i] .. prompt_off[i+1]), completion arrays likewise over comp_off.
//   per_token: n_fields arrays aligned with the completion CSR (may be 0 fields).
//   routed: int16 [routed_off[i] .. routed_off[i+1]) tokens x rl x rk values per item, or null.
// item_idx[m] lists the items of this chunk; bin_of / start_of index by item.
// Every output byte is written exactly once. Returns 0, or -1 if a row would overflow the budget.
TB_HOST_API int tb_pack_fill(const int32_t* item_idx, int m, const int32_t* bin_of, const int32_t* start_of,
                             const int32_t* prompt_ids, const int64_t* prompt_off, const int32_t* comp_ids,
                             const float* comp_mask, const float* adv, const int64_t* comp_off,
                             const float* const* per_token, int n_fields, const int16_t* routed,
                             const int64_t* routed_off, int rl, int rk, int n_bins, int64_t budget, int32_t pad_id,
                             int32_t* out_ids, float* out_prompt_mask, float* out_comp_mask, float* out_adv,
                             int32_t* out_seg, int32_t* out_pos, float* const* out_fields, int16_t* out_routed,
                             int32_t* out_num_segments) {
  std::vector<std::vector<int32_t>> rows(n_bins);
  for (int j = 0; j < m; ++j) {
    const int32_t it = item_idx[j];
    if (bin_of[it] < 0 || bin_of[it] >= n_bins) return -1;
    rows[bin_of[it]].push_back(it);
  }
  const int64_t rstride = (int64_t)rl * rk;
  for (int b = 0; b < n_bins; ++b) {
    auto& items = rows[b];
    std::sort(items.begin(), items.end(), [&](int32_t x, int32_t y) { return start_of[x] < start_of[y]; });
    const int64_t base = (int64_t)b * budget;
    int64_t cursor = 0;
    int seg = 0;
    auto pad_range = [&](int64_t from, int64_t to) {
      if (to <= from) return;
      fill(out_ids + base + from, to - from, pad_id);
      fill(out_prompt_mask + base + from, to - from, 0.f);
      fill(out_comp_mask + base + from, to - from, 0.f);
      fill(out_adv + base + from, to - from, 0.f);
      fill(out_seg + base + from, to - from, (int32_t)0);
      fill(out_pos + base + from, to - from, (int32_t)0);
      for (int f = 0; f < n_fields; ++f) fill(out_fields[f] + base + from, to - from, 0.f);
      if (out_routed) fill(out_routed + (base + from) * rstride, (to - from) * rstride, (int16_t)-1);
    };
    for (int32_t it : items) {
      const int64_t p = prompt_off[it + 1] - prompt_off[it];
      const int64_t c = comp_off[it + 1] - comp_off[it];
      const int64_t start = start_of[it];
      if (start < cursor || start + p + c > budget) return -1;
      pad_range(cursor, start);
      ++seg;
      const int64_t o = base + start;
      std::memcpy(out_ids + o, prompt_ids + prompt_off[it], p * sizeof(int32_t));
      std::memcpy(out_ids + o + p, comp_ids + comp_off[it], c * sizeof(int32_t));
      fill(out_prompt_mask + o, p, 1.f);
      fill(out_prompt_mask + o + p, c, 0.f);
      fill(out_comp_mask + o, p, 0.f);
      std::memcpy(out_comp_mask + o + p, comp_mask + comp_off[it], c * sizeof(float));
      fill(out_adv + o, p, 0.f);
      std::memcpy(out_adv + o + p, adv + comp_off[it], c * sizeof(float));
      fill(out_seg + o, p + c, (int32_t)seg);
      for (int64_t t = 0; t < p + c; ++t) out_pos[o + t] = (int32_t)t;
      for (int f = 0; f < n_fields; ++f) {
        fill(out_fields[f] + o, p, 0.f);
        std::memcpy(out_fields[f] + o + p, per_token[f] + comp_off[it], c * sizeof(float));
      }
      if (out_routed) {
        int64_t have = routed ? (routed_off[it + 1] - routed_off[it]) : 0;
        if (have > p + c) have = p + c;
        if (have > 0) std::memcpy(out_routed + o * rstride, routed + routed_off[it] * rstride, have * rstride * sizeof(int16_t));
        fill(out_routed + (o + have) * rstride, (p + c - have) * rstride, (int16_t)-1);
      }
      cursor = start + p + c;
    }
    pad_range(cursor, budget);
    if (out_num_segments) out_num_segments[b] = seg;
  }
  return 0;
}

// Padded batch: prompts left-padded to p_max (over-long prompts keep their LAST p_max tokens),
// completions right-padded / truncated to c_max. Rows >= n_items are fully padded.
// adv_mode: 0 = one scalar per item (broadcast over kept tokens), 1 = per completion token (CSR with comp_off).
// Returns 0; counts of truncated prompts / completions are written to trunc[0], trunc[1].
TB_HOST_API int tb_assemble_padded(int n_items, int batch, const int32_t* prompt_ids, const int64_t* prompt_off,
                                   const float* prompt_mask /*CSR like prompt_ids or null*/, const int32_t* comp_ids,
                                   const float* comp_mask /*or null*/, const int64_t* comp_off, const float* adv,
                                   int adv_mode, const float* const* per_token, int n_fields, int64_t p_max,
                                   int64_t c_max, int32_t pad_id, int32_t* out_prompt_ids, float* out_prompt_mask,
                                   int32_t* out_comp_ids, float* out_comp_mask, float* out_adv,
                                   float* const* out_fields, int32_t* row_valid_tokens, int32_t* row_num_sequences,
                                   int32_t* trunc) {
  int tp = 0, tc = 0;
  for (int r = 0; r < batch; ++r) {
    int32_t* pi = out_prompt_ids + (int64_t)r * p_max;
    float* pm = out_prompt_mask + (int64_t)r * p_max;
    int32_t* ci = out_comp_ids + (int64_t)r * c_max;
    float* cm = out_comp_mask + (int64_t)r * c_max;
    float* av = out_adv + (int64_t)r * c_max;
    if (r >= n_items) {
      fill(pi, p_max, pad_id);
      fill(pm, p_max, 0.f);
      fill(ci, c_max, pad_id);
      fill(cm, c_max, 0.f);
      fill(av, c_max, 0.f);
      for (int f = 0; f < n_fields; ++f) fill(out_fields[f] + (int64_t)r * c_max, c_max, 0.f);
      if (row_valid_tokens) row_valid_tokens[r] = 0;
      if (row_num_sequences) row_num_sequences[r] = 0;
      continue;
    }
    int64_t p = prompt_off[r + 1] - prompt_off[r];
    int64_t c = comp_off[r + 1] - comp_off[r];
    int64_t pskip = 0;
    if (p > p_max) {
      pskip = p - p_max;
      p = p_max;
      ++tp;
    }
    int64_t ck = c;
    if (ck > c_max) {
      ck = c_max;
      ++tc;
    }
    const int64_t lp = p_max - p;
    fill(pi, lp, pad_id);
    fill(pm, lp, 0.f);
    std::memcpy(pi + lp, prompt_ids + prompt_off[r] + pskip, p * sizeof(int32_t));
    if (prompt_mask) std::memcpy(pm + lp, prompt_mask + prompt_off[r] + pskip, p * sizeof(float));
    else fill(pm + lp, p, 1.f);
    std::memcpy(ci, comp_ids + comp_off[r], ck * sizeof(int32_t));
    fill(ci + ck, c_max - ck, pad_id);
    if (comp_mask) std::memcpy(cm, comp_mask + comp_off[r], ck * sizeof(float));
    else fill(cm, ck, 1.f);
    fill(cm + ck, c_max - ck, 0.f);
    if (adv_mode == 0) fill(av, ck, adv[r]);
    else std::memcpy(av, adv + comp_off[r], ck * sizeof(float));
    fill(av + ck, c_max - ck, 0.f);
    for (int f = 0; f < n_fields; ++f) {
      float* o = out_fields[f] + (int64_t)r * c_max;
      std::memcpy(o, per_token[f] + comp_off[r], ck * sizeof(float));
      fill(o + ck, c_max - ck, 0.f);
    }
    if (row_valid_tokens) row_valid_tokens[r] = (int32_t)(p + ck);
    if (row_num_sequences) row_num_sequences[r] = 1;
  }
  if (trunc) {
    trunc[0] = tp;
    trunc[1] = tc;
  }
  return 0;
}

// Over routed [B,T,L,k] int16 and segment_ids [B,T]: counts real tokens (segment > 0) and those whose
// layer-0 expert list is fully valid (all >= 0, no duplicates). out[0] = real, out[1] = forced.
TB_HOST_API int tb_count_router_replay_forced(const int16_t* routed, const int32_t* segment_ids, int64_t B,
                                              int64_t T, int L, int k, int64_t* out) {
  int64_t real = 0, forced = 0;
  const int64_t stride = (int64_t)L * k;
  for (int64_t i = 0; i < B * T; ++i) {
    if (segment_ids[i] <= 0) continue;
    ++real;
    const int16_t* e = routed + i * stride;
    bool ok = true;
    for (int a = 0; a < k && ok; ++a) {
      if (e[a] < 0) ok = false;
      for (int b = 0; b < a && ok; ++b)
        if (e[a] == e[b]) ok = false;
    }
    if (ok) ++forced;
  }
  out[0] = real;
  out[1] = forced;
  return 0;
}

// Version of this library's C ABI; bumped when an exported signature changes.
extern "C" __attribute__((visibility("default"))) int tb_host_abi_version() { return 2; }
