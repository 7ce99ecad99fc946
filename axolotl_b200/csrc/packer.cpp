// Host-side native helpers (no CUDA): multipack bin packing and attention tile tables.
//
// The packer reproduces the sampler semantics of the reference
// (src/axolotl/utils/samplers/multipack.py:60-241): first-fit in the given (shuffled) order,
// independently per group of `group_size` samples, with at most `bin_size` samples per bin; and
// an order-preserving sequential mode. First-fit uses a tournament tree over the bins' remaining
// capacity, so a group of n samples costs O(n log n) instead of the O(n * bins) scan.
#include <algorithm>
#include <cstdint>
#include <vector>

namespace {

struct FirstFitTree {
  int cap_leaves = 1;
  std::vector<int> mx;  // max remaining capacity in the subtree
  explicit FirstFitTree(int n) {
    while (cap_leaves < n) cap_leaves <<= 1;
    mx.assign(2 * cap_leaves, 0);
  }
  void set(int i, int v) {
    int p = cap_leaves + i;
    mx[p] = v;
    for (p >>= 1; p >= 1; p >>= 1) mx[p] = std::max(mx[2 * p], mx[2 * p + 1]);
  }
  int get(int i) const { return mx[cap_leaves + i]; }
  // leftmost leaf with value >= need, or -1
  int find(int need) const {
    if (mx[1] < need) return -1;
    int p = 1;
    while (p < cap_leaves) p = (mx[2 * p] >= need) ? 2 * p : 2 * p + 1;
    return p - cap_leaves;
  }
};

}  // namespace

extern "C" {

// lengths[n] in sampler order -> bin_of[n] (global bin index, -1 for samples that do not fit a bin
// at all). Returns the number of bins.
int axb_pack_first_fit(const int32_t* lengths, int64_t n, int32_t capacity, int32_t bin_size,
                       int64_t group_size, int32_t* bin_of) {
  if (group_size <= 0) group_size = n > 0 ? n : 1;
  if (bin_size <= 0) bin_size = INT32_MAX;
  int32_t bins_total = 0;
  for (int64_t g0 = 0; g0 < n; g0 += group_size) {
    const int64_t g1 = std::min(n, g0 + group_size);
    const int gn = static_cast<int>(g1 - g0);
    FirstFitTree tree(gn);
    std::vector<int32_t> count;
    count.reserve(gn);
    int nbins = 0;
    for (int64_t i = g0; i < g1; ++i) {
      const int32_t len = lengths[i];
      if (len > capacity || len <= 0) {
        bin_of[i] = -1;
        continue;
      }
      int b = tree.find(len);
      if (b < 0 || b >= nbins) {
        b = nbins++;
        count.push_back(0);
        tree.set(b, capacity);
      }
      bin_of[i] = bins_total + b;
      const int rem = tree.get(b) - len;
      ++count[b];
      tree.set(b, count[b] >= bin_size ? 0 : rem);
    }
    bins_total += nbins;
  }
  return bins_total;
}

// order-preserving greedy fill: a bin is closed as soon as the next sample does not fit.
int axb_pack_sequential(const int32_t* lengths, int64_t n, int32_t capacity, int32_t bin_size,
                        int32_t* bin_of) {
  if (bin_size <= 0) bin_size = INT32_MAX;
  int32_t bin = -1, used = capacity + 1, cnt = 0;
  for (int64_t i = 0; i < n; ++i) {
    const int32_t len = lengths[i];
    if (len > capacity || len <= 0) {
      bin_of[i] = -1;
      continue;
    }
    if (used + len > capacity || cnt >= bin_size) {
      ++bin;
      used = 0;
      cnt = 0;
    }
    bin_of[i] = bin;
    used += len;
    ++cnt;
  }
  return bin + 1;
}

// Tile table for the varlen attention kernels: one int4 (doc_start, doc_len, tile_start, 0) per
// (document, tile of `tile_rows` rows). heavy_first = 1 emits the tiles with the largest
// tile_start first (most causal work for a q tile), 0 emits the smallest first (most work for a
// kv tile). Returns the number of tiles written (at most max_tiles).
int axb_build_attn_tiles(const int32_t* cu_seqlens, int32_t n_docs, int32_t tile_rows,
                         int32_t heavy_first, int32_t* out, int32_t max_tiles) {
  struct T {
    int32_t s, l, t;
  };
  std::vector<T> tiles;
  for (int d = 0; d < n_docs; ++d) {
    const int32_t s = cu_seqlens[d], l = cu_seqlens[d + 1] - cu_seqlens[d];
    for (int32_t t = 0; t < l; t += tile_rows) tiles.push_back({s, l, t});
  }
  if (heavy_first)
    std::stable_sort(tiles.begin(), tiles.end(), [](const T& a, const T& b) { return a.t > b.t; });
  else
    std::stable_sort(tiles.begin(), tiles.end(), [](const T& a, const T& b) {
      return (a.l - a.t) > (b.l - b.t);
    });
  const int n = std::min<int>(static_cast<int>(tiles.size()), max_tiles);
  for (int i = 0; i < n; ++i) {
    out[4 * i + 0] = tiles[i].s;
    out[4 * i + 1] = tiles[i].l;
    out[4 * i + 2] = tiles[i].t;
    out[4 * i + 3] = 0;
  }
  return n;
}

}  // extern "C"
