// Host-side data path in C++: offline bin packing of sequence lengths and assembly of packed rows.
//
// The packing strategies mirror chronicals_b200/data/sequence_packer.py (same bins, same order of items
// inside a bin), so either implementation can serve as the other's oracle.  The reference implements
// these in Python only (chronicals/data/sequence_packer.py:94-322); on a 148-SM GPU that consumes
// ~180 k tokens per second per device the Python packer becomes visible in the input pipeline, hence
// this native version.
//
// C ABI (ctypes):
//   cb_pack_bins(lengths, n, capacity, strategy, bin_of_item, slot_in_bin) -> number of bins (or <0)
//   cb_fill_rows(...)  copies token ids / labels of the packed items into row-major [rows, capacity]
//                      buffers (possibly pinned), writes position ids, sequence ids and cu_seqlens.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <numeric>
#include <queue>
#include <set>
#include <utility>
#include <vector>

namespace {

enum Strategy { FFD = 0, BFD = 1, BFD_HEAP = 2, SPFHP = 3, GREEDY = 4 };

// indices sorted by length; ties keep the original order (Python's sorted() is stable, and with
// reverse=True it keeps the original order among equal keys as well)
std::vector<int64_t> order_by_length(const int64_t* len, int64_t n, bool descending) {
  std::vector<int64_t> idx(n);
  std::iota(idx.begin(), idx.end(), 0);
  if (descending)
    std::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) { return len[a] > len[b]; });
  else
    std::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) { return len[a] < len[b]; });
  return idx;
}

struct Bins {
  std::vector<std::vector<int64_t>> items;
  std::vector<int64_t> used;
  int64_t open() {
    items.emplace_back();
    used.push_back(0);
    return static_cast<int64_t>(items.size()) - 1;
  }
  void add(int64_t b, int64_t i, int64_t L) {
    items[b].push_back(i);
    used[b] += L;
  }
};

void pack_ffd(const int64_t* len, int64_t n, int64_t cap, Bins& bins) {
  // first fit with a segment tree over remaining capacities: O(n log n) instead of the O(n * bins) scan
  const auto ord = order_by_length(len, n, true);
  int64_t leaves = 1;
  while (leaves < std::max<int64_t>(n, 1)) leaves <<= 1;
  std::vector<int64_t> tree(2 * leaves, 0);            // max remaining capacity in the subtree
  int64_t nb = 0;
  for (int64_t i : ord) {
    const int64_t L = std::min(len[i], cap);
    int64_t b;
    if (tree[1] >= L && nb > 0) {
      int64_t node = 1;
      while (node < leaves) node = tree[2 * node] >= L ? 2 * node : 2 * node + 1;
      b = node - leaves;
    } else {
      b = bins.open();
      nb = b + 1;
      tree[leaves + b] = cap;
    }
    bins.add(b, i, L);
    int64_t node = leaves + b;
    tree[node] = cap - bins.used[b];
    for (node >>= 1; node >= 1; node >>= 1) tree[node] = std::max(tree[2 * node], tree[2 * node + 1]);
  }
}

void pack_bfd(const int64_t* len, int64_t n, int64_t cap, Bins& bins) {
  // tightest bin that fits: ordered set of (remaining, bin index), lower_bound((L, -1))
  const auto ord = order_by_length(len, n, true);
  std::set<std::pair<int64_t, int64_t>> rem;
  for (int64_t i : ord) {
    const int64_t L = std::min(len[i], cap);
    auto it = rem.lower_bound({L, -1});
    int64_t b, r;
    if (it != rem.end()) {
      r = it->first;
      b = it->second;
      rem.erase(it);
    } else {
      b = bins.open();
      r = cap;
    }
    bins.add(b, i, L);
    rem.insert({r - L, b});
  }
}

void pack_bfd_heap(const int64_t* len, int64_t n, int64_t cap, Bins& bins) {
  // buckets keyed by exact remaining capacity; within a bucket the most recently inserted bin is reused
  const auto ord = order_by_length(len, n, true);
  std::map<int64_t, std::vector<int64_t>> buckets;
  for (int64_t i : ord) {
    const int64_t L = std::min(len[i], cap);
    auto it = buckets.lower_bound(L);
    int64_t b, r;
    if (it != buckets.end()) {
      r = it->first;
      b = it->second.back();
      it->second.pop_back();
      if (it->second.empty()) buckets.erase(it);
    } else {
      b = bins.open();
      r = cap;
    }
    bins.add(b, i, L);
    buckets[r - L].push_back(b);
  }
}

void pack_spfhp(const int64_t* len, int64_t n, int64_t cap, Bins& bins) {
  // longest first into the least-filled open bin when it fits (min-heap on (used, bin))
  const auto ord = order_by_length(len, n, true);
  using E = std::pair<int64_t, int64_t>;
  std::priority_queue<E, std::vector<E>, std::greater<E>> heap;
  for (int64_t i : ord) {
    const int64_t L = std::min(len[i], cap);
    if (!heap.empty() && heap.top().first + L <= cap) {
      const E top = heap.top();
      heap.pop();
      bins.add(top.second, i, L);
      heap.push({top.first + L, top.second});
    } else {
      const int64_t b = bins.open();
      bins.add(b, i, L);
      heap.push({L, b});
    }
  }
}

void pack_greedy(const int64_t* len, int64_t n, int64_t cap, Bins& bins) {
  const auto ord = order_by_length(len, n, false);
  int64_t cur = -1;
  for (int64_t i : ord) {
    const int64_t L = std::min(len[i], cap);
    if (cur < 0 || (bins.used[cur] + L > cap && !bins.items[cur].empty())) cur = bins.open();
    bins.add(cur, i, L);
  }
}

}  // namespace

extern "C" {

// bin_of_item[i] = bin of item i; slot_in_bin[i] = its position inside that bin.  Returns the bin count,
// -1 for a bad strategy, -2 for bad arguments.
long long cb_pack_bins(const long long* lengths, long long n, long long capacity, int strategy,
                       long long* bin_of_item, long long* slot_in_bin) {
  if (n < 0 || capacity <= 0 || (n > 0 && (!lengths || !bin_of_item || !slot_in_bin))) return -2;
  Bins bins;
  const int64_t* len = reinterpret_cast<const int64_t*>(lengths);
  switch (strategy) {
    case FFD: pack_ffd(len, n, capacity, bins); break;
    case BFD: pack_bfd(len, n, capacity, bins); break;
    case BFD_HEAP: pack_bfd_heap(len, n, capacity, bins); break;
    case SPFHP: pack_spfhp(len, n, capacity, bins); break;
    case GREEDY: pack_greedy(len, n, capacity, bins); break;
    default: return -1;
  }
  for (size_t b = 0; b < bins.items.size(); ++b)
    for (size_t s = 0; s < bins.items[b].size(); ++s) {
      bin_of_item[bins.items[b][s]] = static_cast<long long>(b);
      slot_in_bin[bins.items[b][s]] = static_cast<long long>(s);
    }
  return static_cast<long long>(bins.items.size());
}

// Assemble packed rows.  tokens/labels: concatenated items (labels may be null: labels = tokens);
// offsets[n + 1] delimit the items; row_items lists item indices row by row, row_starts[rows + 1]
// delimits the rows.  Outputs are [rows, capacity] int64 (row-major) except cu_seqlens, which is
// [rows, max_docs + 1] int32 padded with the row's token count, and n_docs[rows].
// Within a document the first label is masked (no target crosses a document boundary).
int cb_fill_rows(const long long* tokens, const long long* labels, const long long* offsets,
                 const long long* row_items, const long long* row_starts, long long rows, long long capacity,
                 long long pad_id, long long ignore_index, int mask_first_label, long long max_docs,
                 long long* out_ids, long long* out_pos, long long* out_labels, long long* out_seq_ids,
                 int* out_cu, int* out_ndocs) {
  if (rows < 0 || capacity <= 0 || max_docs <= 0) return -2;
  for (long long r = 0; r < rows; ++r) {
    long long* ids = out_ids + r * capacity;
    long long* pos = out_pos + r * capacity;
    long long* lab = out_labels + r * capacity;
    long long* sid = out_seq_ids + r * capacity;
    int* cu = out_cu + r * (max_docs + 1);
    long long fill = 0;
    long long doc = 0;
    cu[0] = 0;
    for (long long k = row_starts[r]; k < row_starts[r + 1]; ++k) {
      const long long it = row_items[k];
      long long L = offsets[it + 1] - offsets[it];
      L = std::min(L, capacity - fill);
      if (L <= 0 || doc >= max_docs) break;
      const long long* src = tokens + offsets[it];
      std::memcpy(ids + fill, src, sizeof(long long) * L);
      std::memcpy(lab + fill, labels ? labels + offsets[it] : src, sizeof(long long) * L);
      if (mask_first_label) lab[fill] = ignore_index;
      for (long long j = 0; j < L; ++j) {
        pos[fill + j] = j;
        sid[fill + j] = doc;
      }
      fill += L;
      ++doc;
      cu[doc] = static_cast<int>(fill);
    }
    for (long long j = fill; j < capacity; ++j) {
      ids[j] = pad_id;
      pos[j] = 0;
      lab[j] = ignore_index;
      sid[j] = -1;
    }
    for (long long d = doc + 1; d <= max_docs; ++d) cu[d] = static_cast<int>(fill);
    out_ndocs[r] = static_cast<int>(doc);
  }
  return 0;
}

}  // extern "C"
