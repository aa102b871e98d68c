// Host-side sequence packing: first-fit-decreasing bin packing of variable-length sequences into
// rows of a fixed width, and assembly of the flat static batch (tokens, position ids, cu_seqlens).
//
// Same packing rule and output order as the reference's Python PackingCollator
// (src/nanoplm/pretraining/collator.py:250-327,405-458): sequences sorted by length (descending,
// stable), each placed in the first row with room; output lists rows in order, sequences in the
// order they were placed. First-fit is answered by a max segment tree over the rows' free space,
// so packing n sequences costs O(n log n) instead of O(n * rows).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

namespace {

struct FirstFitTree {
  int size;
  std::vector<int> mx;
  explicit FirstFitTree(int n, int width) {
    size = 1;
    while (size < n) size <<= 1;
    mx.assign(2 * size, 0);
    for (int i = 0; i < n; ++i) mx[size + i] = width;
    for (int i = size - 1; i >= 1; --i) mx[i] = std::max(mx[2 * i], mx[2 * i + 1]);
  }
  // index of the first row with free >= need (always exists: there are as many rows as sequences)
  int place(int need) {
    int i = 1;
    while (i < size) i = (mx[2 * i] >= need) ? 2 * i : 2 * i + 1;
    mx[i] -= need;
    const int row = i - size;
    for (i >>= 1; i >= 1; i >>= 1) mx[i] = std::max(mx[2 * i], mx[2 * i + 1]);
    return row;
  }
};

}  // namespace

extern "C" {

// lens[n] (values > width are truncated to width). Outputs:
//   order[n]   : sequence indices in output order (row by row, placement order inside a row)
//   row_of[n]  : row of order[i]
//   start_of[n]: column where order[i] starts inside its row
// Returns the number of rows used.
int nplm_pack_ffd(const int32_t* lens, int n, int width, int32_t* order, int32_t* row_of,
                  int32_t* start_of) {
  if (n <= 0) return 0;
  std::vector<int> idx(n);
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return lens[a] > lens[b]; });
  FirstFitTree tree(n, width);
  std::vector<int> row(n), fill(n, 0), start(n);
  int n_rows = 0;
  for (int k = 0; k < n; ++k) {
    const int len = std::min<int>(lens[idx[k]], width);
    const int r = tree.place(len);
    row[k] = r;
    start[k] = fill[r];
    fill[r] += len;
    n_rows = std::max(n_rows, r + 1);
  }
  // stable order by row keeps placement order inside each row
  std::vector<int> pos(n);
  std::iota(pos.begin(), pos.end(), 0);
  std::stable_sort(pos.begin(), pos.end(), [&](int a, int b) { return row[a] < row[b]; });
  for (int i = 0; i < n; ++i) {
    order[i] = idx[pos[i]];
    row_of[i] = row[pos[i]];
    start_of[i] = start[pos[i]];
  }
  return n_rows;
}

// Copies the sequences (concatenated in `tokens`, sequence i at offsets[i]..offsets[i+1]) into the
// flat layout given by order[0..n_keep): flat_ids, position ids and cu_seqlens (n_keep+1 entries).
// Sequences longer than width are truncated. Returns the number of tokens written.
int64_t nplm_pack_flatten(const uint8_t* tokens, const int64_t* offsets, const int32_t* order,
                          int n_keep, int width, int64_t* flat_ids, int32_t* pos_ids,
                          int32_t* cu_seqlens) {
  int64_t t = 0;
  cu_seqlens[0] = 0;
  for (int i = 0; i < n_keep; ++i) {
    const int s = order[i];
    int64_t len = offsets[s + 1] - offsets[s];
    if (len > width) len = width;
    const uint8_t* src = tokens + offsets[s];
    for (int64_t j = 0; j < len; ++j) {
      flat_ids[t + j] = src[j];
      pos_ids[t + j] = static_cast<int32_t>(j);
    }
    t += len;
    cu_seqlens[i + 1] = static_cast<int32_t>(t);
  }
  return t;
}

// Deals n = n_bins * per_bin sequences into n_bins bins of exactly per_bin sequences each so that
// the bins' costs are as equal as the greedy rule allows: sequences in order of decreasing cost,
// each to the cheapest bin that still has room (longest-processing-time rule with a cardinality
// limit). cost(len) = len + quad * len^2: the linear part stands for the per-token work of a
// training step, the quadratic part for full attention inside a sequence. Ties go to the lowest
// bin index, so every rank that runs this on the same lengths gets the same answer.
//   bin_of[i]  : bin of sequence i
//   bin_cost[b]: total cost of bin b
// Returns 0, or -1 when n is not n_bins * per_bin.
int nplm_balance_bins(const int32_t* lens, int n, int n_bins, int per_bin, double quad, int32_t* bin_of,
                      double* bin_cost) {
  if (n_bins <= 0 || per_bin <= 0 || n != n_bins * per_bin) return -1;
  std::vector<double> cost(n);
  for (int i = 0; i < n; ++i) cost[i] = lens[i] + quad * static_cast<double>(lens[i]) * lens[i];
  std::vector<int> idx(n);
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return cost[a] > cost[b]; });
  std::vector<int> fill(n_bins, 0);
  for (int b = 0; b < n_bins; ++b) bin_cost[b] = 0.0;
  // n_bins is small (ranks x micro-batches of one optimizer step): a linear scan per sequence is
  // cheaper than keeping a heap consistent with the cardinality limit
  for (int k = 0; k < n; ++k) {
    int best = -1;
    for (int b = 0; b < n_bins; ++b) {
      if (fill[b] >= per_bin) continue;
      if (best < 0 || bin_cost[b] < bin_cost[best]) best = b;
    }
    bin_of[idx[k]] = best;
    bin_cost[best] += cost[idx[k]];
    ++fill[best];
  }
  return 0;
}

}  // extern "C"
