// Byte-pair merges over integer symbol sequences: training (learn the merge table) and encoding (apply it).
//
// The action tokenizer turns every action chunk into a sequence of quantised DCT coefficients and compresses it with
// merges learned on a corpus of such sequences.  Training on a million chunks and encoding every batch of the data
// loader are host-side hot loops; both are linear-ish here:
//
//  * training keeps the corpus as one doubly linked list per sequence, a count per adjacent pair, a lazy max-heap of
//    (count, pair) and, per pair, the list of positions where it was seen.  One merge touches only the occurrences of
//    the chosen pair and their neighbours.  Ties are broken by the smaller left symbol, then the smaller right symbol,
//    and occurrences are merged left to right without overlap ("a a a" -> "N a"), so the table is a pure function of
//    the corpus;
//  * encoding walks each sequence with a min-heap of (rank, position): a pair that contains a merged symbol was
//    learned after that symbol, so new neighbours always rank later and one pass in heap order equals "apply the
//    best-ranked pair everywhere, then look again".  Sequences are independent and are spread over threads.
//
// Plain C entry points (loaded with ctypes), no allocation visible to the caller beyond its own buffers.
#include <algorithm>
#include <cstdint>
#include <queue>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

using Pair = uint64_t;
inline Pair key(int32_t a, int32_t b) { return (uint64_t(uint32_t(a)) << 32) | uint32_t(b); }
inline int32_t left(Pair p) { return int32_t(p >> 32); }
inline int32_t right(Pair p) { return int32_t(p & 0xffffffffu); }

struct HeapEntry {
  int64_t count;
  Pair pair;
};
struct Worse {  // priority_queue keeps the "largest": more frequent first, then smaller left, then smaller right
  bool operator()(const HeapEntry& x, const HeapEntry& y) const {
    if (x.count != y.count) return x.count < y.count;
    return x.pair > y.pair;
  }
};

struct PairInfo {
  int64_t count = 0;
  std::vector<int64_t> where;  // positions of the left symbol; may hold stale or repeated entries
};

}  // namespace

// symbols: all sequences back to back; offsets[n_seq + 1].  merges_out holds 2 * (vocab_size - base) ints.
// Returns the number of merges learned (stops early when the best pair occurs fewer than min_count times).
extern "C" int32_t otb_bpe_train(const int32_t* symbols, const int64_t* offsets, int64_t n_seq, int32_t base,
                                 int32_t vocab_size, int32_t min_count, int32_t* merges_out) {
  if (!symbols || !offsets || !merges_out || n_seq < 0 || vocab_size < base) return -1;
  const int64_t total = offsets[n_seq];
  std::vector<int32_t> sym(symbols, symbols + total);
  std::vector<int64_t> prev(total, -1), next(total, -1);
  std::unordered_map<Pair, PairInfo> pairs;
  pairs.reserve(size_t(total / 4 + 16));
  for (int64_t s = 0; s < n_seq; ++s) {
    for (int64_t i = offsets[s]; i < offsets[s + 1]; ++i) {
      if (i > offsets[s]) prev[i] = i - 1;
      if (i + 1 < offsets[s + 1]) {
        next[i] = i + 1;
        PairInfo& p = pairs[key(sym[i], sym[i + 1])];
        ++p.count;
        p.where.push_back(i);
      }
    }
  }
  std::priority_queue<HeapEntry, std::vector<HeapEntry>, Worse> heap;
  for (auto& kv : pairs) heap.push({kv.second.count, kv.first});

  auto bump = [&](int32_t a, int32_t b, int64_t pos, int64_t delta) {
    PairInfo& p = pairs[key(a, b)];
    p.count += delta;
    if (delta > 0) {
      p.where.push_back(pos);
      heap.push({p.count, key(a, b)});
    }
  };

  int32_t learned = 0;
  while (base + learned < vocab_size && !heap.empty()) {
    const HeapEntry top = heap.top();
    heap.pop();
    auto it = pairs.find(top.pair);
    const int64_t actual = it == pairs.end() ? 0 : it->second.count;
    if (actual != top.count) {  // stale: put the truth back and look again
      if (actual > 0) heap.push({actual, top.pair});
      continue;
    }
    if (actual < min_count) break;
    const int32_t a = left(top.pair), b = right(top.pair), fresh = base + learned;
    merges_out[2 * learned] = a;
    merges_out[2 * learned + 1] = b;
    ++learned;
    std::vector<int64_t> where;
    where.swap(it->second.where);
    std::sort(where.begin(), where.end());
    where.erase(std::unique(where.begin(), where.end()), where.end());
    for (int64_t pos : where) {
      if (sym[pos] != a) continue;
      const int64_t nx = next[pos];
      if (nx < 0 || sym[nx] != b) continue;
      const int64_t pv = prev[pos], nn = next[nx];
      bump(a, b, pos, -1);
      if (pv >= 0) bump(sym[pv], a, pv, -1);
      if (nn >= 0) bump(b, sym[nn], nx, -1);
      sym[pos] = fresh;
      sym[nx] = -1;  // unlinked
      next[pos] = nn;
      if (nn >= 0) prev[nn] = pos;
      if (pv >= 0) bump(sym[pv], fresh, pv, +1);
      if (nn >= 0) bump(fresh, sym[nn], pos, +1);
    }
  }
  return learned;
}

namespace {

void encode_range(const int32_t* symbols, const int64_t* offsets, int64_t lo, int64_t hi,
                  const std::unordered_map<Pair, int32_t>& rank, int32_t base, int32_t* out, int64_t* out_len) {
  using Item = std::pair<int32_t, int64_t>;  // (rank, position of the left symbol), smallest first
  std::vector<int32_t> sym;
  std::vector<int64_t> prev, next;
  for (int64_t s = lo; s < hi; ++s) {
    const int64_t n = offsets[s + 1] - offsets[s];
    sym.assign(symbols + offsets[s], symbols + offsets[s + 1]);
    prev.resize(n);
    next.resize(n);
    std::priority_queue<Item, std::vector<Item>, std::greater<Item>> heap;
    for (int64_t i = 0; i < n; ++i) {
      prev[i] = i - 1;
      next[i] = i + 1 < n ? i + 1 : -1;
      if (i + 1 < n) {
        auto it = rank.find(key(sym[i], sym[i + 1]));
        if (it != rank.end()) heap.push({it->second, i});
      }
    }
    while (!heap.empty()) {
      const Item top = heap.top();
      heap.pop();
      const int64_t pos = top.second;
      if (sym[pos] < 0) continue;
      const int64_t nx = next[pos];
      if (nx < 0) continue;
      auto it = rank.find(key(sym[pos], sym[nx]));
      if (it == rank.end() || it->second != top.first) continue;  // the pair at this position changed since
      const int64_t pv = prev[pos], nn = next[nx];
      sym[pos] = base + top.first;
      sym[nx] = -1;
      next[pos] = nn;
      if (nn >= 0) prev[nn] = pos;
      if (pv >= 0) {
        auto l = rank.find(key(sym[pv], sym[pos]));
        if (l != rank.end()) heap.push({l->second, pv});
      }
      if (nn >= 0) {
        auto r = rank.find(key(sym[pos], sym[nn]));
        if (r != rank.end()) heap.push({r->second, pos});
      }
    }
    int64_t k = 0;
    int32_t* dst = out + offsets[s];
    for (int64_t i = 0; i < n; ++i)
      if (sym[i] >= 0) dst[k++] = sym[i];
    out_len[s] = k;
  }
}

}  // namespace

// out has the size of symbols; sequence s is written at out + offsets[s] with out_len[s] entries.
extern "C" int32_t otb_bpe_encode(const int32_t* symbols, const int64_t* offsets, int64_t n_seq, const int32_t* merges,
                                  int32_t n_merges, int32_t base, int32_t* out, int64_t* out_len, int32_t n_threads) {
  if (!symbols || !offsets || !out || !out_len || n_seq < 0 || n_merges < 0 || (n_merges > 0 && !merges)) return -1;
  std::unordered_map<Pair, int32_t> rank;
  rank.reserve(size_t(n_merges) * 2 + 16);
  for (int32_t r = 0; r < n_merges; ++r) rank.emplace(key(merges[2 * r], merges[2 * r + 1]), r);  // first wins
  const int64_t workers = std::max<int64_t>(1, std::min<int64_t>(n_threads, n_seq));
  if (workers == 1) {
    encode_range(symbols, offsets, 0, n_seq, rank, base, out, out_len);
    return 0;
  }
  std::vector<std::thread> pool;
  const int64_t per = (n_seq + workers - 1) / workers;
  for (int64_t w = 0; w < workers; ++w) {
    const int64_t lo = w * per, hi = std::min(n_seq, lo + per);
    if (lo >= hi) break;
    pool.emplace_back(encode_range, symbols, offsets, lo, hi, std::cref(rank), base, out, out_len);
  }
  for (auto& t : pool) t.join();
  return 0;
}
