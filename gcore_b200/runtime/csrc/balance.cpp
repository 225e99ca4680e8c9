// Host-side combinatorial helpers used every step by the trainer: sequence-length balanced k-way partitioning
// (Karmarkar-Karp largest differencing, as in gpatch_v4/core/seqlen_balancing.py:7-173), first-fit-decreasing
// packing for token-budget micro-batches, and sequential size-capped bucketing (gradient / weight-resync buckets).
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <queue>
#include <vector>

#define RT_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct KKState {
  // k partial sets, kept sorted by descending sum
  std::vector<int64_t> sums;
  std::vector<std::vector<int>> items;
  int64_t spread() const { return sums.front() - sums.back(); }
};

struct KKCmp {
  bool operator()(const KKState* a, const KKState* b) const {
    if (a->spread() != b->spread()) return a->spread() < b->spread();
    return a->sums.front() < b->sums.front();
  }
};

void sort_state(KKState& s) {
  std::vector<int> idx(s.sums.size());
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return s.sums[a] > s.sums[b]; });
  KKState t;
  for (int i : idx) {
    t.sums.push_back(s.sums[i]);
    t.items.push_back(std::move(s.items[i]));
  }
  s = std::move(t);
}

}  // namespace

// assign[i] in [0, k).  equal_size != 0 requires n % k == 0 and gives every part n / k items.
RT_EXPORT int gkrt_kk_partition(const int64_t* lens, int n, int k, int equal_size, int* assign) {
  if (k <= 0 || n < 0) return -1;
  if (equal_size && n % k) return -2;
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lens[a] > lens[b]; });
  std::vector<KKState*> owned;
  std::priority_queue<KKState*, std::vector<KKState*>, KKCmp> heap;
  if (equal_size) {
    // seed states with k items each (one per slot) so that every merge keeps part sizes equal
    for (int base = 0; base < n; base += k) {
      auto* s = new KKState();
      for (int j = 0; j < k; ++j) {
        s->sums.push_back(lens[order[base + j]]);
        s->items.push_back({order[base + j]});
      }
      sort_state(*s);
      owned.push_back(s);
      heap.push(s);
    }
  } else {
    for (int i = 0; i < n; ++i) {
      auto* s = new KKState();
      s->sums.assign(k, 0);
      s->items.assign(k, {});
      s->sums[0] = lens[order[i]];
      s->items[0] = {order[i]};
      owned.push_back(s);
      heap.push(s);
    }
  }
  if (heap.empty()) return 0;
  while (heap.size() > 1) {
    KKState* a = heap.top(); heap.pop();
    KKState* b = heap.top(); heap.pop();
    // largest of a with smallest of b
    for (int j = 0; j < k; ++j) {
      a->sums[j] += b->sums[k - 1 - j];
      auto& dst = a->items[j];
      auto& src = b->items[k - 1 - j];
      dst.insert(dst.end(), src.begin(), src.end());
    }
    sort_state(*a);
    heap.push(a);
  }
  KKState* fin = heap.top();
  for (int j = 0; j < k; ++j)
    for (int it : fin->items[j]) assign[it] = j;
  for (auto* s : owned) delete s;
  return 0;
}

// First-fit decreasing: bins of at most `capacity` tokens (a single longer item gets its own bin).
// Returns the number of bins; bin_of[i] is item i's bin.
RT_EXPORT int gkrt_ffd_pack(const int64_t* lens, int n, int64_t capacity, int* bin_of) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lens[a] > lens[b]; });
  std::vector<int64_t> load;
  for (int i : order) {
    int chosen = -1;
    for (size_t b = 0; b < load.size(); ++b) {
      if (load[b] + lens[i] <= capacity) { chosen = static_cast<int>(b); break; }
    }
    if (chosen < 0) {
      chosen = static_cast<int>(load.size());
      load.push_back(0);
    }
    load[chosen] += lens[i];
    bin_of[i] = chosen;
  }
  return static_cast<int>(load.size());
}

// Sequential buckets in the given order, each at most `cap` bytes (an oversized item is alone in its bucket).
RT_EXPORT int gkrt_plan_buckets(const int64_t* sizes, int n, int64_t cap, int* bucket_of) {
  int b = 0;
  int64_t cur = 0;
  for (int i = 0; i < n; ++i) {
    if (cur > 0 && cur + sizes[i] > cap) {
      ++b;
      cur = 0;
    }
    bucket_of[i] = b;
    cur += sizes[i];
  }
  return n ? b + 1 : 0;
}
