// Token-sequence alignment for reward redistribution: longest common subsequence of two id sequences with the
// O((N + M) * D) greedy algorithm of Myers (1986); D = number of differences, small when one sequence is the other
// after a decode -> re-encode round trip.  The furthest-reaching endpoints of every edit distance are kept (one
// array of 2d + 1 ints per d), and the matched index pairs are read off by walking them backwards.
#include <cstdint>
#include <vector>

#define RT_EXPORT extern "C" __attribute__((visibility("default")))

// Writes up to `cap` matched pairs (a_idx[i], b_idx[i]), increasing in both; returns the LCS length, or -1 when the
// edit distance exceeds `max_d` (the caller then falls back to treating the whole span as one differing region).
RT_EXPORT int gkrt_lcs_match(const int64_t* a, int n, const int64_t* b, int m, int max_d, int* a_idx, int* b_idx,
                             int cap) {
  if (n == 0 || m == 0) return 0;
  const int lim = max_d < n + m ? max_d : n + m;
  std::vector<std::vector<int>> trace;  // trace[d][k + d] = furthest x on diagonal k after d edits
  std::vector<int> v(2 * lim + 3, 0);
  const int off = lim + 1;
  int found_d = -1;
  for (int d = 0; d <= lim && found_d < 0; ++d) {
    for (int k = -d; k <= d; k += 2) {
      int x;
      if (k == -d || (k != d && v[off + k - 1] < v[off + k + 1])) x = v[off + k + 1];  // step down (insert from b)
      else x = v[off + k - 1] + 1;                                                      // step right (delete from a)
      int y = x - k;
      while (x < n && y < m && a[x] == b[y]) { ++x; ++y; }
      v[off + k] = x;
      if (x >= n && y >= m) { found_d = d; break; }
    }
    std::vector<int> snap(2 * d + 1);
    for (int k = -d; k <= d; ++k) snap[k + d] = v[off + k];
    trace.push_back(std::move(snap));
  }
  if (found_d < 0) return -1;
  // backtrack
  std::vector<int> ra, rb;
  int x = n, y = m;
  for (int d = found_d; d > 0; --d) {
    const int k = x - y;
    const std::vector<int>& prev = trace[d - 1];  // diagonals -(d-1) .. (d-1)
    auto pv = [&](int kk) { return prev[kk + (d - 1)]; };
    int pk;
    if (k == -d || (k != d && pv(k - 1) < pv(k + 1))) pk = k + 1; else pk = k - 1;
    const int px = pv(pk), py = px - pk;
    // the snake of this step runs from (sx, sy) to (x, y)
    const int sx = pk == k + 1 ? px : px + 1;
    const int sy = sx - k;
    while (x > sx && y > sy) { --x; --y; ra.push_back(x); rb.push_back(y); }
    x = px; y = py;
  }
  while (x > 0 && y > 0) { --x; --y; ra.push_back(x); rb.push_back(y); }  // the d = 0 snake
  const int len = static_cast<int>(ra.size());
  for (int i = 0; i < len && i < cap; ++i) {
    a_idx[i] = ra[len - 1 - i];
    b_idx[i] = rb[len - 1 - i];
  }
  return len;
}
