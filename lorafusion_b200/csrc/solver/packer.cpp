// Native core of the multi-adapter microbatch solver and the 1F1B pipeline simulator.
//
// Bin packing with per-adapter padding: a microbatch ("bin") holds samples of several
// adapters; the tokens of each adapter inside a bin are padded up to a multiple of the
// kernels' M tile, and the padded sum must not exceed the capacity.
//   lf_pack_ffd    first-fit-decreasing
//   lf_pack_exact  two-phase branch and bound: (1) fewest bins, (2) with that bin count,
//                  the emptiest possible smallest bin (so the leftover bin merges easily
//                  with the next group's microbatches).  Takes a time limit and returns the
//                  best packing found; stands in for the two CBC MILPs of the reference
//                  (lorafusion/solver/proposed_solver.py:1438-1959).
//   lf_simulate_1f1b  event-driven timing of a non-interleaved 1F1B pipeline schedule
//                  (benchmarks_paper/imbalance_simulator/main_random_data.py:71-383).
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

namespace {

using Clock = std::chrono::steady_clock;

struct Problem {
  int n = 0;
  int num_adapters = 0;
  long long capacity = 0;
  long long pad = 1;
  std::vector<long long> len;   // sorted descending
  std::vector<int> adapter;
  std::vector<int> order;       // original index of sorted item
};

inline long long pad_up(long long v, long long m) { return v == 0 ? 0 : ((v + m - 1) / m) * m; }

struct Bin {
  std::vector<long long> per_adapter;  // raw tokens per adapter
  long long padded = 0;
};

inline long long padded_after(const Bin& b, int a, long long add, long long pad) {
  const long long old = pad_up(b.per_adapter[a], pad);
  const long long neu = pad_up(b.per_adapter[a] + add, pad);
  return b.padded - old + neu;
}

Problem make_problem(const long long* lengths, const int* adapters, int n, int num_adapters,
                     long long capacity, long long pad) {
  Problem p;
  p.n = n;
  p.num_adapters = num_adapters;
  p.capacity = capacity;
  p.pad = pad < 1 ? 1 : pad;
  p.order.resize(n);
  std::iota(p.order.begin(), p.order.end(), 0);
  std::stable_sort(p.order.begin(), p.order.end(),
                   [&](int x, int y) { return lengths[x] > lengths[y]; });
  p.len.resize(n);
  p.adapter.resize(n);
  for (int i = 0; i < n; ++i) {
    p.len[i] = lengths[p.order[i]];
    p.adapter[i] = adapters[p.order[i]];
  }
  return p;
}

// FFD on the sorted problem; returns the number of bins, assignment indexed by sorted item.
int ffd(const Problem& p, std::vector<int>& assign) {
  std::vector<Bin> bins;
  assign.assign(p.n, -1);
  for (int i = 0; i < p.n; ++i) {
    int placed = -1;
    for (size_t b = 0; b < bins.size(); ++b) {
      if (padded_after(bins[b], p.adapter[i], p.len[i], p.pad) <= p.capacity) {
        placed = int(b);
        break;
      }
    }
    if (placed < 0) {
      Bin nb;
      nb.per_adapter.assign(p.num_adapters, 0);
      bins.push_back(nb);
      placed = int(bins.size()) - 1;
    }
    Bin& b = bins[placed];
    b.padded = padded_after(b, p.adapter[i], p.len[i], p.pad);
    b.per_adapter[p.adapter[i]] += p.len[i];
    assign[i] = placed;
  }
  return int(bins.size());
}

struct Search {
  const Problem& p;
  Clock::time_point deadline;
  bool timed_out = false;
  long long nodes = 0;

  // phase 1
  int best_bins;
  std::vector<int> best_assign;
  int lower_bound_bins;

  // phase 2
  int fixed_bins = 0;
  long long best_min_load = 0;
  long long min_load_bound = 0;
  bool phase2_done = false;

  std::vector<Bin> bins;
  std::vector<int> assign;
  std::vector<long long> suffix_sum;

  explicit Search(const Problem& prob) : p(prob) {}

  bool out_of_time() {
    if ((++nodes & 0x3ff) == 0 && Clock::now() > deadline) timed_out = true;
    return timed_out;
  }

  void place(int i, int b) {
    Bin& bin = bins[b];
    bin.padded = padded_after(bin, p.adapter[i], p.len[i], p.pad);
    bin.per_adapter[p.adapter[i]] += p.len[i];
    assign[i] = b;
  }
  void unplace(int i, int b) {
    Bin& bin = bins[b];
    bin.per_adapter[p.adapter[i]] -= p.len[i];
    long long tot = 0;
    for (long long v : bin.per_adapter) tot += pad_up(v, p.pad);
    bin.padded = tot;
    assign[i] = -1;
  }

  // ---- phase 1: minimise the number of bins -------------------------------------
  void dfs_bins(int i, int used) {
    if (best_bins == lower_bound_bins || out_of_time()) return;
    if (used >= best_bins) return;
    if (i == p.n) {
      best_bins = used;
      best_assign = assign;
      return;
    }
    // remaining volume bound
    long long free_space = 0;
    for (int b = 0; b < used; ++b) free_space += p.capacity - bins[b].padded;
    const long long need = suffix_sum[i] - free_space;
    if (need > 0) {
      const int extra = int((need + p.capacity - 1) / p.capacity);
      if (used + extra >= best_bins) return;
    }
    for (int b = 0; b < used; ++b) {
      // bins with identical per-adapter loads are interchangeable: try only the first
      bool dup = false;
      for (int c = 0; c < b && !dup; ++c) dup = bins[c].per_adapter == bins[b].per_adapter;
      if (dup) continue;
      if (padded_after(bins[b], p.adapter[i], p.len[i], p.pad) > p.capacity) continue;
      place(i, b);
      dfs_bins(i + 1, used);
      unplace(i, b);
      if (best_bins == lower_bound_bins || timed_out) return;
    }
    if (used + 1 < best_bins) {
      place(i, used);
      dfs_bins(i + 1, used + 1);
      unplace(i, used);
    }
  }

  // ---- phase 2: with `fixed_bins` bins, minimise the smallest padded load ---------
  void dfs_minload(int i, int used) {
    if (phase2_done || out_of_time()) return;
    if (i == p.n) {
      if (used != fixed_bins) return;
      long long mn = bins[0].padded;
      for (int b = 1; b < used; ++b) mn = std::min(mn, bins[b].padded);
      if (mn < best_min_load) {
        best_min_load = mn;
        best_assign = assign;
        if (best_min_load <= min_load_bound) phase2_done = true;
      }
      return;
    }
    // the smallest bin can never drop below what must spill out of the other bins
    for (int b = 0; b < used; ++b) {
      if (padded_after(bins[b], p.adapter[i], p.len[i], p.pad) > p.capacity) continue;
      place(i, b);
      dfs_minload(i + 1, used);
      unplace(i, b);
      if (phase2_done || timed_out) return;
    }
    if (used < fixed_bins) {
      place(i, used);
      dfs_minload(i + 1, used + 1);
      unplace(i, used);
    }
  }
};

}  // namespace

extern "C" {

// out_bin[i] = bin index of sample i (original order).  Returns the number of bins.
int lf_pack_ffd(const long long* lengths, const int* adapters, int n, int num_adapters,
                long long capacity, long long pad_multiple, int* out_bin) {
  if (n <= 0) return 0;
  Problem p = make_problem(lengths, adapters, n, num_adapters, capacity, pad_multiple);
  std::vector<int> assign;
  const int nb = ffd(p, assign);
  for (int i = 0; i < n; ++i) out_bin[p.order[i]] = assign[i];
  return nb;
}

// status bits written to *out_status: 1 = phase 1 proven optimal, 2 = phase 2 reached its
// lower bound, 4 = time limit hit.  Returns the number of bins.
int lf_pack_exact(const long long* lengths, const int* adapters, int n, int num_adapters,
                  long long capacity, long long pad_multiple, double time_limit_s, int* out_bin,
                  int* out_status) {
  if (out_status) *out_status = 0;
  if (n <= 0) return 0;
  Problem p = make_problem(lengths, adapters, n, num_adapters, capacity, pad_multiple);
  Search s(p);
  s.deadline = Clock::now() + std::chrono::microseconds((long long)(time_limit_s * 0.5e6));
  s.suffix_sum.assign(n + 1, 0);
  for (int i = n - 1; i >= 0; --i) s.suffix_sum[i] = s.suffix_sum[i + 1] + p.len[i];
  std::vector<int> greedy;
  s.best_bins = ffd(p, greedy);
  s.best_assign = greedy;
  s.lower_bound_bins = int((s.suffix_sum[0] + capacity - 1) / capacity);
  if (s.lower_bound_bins < 1) s.lower_bound_bins = 1;
  s.bins.assign(n, Bin());
  for (auto& b : s.bins) b.per_adapter.assign(num_adapters, 0);
  s.assign.assign(n, -1);
  int status = 0;
  if (s.best_bins > s.lower_bound_bins) s.dfs_bins(0, 0);
  if (!s.timed_out) status |= 1;

  // phase 2
  const int B = s.best_bins;
  s.fixed_bins = B;
  {
    std::vector<long long> load(B, 0);
    std::vector<std::vector<long long>> per(B, std::vector<long long>(num_adapters, 0));
    for (int i = 0; i < n; ++i) per[s.best_assign[i]][p.adapter[i]] += p.len[i];
    long long mn = -1;
    for (int b = 0; b < B; ++b) {
      for (long long v : per[b]) load[b] += pad_up(v, p.pad);
      mn = (mn < 0 || load[b] < mn) ? load[b] : mn;
    }
    s.best_min_load = mn;
  }
  s.min_load_bound = std::max<long long>(s.suffix_sum[0] - (long long)(B - 1) * capacity, 0);
  s.min_load_bound = std::min(s.min_load_bound, s.best_min_load);
  if (B > 1 && s.best_min_load > s.min_load_bound) {
    const bool p1_timed_out = s.timed_out;
    s.timed_out = false;
    s.deadline = Clock::now() + std::chrono::microseconds((long long)(time_limit_s * 0.5e6));
    for (auto& b : s.bins) {
      std::fill(b.per_adapter.begin(), b.per_adapter.end(), 0);
      b.padded = 0;
    }
    std::fill(s.assign.begin(), s.assign.end(), -1);
    s.dfs_minload(0, 0);
    if (s.phase2_done || !s.timed_out) status |= 2;
    if (s.timed_out || p1_timed_out) status |= 4;
  } else {
    status |= 2;
    if (s.timed_out) status |= 4;
  }
  for (int i = 0; i < n; ++i) out_bin[p.order[i]] = s.best_assign[i];
  if (out_status) *out_status = status;
  return B;
}

// Non-interleaved 1F1B.  fwd/bwd: [M][S] row-major durations.  Outputs (each [M][S]):
// forward start/end and backward start/end times.  Returns the makespan.
double lf_simulate_1f1b(const double* fwd, const double* bwd, int M, int S, double* f_start,
                        double* f_end, double* b_start, double* b_end, double* out_bubble_ratio) {
  if (M <= 0 || S <= 0) return 0.0;
  auto at = [S](int m, int s) { return m * S + s; };
  // per-stage op order: warm-up forwards, steady 1F1B, cool-down backwards
  std::vector<std::vector<std::pair<int, int>>> ops(S);  // (is_backward, microbatch)
  for (int s = 0; s < S; ++s) {
    const int warm = std::min(S - s - 1, M);
    int f = 0, b = 0;
    for (int i = 0; i < warm; ++i) ops[s].push_back({0, f++});
    while (f < M) {
      ops[s].push_back({0, f++});
      ops[s].push_back({1, b++});
    }
    while (b < M) ops[s].push_back({1, b++});
  }
  std::vector<size_t> next(S, 0);
  std::vector<double> free_at(S, 0.0);
  std::vector<char> f_done(M * S, 0), b_done(M * S, 0);
  size_t remaining = 0;
  for (int s = 0; s < S; ++s) remaining += ops[s].size();
  while (remaining > 0) {
    bool progressed = false;
    for (int s = 0; s < S; ++s) {
      while (next[s] < ops[s].size()) {
        const auto [is_b, m] = ops[s][next[s]];
        double ready;
        if (!is_b) {
          if (s > 0 && !f_done[at(m, s - 1)]) break;
          ready = s > 0 ? f_end[at(m, s - 1)] : 0.0;
        } else {
          if (s < S - 1 && !b_done[at(m, s + 1)]) break;
          if (!f_done[at(m, s)]) break;
          ready = s < S - 1 ? b_end[at(m, s + 1)] : f_end[at(m, s)];
        }
        const double start = std::max(ready, free_at[s]);
        if (!is_b) {
          f_start[at(m, s)] = start;
          f_end[at(m, s)] = start + fwd[at(m, s)];
          free_at[s] = f_end[at(m, s)];
          f_done[at(m, s)] = 1;
        } else {
          b_start[at(m, s)] = start;
          b_end[at(m, s)] = start + bwd[at(m, s)];
          free_at[s] = b_end[at(m, s)];
          b_done[at(m, s)] = 1;
        }
        ++next[s];
        --remaining;
        progressed = true;
      }
    }
    if (!progressed) return -1.0;  // inconsistent schedule (cannot happen for 1F1B)
  }
  double makespan = 0.0, busy = 0.0;
  for (int s = 0; s < S; ++s) makespan = std::max(makespan, free_at[s]);
  for (int i = 0; i < M * S; ++i) busy += fwd[i] + bwd[i];
  if (out_bubble_ratio) *out_bubble_ratio = makespan > 0 ? 1.0 - busy / (makespan * S) : 0.0;
  return makespan;
}

}  // extern "C"
