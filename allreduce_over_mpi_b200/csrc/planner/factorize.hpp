// Tree-shape candidate enumeration for FlexTree.
//
// A tree shape is the list of per-level widths, bottom level first; the product of
// the widths is the number of tree ranks.  This header answers "which shapes exist
// for n ranks": every ordered factorisation of n into factors >= 2, the two flat
// sentinels 1*n and n*1, and the "+1 / -1" neighbours used for lonely layouts.
//
// Parity with the reference tool set (paths relative to the reference project):
//   cost_model/GetWidth.h:10-47        -> candidate_shapes()
//   cost_model/GetWidth.h:51-227       -> candidate_shapes_legacy()
//   cost_model/GetPrimeFactor.h:5-19   -> prime_factors()
//   cost_model/IsPrimeNumber.h:4-21    -> is_prime() / is_prime_loose()
//   cost_model/ChooseWidth.h:8-38      -> choose_width()
//   cost_model/PrintTreeStructure.h    -> shape_to_string()
//   topo_count/factor_count.py:1-15    -> count_ordered_factorizations()
//
// Everything here is re-entrant (no file-scope state) and pure host C++17.
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace ft {

using Widths = std::vector<int>;

// Sorted prime factors with multiplicity; n <= 1 gives an empty list.
inline std::vector<int> prime_factors(int n) {
  std::vector<int> out;
  for (int p = 2; n > 1 && (int64_t)p * p <= n; ++p)
    while (n % p == 0) { out.push_back(p); n /= p; }
  if (n > 1) out.push_back(n);
  return out;
}

// Mathematical primality (1 is not prime).
inline bool is_prime(int n) {
  if (n < 2) return false;
  for (int p = 2; (int64_t)p * p <= n; ++p)
    if (n % p == 0) return false;
  return true;
}

// The reference's predicate calls 1 prime and everything <= 0 composite; the
// candidate generator below keeps that behaviour so its output matches for n = 1.
inline bool is_prime_loose(int n) { return n == 1 || is_prime(n); }

namespace detail {
inline void ordered_rec(int rest, Widths& cur, std::vector<Widths>& out) {
  if (rest == 1) { out.push_back(cur); return; }
  for (int f = 2; f <= rest; ++f) {
    if (rest % f) continue;
    cur.push_back(f);
    ordered_rec(rest / f, cur, out);
    cur.pop_back();
  }
}
}  // namespace detail

// All ordered factorisations of n with factors >= 2, in depth-first order with the
// first factor ascending (so the single-factor [n] comes last).  n = 1 -> { [] }.
inline std::vector<Widths> ordered_factorizations(int n) {
  std::vector<Widths> out;
  if (n <= 0) return out;
  Widths cur;
  detail::ordered_rec(n, cur, out);
  return out;
}

// Number of ordered factorisations (0 -> 0, 1 -> 1), memoised.
inline uint64_t count_ordered_factorizations(int n) {
  static thread_local std::map<int, uint64_t> memo;
  if (n <= 0) return 0;
  if (n == 1) return 1;
  auto it = memo.find(n);
  if (it != memo.end()) return it->second;
  uint64_t total = 0;
  for (int f = 2; f <= n; ++f)
    if (n % f == 0) total += count_ordered_factorizations(n / f);
  memo[n] = total;
  return total;
}

// Candidate list for n ranks: the ordered factorisations, except that the trivial
// one-level [n] is replaced by the two flat sentinels [1,n] and [n,1] (a flat tree
// modelled as a degenerate two-level one).  n = 1 -> { [] }, n <= 0 -> {}.
inline std::vector<Widths> candidate_shapes(int n) {
  std::vector<Widths> out;
  for (auto& w : ordered_factorizations(n)) {
    if (w.size() == 1) {
      out.push_back({1, w[0]});
      out.push_back({w[0], 1});
    } else {
      out.push_back(w);
    }
  }
  return out;
}

// Older enumeration strategy: build the set of divisors that are products of prime
// factors, then keep every ordered tuple (up to 9 entries) whose product is n.
// Output is sorted and de-duplicated, with 1*n first and n*1 last.  For any n with
// at most 9 prime factors this is the same *set* as candidate_shapes(n).
inline std::vector<Widths> candidate_shapes_legacy(int n, int max_depth = 9) {
  std::vector<Widths> out;
  if (n <= 1) return candidate_shapes(n);
  std::vector<int> divs;
  for (int d = 2; d < n; ++d)
    if (n % d == 0) divs.push_back(d);
  std::vector<Widths> found;
  Widths cur;
  // iterative deepening over divisor tuples
  struct Rec {
    static void go(int rest, int depth, int max_depth, const std::vector<int>& divs, Widths& cur,
                   std::vector<Widths>& found) {
      if (rest == 1) { if (cur.size() >= 2) found.push_back(cur); return; }
      if (depth == max_depth) return;
      for (int d : divs) {
        if (d > rest) break;
        if (rest % d) continue;
        cur.push_back(d);
        go(rest / d, depth + 1, max_depth, divs, cur, found);
        cur.pop_back();
      }
    }
  };
  Rec::go(n, 0, max_depth, divs, cur, found);
  std::sort(found.begin(), found.end());
  found.erase(std::unique(found.begin(), found.end()), found.end());
  out.push_back({1, n});
  for (auto& w : found) out.push_back(w);
  out.push_back({n, 1});
  return out;
}

// A candidate for a world of `world` ranks: a tree of prod(widths) ranks plus
// `lonely` extra ranks (lonely = -1 means "one phantom rank": a tree one larger than
// the world, which the reference only ever prints and never executes).
struct Candidate {
  Widths widths;
  int lonely = 0;
};

inline std::string shape_to_string(const Widths& w, int lonely = 0) {
  std::string s;
  for (size_t i = 0; i < w.size(); ++i) {
    if (i) s += "*";
    s += std::to_string(w[i]);
  }
  if (lonely > 0) s += "+" + std::to_string(lonely);
  if (lonely < 0) s += std::to_string(lonely);
  return s;
}
inline std::string shape_to_string(const Candidate& c) { return shape_to_string(c.widths, c.lonely); }

// Candidate printer's list for `world` ranks.  A prime world has no tree of its own,
// so it borrows the shapes of world+1 (suffix -1) and of world-1 (suffix +1); a
// composite world lists its own shapes first and then the same two neighbours.
inline std::vector<Candidate> choose_width(int world) {
  std::vector<Candidate> out;
  auto add = [&](int n, int lonely) {
    for (auto& w : candidate_shapes(n)) out.push_back({w, lonely});
  };
  if (!is_prime_loose(world)) add(world, 0);
  add(world + 1, -1);
  add(world - 1, +1);
  return out;
}

}  // namespace ft
