// FlexTree schedule planner: (world, tree shape, lonely count) -> per-rank pull plan.
//
// The schedule is expressed as PULLS, not as matched send/receive pairs: in every
// stage a rank lists, per data block, the ranks whose copy of that block it reads,
// and whether it adds them to its own copy (reduce-scatter half) or just takes the
// first one (all-gather half).  That is the natural form for GPUs that can load from
// each other's memory over NVSwitch: the reader's kernel performs transfer and
// reduction in one pass and no staging buffer or message matching exists.
//
// The algorithm (multi-level tree of widths w0*w1*..., "lonely" ranks for worlds that
// do not factor, and the ring) reproduces the behaviour of the reference planner:
//   allreduce_over_mpi/mpi_mod.hpp:258-347   send lists  (tree, extended groups, lonely)
//   allreduce_over_mpi/mpi_mod.hpp:349-451   receive lists
//   allreduce_over_mpi/mpi_mod.hpp:207-255   lonely predicates (holders, "star", followers)
//   allreduce_over_mpi/mpi_mod.hpp:627-766   element-range adapters (block -> offset,len)
//   allreduce_over_mpi/mpi_mod.hpp:1673-1719 ring
// The all-gather half is derived mechanically as the edge-reversal of the
// reduce-scatter half, which is what the reference does by swapping its send and
// receive lists in reverse stage order (mpi_mod.hpp:661-669, :736-744).
//
// Like the reference planner this file depends only on (world, lonely, rank, widths);
// it knows nothing about transports, CUDA or MPI.  Unlike it, invalid shapes are
// rejected with an error string instead of an assert or a silently wrong schedule.
#pragma once
#include <algorithm>
#include <cstdint>
#include <sstream>
#include <string>
#include <vector>

#include "../api/ft_types.h"
#include "factorize.hpp"

namespace ft {

constexpr int kMaxFanIn = 32;  // sources per reduction incl. own copy (the reference stops at 20)

struct Shape {
  Widths widths;     // bottom-up level widths; product = number of tree ranks
  int lonely = 0;    // extra ranks that sit outside the tree
  bool ring = false; // classic ring instead of a tree (reference: any width == 1)
  int tree_ranks() const {
    int m = 1;
    for (int w : widths) m *= w;
    return m;
  }
  int world() const { return ring ? (widths.empty() ? 0 : widths[0]) : tree_ranks() + lonely; }
  std::string str() const {
    if (ring) return "ring" + std::to_string(world());
    return shape_to_string(widths, lonely);
  }
  static Shape flat(int n) { return Shape{{n}, 0, false}; }
  static Shape make_ring(int n) { return Shape{{n}, 0, true}; }
};

// Empty string when the shape can be executed for `world` ranks, else the reason.
// The lonely rule (>= 2 levels, L <= w0, L*w0 <= tree ranks) is the exact set of
// layouts for which the lonely schedule is complete; the reference only checks the
// first condition (mpi_mod.hpp:1471) and aborts or mis-schedules on the others.
inline std::string validate_shape(int world, const Shape& s) {
  std::ostringstream e;
  if (world < 1) { e << "world size " << world << " < 1"; return e.str(); }
  if (s.ring) {
    if (s.lonely) return "ring takes no lonely ranks";
    if (s.widths.size() != 1 || s.widths[0] != world) return "ring shape must be {world}";
    return "";
  }
  if (s.widths.empty()) return "empty tree shape";
  for (int w : s.widths)
    if (w < 1 || (w == 1 && !(s.widths.size() == 1 && world == 1))) {
      e << "invalid width " << w << " in " << s.str();
      return e.str();
    }
  if (s.lonely < 0) return "negative lonely count";
  const int m = s.tree_ranks();
  if (m + s.lonely != world) {
    e << "shape " << s.str() << " covers " << m + s.lonely << " ranks, world is " << world;
    return e.str();
  }
  for (int w : s.widths)
    if (w > kMaxFanIn - 1) { e << "width " << w << " exceeds max fan-in " << kMaxFanIn - 1; return e.str(); }
  if (s.lonely) {
    if (s.widths.size() < 2) return "lonely ranks need a tree of at least 2 levels";
    if (s.lonely > s.widths[0]) { e << "lonely " << s.lonely << " > bottom width " << s.widths[0]; return e.str(); }
    if (s.lonely * s.widths[0] > m) { e << "lonely*w0 = " << s.lonely * s.widths[0] << " > tree ranks " << m; return e.str(); }
  }
  return "";
}

// One unit of work for one rank in one stage.
struct Pull {
  int block = 0;          // block id in [0, world)
  std::vector<int> srcs;  // ranks read from, in summation order
  bool reduce = false;    // true: mine = mine (+) sum(srcs); false: mine = srcs[0]
};

struct Stage {
  bool reduce_scatter = true;
  std::vector<Pull> pulls;
};

struct Plan {
  int world = 0;
  Shape shape;
  int num_stages = 0;
  // stages[rank][stage]
  std::vector<std::vector<Stage>> stages;
  // sync[stage][rank] = ranks to rendezvous with before running `stage`;
  // sync[num_stages][rank] = the closing rendezvous.  Always symmetric.
  std::vector<std::vector<std::vector<int>>> sync;
  std::string error;  // non-empty => plan is unusable
  bool ok() const { return error.empty(); }
};

// Block geometry: `count` elements cut into `world` blocks of `block_elems`
// (default ceil(count/world)); trailing blocks may be short or empty.
struct Blocks {
  uint64_t count = 0;
  int nblocks = 1;
  uint64_t block_elems = 0;
  Blocks() {}
  Blocks(uint64_t count_, int nblocks_, uint64_t block_elems_ = 0) : count(count_), nblocks(nblocks_) {
    block_elems = block_elems_ ? block_elems_ : (count + nblocks - 1) / (uint64_t)nblocks;
  }
  uint64_t offset(int b) const { return std::min<uint64_t>(count, (uint64_t)b * block_elems); }
  uint64_t length(int b) const {
    uint64_t lo = (uint64_t)b * block_elems;
    if (lo >= count) return 0;
    return std::min<uint64_t>(block_elems, count - lo);
  }
};

namespace detail {

inline void add_pull(std::vector<Stage>& st, int stage, int block, std::vector<int> srcs, bool reduce) {
  if (srcs.empty()) return;
  st[stage].pulls.push_back(Pull{block, std::move(srcs), reduce});
}

// Reduce-scatter half of the tree schedule (stages 0..S-1) for every rank.
inline void build_tree_rs(Plan& p) {
  const Widths& w = p.shape.widths;
  const int S = (int)w.size();
  const int L = p.shape.lonely;
  const int M = p.shape.tree_ranks();
  const int N = p.world;
  const int w0 = w[0];
  const int ext_end = L * w0;  // tree ranks below this index belong to an extended bottom group
  auto star = [&](int j) { return M - w0 + j; };  // tree rank a lonely block "follows"

  // ---- tree ranks
  for (int r = 0; r < M; ++r) {
    int g = 1;
    for (int i = 0; i < S; ++i) {
      const int G = g * w[i];
      const int base = (r / G) * G + r % g;
      std::vector<int> peers;
      for (int k = 0; k < w[i]; ++k)
        if (base + k * g != r) peers.push_back(base + k * g);
      std::vector<int> srcs = peers;
      if (i == 0 && r < ext_end) srcs.push_back(M + r / w0);  // adopted lonely rank, summed last
      for (int b = r % G; b < M; b += G) add_pull(p.stages[r], i, b, srcs, true);

      // partial sums of lonely blocks travel up the tree among non-extended ranks
      const int j = r % w0;
      if (L > 0 && r >= ext_end && j < L && i < S - 1) {
        if (i == 0) {
          add_pull(p.stages[r], 0, M + j, peers, true);
        } else if (r % G == star(j) % G) {
          std::vector<int> holders;
          for (int q : peers)
            if (q >= ext_end) holders.push_back(q);
          add_pull(p.stages[r], i, M + j, holders, true);
        }
      }
      g = G;
    }
  }
  // ---- lonely ranks
  for (int k = 0; k < L; ++k) {
    const int r = M + k;
    std::vector<int> members;
    for (int m = 0; m < w0; ++m) members.push_back(k * w0 + m);
    for (int j = 0; j < L; ++j) add_pull(p.stages[r], 0, M + j, members, true);

    std::vector<int> others;
    for (int q = M; q < N; ++q)
      if (q != r) others.push_back(q);
    std::vector<int> holders;  // tree ranks still holding a partial of block M+k before the last stage
    for (int h = star(k); h >= ext_end; h -= M / w[S - 1]) holders.push_back(h);
    if (S == 2) {
      std::vector<int> srcs = others;
      srcs.insert(srcs.end(), holders.begin(), holders.end());
      add_pull(p.stages[r], 1, r, srcs, true);
    } else {
      add_pull(p.stages[r], 1, r, others, true);
      add_pull(p.stages[r], S - 1, r, holders, true);
    }
  }
}

// All-gather half = every reduce-scatter edge reversed, stages in reverse order.
inline void mirror_rs_into_ag(Plan& p, int S) {
  for (int r = 0; r < p.world; ++r)
    for (int i = 0; i < S; ++i)
      for (const Pull& pl : p.stages[r][i].pulls)
        for (int src : pl.srcs) {
          Stage& st = p.stages[src][2 * S - 1 - i];
          st.reduce_scatter = false;
          st.pulls.push_back(Pull{pl.block, {r}, false});
        }
  for (int r = 0; r < p.world; ++r)
    for (int s = S; s < 2 * S; ++s) {
      auto& v = p.stages[r][s].pulls;
      p.stages[r][s].reduce_scatter = false;
      std::stable_sort(v.begin(), v.end(), [](const Pull& a, const Pull& b) {
        return a.srcs[0] != b.srcs[0] ? a.srcs[0] < b.srcs[0] : a.block < b.block;
      });
    }
}

inline void build_ring(Plan& p) {
  const int N = p.world;
  for (int r = 0; r < N; ++r) {
    const int left = (r + N - 1) % N;
    int blk = left;  // block received (and reduced) in the first step
    for (int s = 0; s < N - 1; ++s) {
      add_pull(p.stages[r], s, blk, {left}, true);
      blk = (blk + N - 1) % N;
    }
    for (int s = 0; s < N - 1; ++s) {
      p.stages[r][N - 1 + s].reduce_scatter = false;
      add_pull(p.stages[r], N - 1 + s, blk, {left}, false);
      blk = (blk + N - 1) % N;
    }
  }
}

// Rendezvous sets: before stage s a rank meets everyone it exchanges data with in
// stage s-1 or s (either direction).  The opening rendezvous is global so that a
// rank entering call k+1 proves that it has left call k.
inline void build_sync(Plan& p) {
  const int N = p.world, T = p.num_stages;
  std::vector<std::vector<std::vector<char>>> touch(T, std::vector<std::vector<char>>(N, std::vector<char>(N, 0)));
  for (int r = 0; r < N; ++r)
    for (int s = 0; s < T; ++s)
      for (const Pull& pl : p.stages[r][s].pulls)
        for (int q : pl.srcs) touch[s][r][q] = touch[s][q][r] = 1;
  p.sync.assign(T + 1, std::vector<std::vector<int>>(N));
  for (int s = 0; s <= T; ++s)
    for (int r = 0; r < N; ++r)
      for (int q = 0; q < N; ++q) {
        if (q == r) continue;
        bool need = (s == 0);
        if (s > 0 && touch[s - 1][r][q]) need = true;
        if (s < T && touch[s][r][q]) need = true;
        if (need) p.sync[s][r].push_back(q);
      }
}

}  // namespace detail

inline Plan build_plan(int world, const Shape& shape) {
  Plan p;
  p.world = world;
  p.shape = shape;
  p.error = validate_shape(world, shape);
  if (!p.ok()) return p;
  if (world == 1) {
    p.num_stages = 0;
    p.stages.assign(1, {});
    p.sync.assign(1, std::vector<std::vector<int>>(1));
    return p;
  }
  if (shape.ring) {
    p.num_stages = 2 * (world - 1);
    p.stages.assign(world, std::vector<Stage>(p.num_stages));
    detail::build_ring(p);
  } else {
    const int S = (int)shape.widths.size();
    p.num_stages = 2 * S;
    p.stages.assign(world, std::vector<Stage>(p.num_stages));
    detail::build_tree_rs(p);
    detail::mirror_rs_into_ag(p, S);
  }
  for (auto& per_rank : p.stages)
    for (auto& st : per_rank)
      for (auto& pl : st.pulls)
        if ((int)pl.srcs.size() + 1 > kMaxFanIn) p.error = "fan-in exceeds " + std::to_string(kMaxFanIn);
  detail::build_sync(p);
  return p;
}

// ---- static checks -------------------------------------------------------------------

// Verifies that the plan is race-free when every rank works in place on one buffer:
// (1) within a stage nobody reads a (rank, block) that its owner rewrites in that stage;
// (2) every read is separated from the write that produced the value, and every
//     overwrite from earlier reads of the old value, by a rendezvous that contains both
//     ranks.  Returns "" or the first violation found.
inline std::string check_hazards(const Plan& p) {
  if (!p.ok()) return p.error;
  const int N = p.world, T = p.num_stages;
  std::ostringstream e;
  auto met = [&](int a, int b, int lo_excl, int hi_incl) {  // rendezvous a<->b at a boundary in (lo, hi]
    for (int s = std::max(lo_excl + 1, 0); s <= hi_incl; ++s)
      if (std::find(p.sync[s][a].begin(), p.sync[s][a].end(), b) != p.sync[s][a].end()) return true;
    return false;
  };
  // last_write[rank][block] = stage of last write (-1 = initial input)
  std::vector<std::vector<int>> last_write(N, std::vector<int>(N, -1));
  // readers[rank][block] = list of (reader, stage) since the last write
  std::vector<std::vector<std::vector<std::pair<int, int>>>> readers(
      N, std::vector<std::vector<std::pair<int, int>>>(N));
  for (int s = 0; s < T; ++s) {
    std::vector<std::vector<char>> written(N, std::vector<char>(N, 0));
    for (int r = 0; r < N; ++r)
      for (const Pull& pl : p.stages[r][s].pulls) {
        if (written[r][pl.block]) { e << "stage " << s << ": rank " << r << " writes block " << pl.block << " twice"; return e.str(); }
        written[r][pl.block] = 1;
      }
    for (int r = 0; r < N; ++r)
      for (const Pull& pl : p.stages[r][s].pulls)
        for (int q : pl.srcs) {
          if (q == r) { e << "stage " << s << ": rank " << r << " pulls from itself"; return e.str(); }
          if (written[q][pl.block]) { e << "stage " << s << ": rank " << r << " reads block " << pl.block << " of rank " << q << " while it is rewritten"; return e.str(); }
          const int lw = last_write[q][pl.block];
          if (!met(r, q, lw, s)) { e << "stage " << s << ": rank " << r << " reads block " << pl.block << " of rank " << q << " (written in stage " << lw << ") without a rendezvous"; return e.str(); }
          readers[q][pl.block].push_back({r, s});
        }
    for (int r = 0; r < N; ++r)
      for (const Pull& pl : p.stages[r][s].pulls) {
        for (auto& rd : readers[r][pl.block])
          if (rd.second < s && !met(r, rd.first, rd.second, s)) {
            e << "stage " << s << ": rank " << r << " overwrites block " << pl.block << " read by rank " << rd.first << " in stage " << rd.second << " without a rendezvous";
            return e.str();
          }
      }
    for (int r = 0; r < N; ++r)
      for (const Pull& pl : p.stages[r][s].pulls) {
        last_write[r][pl.block] = s;
        readers[r][pl.block].clear();
      }
  }
  // closing rendezvous must cover everyone who read from me in the last stages
  for (int r = 0; r < N; ++r)
    for (int b = 0; b < N; ++b)
      for (auto& rd : readers[r][b])
        if (!met(r, rd.first, rd.second, T)) { e << "rank " << rd.first << " may still read block " << b << " of rank " << r << " after the call ends"; return e.str(); }
  return "";
}

struct PlanStats {
  uint64_t total_pulled_blocks = 0;  // over all ranks and stages (remote block transfers)
  int max_fan_in = 0;                // incl. own copy
  std::vector<std::vector<int>> in_blocks;   // [stage][rank] blocks pulled
  std::vector<std::vector<int>> out_blocks;  // [stage][rank] blocks served
};

inline PlanStats plan_stats(const Plan& p) {
  PlanStats st;
  st.in_blocks.assign(p.num_stages, std::vector<int>(p.world, 0));
  st.out_blocks.assign(p.num_stages, std::vector<int>(p.world, 0));
  for (int r = 0; r < p.world; ++r)
    for (int s = 0; s < p.num_stages; ++s)
      for (const Pull& pl : p.stages[r][s].pulls) {
        st.total_pulled_blocks += pl.srcs.size();
        st.in_blocks[s][r] += (int)pl.srcs.size();
        for (int q : pl.srcs) st.out_blocks[s][q] += 1;
        if (pl.reduce) st.max_fan_in = std::max(st.max_fan_in, (int)pl.srcs.size() + 1);
      }
  return st;
}

// Exact number of elements that cross between ranks for a given buffer length.
inline uint64_t plan_traffic_elems(const Plan& p, const Blocks& g) {
  uint64_t t = 0;
  for (int r = 0; r < p.world; ++r)
    for (int s = 0; s < p.num_stages; ++s)
      for (const Pull& pl : p.stages[r][s].pulls) t += pl.srcs.size() * g.length(pl.block);
  return t;
}

// Who holds what after the reduce-scatter half (stages [0, num_stages/2)) alone: holders[b]
// is the set of ranks, as a bit mask, whose copy of block b then contains every rank's
// contribution.  Found by pushing "set of contributors" masks through the plan with the same
// read-before-write semantics as the executors.  These are the blocks a caller of the
// reduce-scatter phase may read, and the blocks the all-gather phase takes as final.
inline std::vector<uint64_t> rs_holders(const Plan& p) {
  std::vector<uint64_t> holders(p.world > 0 ? p.world : 0, 0);
  if (!p.ok() || p.world > 64) return holders;
  const uint64_t all = p.world >= 64 ? ~0ull : ((1ull << p.world) - 1);
  std::vector<std::vector<uint64_t>> have(p.world, std::vector<uint64_t>(p.world, 0));  // [rank][block]
  for (int r = 0; r < p.world; ++r)
    for (int b = 0; b < p.world; ++b) have[r][b] = 1ull << r;
  for (int s = 0; s < p.num_stages / 2; ++s) {
    auto next = have;
    for (int r = 0; r < p.world; ++r)
      for (const Pull& pl : p.stages[r][s].pulls) {
        uint64_t m = pl.reduce ? have[r][pl.block] : 0;
        for (int q : pl.srcs) m |= have[q][pl.block];
        next[r][pl.block] = m;
      }
    have.swap(next);
  }
  for (int b = 0; b < p.world; ++b)
    for (int r = 0; r < p.world; ++r)
      if (have[r][b] == all) holders[b] |= 1ull << r;
  return holders;
}

// Human-readable dump of one rank's schedule (the counterpart of the reference's
// coloured print(), mpi_mod.hpp:159-199 and :585-624).  With count > 0 the element
// ranges "offset+len" are printed next to the block ids.
inline std::string describe(const Plan& p, int rank, uint64_t count = 0, uint64_t block_elems = 0) {
  std::ostringstream os;
  if (!p.ok()) { os << "invalid plan: " << p.error << "\n"; return os.str(); }
  Blocks g(count, p.world, block_elems);
  os << "rank " << rank << " of " << p.world << ", shape " << p.shape.str() << ", " << p.num_stages << " stages\n";
  for (int s = 0; s < p.num_stages; ++s) {
    const Stage& st = p.stages[rank][s];
    os << (s + 1 == p.num_stages ? " `-" : " |-") << " stage " << s << (st.reduce_scatter ? " RS" : " AG") << " sync{";
    for (size_t i = 0; i < p.sync[s][rank].size(); ++i) os << (i ? "," : "") << p.sync[s][rank][i];
    os << "}";
    if (st.pulls.empty()) os << " (idle)";
    for (const Pull& pl : st.pulls) {
      os << " | " << (pl.reduce ? "sum" : "get") << " b" << pl.block;
      if (count) os << "[" << g.offset(pl.block) << "+" << g.length(pl.block) << "]";
      os << " <-";
      for (size_t i = 0; i < pl.srcs.size(); ++i) os << (i ? "," : " ") << pl.srcs[i];
    }
    os << "\n";
  }
  return os.str();
}

}  // namespace ft
