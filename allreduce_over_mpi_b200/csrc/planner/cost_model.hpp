// Tree-width cost models.
//
// v0  cost_v0(): the reference's three-term analytic model with its original
//     constants, restated in closed form (cost_model/CostModel.h:1-120):
//       cost(t) = sum_levels [ 2*lo + (w > 9 ? 100*(w-9)*co : 0) ]         latency + incast
//               + (steps * s / N) * o                                        extra memory passes
//               + ((N-1)/N * s) * bo                                         wire + reduce, shape independent
//       steps   = N + 1 + 2 * sum_{k=1}^{h-1} prod_{j<k} t_j
//     with lo=0.004, co=0.0002, o=0.0004, bo=0.0068.  The incast term really uses the
//     literal chunk 100 whatever `s` is (CostModel.h:92); that quirk is kept behind
//     `V0Params::latency_chunk`.  Two defects are not kept: the accumulator starts at 0
//     (the reference reads it uninitialised for the first candidate) and any depth works
//     (the reference has hand-expanded cases for depth <= 9 only).
//     choose_v0() returns the arg-min over candidate_shapes(N), first minimum wins, which
//     reproduces the reference's printed choice for every N.
//
// v1  cost_v1(): the model re-derived for an NVSwitch box.  There every valid shape
//     moves the same bytes per rank, links do not suffer Ethernet-style incast, and the
//     price of depth is one cross-GPU rendezvous per extra stage.  The model walks the
//     actual plan: per stage it takes the busiest rank's inbound and outbound bytes over
//     the measured link bandwidth (scaled by a measured efficiency for the number of
//     concurrent source peers), the local read+write bytes over HBM bandwidth, and adds
//     one rendezvous latency; plus a launch constant.  One-shot (every rank reads
//     everything once) and NVLS (in-switch reduction) are scored with their own closed
//     forms so that pick_algorithm() can choose per message size.
#pragma once
#include <cmath>
#include <limits>
#include <string>
#include <vector>

#include "plan.hpp"

namespace ft {

struct V0Params {
  double lo = 0.004, co = 0.0002, o = 0.0004, bo = 0.0068;
  double incast_width = 9;
  double latency_chunk = 100;  // <= 0: use the call's chunk size instead of the literal
};

inline double v0_latency_control(double chunk, double width, const V0Params& k = {}) {
  double c = 2 * k.lo;
  if (width > k.incast_width) c += chunk * (width - k.incast_width) * k.co;
  return c;
}
inline double v0_bandwidth_calc(int n, double chunk, const V0Params& k = {}) { return ((n - 1.0) / n * chunk) * k.bo; }
inline double v0_steps(const Widths& t, int n) {
  double steps = n + 1, prod = 1;
  for (size_t j = 0; j + 1 < t.size(); ++j) { prod *= t[j]; steps += 2 * prod; }
  return steps;
}
inline double v0_memory_rw(const Widths& t, int n, double chunk, const V0Params& k = {}) { return (v0_steps(t, n) * chunk / n) * k.o; }

inline double cost_v0(const Widths& t, int n, double chunk, const V0Params& k = {}) {
  double c = 0;
  for (int w : t) c += v0_latency_control(k.latency_chunk > 0 ? k.latency_chunk : chunk, w, k);
  return c + v0_memory_rw(t, n, chunk, k) + v0_bandwidth_calc(n, chunk, k);
}

struct V0Choice { Widths widths; double cost = 0; size_t candidates = 0; };
inline V0Choice choose_v0(int n, double chunk = 100, const V0Params& k = {}) {
  V0Choice best;
  best.cost = 1e9;
  auto cands = candidate_shapes(n);
  best.candidates = cands.size();
  for (auto& t : cands) {
    double c = cost_v0(t, n, chunk, k);
    if (c < best.cost) { best.cost = c; best.widths = t; }
  }
  return best;
}

// ---- v1: measured-parameter model -------------------------------------------------------

struct V1Params {
  double launch_us = 4.0;      // launch + kernel entry/exit
  double sync_us = 2.5;        // one cross-GPU rendezvous
  double link_gbs = 700.0;     // per direction per GPU, pulling from many peers
  double hbm_gbs = 6000.0;     // local read+write
  double stage_floor_us = 0.5; // fixed cost per stage besides the rendezvous
  double nvls_gbs = 0.0;       // in-switch reduce/broadcast bandwidth per GPU; 0 = not available
  double oneshot_max_bytes = 1 << 20;
  double ll_us = 0.0;          // fixed cost of the low-latency push protocol; 0 = not available
  double ll_max_bytes = 256 << 10;
  double push_gain = 0.0;      // > 0: the reduce+push kernel exists; link efficiency of its write half relative to reads
  // link efficiency when a stage pulls from k distinct peers at once (index k, 0 unused)
  std::vector<double> peer_eff = std::vector<double>(FT_MAX_RANKS + 1, 1.0);
};

inline double cost_v1(const Plan& p, uint64_t bytes, const V1Params& k, uint64_t block_bytes = 0) {
  if (!p.ok()) return std::numeric_limits<double>::infinity();
  if (p.world == 1) return k.launch_us;
  Blocks g(bytes, p.world, block_bytes);
  double t = k.launch_us + k.sync_us * (p.num_stages + 1);
  for (int s = 0; s < p.num_stages; ++s) {
    std::vector<double> in(p.world, 0), out(p.world, 0), local(p.world, 0);
    std::vector<int> npeer(p.world, 0);
    for (int r = 0; r < p.world; ++r) {
      std::vector<char> seen(p.world, 0);
      for (const Pull& pl : p.stages[r][s].pulls) {
        const double len = (double)g.length(pl.block);
        in[r] += len * pl.srcs.size();
        local[r] += len * (pl.reduce ? 2 : 1);
        for (int q : pl.srcs) { out[q] += len; if (!seen[q]) { seen[q] = 1; ++npeer[r]; } }
      }
    }
    double worst = 0;
    for (int r = 0; r < p.world; ++r) {
      const double eff = k.peer_eff[std::min<int>(npeer[r], (int)k.peer_eff.size() - 1)];
      const double wire = std::max(in[r] / (k.link_gbs * eff), out[r] / k.link_gbs) * 1e-3;  // bytes/GBps = ns
      worst = std::max({worst, wire, local[r] / k.hbm_gbs * 1e-3});
    }
    t += worst + k.stage_floor_us;
  }
  return t;
}

// Every rank reads all N-1 peer buffers in full: one rendezvous, (N-1)*S inbound.
inline double cost_v1_oneshot(int world, uint64_t bytes, const V1Params& k) {
  if (world == 1) return k.launch_us;
  return k.launch_us + k.sync_us + k.stage_floor_us + (double)bytes * (world - 1) / k.link_gbs * 1e-3;
}
// multimem.ld_reduce of S/N + multimem.st of S/N per rank; the GPU's links carry S*(1+1/N).
inline double cost_v1_nvls(int world, uint64_t bytes, const V1Params& k) {
  if (k.nvls_gbs <= 0) return std::numeric_limits<double>::infinity();
  return k.launch_us + 3 * k.sync_us + (double)bytes * (1.0 + 1.0 / world) / k.nvls_gbs * 1e-3;
}

// One-shot through the switch: one rendezvous, every rank reduces the whole message, so each GPU's links carry N * S.
inline double cost_v1_nvls1(int world, uint64_t bytes, const V1Params& k) {
  if (k.nvls_gbs <= 0) return std::numeric_limits<double>::infinity();
  return k.launch_us + k.sync_us + (double)bytes * world / k.nvls_gbs * 1e-3;
}

// Low-latency push: no rendezvous; every rank writes 2x its payload (data + tags) to each of N-1 peers.
inline double cost_v1_ll(int world, uint64_t bytes, const V1Params& k) {
  if (k.ll_us <= 0 || (double)bytes > k.ll_max_bytes) return std::numeric_limits<double>::infinity();
  return k.ll_us + 2.0 * (double)bytes * (world - 1) / k.link_gbs * 1e-3;
}
// Flat reduce + push: two rendezvous; (N-1)/N*S in by reads and the same again by posted writes.
inline double cost_v1_push(int world, uint64_t bytes, const V1Params& k) {
  if (k.push_gain <= 0 || world < 2) return std::numeric_limits<double>::infinity();
  const double eff = k.peer_eff[std::min<int>(world - 1, (int)k.peer_eff.size() - 1)];
  const double half = (double)bytes * (world - 1) / world;
  return k.launch_us + 2 * k.sync_us + (half / (k.link_gbs * eff) + half / (k.link_gbs * eff * k.push_gain)) * 1e-3;
}

// Shapes that can be executed for `world`: flat, every ordered factorisation with >= 2
// levels, the ring, and every schedulable lonely layout.
inline std::vector<Shape> executable_shapes(int world, int max_lonely = 4) {
  std::vector<Shape> out;
  if (world < 1) return out;
  for (auto& w : ordered_factorizations(world)) {
    Shape s{w, 0, false};
    if (w.empty()) s.widths = {1};
    if (validate_shape(world, s).empty()) out.push_back(s);
  }
  if (world >= 2) out.push_back(Shape::make_ring(world));
  for (int l = 1; l <= max_lonely && l < world; ++l)
    for (auto& w : ordered_factorizations(world - l)) {
      Shape s{w, l, false};
      if (validate_shape(world, s).empty()) out.push_back(s);
    }
  return out;
}

struct V1Choice {
  std::string algo;  // "staged", "oneshot", "nvls", "ll", "push"
  Shape shape;
  double us = std::numeric_limits<double>::infinity();
};

// NVLS and reduce+push work in place on a tensor in the symmetric heap only: allow_nvls says that the
// message qualifies for the switch reduction, allow_push (< 0: same as allow_nvls) that it lives in the heap.
inline V1Choice pick_algorithm(int world, uint64_t bytes, const V1Params& k, bool allow_oneshot = true,
                               bool allow_nvls = true, int allow_push = -1, bool allow_nvls1 = false) {
  V1Choice best;
  for (auto& s : executable_shapes(world)) {
    Plan p = build_plan(world, s);
    double c = cost_v1(p, bytes, k);
    if (c < best.us) { best.us = c; best.shape = s; best.algo = "staged"; }
  }
  if (allow_oneshot && bytes <= k.oneshot_max_bytes) {
    double c = cost_v1_oneshot(world, bytes, k);
    if (c < best.us) { best.us = c; best.shape = Shape::flat(world); best.algo = "oneshot"; }
  }
  if (allow_nvls) {
    double c = cost_v1_nvls(world, bytes, k);
    if (c < best.us) { best.us = c; best.shape = Shape::flat(world); best.algo = "nvls"; }
  }
  if (allow_nvls1) {
    double c = cost_v1_nvls1(world, bytes, k);
    if (c < best.us) { best.us = c; best.shape = Shape::flat(world); best.algo = "nvls1"; }
  }
  if (allow_push < 0 ? allow_nvls : allow_push != 0) {
    double c = cost_v1_push(world, bytes, k);
    if (c < best.us) { best.us = c; best.shape = Shape::flat(world); best.algo = "push"; }
  }
  if (allow_oneshot) {
    double c = cost_v1_ll(world, bytes, k);
    if (c < best.us) { best.us = c; best.shape = Shape::flat(world); best.algo = "ll"; }
  }
  return best;
}

}  // namespace ft
