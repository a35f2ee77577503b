// Device form of one rank's plan, built and validated on the host.
//
// build_dev_plan() flattens a rank's stages into the table the collective kernels walk
// (kernels/comm_dev.h); check_dev_plan() then proves, before anything is uploaded or launched,
// that every descriptor the kernels will follow stays in range: stage and pull indices, block
// ids, fan-in against the kernels' pointer tables, source ranks (in the world, never the rank
// itself, never twice), rendezvous masks (only ranks of the world; every rank a stage reads
// from is one it has met before that stage), and the rendezvous numbering.  The byte offsets
// the kernels derive from a descriptor are block * block_bytes + lane offset with block <
// world, so a tensor that lies inside the heap keeps every access inside the heap.
// The reference has no such check: its schedule lists are trusted and MPI reports a bad peer
// or length at run time (allreduce_over_mpi/mpi_mod.hpp:1254-1305).
#pragma once
#include <algorithm>
#include <string>
#include <vector>

#include "../kernels/comm_dev.h"
#include "../planner/plan.hpp"

namespace ft {

struct HostDevPlan {
  ftk::DevPlan plan{};
  std::vector<ftk::DevPull> pulls;
  std::vector<ftk::DevPush> pushes;
};

// The order in which `rank` works through its pulls of stage `s` on the device.
inline std::vector<Pull> device_order(const Plan& p, int rank, int s) {
  std::vector<Pull> ordered = p.stages[rank][s].pulls;
  // gathers start at the next rank up and wrap around, so that at any moment the ranks of a
  // stage read from different peers instead of all queueing on the lowest-numbered one
  if (std::none_of(ordered.begin(), ordered.end(), [](const Pull& x) { return x.reduce; }))
    std::stable_sort(ordered.begin(), ordered.end(), [&](const Pull& x, const Pull& y) {
      return (x.srcs[0] - rank + p.world) % p.world < (y.srcs[0] - rank + p.world) % p.world;
    });
  return ordered;
}

inline HostDevPlan build_dev_plan(const Plan& p, int rank) {
  HostDevPlan out;
  ftk::DevPlan& hp = out.plan;
  hp.nstages = (uint32_t)p.num_stages;
  auto mask_of = [](const std::vector<int>& v) {
    uint64_t m = 0;
    for (int q : v) m |= 1ull << q;
    return m;
  };
  const int last_rs = p.num_stages / 2 - 1;
  for (int s = 0; s < p.num_stages && s < ftk::kMaxStages; ++s) {
    ftk::DevStage& ds = hp.stages[s];
    ds.pull_begin = (uint32_t)out.pulls.size();
    const std::vector<Pull> ordered = device_order(p, rank, s);
    for (const Pull& pl : ordered) {
      ftk::DevPull dp{};
      dp.block = (uint16_t)pl.block;
      dp.nsrc = (uint8_t)std::min<size_t>(pl.srcs.size(), 255);
      dp.reduce = pl.reduce ? 1 : 0;
      for (size_t i = 0; i < pl.srcs.size() && i < FT_MAX_FANIN; ++i) dp.src[i] = (uint8_t)pl.srcs[i];
      out.pulls.push_back(dp);
    }
    ds.pull_end = (uint32_t)out.pulls.size();
    ds.sync_mask = mask_of(p.sync[s][rank]);
    ds.last_rs = (s == last_rs);
    ds.is_ag = !p.stages[rank][s].reduce_scatter || s > last_rs;
  }
  hp.npulls = (uint32_t)out.pulls.size();
  hp.end_sync_mask = mask_of(p.sync[p.num_stages][rank]);
  // Tagged-word (push) form.  Receive slots of a rank are numbered in the order it consumes them: stage by
  // stage, pull by pull, source by source; a slot is written by exactly one rank in exactly one stage.
  // This rank's pushes are then every pull of another rank that names it as a source.
  std::vector<uint32_t> next_slot(p.world, 0);
  uint32_t my_pull = 0;
  for (int s = 0; s < p.num_stages && s < ftk::kMaxStages; ++s) {
    hp.stages[s].push_begin = (uint32_t)out.pushes.size();
    for (int d = 0; d < p.world; ++d) {
      for (const Pull& pl : device_order(p, d, s)) {
        if (d == rank && my_pull < out.pulls.size()) out.pulls[my_pull++].slot = (uint16_t)next_slot[d];
        for (size_t k = 0; k < pl.srcs.size(); ++k) {
          if (pl.srcs[k] == rank && d != rank) {
            ftk::DevPush ps{};
            ps.block = (uint16_t)pl.block;
            ps.slot = (uint16_t)(next_slot[d] + k);
            ps.dst = (uint8_t)d;
            out.pushes.push_back(ps);
          }
        }
        next_slot[d] += (uint32_t)pl.srcs.size();
      }
    }
    hp.stages[s].push_end = (uint32_t)out.pushes.size();
  }
  hp.npushes = (uint32_t)out.pushes.size();
  hp.nslots = next_slot[rank];
  return out;
}

// Empty string when the table is safe to hand to the kernels, else what is wrong.
inline std::string check_dev_plan(const HostDevPlan& d, int world, int rank) {
  const ftk::DevPlan& hp = d.plan;
  auto bad = [&](int s, const std::string& what) { return "stage " + std::to_string(s) + ": " + what; };
  if (world < 1 || world > FT_MAX_RANKS || rank < 0 || rank >= world) return "rank or world out of range";
  if (hp.nstages > (uint32_t)ftk::kMaxStages) return "more stages than the device table holds";
  if (hp.nstages + 2 > ftk::kCallStride) return "more rendezvous per call than the numbering reserves";
  if (hp.nstages % 2) return "odd number of stages";
  if (hp.npulls != d.pulls.size()) return "pull count does not match the table";
  const uint64_t everyone = world >= 64 ? ~0ull : ((1ull << world) - 1);
  if (hp.end_sync_mask & ~everyone) return "closing rendezvous names a rank outside the world";
  uint32_t next = 0;
  int last_rs_seen = 0;
  for (uint32_t s = 0; s < hp.nstages; ++s) {
    const ftk::DevStage& st = hp.stages[s];
    if (st.pull_begin != next || st.pull_end < st.pull_begin || st.pull_end > hp.npulls) return bad(s, "pull range out of order");
    next = st.pull_end;
    if (st.sync_mask & ~everyone) return bad(s, "rendezvous names a rank outside the world");
    last_rs_seen += st.last_rs ? 1 : 0;
    if (st.last_rs && s + 1 != hp.nstages / 2) return bad(s, "scaling stage is not the last reduce-scatter stage");
    for (uint32_t q = st.pull_begin; q < st.pull_end; ++q) {
      const ftk::DevPull& pl = d.pulls[q];
      if (pl.block >= world) return bad(s, "block id outside the buffer");
      if (pl.nsrc < 1) return bad(s, "pull without a source");
      if (pl.reduce ? pl.nsrc + 1 > FT_MAX_FANIN : pl.nsrc != 1) return bad(s, "fan-in beyond the kernels' pointer table");
      if (pl.reduce && st.is_ag) return bad(s, "reduction inside the all-gather half");
      uint64_t seen = 0;
      for (int i = 0; i < pl.nsrc; ++i) {
        const int src = pl.src[i];
        if (src >= world) return bad(s, "source rank outside the world");
        if (src == rank) return bad(s, "pull from the rank itself");
        if (seen >> src & 1) return bad(s, "source named twice");
        seen |= 1ull << src;
        if (!(st.sync_mask >> src & 1)) return bad(s, "reads from a rank it has not met before this stage");
      }
    }
  }
  if (next != hp.npulls) return "pulls left over after the last stage";
  // tagged-word form: pushes in stage order, destinations in the world and never the rank itself, every receive
  // slot of this rank claimed by exactly one (pull, source)
  if (hp.npushes != d.pushes.size()) return "push count does not match the table";
  uint32_t next_push = 0, slots = 0;
  for (uint32_t s = 0; s < hp.nstages; ++s) {
    const ftk::DevStage& st = hp.stages[s];
    if (st.push_begin != next_push || st.push_end < st.push_begin || st.push_end > hp.npushes) return bad(s, "push range out of order");
    next_push = st.push_end;
    for (uint32_t q = st.push_begin; q < st.push_end; ++q) {
      if (d.pushes[q].dst >= world || d.pushes[q].dst == rank) return bad(s, "push to a rank outside the world or to itself");
      if (d.pushes[q].block >= world) return bad(s, "pushed block id outside the buffer");
    }
    for (uint32_t q = st.pull_begin; q < st.pull_end; ++q) {
      if (d.pulls[q].slot != slots) return bad(s, "receive slots are not consecutive");
      slots += d.pulls[q].nsrc;
    }
  }
  if (next_push != hp.npushes) return "pushes left over after the last stage";
  if (slots != hp.nslots) return "receive slot count does not match the pulls";
  if (hp.nstages && last_rs_seen != 1) return "no single final reduce-scatter stage";
  return "";
}

}  // namespace ft
