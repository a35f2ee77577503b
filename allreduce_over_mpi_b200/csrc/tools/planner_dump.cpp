// Prints the schedule of every rank for a given world and shape:
//     planner_dump [world] [topo] [lonely] [count]        default: 5 "2,2" 1 27
// The default reproduces the case of the reference's visual planner test
// (allreduce_over_mpi/tmp_tree.cpp:736-760: N = 5, one lonely rank, stages {2,2}, 27 elements).
#include <cstdio>
#include <cstdlib>
#include <string>

#include "../planner/config.hpp"
#include "../planner/plan.hpp"

int main(int argc, char** argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 5;
  const std::string topo = argc > 2 ? argv[2] : "2,2";
  const std::string lonely = argc > 3 ? argv[3] : "1";
  const unsigned long long count = argc > 4 ? strtoull(argv[4], nullptr, 10) : 27;
  ft::ShapeConfig cfg = ft::parse_topo(topo, lonely, world);
  if (!cfg.ok()) {
    fprintf(stderr, "%s\n", cfg.error.c_str());
    return 1;
  }
  ft::Plan p = ft::build_plan(world, cfg.shape);
  const std::string hz = ft::check_hazards(p);
  printf("shape %s, %d stages, traffic %llu elements (2*(N-1)*count = %llu), race check: %s\n", cfg.shape.str().c_str(),
         p.num_stages, (unsigned long long)ft::plan_traffic_elems(p, ft::Blocks(count, world)),
         2ull * (world - 1) * count, hz.empty() ? "clean" : hz.c_str());
  for (int r = 0; r < world; ++r) fputs(ft::describe(p, r, count).c_str(), stdout);
  return hz.empty() ? 0 : 2;
}
