// Tree-width cost model printout:
//     cost_model_sweep [n_max=64] [chunk=100] [--csv file]
// For N = 1..n_max prints the number of candidate shapes, the shape the original analytic model
// picks, its cost, and the time the enumeration + scoring took.  The reference's driver does this
// for N = 1..999 into numofstru.csv (cost_model/main.cpp:7-28); its verbose per-candidate log is
// not reproduced.  With a calibration of the NVSwitch model (FT_CALIBRATION-style constants passed
// as --link GB/s --sync us --launch us) the B200 pick for a message size is printed next to it.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../planner/cost_model.hpp"
#include "timer.hpp"

int main(int argc, char** argv) {
  int n_max = 64;
  double chunk = 100;
  const char* csv = nullptr;
  ft::V1Params v1;
  unsigned long long bytes = 64ull << 20;
  int pos = 0;
  for (int i = 1; i < argc; ++i) {
    if (!strcmp(argv[i], "--csv") && i + 1 < argc) csv = argv[++i];
    else if (!strcmp(argv[i], "--link") && i + 1 < argc) v1.link_gbs = atof(argv[++i]);
    else if (!strcmp(argv[i], "--sync") && i + 1 < argc) v1.sync_us = atof(argv[++i]);
    else if (!strcmp(argv[i], "--launch") && i + 1 < argc) v1.launch_us = atof(argv[++i]);
    else if (!strcmp(argv[i], "--bytes") && i + 1 < argc) bytes = strtoull(argv[++i], nullptr, 10);
    else if (pos == 0) { n_max = atoi(argv[i]); ++pos; }
    else if (pos == 1) { chunk = atof(argv[i]); ++pos; }
  }
  FILE* f = csv ? fopen(csv, "w") : nullptr;
  if (f) fprintf(f, "n,candidates,microseconds,shape,cost\n");
  printf("%4s %6s %9s  %-14s %-10s  %s\n", "N", "cands", "us", "v0 shape", "v0 cost", "v1 pick (NVSwitch model)");
  for (int n = 1; n <= n_max; ++n) {
    ft::Timer t;
    t.Start();
    ft::V0Choice c = ft::choose_v0(n, chunk);
    t.Stop();
    std::string v1s = "-";
    if (n >= 2 && n <= FT_MAX_RANKS / 2) {
      ft::V1Choice k = ft::pick_algorithm(n, bytes, v1, true, false);
      char buf[96];
      snprintf(buf, sizeof buf, "%s %s %.1f us", k.algo.c_str(), k.shape.str().c_str(), k.us);
      v1s = buf;
    }
    const std::string shape = ft::shape_to_string(c.widths);
    printf("%4d %6zu %9lld  %-14s %-10.6g  %s\n", n, c.candidates, (long long)t.MicroSeconds(), shape.c_str(), c.cost, v1s.c_str());
    if (f) fprintf(f, "%d,%zu,%lld,%s,%.6g\n", n, c.candidates, (long long)t.MicroSeconds(), shape.c_str(), c.cost);
  }
  if (f) fclose(f);
  return 0;
}
