// Tree-shape configuration from strings / environment.
//
// Same syntax as the reference's get_stages() (allreduce_over_mpi/mpi_mod.hpp:1419-1486):
//   FT_TOPO   = "w0,w1,..."  bottom-up level widths; unset or empty => flat {world};
//               any width equal to 1 => ring
//   FT_LONELY = "L"          number of lonely ranks (default 0)
// A shape is accepted when prod(w) + L == world and lonely layouts have >= 2 levels;
// on top of that this parser refuses the lonely layouts that cannot be scheduled
// (L > w0 or L*w0 > prod(w)) which the reference accepts and then mis-executes.
// Errors come back as a message starting with "invalid FT_TOPO" instead of exit(1).
// The additional value FT_TOPO=auto asks the caller to consult the cost model.
#pragma once
#include <cstdlib>
#include <sstream>
#include <string>

#include "plan.hpp"

namespace ft {

struct ShapeConfig {
  Shape shape;
  bool is_auto = false;
  std::string error;
  bool ok() const { return error.empty(); }
};

inline ShapeConfig parse_topo(const std::string& topo_in, const std::string& lonely_in, int world) {
  ShapeConfig c;
  std::string topo = topo_in;
  if (topo == "auto") {
    c.is_auto = true;
    c.shape = Shape::flat(world);
    return c;
  }
  int lonely = 0;
  if (!lonely_in.empty()) {
    std::istringstream is(lonely_in);
    if (!(is >> lonely) || lonely < 0) { c.error = "invalid FT_LONELY " + lonely_in; return c; }
  }
  Shape s;
  s.lonely = lonely;
  if (topo.empty()) {
    s.widths = {world};
  } else {
    for (char& ch : topo)
      if (ch == ',' || ch == '*' || ch == 'x') ch = ' ';
    std::istringstream is(topo);
    std::string tok;
    while (is >> tok) {
      char* end = nullptr;
      long v = std::strtol(tok.c_str(), &end, 10);
      if (end == tok.c_str() || *end != '\0' || v < 1 || v > 1 << 20) { c.error = "invalid FT_TOPO " + topo_in; return c; }
      if (v == 1) {  // a width of 1 selects the ring, whatever else was listed
        c.shape = Shape::make_ring(world);
        return c;
      }
      s.widths.push_back((int)v);
    }
    if (s.widths.empty()) s.widths = {world};
  }
  std::string why = validate_shape(world, s);
  if (!why.empty()) { c.error = "invalid FT_TOPO " + topo_in + (lonely ? " FT_LONELY " + lonely_in : "") + " (" + why + ")"; return c; }
  c.shape = s;
  return c;
}

inline ShapeConfig shape_from_env(int world) {
  const char* t = std::getenv("FT_TOPO");
  const char* l = std::getenv("FT_LONELY");
  return parse_topo(t ? t : "", l ? l : "", world);
}

}  // namespace ft
