// Which all-reduce algorithm and tree shape to run for a message: ONE policy for every caller.
//
// The reference leaves the choice to a human: its cost model (cost_model/CostModel.h:82-120,
// GetWidth.h:10-47) prints a shape, the operator copies it into FT_TOPO, and the library reads
// that variable on every call (allreduce_over_mpi/mpi_mod.hpp:1419-1486).  Here the link is
// made in code: a calibration file holds, per world size, the measured winner per message size
// plus the fitted parameters of the NVSwitch cost model; choose() answers from the table inside
// the measured range and from the model outside it.  ft_allreduce(FT_ALGO_AUTO), the MPI-style
// entry point, the native benchmark and the Python front end all ask this class.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <tuple>
#include <vector>

#include "cost_model.hpp"
#include "json_min.hpp"

namespace ft {

// "2*4", "2x2+1", "8", "ring8" (the spelling Shape::str() produces).  False on malformed text.
inline bool parse_shape_text(const std::string& text_in, Shape* out) {
  std::string t;
  for (char ch : text_in)
    if (ch != ' ' && ch != '\t') t.push_back((char)(ch >= 'A' && ch <= 'Z' ? ch - 'A' + 'a' : ch));
  Shape s;
  auto to_int = [](const std::string& x, int* v) {
    if (x.empty() || x.size() > 7) return false;
    for (char c : x)
      if (c < '0' || c > '9') return false;
    *v = std::atoi(x.c_str());
    return true;
  };
  if (t.rfind("ring", 0) == 0) {
    int n = 0;
    if (!to_int(t.substr(4), &n) || n < 1) return false;
    *out = Shape::make_ring(n);
    return true;
  }
  const size_t plus = t.find('+');
  if (plus != std::string::npos) {
    if (!to_int(t.substr(plus + 1), &s.lonely)) return false;
    t = t.substr(0, plus);
  }
  std::string tok;
  for (size_t i = 0; i <= t.size(); ++i) {
    if (i == t.size() || t[i] == '*' || t[i] == 'x' || t[i] == ',') {
      if (tok.empty()) continue;
      int w = 0;
      if (!to_int(tok, &w) || w < 1) return false;
      s.widths.push_back(w);
      tok.clear();
    } else {
      tok.push_back(t[i]);
    }
  }
  if (s.widths.empty()) return false;
  *out = s;
  return true;
}

struct PolicyChoice {
  std::string algo;   // "ll", "oneshot", "staged", "push", "nvls", "nvls1", "hybrid"
  Shape shape;        // the plan for "staged"; flat for the others
  double hybrid_bytes = 0.7, hybrid_lanes = 0.5;   // split of "hybrid" (share of each block / of the CTAs in the switch)
  bool from_table = false;
};

class Policy {
 public:
  static constexpr uint64_t kLLMaxBytes = 256u << 10;   // largest message of the low-latency protocol
  static constexpr size_t kCacheEntries = 4096;         // answers remembered per policy before the cache starts over

  explicit Policy(int world) : world_(world) {}
  int world() const { return world_; }

  void set_params(const V1Params& k) { std::lock_guard<std::mutex> lk(mu_); params_ = k; cache_.clear(); }
  V1Params params() const { std::lock_guard<std::mutex> lk(mu_); return params_; }
  void clear_rows() { std::lock_guard<std::mutex> lk(mu_); rows_.clear(); cache_.clear(); }
  size_t num_rows() const { std::lock_guard<std::mutex> lk(mu_); return rows_.size(); }
  // one measured winner: at `bytes`, `algo` ("hybrid-<bytes share>-<lane share>" carries its split) with `shape`
  bool add_row(uint64_t bytes, const std::string& algo, const std::string& shape_text) {
    Row r;
    r.bytes = bytes;
    r.algo = algo;
    if (algo.rfind("hybrid", 0) == 0) {
      r.algo = "hybrid";
      double a = 0.7, b = 0.5;
      if (std::sscanf(algo.c_str(), "hybrid-%lf-%lf", &a, &b) == 2) { r.hybrid_bytes = a; r.hybrid_lanes = b; }
    }
    if (r.algo != "ll" && r.algo != "oneshot" && r.algo != "staged" && r.algo != "push" && r.algo != "nvls" && r.algo != "hybrid" &&
        r.algo != "nvls1")
      return false;
    if (!parse_shape_text(shape_text, &r.shape) || !validate_shape(world_, r.shape).empty()) return false;
    std::lock_guard<std::mutex> lk(mu_);
    rows_.push_back(r);
    cache_.clear();
    return true;
  }

  // Reads {"params": {...}, "table": {"<world>": [[bytes, algo, shape, ...], ...]}}.  Rows that do not
  // parse are skipped and counted in *skipped.  False when the file cannot be read or is not JSON.
  bool load(const std::string& path, std::string* err = nullptr, int* skipped = nullptr) {
    std::ifstream f(path);
    if (!f) { if (err) *err = "cannot open " + path; return false; }
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string text = ss.str();
    Json root;
    JsonParser p(text);
    if (!p.parse(&root)) { if (err) *err = path + ": " + p.err(); return false; }
    if (const Json* pj = root.get("params")) {
      V1Params k = params();
      k.launch_us = field(pj, "launch_us", k.launch_us);
      k.sync_us = field(pj, "sync_us", k.sync_us);
      k.link_gbs = field(pj, "link_gbs", k.link_gbs);
      k.hbm_gbs = field(pj, "hbm_gbs", k.hbm_gbs);
      k.stage_floor_us = field(pj, "stage_floor_us", k.stage_floor_us);
      k.nvls_gbs = field(pj, "nvls_gbs", k.nvls_gbs);
      k.oneshot_max_bytes = field(pj, "oneshot_max_bytes", k.oneshot_max_bytes);
      k.ll_us = field(pj, "ll_us", k.ll_us);
      k.ll_max_bytes = field(pj, "ll_max_bytes", k.ll_max_bytes);
      k.push_gain = field(pj, "push_gain", k.push_gain);
      if (const Json* pe = pj->get("peer_eff"))
        for (auto& kv : pe->obj) {
          const int idx = std::atoi(kv.first.c_str());
          if (idx >= 0 && idx < (int)k.peer_eff.size() && kv.second.kind == Json::Num) k.peer_eff[idx] = kv.second.num;
        }
      set_params(k);
    }
    int bad = 0;
    clear_rows();
    if (const Json* tj = root.get("table"))
      if (const Json* rows = tj->get(std::to_string(world_)))
        for (const Json& r : rows->arr) {
          if (r.kind != Json::Arr || r.arr.size() < 3 || r.arr[0].kind != Json::Num || r.arr[1].kind != Json::Str ||
              r.arr[2].kind != Json::Str || !add_row((uint64_t)r.arr[0].num, r.arr[1].str, r.arr[2].str))
            ++bad;
        }
    if (skipped) *skipped = bad;
    return true;
  }

  // shapes of the staged rows (the plans a communicator builds ahead of the first call)
  std::vector<Shape> table_shapes() const {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<Shape> out;
    for (const Row& r : rows_) {
      if (r.algo != "staged") continue;
      bool seen = false;
      for (const Shape& s : out) seen = seen || s.str() == r.shape.str();
      if (!seen) out.push_back(r.shape);
    }
    return out;
  }

  // in_heap: the tensor is 16-byte aligned inside the symmetric heap (reduce+push and NVLS work in place only);
  // nvls_ok: multicast is bound and the message qualifies (in_heap, float type, multiple of 16 bytes);
  // staging_bytes: size of one staging slot (one-shot must fit); ll_auto_max: below it the low-latency protocol
  // is taken when neither the table nor the model speaks.
  // nvls1_ok: multicast is bound and the type is one the switch reduces (the one-shot form stages through the slots,
  // so the tensor need not live in the heap).
  PolicyChoice choose(uint64_t bytes, bool in_heap, bool nvls_ok, uint64_t staging_bytes, uint64_t ll_auto_max, bool nvls1_ok = false) {
    if (!in_heap) nvls_ok = false;
    const Key key{bytes, in_heap, nvls_ok, staging_bytes, ll_auto_max, nvls1_ok};
    std::lock_guard<std::mutex> lk(mu_);
    auto it = cache_.find(key);
    if (it != cache_.end()) return it->second;
    PolicyChoice c;
    const Row* best = nullptr;
    uint64_t lo = ~0ull, hi = 0;
    double best_d = 0;
    const double lb = std::log((double)(bytes ? bytes : 1));
    for (const Row& r : rows_) {
      if (!nvls_ok && (r.algo == "nvls" || r.algo == "hybrid")) continue;
      if (!in_heap && r.algo == "push") continue;
      if (r.algo == "oneshot" && bytes > staging_bytes) continue;
      if (r.algo == "nvls1" && (!nvls1_ok || bytes > staging_bytes)) continue;
      if (r.algo == "ll" && bytes > kLLMaxBytes) continue;
      lo = r.bytes < lo ? r.bytes : lo;
      hi = r.bytes > hi ? r.bytes : hi;
      const double d = std::fabs(std::log((double)(r.bytes ? r.bytes : 1)) - lb);
      if (!best || d < best_d) { best = &r; best_d = d; }
    }
    // the table speaks only for the range of sizes that was measured (one octave of slack)
    if (best && lo / 2 <= bytes && bytes <= hi * 2) {
      c.algo = best->algo;
      // "staged" runs the row's plan; "ll" with a shape that is not flat runs that plan on tagged words
      c.shape = (best->algo == "staged" || best->algo == "ll") ? best->shape : Shape::flat(world_);
      c.hybrid_bytes = best->hybrid_bytes;
      c.hybrid_lanes = best->hybrid_lanes;
      c.from_table = true;
    } else if (bytes <= ll_auto_max && bytes <= kLLMaxBytes && world_ > 1) {
      c.algo = "ll";
      c.shape = Shape::flat(world_);
    } else {
      V1Choice m = pick_algorithm(world_, bytes, params_, bytes <= staging_bytes, nvls_ok, in_heap, nvls1_ok && bytes <= staging_bytes);
      c.algo = m.algo;
      c.shape = m.shape;
    }
    if (cache_.size() >= kCacheEntries) cache_.clear();   // a caller with endlessly varying sizes must not grow it without bound
    cache_.emplace(key, c);
    return c;
  }

 private:
  struct Row {
    uint64_t bytes = 0;
    std::string algo;
    Shape shape;
    double hybrid_bytes = 0.7, hybrid_lanes = 0.5;
  };
  using Key = std::tuple<uint64_t, bool, bool, uint64_t, uint64_t, bool>;
  static double field(const Json* obj, const char* name, double dflt) {
    const Json* v = obj->get(name);
    return v ? v->number_or(dflt) : dflt;
  }
  int world_;
  mutable std::mutex mu_;
  V1Params params_;
  std::vector<Row> rows_;
  std::map<Key, PolicyChoice> cache_;
};

}  // namespace ft
