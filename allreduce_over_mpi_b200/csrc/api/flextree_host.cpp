// Host half of the C API: planner, cost models, configuration, CPU executors.
// Pure C++17; nothing here touches CUDA, so it runs (and is tested) without a GPU.
#include <dlfcn.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <sstream>
#include <string>

#include "../planner/config.hpp"
#include "../planner/cost_model.hpp"
#include "../planner/cpu_executor.hpp"
#include "../planner/factorize.hpp"
#include "../planner/plan.hpp"
#include "policy_handle.hpp"
#include "../planner/proc_world.hpp"
#include "flextree.h"
#include "../runtime/dev_plan.hpp"

namespace {

size_t put(const std::string& s, char* buf, size_t cap) {
  if (buf && cap) {
    size_t n = s.size() < cap - 1 ? s.size() : cap - 1;
    std::memcpy(buf, s.data(), n);
    buf[n] = '\0';
  }
  return s.size();
}

ft::Shape make_shape(const int* widths, int nw, int lonely, int ring) {
  ft::Shape s;
  if (widths && nw > 0) s.widths.assign(widths, widths + nw);
  s.lonely = lonely;
  s.ring = ring != 0;
  return s;
}

// Plans depend on (world, shape) only; they are built once and shared.
const ft::Plan& cached_plan(int world, const ft::Shape& s) {
  static std::mutex mu;
  static std::map<std::string, ft::Plan> cache;
  std::string key = std::to_string(world) + ":" + s.str();
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it == cache.end()) it = cache.emplace(key, ft::build_plan(world, s)).first;
  return it->second;
}

ft::V1Params to_params(const ft_v1_params* p) {
  ft::V1Params k;
  if (!p) return k;
  k.launch_us = p->launch_us; k.sync_us = p->sync_us; k.link_gbs = p->link_gbs; k.hbm_gbs = p->hbm_gbs;
  k.stage_floor_us = p->stage_floor_us; k.nvls_gbs = p->nvls_gbs; k.oneshot_max_bytes = p->oneshot_max_bytes;
  k.ll_us = p->ll_us; k.ll_max_bytes = p->ll_max_bytes; k.push_gain = p->push_gain;
  k.peer_eff.assign(p->peer_eff, p->peer_eff + FT_MAX_RANKS + 1);
  return k;
}

}  // namespace

struct ft_cpu_world { ft::CpuWorld w; };

// C form of a policy answer (also used by the communicator runtime)
void ft_policy_fill_choice(const ft::PolicyChoice& c, ft_choice* out) {
  std::memset(out, 0, sizeof *out);
  static const char* names[] = {"auto", "staged", "oneshot", "nvls", "hybrid", "ll", "push", "", "", "nvls1"};
  out->algo = FT_ALGO_STAGED;
  for (int i = 1; i < 10; ++i)
    if (names[i][0] && c.algo == names[i]) out->algo = i;
  std::snprintf(out->algo_name, sizeof out->algo_name, "%s", names[out->algo]);
  out->nw = (int)(c.shape.widths.size() < 16 ? c.shape.widths.size() : 16);
  for (int i = 0; i < out->nw; ++i) out->widths[i] = c.shape.widths[i];
  out->lonely = c.shape.lonely;
  out->ring = c.shape.ring ? 1 : 0;
  out->from_table = c.from_table ? 1 : 0;
  out->hybrid_bytes = c.hybrid_bytes;
  out->hybrid_lanes = c.hybrid_lanes;
}

extern "C" {

const char* ft_version(void) { return "flextree-b200 0.1"; }

int ft_prime_factors(int n, int* out, int cap) {
  auto v = ft::prime_factors(n);
  for (int i = 0; i < (int)v.size() && i < cap; ++i) out[i] = v[i];
  return (int)v.size();
}
int ft_is_prime(int n) { return ft::is_prime(n); }
int ft_is_prime_loose(int n) { return ft::is_prime_loose(n); }
uint64_t ft_count_ordered_factorizations(int n) { return ft::count_ordered_factorizations(n); }

size_t ft_candidate_shapes(int n, int legacy, char* buf, size_t cap) {
  std::string s;
  for (auto& w : (legacy ? ft::candidate_shapes_legacy(n) : ft::candidate_shapes(n))) s += ft::shape_to_string(w) + "\n";
  return put(s, buf, cap);
}
size_t ft_choose_width(int world, char* buf, size_t cap) {
  std::string s;
  for (auto& c : ft::choose_width(world)) s += ft::shape_to_string(c) + "\n";
  return put(s, buf, cap);
}

double ft_cost_v0(const int* widths, int nw, int n, double chunk) {
  return ft::cost_v0(ft::Widths(widths, widths + nw), n, chunk);
}
int ft_choose_v0(int n, double chunk, int* widths, int cap, double* cost, uint64_t* ncand) {
  auto c = ft::choose_v0(n, chunk);
  for (int i = 0; i < (int)c.widths.size() && i < cap; ++i) widths[i] = c.widths[i];
  if (cost) *cost = c.cost;
  if (ncand) *ncand = c.candidates;
  return (int)c.widths.size();
}

void ft_v1_defaults(ft_v1_params* p) {
  ft::V1Params k;
  p->launch_us = k.launch_us; p->sync_us = k.sync_us; p->link_gbs = k.link_gbs; p->hbm_gbs = k.hbm_gbs;
  p->stage_floor_us = k.stage_floor_us; p->nvls_gbs = k.nvls_gbs; p->oneshot_max_bytes = k.oneshot_max_bytes;
  p->ll_us = k.ll_us; p->ll_max_bytes = k.ll_max_bytes; p->push_gain = k.push_gain;
  for (int i = 0; i <= FT_MAX_RANKS; ++i) p->peer_eff[i] = 1.0;
}
double ft_cost_v1(int world, const int* widths, int nw, int lonely, int ring, uint64_t bytes, const ft_v1_params* p) {
  return ft::cost_v1(cached_plan(world, make_shape(widths, nw, lonely, ring)), bytes, to_params(p));
}
double ft_cost_v1_oneshot(int world, uint64_t bytes, const ft_v1_params* p) { return ft::cost_v1_oneshot(world, bytes, to_params(p)); }
double ft_cost_v1_nvls(int world, uint64_t bytes, const ft_v1_params* p) { return ft::cost_v1_nvls(world, bytes, to_params(p)); }
int ft_pick_algorithm(int world, uint64_t bytes, const ft_v1_params* p, int allow_oneshot, int allow_nvls, int* widths,
                      int cap, int* lonely, int* ring, char* algo_out, size_t algo_cap, double* us) {
  auto c = ft::pick_algorithm(world, bytes, to_params(p), allow_oneshot != 0, allow_nvls != 0);
  for (int i = 0; i < (int)c.shape.widths.size() && i < cap; ++i) widths[i] = c.shape.widths[i];
  if (lonely) *lonely = c.shape.lonely;
  if (ring) *ring = c.shape.ring;
  if (us) *us = c.us;
  put(c.algo, algo_out, algo_cap);
  return (int)c.shape.widths.size();
}
int ft_pick_algorithm2(int world, uint64_t bytes, const ft_v1_params* p, int allow_oneshot, int allow_nvls, int allow_push,
                       int* widths, int cap, int* lonely, int* ring, char* algo_out, size_t algo_cap, double* us) {
  auto c = ft::pick_algorithm(world, bytes, to_params(p), allow_oneshot != 0, allow_nvls != 0, allow_push != 0);
  for (int i = 0; i < (int)c.shape.widths.size() && i < cap; ++i) widths[i] = c.shape.widths[i];
  if (lonely) *lonely = c.shape.lonely;
  if (ring) *ring = c.shape.ring;
  if (us) *us = c.us;
  put(c.algo, algo_out, algo_cap);
  return (int)c.shape.widths.size();
}

// ---- selection policy
ft_policy* ft_policy_create(int world) {
  if (world < 1 || world > FT_MAX_RANKS) return nullptr;
  return new ft_policy(world);
}
void ft_policy_destroy(ft_policy* p) { delete p; }
size_t ft_policy_default_path(char* buf, size_t cap) {
  std::string path;
  if (const char* e = std::getenv("FT_CALIBRATION"); e && *e) {
    path = e;
  } else {
    Dl_info info;
    if (dladdr((const void*)&ft_policy_default_path, &info) && info.dli_fname) {
      std::string lib = info.dli_fname;   // .../allreduce_over_mpi_b200/lib/libflextree.so
      const size_t slash = lib.rfind('/');
      const std::string dir = slash == std::string::npos ? std::string(".") : lib.substr(0, slash);
      path = dir + "/../parallel/calibration_b200.json";
    }
  }
  return put(path, buf, cap);
}
int ft_policy_load(ft_policy* p, const char* path, char* err, size_t err_cap) {
  if (!p) return FT_ERR_INVALID_ARG;
  char dflt[1024];
  if (!path || !*path) { ft_policy_default_path(dflt, sizeof dflt); path = dflt; }
  std::string why;
  int skipped = 0;
  if (!p->p.load(path, &why, &skipped)) { put(why, err, err_cap); return FT_ERR_NOT_AVAILABLE; }
  put(skipped ? std::to_string(skipped) + " table rows skipped (unknown algorithm or invalid shape)" : "", err, err_cap);
  return FT_OK;
}
int ft_policy_set_params(ft_policy* p, const ft_v1_params* k) {
  if (!p || !k) return FT_ERR_INVALID_ARG;
  p->p.set_params(to_params(k));
  return FT_OK;
}
int ft_policy_get_params(ft_policy* p, ft_v1_params* out) {
  if (!p || !out) return FT_ERR_INVALID_ARG;
  const ft::V1Params k = p->p.params();
  out->launch_us = k.launch_us; out->sync_us = k.sync_us; out->link_gbs = k.link_gbs; out->hbm_gbs = k.hbm_gbs;
  out->stage_floor_us = k.stage_floor_us; out->nvls_gbs = k.nvls_gbs; out->oneshot_max_bytes = k.oneshot_max_bytes;
  out->ll_us = k.ll_us; out->ll_max_bytes = k.ll_max_bytes; out->push_gain = k.push_gain;
  for (int i = 0; i <= FT_MAX_RANKS; ++i) out->peer_eff[i] = i < (int)k.peer_eff.size() ? k.peer_eff[i] : 1.0;
  return FT_OK;
}
void ft_policy_clear_rows(ft_policy* p) { if (p) p->p.clear_rows(); }
int ft_policy_num_rows(ft_policy* p) { return p ? (int)p->p.num_rows() : 0; }
int ft_policy_add_row(ft_policy* p, uint64_t bytes, const char* algo, const char* shape) {
  if (!p || !algo || !shape) return FT_ERR_INVALID_ARG;
  return p->p.add_row(bytes, algo, shape) ? FT_OK : FT_ERR_INVALID_ARG;
}
int ft_policy_choose(ft_policy* p, uint64_t bytes, int in_heap, int nvls_ok, uint64_t staging_bytes, uint64_t ll_auto_max,
                     int nvls1_ok, ft_choice* out) {
  if (!p || !out) return FT_ERR_INVALID_ARG;
  ft_policy_fill_choice(p->p.choose(bytes, in_heap != 0, nvls_ok != 0, staging_bytes, ll_auto_max, nvls1_ok != 0), out);
  return FT_OK;
}

size_t ft_executable_shapes(int world, char* buf, size_t cap) {
  std::string s;
  for (auto& sh : ft::executable_shapes(world)) s += sh.str() + "\n";
  return put(s, buf, cap);
}

int ft_parse_topo(const char* topo, const char* lonely_str, int world, int* widths, int cap, int* nw, int* lonely,
                  int* ring, int* is_auto, char* err, size_t err_cap) {
  auto c = ft::parse_topo(topo ? topo : "", lonely_str ? lonely_str : "", world);
  if (!c.ok()) { put(c.error, err, err_cap); return FT_ERR_INVALID_TOPO; }
  for (int i = 0; i < (int)c.shape.widths.size() && i < cap; ++i) widths[i] = c.shape.widths[i];
  if (nw) *nw = (int)c.shape.widths.size();
  if (lonely) *lonely = c.shape.lonely;
  if (ring) *ring = c.shape.ring;
  if (is_auto) *is_auto = c.is_auto;
  put("", err, err_cap);
  return FT_OK;
}

int ft_validate_shape(int world, const int* widths, int nw, int lonely, int ring, char* err, size_t err_cap) {
  std::string e = ft::validate_shape(world, make_shape(widths, nw, lonely, ring));
  put(e, err, err_cap);
  return e.empty() ? FT_OK : FT_ERR_INVALID_TOPO;
}
int ft_plan_check(int world, const int* widths, int nw, int lonely, int ring, char* err, size_t err_cap) {
  std::string e = ft::check_hazards(cached_plan(world, make_shape(widths, nw, lonely, ring)));
  put(e, err, err_cap);
  return e.empty() ? FT_OK : FT_ERR_INVALID_TOPO;
}
int ft_plan_num_stages(int world, const int* widths, int nw, int lonely, int ring) {
  const auto& p = cached_plan(world, make_shape(widths, nw, lonely, ring));
  return p.ok() ? p.num_stages : -1;
}
int ft_plan_max_fanin(int world, const int* widths, int nw, int lonely, int ring) {
  const auto& p = cached_plan(world, make_shape(widths, nw, lonely, ring));
  return p.ok() ? ft::plan_stats(p).max_fan_in : -1;
}
uint64_t ft_plan_traffic(int world, const int* widths, int nw, int lonely, int ring, uint64_t count,
                         uint64_t block_elems) {
  const auto& p = cached_plan(world, make_shape(widths, nw, lonely, ring));
  if (!p.ok()) return 0;
  return ft::plan_traffic_elems(p, ft::Blocks(count, world, block_elems));
}
size_t ft_plan_describe(int world, const int* widths, int nw, int lonely, int ring, int rank, uint64_t count,
                        uint64_t block_elems, char* buf, size_t cap) {
  const auto& p = cached_plan(world, make_shape(widths, nw, lonely, ring));
  if (p.ok() && (rank < 0 || rank >= world)) return put("invalid rank\n", buf, cap);
  return put(ft::describe(p, rank, count, block_elems), buf, cap);
}
size_t ft_plan_json(int world, const int* widths, int nw, int lonely, int ring, char* buf, size_t cap) {
  const auto& p = cached_plan(world, make_shape(widths, nw, lonely, ring));
  std::ostringstream os;
  if (!p.ok()) {
    os << "{\"error\":\"" << p.error << "\"}";
    return put(os.str(), buf, cap);
  }
  os << "{\"world\":" << p.world << ",\"shape\":\"" << p.shape.str() << "\",\"stages\":" << p.num_stages << ",\"ranks\":[";
  for (int r = 0; r < p.world; ++r) {
    os << (r ? "," : "") << "[";
    for (int s = 0; s < p.num_stages; ++s) {
      const auto& st = p.stages[r][s];
      os << (s ? "," : "") << "{\"rs\":" << (st.reduce_scatter ? 1 : 0) << ",\"sync\":[";
      for (size_t i = 0; i < p.sync[s][r].size(); ++i) os << (i ? "," : "") << p.sync[s][r][i];
      os << "],\"pulls\":[";
      for (size_t i = 0; i < st.pulls.size(); ++i) {
        os << (i ? "," : "") << "[" << st.pulls[i].block << "," << (st.pulls[i].reduce ? 1 : 0) << ",[";
        for (size_t j = 0; j < st.pulls[i].srcs.size(); ++j) os << (j ? "," : "") << st.pulls[i].srcs[j];
        os << "]]";
      }
      os << "]}";
    }
    os << "]";
  }
  os << "],\"end_sync\":[";
  for (int r = 0; r < p.world; ++r) {
    os << (r ? "," : "") << "[";
    for (size_t i = 0; i < p.sync[p.num_stages][r].size(); ++i) os << (i ? "," : "") << p.sync[p.num_stages][r][i];
    os << "]";
  }
  os << "]}";
  return put(os.str(), buf, cap);
}

int ft_cpu_reduce(int op, int dtype, const void* const* src, void* dst, int n, size_t len, int threads) {
  if (n < 0 || (n > 0 && (!src || !dst))) return FT_ERR_INVALID_ARG;
  return ft::reduce_nway_cpu_dispatch((ft_op)op, (ft_dtype)dtype, src, dst, n, len, threads);
}
int ft_run_plan_snapshot(int world, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                         void* const* bufs, uint64_t count, uint64_t block_elems) {
  return ft::run_plan_snapshot(cached_plan(world, make_shape(widths, nw, lonely, ring)), (ft_op)op, (ft_dtype)dtype,
                               bufs, count, block_elems);
}

// ---- process-per-rank world (one host, ranks are processes) ------------------------------------
struct ft_proc_world { ft::ProcWorld w; };

ft_proc_world* ft_proc_world_join(const char* session, int rank, int world, double timeout_s, char* err, size_t err_cap) {
  auto* h = new ft_proc_world;
  if (!session || !h->w.join(session, rank, world, timeout_s)) {
    put(session ? h->w.error : "no session name", err, err_cap);
    delete h;
    return nullptr;
  }
  put("", err, err_cap);
  return h;
}
void ft_proc_world_leave(ft_proc_world* h) { delete h; }
int ft_proc_world_rank(ft_proc_world* h) { return h ? h->w.rank : -1; }
int ft_proc_world_size(ft_proc_world* h) { return h ? h->w.n : 0; }
int ft_proc_barrier(ft_proc_world* h) { return h ? h->w.barrier().code : FT_ERR_INVALID_ARG; }
const char* ft_proc_last_error(ft_proc_world* h) { return h ? h->w.error.c_str() : "null world"; }
int ft_proc_phase(ft_proc_world* h, const int* widths, int nw, int lonely, int ring, int op, int dtype, void* buf,
                  uint64_t count, int phase, int* status_out) {
  if (!h || (phase != 1 && phase != 2)) return FT_ERR_INVALID_ARG;
  const auto& p = cached_plan(h->w.n, make_shape(widths, nw, lonely, ring));
  ft::RankStatus st = h->w.allreduce(p, (ft_op)op, (ft_dtype)dtype, nullptr, buf, count, phase);
  if (status_out) { status_out[0] = st.code; status_out[1] = st.stage; status_out[2] = st.peer; }
  return st.code;
}
int ft_proc_heap_create(ft_proc_world* h, size_t bytes) { return h && h->w.heap_create(bytes) ? FT_OK : FT_ERR_NOT_AVAILABLE; }
void* ft_proc_alloc(ft_proc_world* h, size_t bytes) { return h ? h->w.heap_alloc(bytes) : nullptr; }
int ft_proc_free(ft_proc_world* h, void* p) { return h && h->w.heap_free(p) ? FT_OK : FT_ERR_INVALID_ARG; }
int ft_proc_heap_symmetric(ft_proc_world* h, const void* p) { return h && h->w.heap_symmetric(p) ? 1 : 0; }
int ft_proc_allreduce(ft_proc_world* h, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                      const void* sendbuf, void* recvbuf, uint64_t count, int* status_out) {
  if (!h) return FT_ERR_INVALID_ARG;
  const auto& p = cached_plan(h->w.n, make_shape(widths, nw, lonely, ring));
  ft::RankStatus st = h->w.allreduce(p, (ft_op)op, (ft_dtype)dtype, sendbuf, recvbuf, count);
  if (status_out) { status_out[0] = st.code; status_out[1] = st.stage; status_out[2] = st.peer; }
  return st.code;
}

size_t ft_context_describe(int world, int rank, int lonely, uint64_t count, int dtype, char* buf, size_t cap) {
  // the fields of the reference's per-call context, in its order and spelling (mpi_mod.hpp:776-801)
  const uint64_t split = world > 0 ? (count + world - 1) / (uint64_t)world : 0;
  std::ostringstream os;
  os << "num_nodes=" << world << ", node_label=" << rank << ", num_lonely=" << lonely << ", data_size=" << count
     << ", num_split=" << world - lonely << ", split_size=" << split << ", data_size_aligned=" << split * (uint64_t)world
     << ", type_size=" << ft_dtype_size((ft_dtype)dtype) << ", has_lonely=" << (lonely > 0 ? 1 : 0) << "\n";
  return put(os.str(), buf, cap);
}

int ft_run_plan_snapshot_range(int world, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                               void* const* bufs, uint64_t count, uint64_t block_elems, int stage_begin, int stage_end) {
  return ft::run_plan_snapshot(cached_plan(world, make_shape(widths, nw, lonely, ring)), (ft_op)op, (ft_dtype)dtype,
                               bufs, count, block_elems, stage_begin, stage_end);
}
int ft_plan_rs_holders(int world, const int* widths, int nw, int lonely, int ring, uint64_t* holders) {
  const auto& p = cached_plan(world, make_shape(widths, nw, lonely, ring));
  if (!p.ok() || !holders || world > 64) return FT_ERR_INVALID_TOPO;
  const std::vector<uint64_t> h = ft::rs_holders(p);
  for (int b = 0; b < world; ++b) holders[b] = h[b];
  return FT_OK;
}

int ft_dev_plan_check(int world, const int* widths, int nw, int lonely, int ring, int rank, char* err, size_t err_cap) {
  const auto& p = cached_plan(world, make_shape(widths, nw, lonely, ring));
  if (!p.ok()) { put(p.error, err, err_cap); return FT_ERR_INVALID_TOPO; }
  if (rank < 0 || rank >= world) { put("invalid rank", err, err_cap); return FT_ERR_INVALID_ARG; }
  const std::string e = ft::check_dev_plan(ft::build_dev_plan(p, rank), world, rank);
  put(e, err, err_cap);
  return e.empty() ? FT_OK : FT_ERR_INVALID_TOPO;
}

ft_cpu_world* ft_cpu_world_create(int world, double timeout_s) {
  if (world < 1 || world > 4096) return nullptr;
  auto* w = new ft_cpu_world{ft::CpuWorld(world)};
  if (timeout_s > 0) w->w.timeout_s = timeout_s;
  return w;
}
void ft_cpu_world_destroy(ft_cpu_world* w) { delete w; }
int ft_cpu_allreduce(ft_cpu_world* w, int rank, const int* widths, int nw, int lonely, int ring, int op, int dtype,
                     const void* sendbuf, void* recvbuf, uint64_t count, uint64_t block_elems, int fault_kind,
                     int fault_rank, int fault_stage, int* status_out) {
  if (!w || rank < 0 || rank >= w->w.n) return FT_ERR_INVALID_ARG;
  ft::FaultSpec f;
  f.kind = (ft::Fault)fault_kind;
  f.rank = fault_rank;
  f.stage = fault_stage;
  const auto& p = cached_plan(w->w.n, make_shape(widths, nw, lonely, ring));
  ft::RankStatus st = ft::cpu_allreduce(w->w, rank, p, (ft_op)op, (ft_dtype)dtype, sendbuf, recvbuf, count,
                                        block_elems, fault_kind ? &f : nullptr);
  if (status_out) { status_out[0] = st.code; status_out[1] = st.stage; status_out[2] = st.peer; }
  return st.code;
}
int ft_cpu_phase(ft_cpu_world* w, int rank, const int* widths, int nw, int lonely, int ring, int op, int dtype, void* buf,
                 uint64_t count, uint64_t block_elems, int phase, int* status_out) {
  if (!w || rank < 0 || rank >= w->w.n || (phase != 1 && phase != 2)) return FT_ERR_INVALID_ARG;
  const auto& p = cached_plan(w->w.n, make_shape(widths, nw, lonely, ring));
  ft::RankStatus st = ft::cpu_allreduce(w->w, rank, p, (ft_op)op, (ft_dtype)dtype, nullptr, buf, count, block_elems, nullptr, 1, phase);
  if (status_out) { status_out[0] = st.code; status_out[1] = st.stage; status_out[2] = st.peer; }
  return st.code;
}

}  // extern "C"
